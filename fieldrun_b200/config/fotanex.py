"""Configuration of the Fotanex design, read from its own config.json keys.

The file names the design as ``"architecture": "Fotanex"`` and lists the layers one by one:

    vocab, width                       sizes of the vocabulary and of the residual stream
    norm.eps                           eps of the root-mean-square divisions inside the mixers
    loop {start, stop, times}          layers start .. stop-1 run ``times`` times in a row (absent: every layer once)
    layers[i].type                     "rglru" | "mamba2" | "parallel"
    layers[i].mixer                    the mixer's sizes and constants (below)
    layers[i].mlp                      {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}} or null

    rglru:     width, blocks, conv
    mamba2:    heads, vdim, state, groups, norm_groups, conv
    parallel:  left  {heads, kv_heads, dim, vdim, scale, mask {size}}      attention in chunks, with a sink and a gate
               right {inner, state, dt_rank, conv}                         selective scan

Everything that can differ between two models of the design is read here; what the design fixes (the recurrent
unit's constant 8, the activations, the 1e-20 of the experts' weights) lives with the parts that the plan names
(``models/fotanex.py``).  A key the design does not have is a warning on stderr.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .base import ConfigError, KeyReader, ModelConfig

ARCHITECTURE = "Fotanex"


def _unknown(raw: Mapping[str, Any], allowed: set[str], where: str) -> None:
    extra = sorted(set(raw) - allowed)
    if extra:
        print(f"{where}: warning: keys this design does not have are ignored: {', '.join(extra)}", file=sys.stderr)


def _object(raw: Any, where: str) -> Mapping[str, Any]:
    if not isinstance(raw, Mapping):
        raise ConfigError(f"{where} must be an object")
    return raw


@dataclass(frozen=True)
class FotanexRglru:
    width: int
    blocks: int
    conv: int

    def to_json(self) -> dict[str, Any]:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class FotanexMamba2:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    def to_json(self) -> dict[str, Any]:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                "norm_groups": self.norm_groups, "conv": self.conv}


@dataclass(frozen=True)
class FotanexChunkAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int]                  # None: a file without a mask; every earlier key is seen

    def to_json(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        return out


@dataclass(frozen=True)
class FotanexScan:
    inner: int
    state: int
    dt_rank: int
    conv: int

    def to_json(self) -> dict[str, Any]:
        return {"inner": self.inner, "state": self.state, "dt_rank": self.dt_rank, "conv": self.conv}


@dataclass(frozen=True)
class FotanexParallel:
    left: FotanexChunkAttention
    right: FotanexScan

    def to_json(self) -> dict[str, Any]:
        return {"left": self.left.to_json(), "right": self.right.to_json()}


@dataclass(frozen=True)
class FotanexExperts:
    experts: int
    top: int
    ff: int

    def to_json(self) -> dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class FotanexLayer:
    type: str
    mixer: Any                            # FotanexRglru | FotanexMamba2 | FotanexParallel
    mlp: Optional[FotanexExperts]

    def to_json(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": self.mlp.to_json() if self.mlp else None}


@dataclass(frozen=True)
class FotanexLoop:
    start: int
    stop: int
    times: int

    def to_json(self) -> dict[str, Any]:
        return {"start": self.start, "stop": self.stop, "times": self.times}


def _rglru(raw: Mapping[str, Any], where: str) -> FotanexRglru:
    _unknown(raw, {"width", "blocks", "conv"}, where)
    r = KeyReader(raw, where)
    width, blocks = r.integer("width", minimum=1), r.integer("blocks", default=1, minimum=1)
    if width % blocks:
        raise ConfigError(f"{where}: a width of {width} does not divide into {blocks} blocks")
    return FotanexRglru(width, blocks, r.integer("conv", minimum=1))


def _mamba2(raw: Mapping[str, Any], where: str) -> FotanexMamba2:
    _unknown(raw, {"heads", "vdim", "state", "groups", "norm_groups", "conv"}, where)
    r = KeyReader(raw, where)
    heads, vdim = r.integer("heads", minimum=1), r.integer("vdim", minimum=1)
    groups = r.integer("groups", default=1, minimum=1)
    norm_groups = r.integer("norm_groups", default=1, minimum=1)
    if heads % groups:
        raise ConfigError(f"{where}: {heads} heads are not a multiple of {groups} groups")
    if (heads * vdim) % norm_groups:
        raise ConfigError(f"{where}: {heads} x {vdim} channels do not divide into {norm_groups} norm_groups")
    return FotanexMamba2(heads, vdim, r.integer("state", minimum=1), groups, norm_groups, r.integer("conv", minimum=1))


def _parallel(raw: Mapping[str, Any], where: str) -> FotanexParallel:
    _unknown(raw, {"left", "right"}, where)
    left, right = _object(raw.get("left"), where + ".left"), _object(raw.get("right"), where + ".right")
    _unknown(left, {"heads", "kv_heads", "dim", "vdim", "scale", "mask"}, where + ".left")
    _unknown(right, {"inner", "state", "dt_rank", "conv"}, where + ".right")
    a = KeyReader(left, where + ".left")
    heads = a.integer("heads", minimum=1)
    kv_heads = a.integer("kv_heads", default=heads, minimum=1)
    if heads % kv_heads:
        raise ConfigError(f"{where}.left: {heads} heads are not a multiple of {kv_heads} kv_heads")
    dim = a.integer("dim", minimum=1)
    chunk = None
    if left.get("mask") is not None:
        _unknown(_object(left["mask"], where + ".left.mask"), {"size"}, where + ".left.mask")
        chunk = a.integer("mask.size", minimum=1)
    attention = FotanexChunkAttention(heads, kv_heads, dim, a.integer("vdim", default=dim, minimum=1),
                                      a.real("scale", default=float(dim) ** -0.5, positive=True), chunk)
    s = KeyReader(right, where + ".right")
    scan = FotanexScan(s.integer("inner", minimum=1), s.integer("state", minimum=1), s.integer("dt_rank", minimum=1),
                       s.integer("conv", minimum=1))
    return FotanexParallel(attention, scan)


_MIXERS = {"rglru": _rglru, "mamba2": _mamba2, "parallel": _parallel}


@dataclass(frozen=True)
class FotanexConfig(ModelConfig):
    norm_eps: float = 1e-6
    layers: tuple[FotanexLayer, ...] = ()
    loop: Optional[FotanexLoop] = None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "FotanexConfig":
        _unknown(raw, {"architecture", "architectures", "model_type", "vocab", "width", "norm", "layers", "loop",
                       "eos_token_id"}, where)
        r = KeyReader(raw, where)
        if isinstance(raw.get("norm"), Mapping):
            _unknown(raw["norm"], {"eps"}, f"{where}: norm")
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError(f"{where}: key 'layers' must be a list of at least one layer")
        layers: list[FotanexLayer] = []
        for index, entry in enumerate(listed):
            at = f"{where}: layers[{index}]"
            entry = _object(entry, at)
            _unknown(entry, {"type", "mixer", "mlp"}, at)
            kind = entry.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"{at}.type is {kind!r}: this design has {', '.join(sorted(_MIXERS))}")
            mixer = _MIXERS[kind](_object(entry.get("mixer"), at + ".mixer"), at + ".mixer")
            mlp = None
            if entry.get("mlp") is not None:
                m = _object(entry["mlp"], at + ".mlp")
                _unknown(m, {"kind", "expert", "router"}, at + ".mlp")
                if m.get("kind", "moe") != "moe":
                    raise ConfigError(f"{at}.mlp.kind is {m.get('kind')!r}: this design has 'moe'")
                k = KeyReader(m, at + ".mlp")
                experts = k.integer("router.experts", minimum=1)
                top = k.integer("router.top", minimum=1)
                if top > experts:
                    raise ConfigError(f"{at}.mlp.router: top {top} of {experts} experts")
                mlp = FotanexExperts(experts, top, k.integer("expert.ff", minimum=1))
            layers.append(FotanexLayer(kind, mixer, mlp))
        loop = None
        if raw.get("loop") is not None:
            lp = _object(raw["loop"], f"{where}: loop")
            _unknown(lp, {"start", "stop", "times"}, f"{where}: loop")
            k = KeyReader(lp, f"{where}: loop")
            loop = FotanexLoop(k.integer("start", default=0, minimum=0), k.integer("stop", default=len(layers), minimum=0),
                               k.integer("times", default=1, minimum=1))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"{where}: loop runs layers {loop.start} .. {loop.stop - 1} of {len(layers)}")
        return cls(
            architecture=ARCHITECTURE,
            vocab_size=r.integer("vocab", minimum=1),
            hidden_size=r.integer("width", minimum=1),
            num_hidden_layers=len(layers),
            eos_token_id=tuple(t for t in r.integer_list("eos_token_id", default=()) if t >= 0),
            norm_eps=r.real("norm.eps", positive=True),
            layers=tuple(layers),
            loop=loop,
        )

    def to_json_dict(self) -> dict[str, Any]:
        """The config.json that reads back to this configuration."""
        out: dict[str, Any] = {
            "architecture": ARCHITECTURE,
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "norm": {"eps": self.norm_eps},
            "layers": [layer.to_json() for layer in self.layers],
        }
        if self.loop is not None:
            out["loop"] = self.loop.to_json()
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
