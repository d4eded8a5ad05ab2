"""Configuration of the Bamasun design, read from its own config.json keys.

The file names the design as ``"architecture": "Bamasun"`` and lists the layers one by one:

    vocab, width                       sizes of the vocabulary and of the residual stream
    embedding.scale                    multiplier on the embedding rows
    norm.eps                           eps of every norm of a layer and of the model
    logit_softcap                      cap of the logits (absent or null: none)
    layers[i].type                     "attention" | "gla"
    layers[i].mixer                    the mixer's sizes and constants (below)
    layers[i].mlp                      {"kind": "dense", "ff": n} or null for a layer without feed-forward

    attention:  heads, kv_heads, dim, vdim, scale, q_temp {coef, every} (optional), kv_from (optional: the index
                of the earlier attention layer whose keys and values this layer reads instead of making its own)
    gla:        heads, dim, vdim, tau  (the rank of the decay's inner product is the shape of its tensor)

Everything that can differ between two models of the design is read here; the constants that the design fixes
(the slopes' exponent, the activations) live with the plan in ``models/bamasun.py``.  Inside a layer, the
embedding and the norm a key the design does not have is refused, so that a file of another design (a window, a
sink, a cap on the scores) is not run as this one; at the top level such a key is a warning.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .base import ConfigError, KeyReader, ModelConfig

ARCHITECTURE = "Bamasun"


@dataclass(frozen=True)
class BamasunAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp_coef: Optional[float] = None
    q_temp_every: Optional[int] = None
    kv_from: Optional[int] = None

    def to_json(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.q_temp_coef is not None:
            out["q_temp"] = {"coef": self.q_temp_coef, "every": self.q_temp_every}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class BamasunGla:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int] = None          # not a key of the file: taken from the decay tensor's shape at load

    def to_json(self) -> dict[str, Any]:
        out: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.rank is not None:
            out["rank"] = self.rank
        return out


@dataclass(frozen=True)
class BamasunLayer:
    type: str
    mixer: Any                           # BamasunAttention | BamasunGla
    ff: Optional[int]                    # width of the dense feed-forward; None: the layer has none

    def to_json(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_json(),
                "mlp": {"kind": "dense", "ff": self.ff} if self.ff is not None else None}


def _only(raw: Mapping[str, Any], allowed: set[str], where: str) -> None:
    extra = sorted(set(raw) - allowed)
    if extra:
        raise ConfigError(f"{where}: keys this design does not have: {', '.join(extra)}")


def _attention(raw: Mapping[str, Any], where: str, index: int, before: list[BamasunLayer]) -> BamasunAttention:
    _only(raw, {"heads", "kv_heads", "dim", "vdim", "scale", "q_temp", "kv_from"}, where)
    r = KeyReader(raw, where)
    heads = r.integer("heads", minimum=1)
    kv_heads = r.integer("kv_heads", default=heads, minimum=1)
    if heads % kv_heads:
        raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
    dim = r.integer("dim", minimum=1)
    vdim = r.integer("vdim", default=dim, minimum=1)
    coef = every = None
    if r.present("q_temp"):
        _only(raw["q_temp"], {"coef", "every"}, where + ".q_temp")
        coef = r.real("q_temp.coef")
        every = r.integer("q_temp.every", minimum=1)
    kv_from = None
    if r.present("kv_from"):
        kv_from = r.integer("kv_from", minimum=0)
        if kv_from >= index:
            raise ConfigError(f"{where}: kv_from {kv_from} must name an earlier layer")
        source = before[kv_from]
        if source.type != "attention" or source.mixer.kv_from is not None:
            raise ConfigError(f"{where}: kv_from {kv_from} must name an attention layer with keys and values of its own")
        if (source.mixer.kv_heads, source.mixer.dim, source.mixer.vdim) != (kv_heads, dim, vdim):
            raise ConfigError(f"{where}: layer {kv_from}'s keys and values ({source.mixer.kv_heads} heads of "
                              f"{source.mixer.dim}/{source.mixer.vdim}) do not fit this layer's ({kv_heads} of {dim}/{vdim})")
    return BamasunAttention(heads, kv_heads, dim, vdim, r.real("scale", default=float(dim) ** -0.5, positive=True),
                            coef, every, kv_from)


def _gla(raw: Mapping[str, Any], where: str) -> BamasunGla:
    _only(raw, {"heads", "dim", "vdim", "tau", "rank"}, where)
    r = KeyReader(raw, where)
    dim = r.integer("dim", minimum=1)
    rank = r.integer("rank", minimum=1) if r.present("rank") else None
    return BamasunGla(r.integer("heads", minimum=1), dim, r.integer("vdim", default=dim, minimum=1),
                      r.real("tau", positive=True), rank)


@dataclass(frozen=True)
class BamasunConfig(ModelConfig):
    embedding_scale: float = 1.0
    norm_eps: float = 1e-6
    logit_softcap: Optional[float] = None
    layers: tuple[BamasunLayer, ...] = ()

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "BamasunConfig":
        known = {"architecture", "architectures", "model_type", "vocab", "width", "embedding", "norm", "logit_softcap",
                 "layers", "eos_token_id"}
        extra = sorted(set(raw) - known)
        if extra:
            # beside the model's sizes a file may carry notes of its writer (a name, a seed); inside a layer,
            # where every key is arithmetic, an unknown key is refused
            print(f"{where}: warning: top-level keys this design does not have are ignored: {', '.join(extra)}", file=sys.stderr)
        for name in ("embedding", "norm"):
            if isinstance(raw.get(name), Mapping):
                _only(raw[name], {"scale"} if name == "embedding" else {"eps"}, f"{where}: {name}")
        r = KeyReader(raw, where)
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError(f"{where}: key 'layers' must be a list of at least one layer")
        layers: list[BamasunLayer] = []
        for index, entry in enumerate(listed):
            at = f"{where}: layers[{index}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{at} must be an object")
            _only(entry, {"type", "mixer", "mlp"}, at)
            kind = entry.get("type")
            mixer_raw = entry.get("mixer")
            if not isinstance(mixer_raw, Mapping):
                raise ConfigError(f"{at}.mixer must be an object")
            if kind == "attention":
                mixer: Any = _attention(mixer_raw, at + ".mixer", index, layers)
            elif kind == "gla":
                mixer = _gla(mixer_raw, at + ".mixer")
            else:
                raise ConfigError(f"{at}.type is {kind!r}: this design has 'attention' and 'gla'")
            ff = None
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"{at}.mlp must be an object or null")
                _only(mlp, {"kind", "ff"}, at + ".mlp")
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{at}.mlp.kind is {mlp.get('kind')!r}: this design has 'dense'")
                ff = KeyReader(mlp, at + ".mlp").integer("ff", minimum=1)
            layers.append(BamasunLayer(kind, mixer, ff))
        cap = r.real("logit_softcap", positive=True) if r.present("logit_softcap") else None
        return cls(
            architecture=ARCHITECTURE,
            vocab_size=r.integer("vocab", minimum=1),
            hidden_size=r.integer("width", minimum=1),
            num_hidden_layers=len(layers),
            eos_token_id=tuple(t for t in r.integer_list("eos_token_id", default=()) if t >= 0),
            embedding_scale=r.real("embedding.scale", default=1.0),
            norm_eps=r.real("norm.eps", positive=True),
            logit_softcap=cap,
            layers=tuple(layers),
        )

    def to_json_dict(self) -> dict[str, Any]:
        """The config.json that reads back to this configuration."""
        out: dict[str, Any] = {
            "architecture": ARCHITECTURE,
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "embedding": {"scale": self.embedding_scale},
            "norm": {"eps": self.norm_eps},
            "layers": [layer.to_json() for layer in self.layers],
        }
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
