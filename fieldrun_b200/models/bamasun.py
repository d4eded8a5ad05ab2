"""Bamasun as a plan of parts.

A decoder whose layers are listed one by one in the configuration and differ from one another.  Every layer
has the norm on the sublayer's output (block ``output_norm``): x <- x + LN(mixer(x)), then, if it has a
feed-forward, x <- x + LN(W_down relu(W_up x)^2); the norms are layer norms with weight and bias.  Two mixers:

* ``attention``: grouped-query softmax attention without rotation; q, k and v projections with biases; one RMS
  norm over the whole q row and one over the whole k row; the query multiplied by a temperature that grows with
  the logarithm of the position; a score scale from the configuration; the score of key j for query i lowered by
  slope_h * (i - j) with slope_h = 2^(-8 (h + 1) / H).  A layer with ``kv_from`` has no keys and values of its
  own: its run reads the cache line that the named layer's run writes.
* ``gla``: gated linear attention with a decay per key channel (``gated_linear_attention``), its state in the
  cache line's state area.

The embedding rows are multiplied by a constant; the model's last norm is a layer norm too; the logits are capped
by cap * tanh(logits / cap).  Tensor names: ``embed``, ``head``, ``final.norm[.b]``, and per layer i ``l<i>.norm1[.b]``,
``l<i>.norm2[.b]``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``.
"""
from __future__ import annotations

from dataclasses import replace
from typing import Mapping

from ..config.bamasun import ARCHITECTURE, BamasunConfig, BamasunGla
from ..config.base import ConfigError
from ..config.plan import LayerSpec, ModelPlan, PartSpec, RunSpec
from ..config.registry import Architecture, register_architecture

SLOPE_EXPONENT = 8.0          # slope of head h (0-based) of H: 2^(-SLOPE_EXPONENT * (h + 1) / H)
FEED_FORWARD_ACTIVATION = "relu_squared"


def distance_slopes(num_heads: int) -> tuple[float, ...]:
    return tuple(2.0 ** (-SLOPE_EXPONENT * (h + 1) / num_heads) for h in range(num_heads))


def _layer_norm(width: int, eps: float, name: str) -> PartSpec:
    return PartSpec("layernorm", {"width": width, "eps": eps, "bias": True}, {"weight": name, "bias": name + ".b"})


def bamasun_plan(cfg: BamasunConfig) -> ModelPlan:
    d = cfg.hidden_size
    layers = []
    runs = []
    line_of: dict[int, int] = {}
    for index, layer in enumerate(cfg.layers):
        p = f"l{index}."
        m = layer.mixer
        if layer.type == "attention":
            tensors = {"q_proj": p + "mix.q", "q_bias": p + "mix.q.b", "q_norm": p + "mix.q.norm", "o_proj": p + "mix.o",
                       "k_proj": p + "mix.k", "k_bias": p + "mix.k.b", "k_norm": p + "mix.k.norm",
                       "v_proj": p + "mix.v", "v_bias": p + "mix.v.b"}
            mixer = PartSpec(
                kind="gqa_attention",
                args={
                    "hidden_size": d, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "bias": True,
                    "qk_norm": "full_width", "qk_norm_eps": cfg.norm_eps,
                    "position": None,                                   # no rotation: positions enter through the two below
                    "query_temperature": ({"coef": m.q_temp_coef, "every": m.q_temp_every}
                                          if m.q_temp_coef is not None else None),
                    "distance_slopes": distance_slopes(m.heads),
                    "softmax_scale": m.scale, "window": None,
                    "shares_kv": m.kv_from is not None,
                },
                tensors=tensors,
            )
            if m.kv_from is None:
                line_of[index] = max(line_of.values(), default=-1) + 1
                runs.append(RunSpec(layer=index, cache_line=line_of[index], writes_cache=True))
            else:
                line_of[index] = line_of[m.kv_from]
                runs.append(RunSpec(layer=index, cache_line=line_of[m.kv_from], writes_cache=False))
        else:
            if m.rank is None:
                raise ConfigError(f"layer {index}: the rank of the decay's inner product is not known; it is the first "
                                  f"size of tensor {p}mix.a1 (or the key 'rank' of the mixer)")
            mixer = PartSpec(
                kind="gated_linear_attention",
                args={"hidden_size": d, "num_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "decay_rank": m.rank,
                      "tau": m.tau, "q_scale": float(m.dim) ** -0.5, "norm_eps": cfg.norm_eps},
                tensors={"q_proj": p + "mix.q", "k_proj": p + "mix.k", "v_proj": p + "mix.v", "gate_proj": p + "mix.g",
                         "decay_in": p + "mix.a1", "decay_out": p + "mix.a2", "decay_bias": p + "mix.a2.b",
                         "out_norm": p + "mix.norm", "o_proj": p + "mix.o"},
            )
            line = max(line_of.values(), default=-1) + 1
            line_of[index] = line
            runs.append(RunSpec(layer=index, cache_line=line, writes_cache=True))
        feed_forward = feed_forward_norm = None
        if layer.ff is not None:
            feed_forward = PartSpec("dense_unit", {"hidden_size": d, "width": layer.ff, "activation": FEED_FORWARD_ACTIVATION},
                                    {"w_up": p + "mlp.up", "w_down": p + "mlp.down"})
            feed_forward_norm = _layer_norm(d, cfg.norm_eps, p + "norm2")
        layers.append(LayerSpec(block="output_norm", mixer=mixer, feed_forward=feed_forward,
                                mixer_norm=_layer_norm(d, cfg.norm_eps, p + "norm1"), feed_forward_norm=feed_forward_norm))
    plan = ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=d,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": d, "scale": cfg.embedding_scale,
                                               "typed_copy": True}, {"weight": "embed"}),
        layers=tuple(layers),
        run_order=tuple(runs),
        final_norm=_layer_norm(d, cfg.norm_eps, "final.norm"),
        head=PartSpec("vocab_head", {"vocab_size": cfg.vocab_size, "width": d, "softcap": cfg.logit_softcap},
                      {"weight": "head"}),
        eos_token_id=cfg.eos_token_id,
    )
    plan.check()
    return plan


def sizes_from_tensors(cfg: BamasunConfig, shapes: Mapping[str, tuple[int, ...]]) -> BamasunConfig:
    """The one size that only a tensor's shape gives: the rank of a gla layer's decay, rows of ``l<i>.mix.a1``."""
    layers = []
    for index, layer in enumerate(cfg.layers):
        shape = shapes.get(f"l{index}.mix.a1")
        if isinstance(layer.mixer, BamasunGla) and shape is not None and len(shape) == 2:
            if layer.mixer.rank is not None and layer.mixer.rank != shape[0]:
                raise ConfigError(f"layer {index}: the configuration says rank {layer.mixer.rank}, tensor l{index}.mix.a1 "
                                  f"has {shape[0]} rows")
            layer = replace(layer, mixer=replace(layer.mixer, rank=int(shape[0])))
        layers.append(layer)
    return replace(cfg, layers=tuple(layers))


register_architecture(Architecture(
    name=ARCHITECTURE,
    config_from_dict=BamasunConfig.from_dict,
    plan=bamasun_plan,
    model_type_prefixes=("bamasun",),
    sizes_from_tensors=sizes_from_tensors,
), replace=True)
