"""Fotanex as a plan of parts.

A decoder whose layers are listed one by one in the configuration.  Every layer is parallel with two norms
(block ``parallel_pre_norm``): x <- x + mixer(norm1(x)) + experts(norm2(x)), both norms reading the same x; the
norms, and the model's last one, are dynamic tanh (``dynamic_tanh``: tanh(alpha v) * w + b, no statistics).  The
feed-forward is a set of routed experts with softmax scores.  Three mixers:

* ``rglru``: the recurrent block with a real-gated linear recurrent unit (``gated_linear_recurrence``);
* ``mamba2``: a state per head with one decay per head and token (``scalar_decay_state_space``);
* ``parallel``: two mixers side by side (``mixer_pair``), each output divided by its root mean square and weighted,
  half their sum: attention without positions in chunks, with a sink in the softmax and a gate per head
  (``gqa_attention`` with ``chunk``, ``sink``, ``head_gate``), beside a selective scan (``selective_scan``).

``loop``: a stretch of layers runs several times with the same weights; every pass has cache lines of its own
and begins with a connector (``stream_reentry``): x <- W_in [x ; x0] + step[pass], x0 being the embedding's rows.

Tensor names: ``embed``, ``head``, ``final.norm[.b|.alpha]``, ``loop.in``, ``loop.step``, and per layer i
``l<i>.norm1|norm2[.b|.alpha]``, ``l<i>.mix.*``, ``l<i>.mlp.router``, ``l<i>.mlp.e<e>.gate|up|down``.
"""
from __future__ import annotations

from ..config.fotanex import ARCHITECTURE, FotanexConfig
from ..config.plan import LayerSpec, ModelPlan, PartSpec, RunSpec
from ..config.registry import Architecture, register_architecture

RECURRENT_GATE_CONSTANT = 8.0          # log a = -RECURRENT_GATE_CONSTANT * r * softplus(lam)
EXPERT_WEIGHT_FLOOR = 1e-20            # added to the sum of the chosen experts' scores before the division


def _dyt(width: int, name: str) -> PartSpec:
    return PartSpec("dynamic_tanh", {"width": width}, {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})


def _mixer(cfg: FotanexConfig, index: int) -> PartSpec:
    d = cfg.hidden_size
    layer = cfg.layers[index]
    m = layer.mixer
    p = f"l{index}.mix."
    if layer.type == "rglru":
        return PartSpec(
            "gated_linear_recurrence",
            {"hidden_size": d, "width": m.width, "blocks": m.blocks, "conv": m.conv, "gate_constant": RECURRENT_GATE_CONSTANT,
             "activation": "gelu_tanh"},
            {"y_proj": p + "y", "y_bias": p + "y.b", "x_proj": p + "x", "x_bias": p + "x.b", "conv": p + "conv",
             "conv_bias": p + "conv.b", "a_gate": p + "ra", "a_gate_bias": p + "ra.b", "i_gate": p + "ri",
             "i_gate_bias": p + "ri.b", "lam": p + "lam", "o_proj": p + "o"})
    if layer.type == "mamba2":
        return PartSpec(
            "scalar_decay_state_space",
            {"hidden_size": d, "num_heads": m.heads, "value_dim": m.vdim, "state": m.state, "groups": m.groups,
             "norm_groups": m.norm_groups, "conv": m.conv, "norm_eps": cfg.norm_eps},
            {"in_proj": p + "in", "conv": p + "conv", "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias",
             "a_log": p + "A_log", "d": p + "D", "norm": p + "norm", "o_proj": p + "o"})
    a, s = m.left, m.right
    left = PartSpec(
        "gqa_attention",
        {"hidden_size": d, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim,
         "qk_norm": "none", "position": None, "softmax_scale": a.scale, "window": None, "chunk": a.chunk, "sink": True,
         "head_gate": True},
        {"q_proj": p + "left.q", "k_proj": p + "left.k", "v_proj": p + "left.v", "o_proj": p + "left.o",
         "sink": p + "left.sink", "gate_proj": p + "left.g"})
    right = PartSpec(
        "selective_scan",
        {"hidden_size": d, "inner": s.inner, "state": s.state, "dt_rank": s.dt_rank, "conv": s.conv},
        {"in_proj": p + "right.in", "conv": p + "right.conv", "conv_bias": p + "right.conv.b", "x_proj": p + "right.x",
         "dt_proj": p + "right.dt", "dt_bias": p + "right.dt.b", "a_log": p + "right.A_log", "d": p + "right.D",
         "o_proj": p + "right.o"})
    return PartSpec("mixer_pair", {"hidden_size": d, "left": left, "right": right, "norm_eps": cfg.norm_eps, "share": 0.5},
                    {"left_norm": p + "left.out", "right_norm": p + "right.out"})


def fotanex_plan(cfg: FotanexConfig) -> ModelPlan:
    d = cfg.hidden_size
    layers = []
    for index, layer in enumerate(cfg.layers):
        p = f"l{index}."
        feed_forward = feed_forward_norm = None
        if layer.mlp is not None:
            feed_forward = PartSpec(
                "routed_experts",
                {"hidden_size": d, "num_experts": layer.mlp.experts, "top_k": layer.mlp.top, "expert_width": layer.mlp.ff,
                 "score": "softmax", "choice_bias": False, "renormalize": True, "weight_floor": EXPERT_WEIGHT_FLOOR},
                {"router": p + "mlp.router", "w_gate": p + "mlp.e{e}.gate", "w_up": p + "mlp.e{e}.up",
                 "w_down": p + "mlp.e{e}.down"})
            feed_forward_norm = _dyt(d, p + "norm2")
        layers.append(LayerSpec(block="parallel_pre_norm", mixer=_mixer(cfg, index), feed_forward=feed_forward,
                                mixer_norm=_dyt(d, p + "norm1"), feed_forward_norm=feed_forward_norm))
    # the run order: layers before the loop once, the loop's layers ``times`` times (a cache line per run: every pass
    # has keys, values and states of its own), the rest once
    count = len(cfg.layers)
    loop = cfg.loop
    order: list[tuple[int, int | None]] = []
    if loop is None:
        order = [(i, None) for i in range(count)]
    else:
        order += [(i, None) for i in range(loop.start)]
        for t in range(loop.times):
            order += [(i, t if i == loop.start else None) for i in range(loop.start, loop.stop)]
        order += [(i, None) for i in range(loop.stop, count)]
    runs = tuple(RunSpec(layer=i, cache_line=line, writes_cache=True, connector=(0, opens) if opens is not None else None)
                 for line, (i, opens) in enumerate(order))
    connectors = ()
    if loop is not None:
        connectors = (PartSpec("stream_reentry", {"width": d, "passes": loop.times}, {"weight": "loop.in", "step": "loop.step"}),)
    plan = ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=d,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": d}, {"weight": "embed"}),
        layers=tuple(layers),
        run_order=runs,
        final_norm=_dyt(d, "final.norm"),
        head=PartSpec("vocab_head", {"vocab_size": cfg.vocab_size, "width": d}, {"weight": "head"}),
        eos_token_id=cfg.eos_token_id,
        connectors=connectors,
    )
    plan.check()
    return plan


register_architecture(Architecture(
    name=ARCHITECTURE,
    config_from_dict=FotanexConfig.from_dict,
    plan=fotanex_plan,
    model_type_prefixes=("fotanex",),
), replace=True)
