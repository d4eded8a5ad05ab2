"""Gated linear attention: a recurrence over a float32 state per sequence instead of keys and values.

Per head, with q and k of ``head_dim`` channels and v of ``value_dim``:

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,    o_t = S_t^T (q_t * q_scale)
    alpha_t = sigmoid(z_t)^(1/tau),              z_t = A2 (A1 x_t) + b        (one decay per key channel)

then each head's o_t is divided by its root mean square over ``value_dim`` and multiplied by one weight vector
shared by the heads, the heads side by side are multiplied by silu(G x_t), and the output projection follows.
The state starts at zero (the cache zeroes a slot's state when it hands the slot out) and is carried from step
to step in the cache line's state area, which holds two copies per slot so that a step of one token reads one
and writes the other (see gla.cu).  q, k, v, the gate and A1 x come from one product; everything between that
product and the output projection is one kernel in float32 (three launches of it for a long prompt, whose tokens
are cut into segments that run side by side).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed, LineView
from ..csrc import ops
from ..weights.loader import MATRIX, VECTOR, TensorNeed, TensorSource
from .base import Mixer, register_part
from .linear import linear


SEGMENT_TOKENS = 128        # a long prompt's tokens run in segments of this many, side by side (see gla.cu)


class GatedLinearAttention(Mixer):
    replayable = True
    kernel_groups = ("common", "streams", "recurrent")

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size = int(a["hidden_size"])
        self.num_heads = int(a["num_heads"])
        self.head_dim = int(a["head_dim"])
        self.value_dim = int(a.get("value_dim") or self.head_dim)
        self.decay_rank = int(a["decay_rank"])
        self.tau = float(a["tau"])
        self.q_scale = float(a.get("q_scale", self.head_dim ** -0.5))
        self.norm_eps = float(a.get("norm_eps", 1e-6))
        if min(self.num_heads, self.head_dim, self.value_dim, self.decay_rank) < 1:
            raise ValueError("gated linear attention needs heads, head_dim, value_dim and decay_rank of at least 1")
        if not self.tau > 0.0:
            raise ValueError(f"a decay exponent 1/tau with tau = {self.tau}")
        self.qk_width = self.num_heads * self.head_dim
        self.v_width = self.num_heads * self.value_dim
        # rows of the joint projection: q | k | v | gate | decay's inner rows
        self.offsets = (0, self.qk_width, 2 * self.qk_width, 2 * self.qk_width + self.v_width,
                        2 * self.qk_width + 2 * self.v_width)
        self.w_in: Optional[torch.Tensor] = None
        self.w_decay: Optional[torch.Tensor] = None
        self.decay_bias: Optional[torch.Tensor] = None
        self.norm_weight: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def _needs(self) -> dict[str, TensorNeed]:
        d = self.hidden_size
        return {
            "q_proj": TensorNeed(self.name_of("q_proj"), (self.qk_width, d), MATRIX, "normal"),
            "k_proj": TensorNeed(self.name_of("k_proj"), (self.qk_width, d), MATRIX, "normal"),
            "v_proj": TensorNeed(self.name_of("v_proj"), (self.v_width, d), MATRIX, "normal"),
            "gate_proj": TensorNeed(self.name_of("gate_proj"), (self.v_width, d), MATRIX, "normal"),
            "decay_in": TensorNeed(self.name_of("decay_in"), (self.decay_rank, d), MATRIX, "normal"),
            "decay_out": TensorNeed(self.name_of("decay_out"), (self.qk_width, self.decay_rank), MATRIX, "normal"),
            "decay_bias": TensorNeed(self.name_of("decay_bias"), (self.qk_width,), VECTOR, "bias"),
            "out_norm": TensorNeed(self.name_of("out_norm"), (self.value_dim,), VECTOR, "around_one"),
            "o_proj": TensorNeed(self.name_of("o_proj"), (d, self.v_width), MATRIX, "normal"),
        }

    def tensor_needs(self):
        return list(self._needs().values())

    def load(self, source: TensorSource) -> None:
        needs = self._needs()
        self.w_in = torch.cat([source.fetch(needs[n]) for n in ("q_proj", "k_proj", "v_proj", "gate_proj", "decay_in")],
                              dim=0).contiguous()
        self.w_decay = source.fetch(needs["decay_out"])
        self.decay_bias = source.fetch(needs["decay_bias"])
        self.norm_weight = source.fetch(needs["out_norm"])
        self.w_o = source.fetch(needs["o_proj"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state_shape=(2, self.num_heads, self.head_dim, self.value_dim), state_dtype="float32")

    def segments(self, ctx):
        """Tables that cut the step's prompts into segments of ``SEGMENT_TOKENS``, or None when the sequences as they
        are give the device enough blocks (or are short).  Only a step of prompts comes here, and such a step is never
        recorded, so the lengths may be read on the host."""
        if ctx.is_decode or ctx.max_q_len < 2 * SEGMENT_TOKENS:
            return None
        if ctx.num_seqs * self.num_heads >= 2 * ops.sm_count(ctx.device):
            return None
        cached = getattr(ctx, "_token_segments", None)          # the same for every recurrent layer of the step
        if cached is None:
            seqs, begins, ends, first = [], [], [], [0]
            for b, n in enumerate(ctx.seq_q_lens):
                for lo in range(0, n, SEGMENT_TOKENS):
                    seqs.append(b)
                    begins.append(lo)
                    ends.append(min(lo + SEGMENT_TOKENS, n))
                first.append(len(seqs))
            flat = torch.tensor(seqs + begins + ends + first, dtype=torch.int32).to(ctx.device)
            count = len(seqs)
            cached = ctx._token_segments = (flat[:count], flat[count:2 * count], flat[2 * count:3 * count], flat[3 * count:])
        return cached

    def forward(self, ctx, act: torch.Tensor, line: LineView, writes_cache: bool) -> torch.Tensor:
        if not writes_cache:
            raise ValueError("a recurrent layer cannot read another layer's state: it has to write its own")
        proj = linear(act, self.w_in)                                       # float32 [T, 2 qk + 2 v + rank]
        out = ctx.buffer("linear_attention.out", (act.shape[0], self.v_width), self.dtype)
        segments = self.segments(ctx)
        scratch = None
        if segments is not None:
            floats = ops.gla_scratch_floats(segments[0].numel(), self.num_heads, self.head_dim, self.value_dim)
            scratch = ctx.buffer("linear_attention.segments", (floats,), torch.float32)
        ops.gla_scan(proj, self.offsets, self.w_decay, self.decay_bias, self.norm_weight, line.state, ctx.seq_slot,
                     ctx.seq_start, ctx.cu_q_len, out, heads=self.num_heads, dim=self.head_dim, vdim=self.value_dim,
                     tau=self.tau, q_scale=self.q_scale, eps=self.norm_eps, segments=segments, scratch=scratch)
        return linear(out, self.w_o)


register_part("mixer", "gated_linear_attention", GatedLinearAttention, replace=True)
