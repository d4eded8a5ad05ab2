"""RMSNorm: x * (1 / sqrt(mean(x^2) + eps)) * w per row, the weight used as it is
(src/minimax.rs:56-66).  The kernel also performs the residual sum that precedes
the norm, in float32, so the update of the stream and the norm read it once."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import VECTOR, TensorNeed, TensorSource
from .base import Norm, UpdateSum, WeightedRows, as_tensor, register_part


class RMSNorm(Norm):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.width = int(spec.args["width"])
        self.eps = float(spec.args["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.width,), VECTOR, "around_one")]

    def load(self, source: TensorSource) -> None:
        self.weight = source.fetch(self.tensor_needs()[0])

    accepts_deferred = True

    def forward(self, ctx, x, *, delta=None, rows=None, want32=False, write_back=True):
        experts = None
        if isinstance(delta, WeightedRows) and delta.top_k <= ops.NORM_MAX_SUMMED_ROWS:
            experts, delta = (delta.rows, delta.weights, delta.row_map), None      # the kernel sums them as it reads x
        else:
            delta = as_tensor(ctx, delta)
        count = rows.numel() if rows is not None else x.shape[0]
        out = ctx.buffer(f"norm.out.{self.width}", (count, self.width), self.dtype)
        out32 = None
        if want32:
            out32 = out if self.dtype == torch.float32 else ctx.buffer(f"norm.out32.{self.width}", (count, self.width),
                                                                       torch.float32)
        ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows, out32=None if out32 is out else out32,
                    write_back=write_back and (delta is not None or experts is not None), experts=experts)
        return out, out32


class LayerNorm(Norm):
    """(v - mean) / sqrt(var + eps) * weight + bias per row, var the mean of the squared deviations, float32
    statistics; the bias is optional (``bias: False``).  It serves in both places of a norm: on the stream
    (``forward``: a model's last norm, or a pre-norm block) and on a sublayer's output (``add_normed``), where
    one kernel norms the update, adds it to the float32 stream and writes the stream's copy in the model dtype."""

    replayable = True
    STREAM_COPY = "stream.act"           # the workspace buffer that holds the stream in the model dtype

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.width = int(spec.args["width"])
        self.eps = float(spec.args["eps"])
        self.has_bias = bool(spec.args.get("bias", True))
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_needs(self):
        needs = [TensorNeed(self.name_of("weight"), (self.width,), VECTOR, "around_one")]
        if self.has_bias:
            needs.append(TensorNeed(self.name_of("bias"), (self.width,), VECTOR, "bias"))
        return needs

    def load(self, source: TensorSource) -> None:
        needs = self.tensor_needs()
        self.weight = source.fetch(needs[0])
        self.bias = source.fetch(needs[1]) if self.has_bias else None

    def forward(self, ctx, x, *, delta=None, rows=None, want32=False, write_back=True):
        delta = as_tensor(ctx, delta)
        if delta is not None:
            if write_back:
                ops.add_rows(x, delta)
            else:
                x = x + delta
        count = rows.numel() if rows is not None else x.shape[0]
        out = ctx.buffer(f"norm.out.{self.width}", (count, self.width), self.dtype)
        ops.layernorm(x, self.weight, self.bias, self.eps, rows=rows, act=out)
        out32 = None
        if want32:
            out32 = out
            if self.dtype != torch.float32:
                out32 = ctx.buffer(f"norm.out32.{self.width}", (count, self.width), torch.float32)
                ops.layernorm(x, self.weight, self.bias, self.eps, rows=rows, act=out32)
        return out, out32

    def add_normed(self, ctx, update, x):
        if self.dtype == torch.float32:
            ops.layernorm(update, self.weight, self.bias, self.eps, stream=x)
            return x
        act = ctx.buffer(self.STREAM_COPY, tuple(x.shape), self.dtype)
        ops.layernorm(update, self.weight, self.bias, self.eps, stream=x, act=act)
        return act


class DynamicTanh(Norm):
    """tanh(alpha v) * weight + bias with one learned scalar alpha: a norm without statistics.  Two of them that read
    the same stream (a block whose sublayers run side by side) go through one kernel (``forward_pair``), which also
    adds the updates that the block before left: float32 tensors and the experts' weighted rows."""

    replayable = True
    accepts_deferred = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.width = int(spec.args["width"])
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.alpha: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.width,), VECTOR, "around_one"),
                TensorNeed(self.name_of("bias"), (self.width,), VECTOR, "bias"),
                TensorNeed(self.name_of("alpha"), (), VECTOR, "around_half")]

    def load(self, source: TensorSource) -> None:
        self.weight, self.bias, alpha = (source.fetch(need) for need in self.tensor_needs())
        self.alpha = alpha.reshape(1)                    # stays on the device: the kernel reads it there

    def triple(self):
        return self.weight, self.bias, self.alpha

    @staticmethod
    def split(ctx, delta):
        """(float32 tensors, experts' rows or None) of whatever form the update came in."""
        if delta is None:
            return (), None
        if isinstance(delta, torch.Tensor):
            return (delta,), None
        if isinstance(delta, WeightedRows) and delta.top_k <= ops.NORM_MAX_SUMMED_ROWS:
            return (), (delta.rows, delta.weights, delta.row_map)
        if isinstance(delta, UpdateSum) and len(delta.tensors) <= 2 and all(
                w.top_k <= ops.NORM_MAX_SUMMED_ROWS for w in delta.weighted):
            weighted = delta.weighted[0] if delta.weighted else None
            return tuple(delta.tensors), (weighted.rows, weighted.weights, weighted.row_map) if weighted else None
        return (as_tensor(ctx, delta),), None

    def forward(self, ctx, x, *, delta=None, rows=None, want32=False, write_back=True):
        deltas, experts = self.split(ctx, delta)
        count = rows.numel() if rows is not None else x.shape[0]
        out = ctx.buffer(f"norm.out.{self.width}", (count, self.width), self.dtype)
        ops.dyt_norm(x, self.triple(), out, deltas=deltas, experts=experts, rows=rows,
                     write_back=write_back and rows is None and (bool(deltas) or experts is not None))
        out32 = None
        if want32:
            out32 = out
            if self.dtype != torch.float32:
                out32 = ctx.buffer(f"norm.out32.{self.width}", (count, self.width), torch.float32)
                ops.dyt_norm(x, self.triple(), out32, rows=rows)       # x holds the sum by now (or nothing was added)
        return out, out32

    def forward_pair(self, ctx, x, other: "DynamicTanh", *, delta=None, want32=False):
        """This norm and ``other`` of the same x + delta (the sum stored back): (out, other's out, other's out in
        float32 or None)."""
        deltas, experts = self.split(ctx, delta)
        rows = x.shape[0]
        out1 = ctx.buffer(f"norm.out.{self.width}", (rows, self.width), self.dtype)
        out2 = ctx.buffer(f"norm.out2.{self.width}", (rows, self.width), self.dtype)
        out2_32 = None
        if want32 and self.dtype != torch.float32:
            out2_32 = ctx.buffer(f"norm.out32.{self.width}", (rows, self.width), torch.float32)
        ops.dyt_norm(x, self.triple(), out1, second=other.triple(), out2=out2, out2_32=out2_32, deltas=deltas, experts=experts,
                     write_back=bool(deltas) or experts is not None)
        return out1, out2, (out2 if self.dtype == torch.float32 else out2_32) if want32 else None


register_part("norm", "dynamic_tanh", DynamicTanh, replace=True)
register_part("norm", "rmsnorm", RMSNorm, replace=True)
register_part("norm", "layernorm", LayerNorm, replace=True)
