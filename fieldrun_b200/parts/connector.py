"""Connectors: parts that stand between two runs of the run order and rewrite the whole stream.

``stream_reentry``: x <- W [x ; x0] + step[index], with x0 the embedding's rows, W [width, 2 width] (x's columns
first) and one vector ``step[index]`` per pass.  A model that runs a stretch of its layers several times with the
same weights puts this in front of every pass."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import MATRIX, VECTOR, TensorNeed, TensorSource
from .base import Connector, as_tensor, register_part
from .linear import linear


class StreamReentry(Connector):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.width = int(spec.args["width"])
        self.passes = int(spec.args["passes"])
        self.weight: Optional[torch.Tensor] = None
        self.step: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.width, 2 * self.width), MATRIX, "normal"),
                TensorNeed(self.name_of("step"), (self.passes, self.width), VECTOR, "bias")]

    def load(self, source: TensorSource) -> None:
        self.weight, self.step = (source.fetch(need) for need in self.tensor_needs())

    def forward(self, ctx, x, pending, first, index):
        if not 0 <= index < self.passes:
            raise ValueError(f"pass {index} of {self.passes}")
        both = ctx.buffer("reentry.rows", (x.shape[0], 2 * self.width), self.dtype)
        ops.concat_rows(x, first, both, delta=as_tensor(ctx, pending))      # the update a block left is added on the way
        ops.add_row_vector(linear(both, self.weight), self.step[index], x)
        return x


register_part("connector", "stream_reentry", StreamReentry, replace=True)
