"""Token embedding rows into the float32 residual stream (no multiplier, src/minimax.rs:132)
and the vocabulary head: logits = rows @ W^T in float32, W the head's own matrix or the
embedding's when tied (src/minimax.rs:54,373-376).  Two optional constants that the reference's
model does not have: the embedding's ``scale`` (rows are multiplied by it) and the head's
``softcap`` (logits <- cap * tanh(logits / cap)); ``typed_copy`` makes the embedding write the
stream a second time in the model dtype, for blocks whose sublayers read the stream itself."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import MATRIX, TensorNeed, TensorSource
from .base import Part, register_part
from .linear import linear
from .norm import LayerNorm


class TokenEmbedding(Part):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.vocab_size = int(spec.args["vocab_size"])
        self.width = int(spec.args["width"])
        self.scale = float(spec.args.get("scale", 1.0))
        self.typed_copy = bool(spec.args.get("typed_copy", False))
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.vocab_size, self.width), MATRIX, "normal")]

    def load(self, source: TensorSource) -> None:
        self.weight = source.fetch(self.tensor_needs()[0])

    def forward(self, ctx, tokens: torch.Tensor) -> torch.Tensor:
        x = ctx.buffer("stream", (tokens.numel(), self.width), torch.float32)
        act = None
        ctx.stream_copy_rows = -1
        if self.typed_copy and self.dtype != torch.float32:
            act = ctx.buffer(LayerNorm.STREAM_COPY, (tokens.numel(), self.width), self.dtype)
            ctx.stream_copy_rows = tokens.numel()
        ops.embed_rows(tokens, self.weight, x, self.scale, act)
        return x


class VocabHead(Part):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.vocab_size = int(spec.args["vocab_size"])
        self.width = int(spec.args["width"])
        self.softcap = spec.args.get("softcap")
        if self.softcap is not None and not float(self.softcap) > 0.0:
            raise ValueError(f"a logit cap of {self.softcap}")
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.vocab_size, self.width), MATRIX, "normal")]

    def load(self, source: TensorSource, shared: Optional[torch.Tensor] = None) -> None:
        self.weight = shared if shared is not None else source.fetch(self.tensor_needs()[0])

    def forward(self, ctx, rows: torch.Tensor) -> torch.Tensor:
        logits = linear(rows, self.weight)
        if self.softcap is not None:
            ops.softcap(logits, float(self.softcap))
        return logits


register_part("embedding", "token_embedding", TokenEmbedding, replace=True)
register_part("head", "vocab_head", VocabHead, replace=True)
