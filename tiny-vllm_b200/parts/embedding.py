"""Token embedding and the language-model head.

h = E[ids] (tinyvllm/models/qwen3.py:427-432, :480); logits = h . W^T with W the
embedding itself when tied (:514-525, :703-717).  Logits leave in float32.
"""

from __future__ import annotations

import torch

from ..ops import kernels, linear
from .base import BuildContext, ParamSpec, Part
from .registry import register_part


class TokenEmbedding(Part):
    """h = E[ids]; with ``norm`` (a norm part that offers ``start``) the rows are normed at once and leave
    in float32, as the first tensor of a float32 residual stream."""

    def __init__(self, ctx: BuildContext, *, vocab_size: int, width: int, name: str, norm=None) -> None:
        self.vocab_size, self.width, self.name = vocab_size, width, name
        self.weight = None
        self.norm = ctx.build("norm", norm, ctx) if norm is not None else None
        if self.norm is not None and not hasattr(self.norm, "start"):
            raise ValueError("an embedding's norm must offer start(x)")

    def param_specs(self):
        return [ParamSpec.single("weight", self.name, (self.vocab_size, self.width), role="table")]

    def children(self):
        return [self.norm] if self.norm is not None else []

    def forward(self, token_ids):
        rows = kernels.embed_rows(self.weight, token_ids)
        return rows if self.norm is None else self.norm.start(rows)


class LMHead(Part):
    def __init__(self, ctx: BuildContext, *, vocab_size: int, width: int, name: str,
                 tied_to: str | None, scale: float = 1.0) -> None:
        self.vocab_size, self.width, self.name, self.tied_to = vocab_size, width, name, tied_to
        self.scale = float(scale)          # the float32 logits are multiplied by it
        self.weight = None

    def param_specs(self):
        if self.tied_to is not None:
            return []
        return [ParamSpec.single("weight", self.name, (self.vocab_size, self.width))]

    def streamed_weights(self):
        return [self.weight]

    def forward(self, hidden_rows):
        logits = linear(hidden_rows, self.weight, out_dtype=torch.float32)
        return logits if self.scale == 1.0 else kernels.scale_float32(logits, self.scale)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
