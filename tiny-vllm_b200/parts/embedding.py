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
    def __init__(self, ctx: BuildContext, *, vocab_size: int, width: int, name: str) -> None:
        self.vocab_size, self.width, self.name = vocab_size, width, name
        self.weight = None

    def param_specs(self):
        return [ParamSpec.single("weight", self.name, (self.vocab_size, self.width), role="table")]

    def forward(self, token_ids):
        return kernels.embed_rows(self.weight, token_ids)


class LMHead(Part):
    def __init__(self, ctx: BuildContext, *, vocab_size: int, width: int, name: str,
                 tied_to: str | None) -> None:
        self.vocab_size, self.width, self.name, self.tied_to = vocab_size, width, name, tied_to
        self.weight = None

    def param_specs(self):
        if self.tied_to is not None:
            return []
        return [ParamSpec.single("weight", self.name, (self.vocab_size, self.width))]

    def streamed_weights(self):
        return [self.weight]

    def forward(self, hidden_rows):
        return linear(hidden_rows, self.weight, out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
