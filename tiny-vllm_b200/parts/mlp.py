"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases.

gate and up are one packed projection [gate | up]
(tinyvllm/models/qwen3.py:316-346; activation tinyvllm/kernels/pointwise.cu:274-285).
"""

from __future__ import annotations

from ..ops import linear, linear_into_stream, linear_norm, linear_silu
from .base import BuildContext, ParamSpec, Part
from .registry import register_part


class SwiGLU(Part):
    def __init__(self, ctx: BuildContext, *, hidden_size: int, intermediate_size: int,
                 names: dict | None = None) -> None:
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        n = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight",
             **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.gate_up_weight = self.down_weight = None

    def param_specs(self):
        return [
            ParamSpec.packed("gate_up_weight", [(self.names["gate"], self.intermediate_size),
                                                (self.names["up"], self.intermediate_size)],
                             self.hidden_size),
            ParamSpec.single("down_weight", self.names["down"],
                             (self.hidden_size, self.intermediate_size)),
        ]

    def streamed_weights(self):
        return [self.gate_up_weight, self.down_weight]

    def forward(self, x, ctx):
        return linear(linear_silu(x, self.gate_up_weight), self.down_weight)

    def forward_normed(self, hidden, residual, norm, ctx):
        """forward(norm(hidden + residual)) and the new residual stream; the output is None when
        the down projection has added it to the stream itself."""
        activated, residual = linear_norm(hidden, residual, norm, self.gate_up_weight, silu=True)
        return linear_into_stream(activated, self.down_weight, residual)


register_part("feed_forward", "swiglu", SwiGLU)
