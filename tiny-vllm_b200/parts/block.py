"""Arrangement of a layer's parts: pre-norm with a deferred residual sum.

The first layer keeps its input as the residual stream and norms it; every
later norm first adds the previous part's output to the stream.  The
feed-forward output is NOT added here: the next block's first norm (or the
model's final norm) adds it (tinyvllm/models/qwen3.py:386-412).
"""

from __future__ import annotations

from .base import Block, BuildContext
from .registry import register_part


class PreNormResidualBlock(Block):
    def __init__(self, ctx: BuildContext, *, mixer, feed_forward, norm, mixer_norm_name: str,
                 feed_forward_norm_name: str, mixer_name: str, feed_forward_name: str) -> None:
        self.mixer_norm = ctx.build("norm", norm, ctx.child(mixer_norm_name))
        self.mixer = ctx.build("mixer", mixer, ctx.child(mixer_name))
        self.feed_forward_norm = ctx.build("norm", norm, ctx.child(feed_forward_norm_name))
        self.feed_forward = ctx.build("feed_forward", feed_forward, ctx.child(feed_forward_name))

    def children(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, hidden, residual, ctx, run: int):
        # a part that can take its norm into its first projection does so (forward_normed
        # returns its output and the new residual stream); the others get a normalised input
        # A forward_normed may return None as its output: it has added it to the stream already.
        if hasattr(self.mixer, "forward_normed"):
            mixed, residual = self.mixer.forward_normed(hidden, residual, self.mixer_norm, ctx, run)
        else:
            x, residual = _normed(self.mixer_norm, hidden, residual)
            mixed = self.mixer.forward(x, ctx, run)
        if hasattr(self.feed_forward, "forward_normed"):
            return self.feed_forward.forward_normed(mixed, residual, self.feed_forward_norm, ctx)
        x, residual = _normed(self.feed_forward_norm, mixed, residual)
        return self.feed_forward.forward(x, ctx), residual


def _normed(norm, hidden, residual):
    """(norm(hidden + residual), hidden + residual); either of the two may be missing: the first
    layer has no residual yet, and a part that added its output to the stream returns no output."""
    if hidden is None:
        return norm.forward(residual), residual
    if residual is None:
        return norm.forward(hidden), hidden
    return norm.add(hidden, residual)


register_part("block", "prenorm_residual", PreNormResidualBlock)
