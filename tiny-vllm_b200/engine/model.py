"""A model put together from a :class:`ModelSpec`, and its forward over one step.

The model owns the parts and the run list and nothing else: the cache belongs
to the cache storage, the batch to the step context.  Weights are bound by the
loader or drawn at random.  Layer arrangement and final norm follow
tinyvllm/models/qwen3.py:458-494 and :703-717.
"""

from __future__ import annotations

from pathlib import Path

import torch

from ..config.spec import ModelSpec
from ..parts import BuildContext, build_part
from ..parts.base import Part
from ..weights.loader import bind_tensors, load_checkpoint
from ..weights.random_init import random_tensors


class Model:
    def __init__(self, spec: ModelSpec, *, device, dtype: torch.dtype) -> None:
        self.spec = spec
        self.device = torch.device(device)
        self.dtype = dtype
        top = BuildContext(self.device, dtype, "", build_part)
        self.embedding = build_part("embedding", spec.embedding, top)
        self.blocks = []
        for layer in spec.layers:
            ctx = BuildContext(self.device, dtype, layer.prefix, build_part)
            self.blocks.append(build_part(
                "block", layer.block, ctx,
                mixer=layer.mixer, feed_forward=layer.feed_forward, norm=layer.norm))
        self.final_norm = build_part("norm", spec.final_norm, top)
        self.head = build_part("head", spec.head, top)
        self.order = spec.order

    # ---------------------------------------------------------------- parts
    def parts(self) -> list[Part]:
        found = self.embedding.all_parts()
        for block in self.blocks:
            found.extend(block.all_parts())
        found.extend(self.final_norm.all_parts())
        found.extend(self.head.all_parts())
        return found

    def param_targets(self):
        """(part, ParamSpec) of every tensor, in declaration order."""
        return [(part, spec) for part in self.parts() for spec in part.param_specs()]

    def cache_needs(self) -> list:
        """What each entry of the run list needs of the cache."""
        return [self.blocks[step.layer].cache_need() for step in self.order]

    def cache_sources(self) -> list:
        return [step.cache_from for step in self.order]

    # -------------------------------------------------------------- weights
    def _after_binding(self) -> None:
        tied = getattr(self.head, "tied_to", None)
        if tied is not None:
            if tied != getattr(self.embedding, "name", None):
                raise ValueError(f"the head is tied to {tied}, which is not the embedding")
            self.head.bind("weight", self.embedding.weight)
        for part in self.parts():
            finalize = getattr(part, "finalize", None)
            if finalize is not None:
                finalize()
        if self.device.type == "cuda":
            # the order in which a step streams the large weights: each product fetches the next
            from ..ops.gemm import chain_weights
            streamed = []
            for step in self.order:
                block = self.blocks[step.layer]
                for part in block.all_parts():
                    streamed.extend(getattr(part, "streamed_weights", lambda: [])())
            streamed.extend(getattr(self.head, "streamed_weights", lambda: [])())
            chain_weights(streamed)

    def _name_aliases(self) -> dict[str, str]:
        # a tied head may be stored under its own name, beside the embedding or instead of it: it is
        # the embedding (tinyvllm/models/qwen3.py:637-641, :682-686)
        tied = getattr(self.head, "tied_to", None)
        return {self.head.name: tied} if tied is not None else {}

    def load(self, folder: str | Path) -> "Model":
        load_checkpoint(self.param_targets(), folder, dtype=self.dtype, device=self.device,
                        aliases=self._name_aliases())
        self._after_binding()
        return self

    def init_random(self, seed: int) -> "Model":
        """Draw every tensor on the device; values differ from a folder written with
        the same seed on the host, the laws are the same."""
        targets = self.param_targets()
        bind_tensors(targets, random_tensors(targets, seed, device=self.device),
                     dtype=self.dtype, device=self.device)
        self._after_binding()
        return self

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for part, spec in self.param_targets():
            tensor = getattr(part, spec.attr)
            if tensor is not None and tensor.data_ptr() not in seen:
                seen.add(tensor.data_ptr())
                total += tensor.numel() * tensor.element_size()
        return total

    # -------------------------------------------------------------- forward
    def forward(self, ctx) -> torch.Tensor | None:
        """Logits (float32, [wanted rows, vocab]) of the step described by ``ctx``,
        or None when no row is wanted.  Keys and values of all tokens are written."""
        hidden = self.embedding.forward(ctx.token_ids)
        residual = None
        for run, step in enumerate(self.order):
            hidden, residual = self.blocks[step.layer].forward(hidden, residual, ctx, run)
        if ctx.num_wanted == 0:
            return None
        if hidden is None:          # the last block added its output to the stream itself
            hidden, residual = residual, None
        rows = self.final_norm.add_rows(hidden, residual, ctx.want_rows)
        return self.head.forward(rows)
