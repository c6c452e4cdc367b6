"""Arrangements of mixer, feed-forward and norms in one layer."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200.parts.base import (
    Block,
    BuildContext,
    LayerCache,
    PartSpec,
    StepContext,
    TensorSpec,
    build_part,
    register_part,
)


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """h = h + Mixer(Norm_a(h)); h = h + FeedForward(Norm_f(h))  (engine/nn/layers.py:111-121).

    The residual stream is float32.  Each branch output is handed on as `pending` and
    added by the next norm in the same pass that norms it, so a residual sum never costs
    a pass over memory of its own.
    """

    def __init__(self, ctx: BuildContext, *, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, ffn_norm: PartSpec) -> None:
        self.dtype = ctx.dtype
        self.mixer = build_part("mixer", mixer, ctx)
        self.feed_forward = build_part("feed_forward", feed_forward, ctx)
        self.mixer_norm = build_part("norm", mixer_norm, ctx)
        self.ffn_norm = build_part("norm", ffn_norm, ctx)
        self._parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)
        self.graph_safe = all(p.graph_safe for p in self._parts)

    def tensor_specs(self) -> list[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load(tensors)

    def forward(self, hidden, pending, step: StepContext, cache: LayerCache) -> Optional[torch.Tensor]:
        normed = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
        after_block = step.weight_after
        self.mixer_norm.forward(hidden, pending, normed)
        step.weight_after = self.feed_forward.first_weight()
        mixed = self.mixer.forward(normed, step, cache)
        self.ffn_norm.forward(hidden, mixed, normed)
        step.weight_after = after_block
        return self.feed_forward.forward(normed, step)

    def first_weight(self):
        return self.mixer.first_weight()
