"""Arrangements of mixer, feed-forward and norms in one layer."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import (
    Block,
    BuildContext,
    LayerCache,
    PartSpec,
    PreNormed,
    ResidualNorm,
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
        # the block itself only hands tensors on; before a part that reads them by other means
        # than this package's ops, products that still wait in a chain are launched
        self.reads_through_ops = True

    def tensor_specs(self) -> list[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load(tensors)

    def entry_norm(self):
        return self.mixer_norm

    def forward(self, hidden, pending, step: StepContext, cache: LayerCache):
        """`pending`: None, the last branch output not yet added to `hidden`, or a PreNormed that
        stands for mixer_norm(hidden) (the part before prepared it; `hidden` is then complete).

        Where mixer and feed-forward offer it (`folds_norms`, and `can_fold` for this step), the
        norms and residual sums between them are folded into their products: the mixer's last
        product adds into `hidden` and prepares the feed-forward's input, the feed-forward's last
        product does the same for `step.norm_after`.  Otherwise every norm is a step of its own."""
        T = hidden.shape[0]
        after_block, norm_after = step.weight_after, step.norm_after
        mixer_folds = self.mixer.folds_norms and self.mixer.can_fold(T, self.dtype)
        ffn_folds = self.feed_forward.folds_norms and self.feed_forward.can_fold(T, self.dtype)

        if isinstance(pending, PreNormed) and mixer_folds:
            x = pending
        else:
            x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
            self._before(self.mixer_norm)
            self.mixer_norm.forward(hidden, None if isinstance(pending, PreNormed) else pending, x)
        step.weight_after = self.feed_forward.first_weight()
        ffn_norm = self.ffn_norm.params()
        self._before(self.mixer)
        if mixer_folds and ffn_folds and ffn_norm is not None:
            x = self.mixer.forward(x, step, cache, fold=ResidualNorm(hidden, ffn_norm))
        else:
            mixed = self.mixer.forward(x, step, cache)
            x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
            self._before(self.ffn_norm)
            self.ffn_norm.forward(hidden, mixed, x)
        step.weight_after = after_block
        next_norm = norm_after.params() if norm_after is not None else None
        self._before(self.feed_forward)
        if ffn_folds and next_norm is not None:
            return self.feed_forward.forward(x, step, fold=ResidualNorm(hidden, next_norm))
        return self.feed_forward.forward(x, step)

    @staticmethod
    def _before(part) -> None:
        if not part.reads_through_ops:
            ops.flush_gemm_chain()

    def first_weight(self):
        return self.mixer.first_weight()
