"""Rotary position encoding (rotate-half pairing) as a part of its own."""

from __future__ import annotations

from typing import Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, PositionEncoding, StepContext, register_part


def rope_inverse_frequencies(dim: int, theta: float) -> torch.Tensor:
    """inv_freq[j] = 1 / theta^(2j/dim), j = 0..dim/2-1, float32 on the host.

    The reference's formula and dtype (engine/nn/rope.py:28-29).
    """
    idx = torch.arange(0, dim, step=2, dtype=torch.float32)
    return 1.0 / (theta ** (idx / dim))


@register_part("position_encoding", "rotary")
class RotaryEncoding(PositionEncoding):
    """x'[j] = x[j] cos - x[j+r/2] sin, x'[j+r/2] = x[j+r/2] cos + x[j] sin over the first
    `dim` (= r) entries of each head, angle = position * inv_freq[j] in float32
    (engine/nn/rope.py:105-123, engine/kernels/triton/rope.py:22-65).  The rotation
    itself runs inside the fused q/k kernel; this part owns the frequencies."""

    graph_safe = True

    def __init__(self, ctx: BuildContext, *, dim: int, theta: float) -> None:
        if dim % 2:
            raise ValueError(f"rotary width must be even, got {dim}")
        self.dim, self.theta = int(dim), float(theta)
        self.inv_freq = rope_inverse_frequencies(self.dim, self.theta).to(ctx.device)

    def rotary_inv_freq(self) -> Optional[torch.Tensor]:
        return self.inv_freq

    def rotary_cos_sin(self, step: StepContext) -> Optional[torch.Tensor]:
        """The table of the step, made by the first layer that asks and used by all layers with the
        same width and base (angles, cosines and sines in float32, as in the rotating kernels)."""
        key = ("rotary_cos_sin", self.dim, self.theta)
        table = step.shared.get(key)
        if table is None:
            table = step.shared[key] = ops.rope_cos_sin(step.positions, self.inv_freq, step.num_tokens)
        return table
