"""Dense SwiGLU feed-forward."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, FeedForward, StepContext, TensorSpec, register_part
from tokensprint_b200.parts.linear import linear


@register_part("feed_forward", "swiglu")
class SwiGLUFeedForward(FeedForward):
    """f = (silu(x Wg^T) * (x Wu^T)) Wd^T (engine/nn/layers.py:61-66), no biases.

    Gate and up weights are stacked at load into one [2I, H] matrix so one product
    gives both halves and the activation kernel reads them side by side.
    """

    graph_safe = True

    def __init__(self, ctx: BuildContext, *, hidden_size: int, intermediate_size: int, gate: str, up: str, down: str) -> None:
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.names = {"gate": gate, "up": up, "down": down}
        self.gate_up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.gate_up

    def tensor_specs(self) -> list[TensorSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return [
            TensorSpec(self.names["gate"], (I, H)),
            TensorSpec(self.names["up"], (I, H)),
            TensorSpec(self.names["down"], (H, I)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.gate_up = torch.cat([tensors[self.names["gate"]], tensors[self.names["up"]]], dim=0).contiguous()
        self.down = tensors[self.names["down"]]

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        gu = linear(x, self.gate_up, next_weight=self.down)
        act = torch.empty((x.shape[0], self.intermediate_size), device=x.device, dtype=x.dtype)
        ops.swiglu(gu, act)
        return linear(act, self.down, next_weight=step.weight_after if step is not None else None)
