"""Dense SwiGLU feed-forward."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, FeedForward, ResidualNorm, StepContext, TensorSpec, register_part
from tokensprint_b200.parts.linear import folding_possible, linear, linear_into_residual, linear_swiglu


@register_part("feed_forward", "swiglu")
class SwiGLUFeedForward(FeedForward):
    """f = (silu(x Wg^T) * (x Wu^T)) Wd^T (engine/nn/layers.py:61-66), no biases.

    Gate and up weights are stacked at load into one [2I, H] matrix so one product
    gives both halves.  When the width allows it the rows are stacked in blocks of 64 gate rows
    followed by the 64 up rows of the same outputs: a 128-row tile of the engine's own GEMM then
    holds both operands of 64 activations, and steps of few tokens get the activation from the
    GEMM's epilogue instead of from a kernel of its own.
    """

    graph_safe = True
    reads_through_ops = True
    folds_norms = True

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
        gate, up = tensors[self.names["gate"]], tensors[self.names["up"]]
        I, H = self.intermediate_size, self.hidden_size
        self.block = 64 if I % 64 == 0 else 0
        if self.block:
            self.gate_up = torch.stack([gate.view(I // 64, 64, H), up.view(I // 64, 64, H)], dim=1).reshape(2 * I, H).contiguous()
        else:
            self.gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.down = tensors[self.names["down"]]

    def forward(self, x, step: StepContext, fold: Optional[ResidualNorm] = None):
        """x: [T, H], or a PreNormed (then the products are the engine's own and apply the missing
        1/rms).  With `fold` the result is added into fold.hidden here and the PreNormed of the
        norm that follows is returned instead of the branch output."""
        after = step.weight_after if step is not None else None
        T = (x if isinstance(x, torch.Tensor) else x.x).shape[0]
        dtype = (x if isinstance(x, torch.Tensor) else x.x).dtype
        own = self.block == 64 and folding_possible(T, dtype, self.gate_up, self.down)
        if not isinstance(x, torch.Tensor) and not own:
            raise ops.KernelError("swiglu feed-forward: a PreNormed input needs the engine's own GEMM for both products")
        if own:
            act = linear_swiglu(x, self.gate_up, next_weight=self.down)
        else:
            gu = linear(x, self.gate_up, next_weight=self.down)
            act = torch.empty((T, self.intermediate_size), device=gu.device, dtype=gu.dtype)
            ops.swiglu(gu, act, self.block)
        if fold is not None:
            if not own:
                raise ops.KernelError("swiglu feed-forward: folding the residual sum needs the engine's own GEMM")
            return linear_into_residual(act, self.down, fold, next_weight=after)
        return linear(act, self.down, next_weight=after)

    def can_fold(self, num_tokens: int, dtype: torch.dtype) -> bool:
        return self.block == 64 and folding_possible(num_tokens, dtype, self.gate_up, self.down)
