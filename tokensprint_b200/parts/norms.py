"""RMSNorm over the float32 residual stream, fused with the residual sum before it."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import NormParams, BuildContext, Norm, TensorSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * weight, plain weight (not 1 + w), no bias.

    Reference: engine/nn/base_layers.py:38-46 and engine/kernels/triton/rmsnorm.py:19-42.
    """

    graph_safe = True
    reads_through_ops = True

    def __init__(self, ctx: BuildContext, *, dim: int, eps: float, weight: str) -> None:
        self.dim, self.eps, self.weight_name = int(dim), float(eps), weight
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.dim,), "vector")]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]

    def params(self) -> Optional[NormParams]:
        return NormParams(self.weight, self.eps, self.dim)

    def forward(self, hidden, delta, out, row_index=None) -> None:
        ops.add_rmsnorm(hidden, delta, self.weight, out, self.eps, row_index)
