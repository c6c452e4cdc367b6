"""Matrix product of activations with a row-major [out, in] weight.

bfloat16: steps of up to SKINNY_ROWS tokens (decode, short portions) stream the weights through
the engine's own tcgen05 kernel (csrc/gemm_tcgen05.cu); larger steps use the library
GEMM (cuBLAS through torch.mm), as the reference does with nn.Linear
(engine/nn/attention.py:122-135, engine/nn/layers.py:61-66).  float32 runs use the
engine's own FFMA kernel, so no reduced-precision matrix mode can slip into the 32-bit
path whatever torch's global switches say.
"""

from __future__ import annotations

from typing import Optional

import torch

from tokensprint_b200 import ops


# Up to this many rows the engine's own weight-streaming kernel is used; above it the
# library GEMM is (measured on B200 at Qwen3-8B sizes: the own kernel wins while the step is
# bound by reading the weights).
SKINNY_ROWS = 32


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           next_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, in] @ weight[out, in]^T -> [T, out] in x's dtype.  `next_weight`: the matrix the
    following product reads, if the caller knows it (a hint for prefetching, never needed)."""
    if x.dtype != weight.dtype:
        raise ops.KernelError(f"linear: activation {x.dtype} and weight {weight.dtype} differ")
    T, N = x.shape[0], weight.shape[0]
    if out is None:
        out = torch.empty((T, N), device=x.device, dtype=x.dtype)
    if T == 0:
        return out
    if x.dtype == torch.float32:
        ops.sgemm_nt(x, weight, out)
    elif x.dtype == torch.bfloat16:
        if not x.is_cuda:
            raise ops.KernelError("linear: there is no CPU path")
        if T <= SKINNY_ROWS and ops.gemm_skinny_supported(x, weight):
            ops.gemm_skinny_bf16(x, weight, out, next_weight)
        else:
            torch.mm(x, weight.t(), out=out)
    else:
        raise ops.KernelError(f"linear: unsupported dtype {x.dtype}")
    return out


def linear_float32_out(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Same product with a float32 result (the logits)."""
    if x.dtype == torch.float32:
        return linear(x, weight)
    if x.shape[0] <= SKINNY_ROWS and ops.gemm_skinny_supported(x, weight):
        out = torch.empty((x.shape[0], weight.shape[0]), device=x.device, dtype=torch.float32)
        ops.gemm_skinny_bf16(x, weight, out)
        return out
    return linear(x, weight).float()
