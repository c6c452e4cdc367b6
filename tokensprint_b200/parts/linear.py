"""Matrix product of activations with a row-major [out, in] weight.

bfloat16: steps of up to SKINNY_ROWS tokens (decode, short portions) stream the weights through
the engine's own tcgen05 kernel (csrc/gemm_tcgen05.cu); larger steps use the library
GEMM (cuBLAS through torch.mm), as the reference does with nn.Linear
(engine/nn/attention.py:122-135, engine/nn/layers.py:61-66).  float32 runs use the
engine's own FFMA kernel, so no reduced-precision matrix mode can slip into the 32-bit
path whatever torch's global switches say.
"""

from __future__ import annotations

import os
from typing import Optional

import torch

from tokensprint_b200 import ops


# Up to this many rows the engine's own weight-streaming kernel is used; above it the
# library GEMM is (measured on B200 at Qwen3-8B sizes: the own kernel wins while the step is
# bound by reading the weights).
SKINNY_ROWS = int(os.environ.get("TS_SKINNY_ROWS", "32"))  # the variable is for measurements


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
            ops.library_mm(x, weight, out=out)
    else:
        raise ops.KernelError(f"linear: unsupported dtype {x.dtype}")
    return out


FOLD_NORMS = os.environ.get("TS_FOLD_NORMS", "1") != "0"  # 0: every norm and activation stays a kernel of its own


def folding_possible(num_tokens: int, dtype: torch.dtype, *weights: torch.Tensor) -> bool:
    """Whether the products of a step of `num_tokens` rows with these weights run through the
    engine's own GEMM with fused epilogues (so norms, residual sums and the activation can be
    folded into them): bfloat16, few rows, shapes the kernel takes."""
    if not FOLD_NORMS or dtype != torch.bfloat16 or not 0 < num_tokens <= min(SKINNY_ROWS, ops.GEMM_FUSED_MAX_ROWS):
        return False
    for w in weights:
        if not ops.matrix_streams_through_own_gemm(w):
            return False
    return True


def linear_scaled(x: "PreNormed | torch.Tensor", weight: torch.Tensor, next_weight: Optional[torch.Tensor] = None,
                  float32_out: bool = False) -> torch.Tensor:
    """linear() for an input whose norm still lacks its 1/rms (a PreNormed): the factor is applied
    to the rows of the product.  A plain tensor is passed on to linear()."""
    if isinstance(x, torch.Tensor):
        return linear_float32_out(x, weight) if float32_out else linear(x, weight, next_weight=next_weight)
    out = torch.empty((x.x.shape[0], weight.shape[0]), device=x.x.device, dtype=torch.float32 if float32_out else x.x.dtype)
    ops.gemm_skinny_fused(x.x, weight, out=out, scale_ssq=x.ssq, scale_width=x.width, scale_eps=x.eps, prefetch=next_weight)
    return out


def linear_swiglu(x: "PreNormed | torch.Tensor", gate_up_blocks: torch.Tensor, next_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) in one kernel; the rows of `gate_up_blocks` come in blocks of 64
    gate rows and the 64 up rows of the same outputs."""
    xt = x if isinstance(x, torch.Tensor) else x.x
    out = torch.empty((xt.shape[0], gate_up_blocks.shape[0] // 2), device=xt.device, dtype=xt.dtype)
    if isinstance(x, torch.Tensor):
        ops.gemm_skinny_fused(x, gate_up_blocks, out=out, mode=ops.GEMM_EPILOGUE_SWIGLU, prefetch=next_weight)
    else:
        ops.gemm_skinny_fused(x.x, gate_up_blocks, out=out, mode=ops.GEMM_EPILOGUE_SWIGLU, scale_ssq=x.ssq, scale_width=x.width,
                              scale_eps=x.eps, prefetch=next_weight)
    return out


def linear_into_residual(x: torch.Tensor, weight: torch.Tensor, fold: "ResidualNorm", next_weight: Optional[torch.Tensor] = None) -> "PreNormed":
    """fold.hidden += x @ weight^T, and the input of the norm that follows, all in the product's
    kernel.  Returns the PreNormed that stands for norm(hidden)."""
    from tokensprint_b200.parts.base import PreNormed

    T, N = x.shape[0], weight.shape[0]
    xprime = torch.empty((T, N), device=x.device, dtype=x.dtype)
    ssq = torch.empty((-(-N // 128), T), device=x.device, dtype=torch.float32)
    ops.gemm_skinny_fused(x, weight, mode=ops.GEMM_EPILOGUE_RESIDUAL_NORM, hidden=fold.hidden, norm_weight=fold.norm.weight,
                          xprime=xprime, ssq_out=ssq, prefetch=next_weight)
    return PreNormed(xprime, ssq, fold.norm.width, fold.norm.eps)


def linear_float32_out(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Same product with a float32 result (the logits)."""
    if x.dtype == torch.float32:
        return linear(x, weight)
    if x.shape[0] <= SKINNY_ROWS and ops.gemm_skinny_supported(x, weight):
        out = torch.empty((x.shape[0], weight.shape[0]), device=x.device, dtype=torch.float32)
        ops.gemm_skinny_bf16(x, weight, out)
        return out
    if not x.is_cuda or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise ops.KernelError(f"linear: bfloat16 CUDA tensors wanted (there is no CPU path), got {x.dtype} on {x.device}")
    # the library product with a float32 result: the sums are not rounded to bfloat16 on the way out
    return ops.library_mm(x, weight, float32_out=True)
