// SwiGLU activation on the fused gate/up product: out[t, i] = silu(gate[t, i]) * up[t, i],
// silu(z) = z * sigmoid(z), evaluated in float32 (engine/nn/layers.py:66 of the reference:
// `F.silu(self.gate_proj(seqs)) * self.up_proj(seqs)`).  The product's 2 I columns come in one
// of two orders: `block` = 0: all gates, then all ups (gate i at column i, up at I + i);
// `block` = 64: blocks of 128 columns, the gates of 64 outputs and then their ups (gate i at
// column 128 (i / 64) + i % 64, up 64 further), the order the fused GEMM epilogue wants its
// weight rows in.
#include "common.cuh"

template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I, size_t total, int block) {
  ts_pdl_prologue();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  size_t t = idx / I;
  int i = (int)(idx - t * I);
  const TA* row = gu + t * (size_t)(2 * I);
  const int gi = block ? (i / block) * 2 * block + i % block : i;
  float g = ts_to_float(row[gi]);
  float u = ts_to_float(row[gi + (block ? block : I)]);
  float s = g / (1.f + expf(-g));
  out[idx] = ts_from_float<TA>(s * u);
}

// Eight bfloat16 per thread (16-byte loads) when the inner size allows it; the row comes from
// the grid (no division per thread), and the sigmoid uses the fast exponential and reciprocal:
// their error (2 ulp of float32) disappears in the rounding to bfloat16.
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I, int T, int block) {
  ts_pdl_prologue();
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) << 3;
  if (i >= I) return;
  const int gi = block ? (i / block) * 2 * block + i % block : i;  // eight outputs never straddle a block of 64
  const int ui = gi + (block ? block : I);
  for (int t = blockIdx.y; t < T; t += gridDim.y) {
    const __nv_bfloat16* row = gu + (size_t)t * (size_t)(2 * I);
    const uint4 g4 = *reinterpret_cast<const uint4*>(row + gi);
    const uint4 u4 = *reinterpret_cast<const uint4*>(row + ui);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
      o2[k] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x, __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * (size_t)I + i) = o4;
  }
}

TS_EXPORT int ts_swiglu(const void* gu, void* out, int act_dtype, int T, int I, int block, void* stream) {
  if (T <= 0) return 0;
  if (I <= 0 || (block != 0 && (block != 64 || I % 64))) return TS_ERR_BAD_ARGUMENT;
  size_t total = (size_t)T * I;
  unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, I, total, block);
  else if (act_dtype == TS_DTYPE_BF16 && I % 8 == 0 && ((uintptr_t)gu | (uintptr_t)out) % 16 == 0) {
    const int threads = I / 8 >= 256 ? 256 : 64;
    return ts_launch(swiglu_bf16x8_kernel, dim3((unsigned)((I / 8 + threads - 1) / threads), (unsigned)(T < 65535 ? T : 65535)), dim3(threads), 0, s,
                     (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, T, block);
  } else if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, total, block);
  else
    return TS_ERR_BAD_ARGUMENT;
  return ts_launch_status();
}
