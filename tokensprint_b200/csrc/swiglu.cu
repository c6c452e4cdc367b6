// SwiGLU activation on the fused gate/up product: out[t, i] = silu(gu[t, i]) * gu[t, I + i],
// silu(z) = z * sigmoid(z), evaluated in float32 (engine/nn/layers.py:66 of the reference:
// `F.silu(self.gate_proj(seqs)) * self.up_proj(seqs)`).
#include "common.cuh"

template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  size_t t = idx / I;
  int i = (int)(idx - t * I);
  const TA* row = gu + t * (size_t)(2 * I);
  float g = ts_to_float(row[i]);
  float u = ts_to_float(row[I + i]);
  float s = g / (1.f + expf(-g));
  out[idx] = ts_from_float<TA>(s * u);
}

TS_EXPORT int ts_swiglu(const void* gu, void* out, int act_dtype, int T, int I, void* stream) {
  if (T <= 0) return 0;
  if (I <= 0) return TS_ERR_BAD_ARGUMENT;
  size_t total = (size_t)T * I;
  unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    swiglu_kernel<float><<<blocks, 256, 0, s>>>((const float*)gu, (float*)out, I, total);
  else if (act_dtype == TS_DTYPE_BF16)
    swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, total);
  else
    return TS_ERR_BAD_ARGUMENT;
  return ts_launch_status();
}
