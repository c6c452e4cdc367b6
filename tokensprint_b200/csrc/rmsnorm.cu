// Residual add + RMSNorm over the float32 residual stream.
//
//   h = hidden[row] (+ delta[row]);  hidden[row] = h (when a delta was added);
//   out[r] = h * rsqrt(mean(h^2) + eps) * weight
//
// Sums, mean, rsqrt and the scaling are float32 with one rounding at the store, as in the
// reference's kernel (engine/kernels/triton/rmsnorm.py:19-42); the residual sum is float32
// too (the reference adds in the model dtype, engine/nn/layers.py:112,121).  With
// `row_index` the kernel reads only the listed rows (the rows whose logits are wanted
// before the final norm) and leaves `hidden` untouched.
#include "common.cuh"

template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ hidden, const TA* __restrict__ delta,
                                   const float* __restrict__ weight, TA* __restrict__ out,
                                   const int* __restrict__ row_index, int H, float eps) {
  ts_pdl_prologue();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = row_index ? row_index[r] : r;
  float* h = hidden + (size_t)row * H;
  const TA* d = delta ? delta + (size_t)row * H : nullptr;
  TA* o = out + (size_t)r * H;
  const bool write_back = (d != nullptr) && (row_index == nullptr);

  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = h[i];
    if (d) v += ts_to_float(d[i]);
    if (write_back) h[i] = v;
    ss += v * v;
  }
  ss = ts_block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = h[i];
    if (d && !write_back) v += ts_to_float(d[i]);
    o[i] = ts_from_float<TA>(v * rstd * weight[i]);
  }
}

// Fast path for widths that are a multiple of 4: every thread keeps its (up to
// RN_MAX_CHUNKS) float4 pieces of the row in registers between the two passes, so the row
// is read once, with 16-byte loads issued back to back.
#define RN_MAX_CHUNKS 4

__device__ __forceinline__ float4 ts_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ts_load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void ts_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void ts_store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&a);
  raw.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TA>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ hidden, const TA* __restrict__ delta,
                                       const float* __restrict__ weight, TA* __restrict__ out,
                                       const int* __restrict__ row_index, int H, float eps) {
  ts_pdl_prologue();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = row_index ? row_index[r] : r;
  float* h = hidden + (size_t)row * H;
  const TA* d = delta ? delta + (size_t)row * H : nullptr;
  TA* o = out + (size_t)r * H;
  const bool write_back = (d != nullptr) && (row_index == nullptr);
  const int chunks = H >> 2;
  float4 v[RN_MAX_CHUNKS];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      v[k] = ts_load4(h + 4 * c);
      if (d) {
        const float4 dv = ts_load4(d + 4 * c);
        v[k].x += dv.x; v[k].y += dv.y; v[k].z += dv.z; v[k].w += dv.w;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      if (write_back) ts_store4(h + 4 * c, v[k]);
      ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  ss = ts_block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
#pragma unroll
  for (int k = 0; k < RN_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      const float4 w = ts_load4(weight + 4 * c);
      ts_store4(o + 4 * c, make_float4(v[k].x * rstd * w.x, v[k].y * rstd * w.y, v[k].z * rstd * w.z, v[k].w * rstd * w.w));
    }
  }
}

template <typename TA>
static int launch_add_rmsnorm(float* hidden, const void* delta, const float* weight, void* out,
                              const int* row_index, int rows, int H, float eps, cudaStream_t s) {
  const int chunks = H >> 2;
  const bool aligned = (H % 4 == 0) && (((uintptr_t)hidden | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) % 16 == 0);
  if (aligned && chunks <= RN_MAX_CHUNKS * 1024) {
    int threads = (chunks + RN_MAX_CHUNKS - 1) / RN_MAX_CHUNKS;
    if (rows <= 512) threads = chunks;  // few rows: one piece per thread, shortest latency
    threads = min(1024, max(32, (threads + 31) / 32 * 32));
    return ts_launch(add_rmsnorm_vec_kernel<TA>, dim3(rows), dim3(threads), 0, s, hidden, (const TA*)delta, weight, (TA*)out, row_index, H, eps);
  } else {
    int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : (H >= 256 ? 128 : 64));
    return ts_launch(add_rmsnorm_kernel<TA>, dim3(rows), dim3(threads), 0, s, hidden, (const TA*)delta, weight, (TA*)out, row_index, H, eps);
  }
}

TS_EXPORT int ts_add_rmsnorm(float* hidden, const void* delta, int act_dtype, const float* weight,
                             void* out, const int* row_index, int rows, int H, float eps,
                             void* stream) {
  if (rows <= 0) return 0;
  if (H <= 0) return TS_ERR_BAD_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return launch_add_rmsnorm<float>(hidden, delta, weight, out, row_index, rows, H, eps, s);
  if (act_dtype == TS_DTYPE_BF16)
    return launch_add_rmsnorm<__nv_bfloat16>(hidden, delta, weight, out, row_index, rows, H, eps, s);
  return TS_ERR_BAD_ARGUMENT;
}

// hidden[row] += delta[row] without a norm (the last residual sum when nothing follows it).
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ hidden, const TA* __restrict__ delta, size_t n) {
  ts_pdl_prologue();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) hidden[i] += ts_to_float(delta[i]);
}

TS_EXPORT int ts_residual_add(float* hidden, const void* delta, int act_dtype, long long n, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  unsigned blocks = (unsigned)((n + 255) / 256);
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, s, hidden, (const float*)delta, (size_t)n);
  else if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(residual_add_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, hidden, (const __nv_bfloat16*)delta, (size_t)n);
  else
    return TS_ERR_BAD_ARGUMENT;
  return ts_launch_status();
}
