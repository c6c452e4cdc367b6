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

TS_EXPORT int ts_add_rmsnorm(float* hidden, const void* delta, int act_dtype, const float* weight,
                             void* out, const int* row_index, int rows, int H, float eps,
                             void* stream) {
  if (rows <= 0) return 0;
  if (H <= 0) return TS_ERR_BAD_ARGUMENT;
  int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : (H >= 256 ? 128 : 64));
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    add_rmsnorm_kernel<float><<<rows, threads, 0, s>>>(hidden, (const float*)delta, weight, (float*)out,
                                                       row_index, H, eps);
  else if (act_dtype == TS_DTYPE_BF16)
    add_rmsnorm_kernel<__nv_bfloat16><<<rows, threads, 0, s>>>(
        hidden, (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)out, row_index, H, eps);
  else
    return TS_ERR_BAD_ARGUMENT;
  return ts_launch_status();
}

// hidden[row] += delta[row] without a norm (the last residual sum when nothing follows it).
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ hidden, const TA* __restrict__ delta, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) hidden[i] += ts_to_float(delta[i]);
}

TS_EXPORT int ts_residual_add(float* hidden, const void* delta, int act_dtype, long long n, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  unsigned blocks = (unsigned)((n + 255) / 256);
  if (act_dtype == TS_DTYPE_F32)
    residual_add_kernel<float><<<blocks, 256, 0, s>>>(hidden, (const float*)delta, (size_t)n);
  else if (act_dtype == TS_DTYPE_BF16)
    residual_add_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(hidden, (const __nv_bfloat16*)delta, (size_t)n);
  else
    return TS_ERR_BAD_ARGUMENT;
  return ts_launch_status();
}
