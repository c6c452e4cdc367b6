// Token embedding: hidden[t, :] = table[ids[t], :], widened to the float32 residual stream.
// (engine/model.py:65 of the reference: `seqs = self.embedding(seqs)`.)
#include "common.cuh"

template <typename TW>
__global__ void embed_gather_kernel(float* __restrict__ hidden, const TW* __restrict__ table,
                                    const int* __restrict__ ids, int H, int V) {
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = hidden + (size_t)t * H;
  if (id < 0 || id >= V) {
    // An id outside the table is the caller's fault; make it loud, never silent.
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __int_as_float(0x7fc00000);
    return;
  }
  const TW* src = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ts_to_float(src[i]);
}

TS_EXPORT int ts_embed_gather(float* hidden, const void* table, int table_dtype, const int* ids,
                              int T, int H, int V, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || V <= 0) return TS_ERR_BAD_ARGUMENT;
  int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  cudaStream_t s = (cudaStream_t)stream;
  if (table_dtype == TS_DTYPE_F32)
    embed_gather_kernel<float><<<T, threads, 0, s>>>(hidden, (const float*)table, ids, H, V);
  else if (table_dtype == TS_DTYPE_BF16)
    embed_gather_kernel<__nv_bfloat16><<<T, threads, 0, s>>>(hidden, (const __nv_bfloat16*)table, ids, H, V);
  else
    return TS_ERR_BAD_ARGUMENT;
  return ts_launch_status();
}
