// Token embedding: hidden[t, :] = table[ids[t], :], widened to the float32 residual stream.
// (engine/model.py:65 of the reference: `seqs = self.embedding(seqs)`.)
#include "common.cuh"

template <typename TW>
__global__ void embed_gather_kernel(float* __restrict__ hidden, const TW* __restrict__ table,
                                    const int* __restrict__ ids, int H, int V) {
  ts_pdl_prologue();
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

__global__ void embed_gather_bf16x8_kernel(float* __restrict__ hidden, const __nv_bfloat16* __restrict__ table,
                                           const int* __restrict__ ids, int H, int V) {
  ts_pdl_prologue();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = hidden + (size_t)t * H;
  const bool ok = id >= 0 && id < V;
  const __nv_bfloat16* src = table + (size_t)(ok ? id : 0) * H;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float4 a, b;
    if (ok) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + i);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
      const float2 f2 = __bfloat1622float2(h2[2]), f3 = __bfloat1622float2(h2[3]);
      a = make_float4(f0.x, f0.y, f1.x, f1.y);
      b = make_float4(f2.x, f2.y, f3.x, f3.y);
    } else {
      const float nan = __int_as_float(0x7fc00000);
      a = b = make_float4(nan, nan, nan, nan);
    }
    *reinterpret_cast<float4*>(dst + i) = a;
    *reinterpret_cast<float4*>(dst + i + 4) = b;
  }
}

TS_EXPORT int ts_embed_gather(float* hidden, const void* table, int table_dtype, const int* ids,
                              int T, int H, int V, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || V <= 0) return TS_ERR_BAD_ARGUMENT;
  int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  cudaStream_t s = (cudaStream_t)stream;
  if (table_dtype == TS_DTYPE_F32)
    return ts_launch(embed_gather_kernel<float>, dim3(T), dim3(threads), 0, s, hidden, (const float*)table, ids, H, V);
  else if (table_dtype == TS_DTYPE_BF16 && H % 8 == 0 && ((uintptr_t)hidden | (uintptr_t)table) % 16 == 0)
    return ts_launch(embed_gather_bf16x8_kernel, dim3(T), dim3(min(1024, max(32, (H / 8 + 31) / 32 * 32))), 0, s, hidden, (const __nv_bfloat16*)table, ids, H, V);
  else if (table_dtype == TS_DTYPE_BF16)
    return ts_launch(embed_gather_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, s, hidden, (const __nv_bfloat16*)table, ids, H, V);
  else
    return TS_ERR_BAD_ARGUMENT;
  return ts_launch_status();
}

// Token ids that an earlier kernel left on the device (the ids the step before sampled): lane
// lanes[i] of `ids` takes source[rows[i]].  The other lanes of `ids` come from the host.
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ source, const int* __restrict__ lanes,
                                   const int* __restrict__ rows, int n) {
  ts_pdl_prologue();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) ids[lanes[i]] = source[rows[i]];
}

TS_EXPORT int ts_feed_tokens(int* ids, const int* source, const int* lanes, const int* rows, int n, void* stream) {
  if (n <= 0) return 0;
  return ts_launch(feed_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, ids, (const int*)source, lanes, rows, n);
}
