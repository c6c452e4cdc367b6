// Paged causal attention on CUDA cores, any element type: the float32 path's attention
// and the yardstick of the tensor-core kernels.
//
// For the query of token t (sequence b = seq_index[t], absolute position p = positions[t],
// head g): keys lo..p of the same sequence from KV head g / (nq / nkv), where lo = 0 or
// p - window + 1 for a sliding layer; s = (q . k) * scale; softmax over the keys;
// o = sum p * v.  Scores, running max and sum, and the output accumulate in float32
// (engine/nn/sdpa.py:56,85-102 of the reference: scale head_dim^-0.5, causal, GQA by head
// ratio, keys and values read through the block table).  Key j of sequence b lives at
// slot block_table[b][j / page] * page + j % page.
//
// One warp per (token, head).  Keys are taken 32 at a time: each lane scores one key,
// the warp agrees on the new running max, then all lanes walk the 32 values together,
// each owning head dims lane, lane + 32, ...  The order of the sums for one query depends
// only on its own keys, never on the batch around it.
#include "common.cuh"

#define ATS_MAX_HEAD_DIM 512
#define ATS_WARPS 4

template <typename TA>
__global__ void attention_paged_simple_kernel(
    const TA* __restrict__ q, const TA* __restrict__ kcache, const TA* __restrict__ vcache,
    TA* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ seq_index,
    const int* __restrict__ block_table, int max_blocks, int page, int T, int nq, int nkv, int d,
    float scale, int window) {
  ts_pdl_prologue();
  __shared__ float qs[ATS_WARPS][ATS_MAX_HEAD_DIM];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * ATS_WARPS + warp;
  if (item >= (long long)T * nq) return;
  const int t = (int)(item / nq);
  const int g = (int)(item - (long long)t * nq);
  const int hk = g / (nq / nkv);
  const int b = seq_index[t];
  if (b < 0) {  // a padded lane of a fixed-size batch: no sequence behind it
    TA* orow = out + ((size_t)t * nq + g) * d;
    for (int i = lane; i < d; i += 32) orow[i] = ts_from_float<TA>(0.f);
    return;
  }
  const int p = positions[t];
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int* table = block_table + (size_t)b * max_blocks;

  const TA* qrow = q + ((size_t)t * nq + g) * d;
  for (int i = lane; i < d; i += 32) qs[warp][i] = ts_to_float(qrow[i]) * scale;
  __syncwarp();

  constexpr int ACC = ATS_MAX_HEAD_DIM / 32;
  float acc[ACC];
#pragma unroll
  for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int base = lo; base <= p; base += 32) {
    const int j = base + lane;
    float s = -INFINITY;
    size_t slot = 0;
    if (j <= p) {
      slot = (size_t)table[j / page] * page + (j % page);
      const TA* krow = kcache + (slot * nkv + hk) * d;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot += qs[warp][i] * ts_to_float(krow[i]);
      s = dot;
    }
    const float m_new = fmaxf(m, ts_warp_max(s));
    const float corr = expf(m - m_new);  // m = -inf on the first round: exp(-inf) = 0
    const float pj = (j <= p) ? expf(s - m_new) : 0.f;
    l = l * corr + ts_warp_sum(pj);
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] *= corr;
    const int n = min(32, p - base + 1);
    for (int kk = 0; kk < n; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, pj, kk);
      const size_t sk = __shfl_sync(0xffffffffu, (unsigned long long)slot, kk);
      const TA* vrow = vcache + (sk * nkv + hk) * d;
#pragma unroll
      for (int i = 0; i < ACC; ++i) {
        const int dim = lane + 32 * i;
        if (dim < d) acc[i] += pk * ts_to_float(vrow[dim]);
      }
    }
    m = m_new;
  }
  TA* orow = out + ((size_t)t * nq + g) * d;
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < ACC; ++i) {
    const int dim = lane + 32 * i;
    if (dim < d) orow[dim] = ts_from_float<TA>(acc[i] * inv);
  }
}

TS_EXPORT int ts_attention_paged_simple(const void* q, const void* kcache, const void* vcache,
                                        int act_dtype, void* out, const int* positions,
                                        const int* seq_index, const int* block_table,
                                        int max_blocks, int page, int T, int nq, int nkv, int d,
                                        float scale, int window, void* stream) {
  if (T <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || d <= 0 || page <= 0 || max_blocks <= 0)
    return TS_ERR_BAD_ARGUMENT;
  if (d > ATS_MAX_HEAD_DIM) return TS_ERR_UNSUPPORTED_SIZE;
  long long items = (long long)T * nq;
  unsigned blocks = (unsigned)((items + ATS_WARPS - 1) / ATS_WARPS);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(attention_paged_simple_kernel<float>, dim3(blocks), dim3(ATS_WARPS * 32), 0, s,
        (const float*)q, (const float*)kcache, (const float*)vcache, (float*)out, positions,
        seq_index, block_table, max_blocks, page, T, nq, nkv, d, scale, window);
  else if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(attention_paged_simple_kernel<__nv_bfloat16>, dim3(blocks), dim3(ATS_WARPS * 32), 0, s,
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache,
        (__nv_bfloat16*)out, positions, seq_index, block_table, max_blocks, page, T, nq, nkv, d,
        scale, window);
  else
    return TS_ERR_BAD_ARGUMENT;
  return ts_launch_status();
}
