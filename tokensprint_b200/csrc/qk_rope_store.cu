// Per-head q/k RMSNorm, rotary position encoding and the store of keys and values into
// the paged cache, in one pass over the fused q|k|v projection.
//
// Reference order (engine/nn/attention.py:171-188): unflatten heads, q_norm/k_norm over
// head_dim with one [head_dim] weight shared by all heads, then RoPE on q and k, then
// store_kvcache(k, v) by slot.  RoPE is the rotate-half pairing (j, j + rot/2) with
// angle = position * inv_freq[j], all float32 (engine/kernels/triton/rope.py:22-65,
// engine/nn/rope.py:28-29,116-123).  Here the normed value is not rounded to the model
// dtype before the rotation: one rounding at the store instead of two.
//
// One warp per (token, head).  Heads 0..nq-1 are queries (written to q_out), the next nkv
// are keys, the last nkv are values (copied).  A slot of -1 skips the key/value store.
// Without `slot_mapping` keys and values go to dense [T, nkv, d] buffers.
#include "common.cuh"

#define QKR_MAX_HEAD_DIM 512
#define QKR_WARPS 4

template <typename TA>
__global__ void qk_norm_rope_store_kernel(const TA* __restrict__ qkv, TA* __restrict__ q_out,
                                          TA* __restrict__ k_dst, TA* __restrict__ v_dst,
                                          const int* __restrict__ slot_mapping,
                                          const int* __restrict__ positions,
                                          const float* __restrict__ q_norm_w,
                                          const float* __restrict__ k_norm_w, float eps,
                                          const float* __restrict__ inv_freq, int rot_dim, int T,
                                          int nq, int nkv, int d) {
  ts_pdl_prologue();
  __shared__ float buf[QKR_WARPS][QKR_MAX_HEAD_DIM];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const long long item = (long long)blockIdx.x * QKR_WARPS + warp;
  if (item >= (long long)T * heads) return;
  const int t = (int)(item / heads);
  const int head = (int)(item - (long long)t * heads);
  const TA* src = qkv + ((size_t)t * heads + head) * d;

  const bool is_q = head < nq;
  const bool is_k = !is_q && head < nq + nkv;
  int slot = -1;
  if (!is_q) {
    slot = slot_mapping ? slot_mapping[t] : t;
    if (slot < 0) return;
  }
  if (!is_q && !is_k) {  // value head: plain copy
    TA* dst = v_dst + ((size_t)slot * nkv + (head - nq - nkv)) * d;
    for (int i = lane; i < d; i += 32) dst[i] = src[i];
    return;
  }

  float* x = buf[warp];
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    float v = ts_to_float(src[i]);
    x[i] = v;
    ss += v * v;
  }
  const float* w = is_q ? q_norm_w : k_norm_w;
  if (w) {
    ss = ts_warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)d + eps);
    for (int i = lane; i < d; i += 32) x[i] = x[i] * rstd * w[i];
  }
  __syncwarp();

  TA* dst = is_q ? q_out + ((size_t)t * nq + head) * d
                 : k_dst + ((size_t)slot * nkv + (head - nq)) * d;
  const int half = inv_freq ? rot_dim / 2 : 0;
  if (half > 0) {
    const float pos = (float)positions[t];
    for (int j = lane; j < half; j += 32) {
      float s, c;
      sincosf(pos * inv_freq[j], &s, &c);
      const float re = x[j], im = x[j + half];
      dst[j] = ts_from_float<TA>(re * c - im * s);
      dst[j + half] = ts_from_float<TA>(im * c + re * s);
    }
  }
  for (int i = 2 * half + lane; i < d; i += 32) dst[i] = ts_from_float<TA>(x[i]);
}

// Fast path: full-width rotation (or none), head_dim a multiple of 4.  A lane owns the element
// pairs (2l, 2l+1) (+64 per round) of the lower half and their partners in the upper half, keeps
// them in registers from the norm to the rotation, and moves them with 4- or 8-byte accesses.
#define QKR_ROUNDS 4

__device__ __forceinline__ float2 ts_load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 ts_load2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void ts_store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void ts_store2(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename TA>
__global__ void qk_norm_rope_store_pairs_kernel(const TA* __restrict__ qkv, TA* __restrict__ q_out,
                                                TA* __restrict__ k_dst, TA* __restrict__ v_dst,
                                                const int* __restrict__ slot_mapping,
                                                const int* __restrict__ positions,
                                                const float* __restrict__ q_norm_w,
                                                const float* __restrict__ k_norm_w, float eps,
                                                const float* __restrict__ inv_freq, int T, int nq, int nkv, int d,
                                                int heads_per_warp) {
  ts_pdl_prologue();
  // A warp takes `heads_per_warp` consecutive heads of one token: the sines and cosines of the
  // token's position are computed once and serve all of them.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const int groups = (heads + heads_per_warp - 1) / heads_per_warp;
  const long long item = (long long)blockIdx.x * QKR_WARPS + warp;
  if (item >= (long long)T * groups) return;
  const int t = (int)(item / groups);
  const int head0 = (int)(item - (long long)t * groups) * heads_per_warp;
  const int head1 = min(heads, head0 + heads_per_warp);
  const int half = d >> 1;
  const int slot = slot_mapping ? slot_mapping[t] : t;

  float cs[QKR_ROUNDS][4];  // cos, sin of the two pairs this lane owns in every round
  if (inv_freq && head0 < nq + nkv) {
    const float pos = (float)positions[t];
#pragma unroll
    for (int r = 0; r < QKR_ROUNDS; ++r) {
      const int j = 2 * lane + 64 * r;
      if (j < half) {
        const float2 f = ts_load2(inv_freq + j);
        sincosf(pos * f.x, &cs[r][1], &cs[r][0]);
        sincosf(pos * f.y, &cs[r][3], &cs[r][2]);
      }
    }
  }

  // Heads are taken four at a time: all loads of the four first, then the math and the stores,
  // so four rows are in flight per warp instead of one.
  constexpr int BATCH = 4;
  for (int hb = head0; hb < head1; hb += BATCH) {
    float2 lo[BATCH][QKR_ROUNDS], hi[BATCH][QKR_ROUNDS];
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
      const int head = hb + u;
      if (head >= head1) continue;
      if (head >= nq && slot < 0) continue;
      const TA* src = qkv + ((size_t)t * heads + head) * d;
#pragma unroll
      for (int r = 0; r < QKR_ROUNDS; ++r) {
        const int j = 2 * lane + 64 * r;
        if (j < half) {
          lo[u][r] = ts_load2(src + j);
          hi[u][r] = ts_load2(src + half + j);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
      const int head = hb + u;
      if (head >= head1) continue;
      const bool is_q = head < nq;
      const bool is_k = !is_q && head < nq + nkv;
      if (!is_q && slot < 0) continue;
      if (!is_q && !is_k) {  // value head: plain copy
        TA* dst = v_dst + ((size_t)slot * nkv + (head - nq - nkv)) * d;
#pragma unroll
        for (int r = 0; r < QKR_ROUNDS; ++r) {
          const int j = 2 * lane + 64 * r;
          if (j < half) {
            ts_store2(dst + j, lo[u][r].x, lo[u][r].y);
            ts_store2(dst + half + j, hi[u][r].x, hi[u][r].y);
          }
        }
        continue;
      }
      float ss = 0.f;
#pragma unroll
      for (int r = 0; r < QKR_ROUNDS; ++r) {
        const int j = 2 * lane + 64 * r;
        if (j < half)
          ss += lo[u][r].x * lo[u][r].x + lo[u][r].y * lo[u][r].y + hi[u][r].x * hi[u][r].x + hi[u][r].y * hi[u][r].y;
      }
      const float* w = is_q ? q_norm_w : k_norm_w;
      float rstd = 1.f;
      if (w) {
        ss = ts_warp_sum(ss);
        rstd = rsqrtf(ss / (float)d + eps);
      }
      TA* dst = is_q ? q_out + ((size_t)t * nq + head) * d : k_dst + ((size_t)slot * nkv + (head - nq)) * d;
#pragma unroll
      for (int r = 0; r < QKR_ROUNDS; ++r) {
        const int j = 2 * lane + 64 * r;
        if (j < half) {
          float2 a = lo[u][r], b = hi[u][r];
          if (w) {
            const float2 wl = ts_load2(w + j), wh = ts_load2(w + half + j);
            a.x *= rstd * wl.x; a.y *= rstd * wl.y;
            b.x *= rstd * wh.x; b.y *= rstd * wh.y;
          }
          if (inv_freq) {
            const float2 ra = make_float2(a.x * cs[r][0] - b.x * cs[r][1], a.y * cs[r][2] - b.y * cs[r][3]);
            const float2 rb = make_float2(b.x * cs[r][0] + a.x * cs[r][1], b.y * cs[r][2] + a.y * cs[r][3]);
            a = ra;
            b = rb;
          }
          ts_store2(dst + j, a.x, a.y);
          ts_store2(dst + half + j, b.x, b.y);
        }
      }
    }
  }
}

// Prompt-sized batches, bfloat16, a head size that is a power of two: LPR = d / 16 lanes share
// one head row (16-byte loads: 8 elements of the lower half and their 8 partners in the upper
// half per lane), so a warp works on 32 / LPR heads of one token at a time; the sines and
// cosines of the token's position are computed once per warp and serve all its heads.
template <int LPR>
__global__ void qk_norm_rope_store_vec8_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                               __nv_bfloat16* __restrict__ k_dst, __nv_bfloat16* __restrict__ v_dst,
                                               const int* __restrict__ slot_mapping, const int* __restrict__ positions,
                                               const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                                               float eps, const float* __restrict__ inv_freq, int T, int nq, int nkv,
                                               int warps_per_token) {
  ts_pdl_prologue();
  constexpr int D = LPR * 16, HALF = D / 2, ROWS = 32 / LPR;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * QKR_WARPS + warp;
  if (item >= (long long)T * warps_per_token) return;
  const int t = (int)(item / warps_per_token);
  const int part = (int)(item - (long long)t * warps_per_token);
  const int heads = nq + 2 * nkv;
  const int per_part = (heads + warps_per_token - 1) / warps_per_token;
  const int h0 = part * per_part, h1 = min(heads, h0 + per_part);
  const int sub = lane / LPR, l = lane % LPR;
  const int slot = slot_mapping ? slot_mapping[t] : t;

  float cs[8], sn[8];
  if (inv_freq && h0 < nq + nkv) {
    const float pos = (float)positions[t];
#pragma unroll
    for (int i = 0; i < 8; ++i) sincosf(pos * inv_freq[8 * l + i], &sn[i], &cs[i]);
  }

  for (int base = h0; base < h1; base += ROWS) {
    const int head = base + sub;
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    const bool active = head < h1 && (is_q || slot >= 0);
    uint4 raw_lo = make_uint4(0u, 0u, 0u, 0u), raw_hi = raw_lo;
    if (active) {
      const __nv_bfloat16* src = qkv + ((size_t)t * heads + head) * D + 8 * l;
      raw_lo = *reinterpret_cast<const uint4*>(src);
      raw_hi = *reinterpret_cast<const uint4*>(src + HALF);
    }
    __nv_bfloat16* dst = nullptr;
    if (active)
      dst = (is_q ? q_out + ((size_t)t * nq + head) * D
                  : is_k ? k_dst + ((size_t)slot * nkv + (head - nq)) * D : v_dst + ((size_t)slot * nkv + (head - nq - nkv)) * D) + 8 * l;
    float a[8], b[8];
    {
      const __nv_bfloat162* pl = reinterpret_cast<const __nv_bfloat162*>(&raw_lo);
      const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&raw_hi);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(pl[i]), y = __bfloat1622float2(ph[i]);
        a[2 * i] = x.x; a[2 * i + 1] = x.y;
        b[2 * i] = y.x; b[2 * i + 1] = y.y;
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
    // every lane takes part in the shuffles; the sums stay inside the LPR lanes of a row
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!active) continue;
    if (is_q || is_k) {
      const float* w = is_q ? q_norm_w : k_norm_w;
      if (w) {
        const float rstd = rsqrtf(ss / (float)D + eps);
        const float4 w0 = *reinterpret_cast<const float4*>(w + 8 * l), w1 = *reinterpret_cast<const float4*>(w + 8 * l + 4);
        const float4 w2 = *reinterpret_cast<const float4*>(w + HALF + 8 * l), w3 = *reinterpret_cast<const float4*>(w + HALF + 8 * l + 4);
        const float wl[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const float wh[8] = {w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          a[i] *= rstd * wl[i];
          b[i] *= rstd * wh[i];
        }
      }
      if (inv_freq) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float ra = a[i] * cs[i] - b[i] * sn[i];
          const float rb = b[i] * cs[i] + a[i] * sn[i];
          a[i] = ra;
          b[i] = rb;
        }
      }
      uint4 out_lo, out_hi;
      __nv_bfloat162* ol = reinterpret_cast<__nv_bfloat162*>(&out_lo);
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out_hi);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ol[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
        oh[i] = __floats2bfloat162_rn(b[2 * i], b[2 * i + 1]);
      }
      *reinterpret_cast<uint4*>(dst) = out_lo;
      *reinterpret_cast<uint4*>(dst + HALF) = out_hi;
    } else {  // value head: plain copy
      *reinterpret_cast<uint4*>(dst) = raw_lo;
      *reinterpret_cast<uint4*>(dst + HALF) = raw_hi;
    }
  }
}

template <int LPR>
static int launch_vec8(const void* qkv, void* q_out, void* k_dst, void* v_dst, const int* slot_mapping, const int* positions,
                       const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq, int T, int nq, int nkv,
                       cudaStream_t s) {
  // A warp takes `rows` heads of a token at a time.  Many tokens: two warps per token where a token
  // has enough heads for both; fewer tokens (a decode step of a large batch): more warps per token,
  // up to one per `rows` heads, so that a few thousand warps are in flight all the same.
  const int rows = 32 / LPR;
  const int heads = nq + 2 * nkv;
  int warps_per_token = heads >= 4 * rows ? 2 : 1;
  const int most = (heads + rows - 1) / rows;
  const int wanted = (int)((2048 + (long long)T - 1) / T);
  if (wanted > warps_per_token) warps_per_token = wanted < most ? wanted : most;
  const unsigned blocks = (unsigned)(((long long)T * warps_per_token + QKR_WARPS - 1) / QKR_WARPS);
  return ts_launch(qk_norm_rope_store_vec8_kernel<LPR>, dim3(blocks), dim3(QKR_WARPS * 32), 0, s, (const __nv_bfloat16*)qkv,
                   (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_dst, (__nv_bfloat16*)v_dst, slot_mapping, positions, q_norm_w, k_norm_w,
                   eps, inv_freq, T, nq, nkv, warps_per_token);
}

TS_EXPORT int ts_qk_norm_rope_store(const void* qkv, int act_dtype, void* q_out, void* k_dst,
                                    void* v_dst, const int* slot_mapping, const int* positions,
                                    const float* q_norm_w, const float* k_norm_w, float eps,
                                    const float* inv_freq, int rot_dim, int T, int nq, int nkv,
                                    int d, void* stream) {
  if (T <= 0) return 0;
  if (nq < 0 || nkv < 0 || nq + nkv <= 0 || d <= 0) return TS_ERR_BAD_ARGUMENT;
  if (d > QKR_MAX_HEAD_DIM) return TS_ERR_UNSUPPORTED_SIZE;
  if (inv_freq && (rot_dim <= 0 || rot_dim > d || (rot_dim & 1))) return TS_ERR_BAD_ARGUMENT;
  long long items = (long long)T * (nq + 2 * nkv);
  unsigned blocks = (unsigned)((items + QKR_WARPS - 1) / QKR_WARPS);
  cudaStream_t s = (cudaStream_t)stream;
  const bool pairs = (d % 4 == 0) && (d / 2 <= 64 * QKR_ROUNDS) && (!inv_freq || rot_dim == d) &&
                     (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_dst | (uintptr_t)v_dst | (uintptr_t)q_norm_w |
                       (uintptr_t)k_norm_w | (uintptr_t)inv_freq) % 8 == 0);
  // Many tokens: a warp takes 8 heads of a token and shares the trigonometry among them; few
  // tokens (decode): one head per warp, for the most warps in flight.
  const int heads_per_warp = T >= 256 ? 8 : 1;
  const int groups = (nq + 2 * nkv + heads_per_warp - 1) / heads_per_warp;
  const unsigned pair_blocks = (unsigned)(((long long)T * groups + QKR_WARPS - 1) / QKR_WARPS);
  // bfloat16 batches of 48 tokens or more with a power-of-two head size: 16-byte accesses, several heads per warp
  const bool vec8 = pairs && act_dtype == TS_DTYPE_BF16 && T >= 48 && d >= 16 && (d & (d - 1)) == 0 &&
                    (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_dst | (uintptr_t)v_dst | (uintptr_t)q_norm_w |
                      (uintptr_t)k_norm_w) % 16 == 0) && ((uintptr_t)inv_freq % 4 == 0);
  if (vec8) {
    switch (d) {
      case 16: return launch_vec8<1>(qkv, q_out, k_dst, v_dst, slot_mapping, positions, q_norm_w, k_norm_w, eps, inv_freq, T, nq, nkv, s);
      case 32: return launch_vec8<2>(qkv, q_out, k_dst, v_dst, slot_mapping, positions, q_norm_w, k_norm_w, eps, inv_freq, T, nq, nkv, s);
      case 64: return launch_vec8<4>(qkv, q_out, k_dst, v_dst, slot_mapping, positions, q_norm_w, k_norm_w, eps, inv_freq, T, nq, nkv, s);
      case 128: return launch_vec8<8>(qkv, q_out, k_dst, v_dst, slot_mapping, positions, q_norm_w, k_norm_w, eps, inv_freq, T, nq, nkv, s);
      case 256: return launch_vec8<16>(qkv, q_out, k_dst, v_dst, slot_mapping, positions, q_norm_w, k_norm_w, eps, inv_freq, T, nq, nkv, s);
      case 512: return launch_vec8<32>(qkv, q_out, k_dst, v_dst, slot_mapping, positions, q_norm_w, k_norm_w, eps, inv_freq, T, nq, nkv, s);
    }
  }
  if (pairs && act_dtype == TS_DTYPE_F32) {
    return ts_launch(qk_norm_rope_store_pairs_kernel<float>, dim3(pair_blocks), dim3(QKR_WARPS * 32), 0, s,
        (const float*)qkv, (float*)q_out, (float*)k_dst, (float*)v_dst, slot_mapping, positions, q_norm_w,
        k_norm_w, eps, inv_freq, T, nq, nkv, d, heads_per_warp);
  }
  if (pairs && act_dtype == TS_DTYPE_BF16) {
    return ts_launch(qk_norm_rope_store_pairs_kernel<__nv_bfloat16>, dim3(pair_blocks), dim3(QKR_WARPS * 32), 0, s,
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_dst, (__nv_bfloat16*)v_dst,
        slot_mapping, positions, q_norm_w, k_norm_w, eps, inv_freq, T, nq, nkv, d, heads_per_warp);
  }
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(qk_norm_rope_store_kernel<float>, dim3(blocks), dim3(QKR_WARPS * 32), 0, s,
        (const float*)qkv, (float*)q_out, (float*)k_dst, (float*)v_dst, slot_mapping, positions,
        q_norm_w, k_norm_w, eps, inv_freq, rot_dim, T, nq, nkv, d);
  else if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(qk_norm_rope_store_kernel<__nv_bfloat16>, dim3(blocks), dim3(QKR_WARPS * 32), 0, s,
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_dst,
        (__nv_bfloat16*)v_dst, slot_mapping, positions, q_norm_w, k_norm_w, eps, inv_freq, rot_dim,
        T, nq, nkv, d);
  else
    return TS_ERR_BAD_ARGUMENT;
  return ts_launch_status();
}

// The rotation's cosines and sines for every token of a step, once for all layers that rotate with
// the same frequencies: out[t][j] = (cos, sin)(positions[t] * inv_freq[j]), j < half, with the
// same float32 product and the same sincosf as the kernels that rotate by themselves
// (engine/nn/rope.py:105-123 of the reference: angles and trigonometry in float32).
__global__ void rope_cos_sin_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int T, int half,
                                    float2* __restrict__ out) {
  ts_pdl_prologue();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const int t = i / half, j = i - t * half;
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
  out[i] = make_float2(cs, sn);
}

TS_EXPORT int ts_rope_cos_sin(const int* positions, const float* inv_freq, int T, int half, float* out, void* stream) {
  if (T <= 0 || half <= 0) return 0;
  if (positions == nullptr || inv_freq == nullptr || out == nullptr || ((uintptr_t)out % 8)) return TS_ERR_BAD_ARGUMENT;
  const int n = T * half;
  return ts_launch(rope_cos_sin_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, positions, inv_freq, T, half,
                   reinterpret_cast<float2*>(out));
}
