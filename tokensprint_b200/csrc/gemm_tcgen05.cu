// Skinny bfloat16 GEMM for decode steps on the 5th-generation tensor cores:
//   out[M, N] = X[M, K] * W[N, K]^T,  M <= 128 tokens, float32 accumulation in tensor memory.
//
// A decode step reads every weight once and does little math with it, so the kernel is built
// to stream W at HBM speed from every SM at once.  The roles are swapped against the usual
// picture: the 128 rows of a W tile are the MMA's M dimension, the (padded) tokens its N
// dimension, so even one token fills the tensor core's rows.
//
// Work is counted in units of (128-row tile of W) x (64-wide chunk of K).  The grid is one
// persistent CTA per SM; CTA c takes the contiguous unit range [c * U/P, (c+1) * U/P), which
// may start and end in the middle of a tile (stream-K), so all SMs stream the same number of
// bytes whatever the layer's shape.  Inside a CTA, six warps:
//   * warp 0, one thread: TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of [128 x 64] W
//     tiles and [MPAD x 64] X tiles into a ring of shared-memory stages, running ahead
//     across tile boundaries;
//   * warp 1, one thread: tcgen05.mma (cta_group::1, kind::f16, M=128, N=MPAD, K=16) from the
//     stages into one of two TMEM accumulators; tcgen05.commit frees each stage and hands
//     each finished accumulator over;
//   * warps 2-5: read an accumulator back with tcgen05.ld while the next one fills, and
//     store it.  A tile that one CTA covered alone goes straight to the output.  A tile
//     shared by several CTAs goes to a float32 scratch slot; each contributor takes a
//     ticket, and the one that arrives last adds the slots in contributor order and writes
//     the result.  Nobody waits for another CTA.
// Every wait is on an mbarrier fed by this CTA's own copies and MMAs and gives up after a
// bounded number of tries; then the CTA raises the error word, frees its tensor memory and
// returns.
//
// The split of the work depends on the weight's shape and the SM count only, so a token's
// result does not depend on what else is in the batch.
//
// Chains.  Up to MAX_PHASES products that feed one another (a decode layer's output projection,
// gate/up, down, and the next layer's q/k/v) run as phases of ONE launch: every CTA works through
// its share of phase after phase.  The copies of a phase's weights start while the phase before
// is still being finished elsewhere (weights depend on nothing); only the copies of its
// activations wait, at a barrier over the whole grid that the CTAs pass when everyone has stored
// the phase before: a counter in device memory that every CTA raises once per phase and polls
// with a bounded wait.  All CTAs of the grid are resident together (one per SM, never more CTAs
// than SMs), and a kernel launched behind this one cannot take an SM before all of them are,
// because it may start only when every CTA here has begun.  The last CTA to leave the kernel
// zeroes the counters for the next launch.
//
// The reference runs these products through nn.Linear (engine/nn/attention.py:122-135,
// engine/nn/layers.py:61-66); W is row-major [out, in] as there.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

// Optional timestamps for tuning (compile with -DTS_GEMM_PROBE): every CTA records the
// nanosecond timer at a few points into args.probe[cta * 64 + i] (8 + 8 * phase + k for the stamps of a phase;
// 40..43 for the end of the CTA's last shared tile: partial sums fenced, ticket known, sums added, epilogue done).
#ifdef TS_GEMM_PROBE
#define TS_PROBE(i) do { if (args.probe) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); args.probe[blockIdx.x * 64 + (i)] = t_; } } while (0)
#else
#define TS_PROBE(i) do { } while (0)
#endif

namespace {

constexpr int TILE_N = 128;   // W rows per tile (the MMA's M)
// Boxes side by side per stage.  Two (256 contiguous bytes of every W row asked for at once, half
// as many stages of twice the size) measured the same alone and 4 % slower inside the decode step.
// Tiles of W and X in flight per CTA, for up to 64 rows (a build option for measurements: 6, 10
// and 12 were measured no better than 8).
#ifndef TS_GEMM_STAGES
#define TS_GEMM_STAGES 8
#endif
#ifndef TS_GEMM_KATOMS
#define TS_GEMM_KATOMS 1
#endif
constexpr int ATOM_K = 64;                       // bf16 per row of one TMA box: one 128-byte swizzle atom
constexpr int KATOMS = TS_GEMM_KATOMS;
constexpr int TILE_K = ATOM_K * KATOMS;          // bf16 per stage and row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int MAX_CONTRIB = 8;   // most CTAs that may share one tile
constexpr int EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_RESIDUAL_NORM = 2, EPI_QK_ROPE = 3;
constexpr int FUSED_MAX_ROWS = 32;
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int MAX_PHASES = 4;            // products per chained launch
constexpr uint32_t GRID_SPIN_LIMIT = 1u << 23;  // polls of the grid barrier (each a tenth of a microsecond or more)

template <int MPAD>
struct Cfg {
  static constexpr uint32_t A_BYTES = TILE_N * TILE_K * 2;
  static constexpr uint32_t B_BYTES = MPAD * TILE_K * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + ((B_BYTES + 1023) / 1024) * 1024;
  // Stages of the ring.  Measured inside the decode step (8 rows, Qwen3-8B sizes): 6 stages
  // 4.52 ms, 8 4.39 ms, 10 4.40 ms, 12 4.47 ms per step: more bytes in flight than the memory
  // system turns around only queue up.
  static constexpr int STAGES = (MPAD <= 64 ? TS_GEMM_STAGES : 6) / KATOMS;
  static constexpr uint32_t A_ATOM = TILE_N * ATOM_K * 2;  // one box of W
  static constexpr uint32_t B_ATOM = MPAD * ATOM_K * 2;    // one box of X
  static constexpr uint32_t TMEM_COLS = 2 * MPAD < 32 ? 32 : 2 * MPAD;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
};

struct GemmArgs {
  void* out;             // [M, ldo] bf16 or f32
  float* partial;        // [ctas, 2, M, 128] f32: at most two shared tiles per CTA
  int* counters;         // [n_tiles] zero before the first launch, zero again after each
  int* error;            // set to 1 when a wait gave up
  int M, N, K, ldo, out_f32;
  int tiles, chunks, units_per;  // chunks of K per tile; units (tile x chunk) per CTA
  const char* prefetch;          // weights of the GEMM that follows (may be null)
  unsigned long long prefetch_bytes;
  // Fused epilogues (M <= 32), see ts_gemm_skinny_fused:
  int mode;                      // EPI_PLAIN, EPI_SWIGLU or EPI_RESIDUAL_NORM
  const float* scale_ssq;        // [scale_tiles, M] sums of squares of the rows of x's source, or null
  int scale_tiles;
  float scale_width, scale_eps;  // rstd[m] = rsqrt(sum / scale_width + scale_eps) multiplies row m of the product
  float* hidden;                 // EPI_RESIDUAL_NORM: [M, ldh] float32 residual, += the product
  const float* norm_w;           //   [N] weight of the norm that follows
  __nv_bfloat16* xprime;         //   [M, ldh] bf16(hidden * norm_w)
  float* ssq_out;                //   [tiles, M] sums of squares of the new hidden rows, per tile of 128 columns
  long long ldh;
  // EPI_QK_ROPE (head size 128 = one tile per head; rows of W: nq query heads, nkv key heads, nkv value heads):
  __nv_bfloat16* q_out;          //   [M, nq * 128]
  __nv_bfloat16* k_cache;        //   [slots, nkv, 128]
  __nv_bfloat16* v_cache;
  const int* slot_mapping;       //   [M] cache slot of every row, -1: no store
  const int* positions;          //   [M]
  const float* q_norm_w;         //   [128] or null
  const float* k_norm_w;
  const float* inv_freq;         //   [64] or null (no rotation)
  const float2* rope_cs;         //   [M, 64] (cos, sin) of positions[m] * inv_freq[j], or null: computed here
  float qk_eps;
  int nq, nkv;
#ifdef TS_GEMM_PROBE
  unsigned long long* probe;
#endif
};

// A chain of products: per phase its arguments and tensor maps, the grid barrier's counters
// (ts_gemm_chain_sync_words() unsigned ints, zero before the first launch; the kernel leaves them zero).
// (Templated on the most phases a launch holds: a product launched alone takes the one-phase
// form, whose parameters are as small as a single product's and are read at fixed offsets.)
template <int NPH>
struct ChainArgsT {
  GemmArgs g[NPH];
  int n;
  int hold;   // 1: a phase's copies start only when this CTA has stored the phase before
  int ahead;  // W tiles asked into the L2 beyond the ring while a phase waits for its inputs
  unsigned int* sync;
};
template <int NPH>
struct ChainMapsT {
  CUtensorMap w[NPH];
  CUtensorMap x[NPH];
};
using ChainArgs = ChainArgsT<MAX_PHASES>;
using ChainMaps = ChainMapsT<MAX_PHASES>;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait for a phase of an mbarrier.  False: gave up (or another role already did).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t limit = SPIN_LIMIT) {
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
// Grid barrier.  Per phase a counter that every CTA raises once its stores of the phase are done
// (and visible to the other SMs and their copy engines) and a flag that the last one to arrive
// sets; waiters poll the flag only, one thread per CTA, with a pause between polls, so that the
// arrivals do not queue behind the polls.  Each word has a 128-byte line of its own.  Wait: a
// bounded number of polls; false: gave up (or another role already did).
constexpr int SYNC_LINE = 32;  // unsigned ints per line
__device__ __forceinline__ unsigned int* sync_counter(unsigned int* sync, int phase) { return sync + (size_t)(2 * phase) * SYNC_LINE; }
__device__ __forceinline__ unsigned int* sync_flag(unsigned int* sync, int phase) { return sync + (size_t)(2 * phase + 1) * SYNC_LINE; }
__device__ __forceinline__ unsigned int* sync_departed(unsigned int* sync) { return sync + (size_t)(2 * MAX_PHASES) * SYNC_LINE; }
__device__ __forceinline__ void grid_arrive(unsigned int* sync, int phase, unsigned int ctas) {
  __threadfence();
  if (atomicAdd(sync_counter(sync, phase), 1u) == ctas - 1) {
    __threadfence();
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(sync_flag(sync, phase)), "r"(1u) : "memory");
  }
}
__device__ __forceinline__ bool grid_wait(unsigned int* sync, int phase, volatile int* abort_flag) {
  const unsigned int* flag = sync_flag(sync, phase);
  for (uint32_t i = 0; i < GRID_SPIN_LIMIT; ++i) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v != 0) return true;
    if (*abort_flag) return false;
    __nanosleep(100);
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// The same with a cache policy for the L2 (weights pass through once per step: "evict first"
// leaves the L2 to what is read again, the activations and what was asked ahead).
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "l"(policy) : "memory");
}
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart; descriptor version 1 (sm_100).
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// The share of one CTA: units [u0, u1) of tiles * chunks.
struct Range {
  int u0, u1;
};
__device__ __forceinline__ Range cta_range(const GemmArgs& a, int cta) {
  const long long total = (long long)a.tiles * a.chunks;
  Range r;
  r.u0 = (int)min(total, (long long)cta * a.units_per);
  r.u1 = (int)min(total, (long long)(cta + 1) * a.units_per);
  return r;
}

// What the fused epilogues do with a finished tile (`tile`: [M][128] float32 sums of the
// products, rows of W down the 128).  Called by the 128 epilogue threads together.
//   EPI_PLAIN with a row scale: out = rstd[m] * sum.
//   EPI_SWIGLU: the tile's first 64 rows of W are gate rows and the last 64 the up rows of the
//     same 64 outputs: out[m][64 t + j] = silu(rstd g) * (rstd u).
//   EPI_RESIDUAL_NORM: hidden[m][n] += sum; xprime = bf16(hidden * norm_w[n]); ssq_out[t][m] =
//     the sum over the tile's columns of hidden^2 (a warp takes a whole row of the tile, so
//     the sum needs shuffles only and is the same in every run).
// `ahead` (EPI_RESIDUAL_NORM): what this thread will need from device memory, asked for when the
// tile's accumulator was taken (hidden values in the order of the loop below, then the norm's four
// weights), so that the trips are over when the sums are there.
template <int MPAD>
struct EpilogueAhead {
  static constexpr int ROUNDS = MPAD / 4;  // passes of the 128 threads over a tile of MPAD rows x 32 pieces
  float4 hidden[ROUNDS];
  float4 norm_w;
};
template <int MPAD>
__device__ __forceinline__ void load_ahead(const GemmArgs& args, int t, int etid, EpilogueAhead<MPAD>& ahead) {
  const int nl = (etid & 31) * 4, n0 = t * TILE_N + nl;
  const bool whole = n0 + 3 < args.N && (args.ldh & 3) == 0;  // the four columns exist and the rows are 16-byte aligned
#pragma unroll
  for (int it = 0; it < EpilogueAhead<MPAD>::ROUNDS; ++it) {
    const int m = (etid + it * 128) >> 5;
    float4 h = make_float4(0.f, 0.f, 0.f, 0.f);
    if (m < args.M) {
      const float* hp = args.hidden + (size_t)m * args.ldh + n0;
      if (whole) {
        h = __ldcg(reinterpret_cast<const float4*>(hp));
      } else {
        if (n0 < args.N) h.x = __ldcg(hp);
        if (n0 + 1 < args.N) h.y = __ldcg(hp + 1);
        if (n0 + 2 < args.N) h.z = __ldcg(hp + 2);
        if (n0 + 3 < args.N) h.w = __ldcg(hp + 3);
      }
    }
    ahead.hidden[it] = h;
  }
  float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
  if (n0 < args.N) w.x = args.norm_w[n0];
  if (n0 + 1 < args.N) w.y = args.norm_w[n0 + 1];
  if (n0 + 2 < args.N) w.z = args.norm_w[n0 + 2];
  if (n0 + 3 < args.N) w.w = args.norm_w[n0 + 3];
  ahead.norm_w = w;
}

template <int MPAD>
__device__ __forceinline__ void fused_epilogue(const GemmArgs& args, int t, int etid, int lane, const float* tile, const float* rstd,
                                               const EpilogueAhead<MPAD>& ahead) {
  if (args.mode == EPI_SWIGLU) {
    const int half_n = args.N >> 1;
    for (int idx = etid; idx < args.M * 16; idx += 128) {
      const int m = idx >> 4, j = (idx & 15) * 4;
      const float4 g = *reinterpret_cast<const float4*>(tile + m * TILE_N + j);
      const float4 u = *reinterpret_cast<const float4*>(tile + m * TILE_N + 64 + j);
      const float r = rstd[m];
      const float gs[4] = {g.x * r, g.y * r, g.z * r, g.w * r}, us[4] = {u.x * r, u.y * r, u.z * r, u.w * r};
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(args.out) + (size_t)m * args.ldo + t * 64 + j;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (t * 64 + j + i < half_n) dst[i] = __float2bfloat16_rn(gs[i] / (1.f + __expf(-gs[i])) * us[i]);
    }
  } else if (args.mode == EPI_RESIDUAL_NORM) {
    const int nl = (etid & 31) * 4, n0 = t * TILE_N + nl;  // the 32 lanes of a warp share m
    const bool whole = n0 + 3 < args.N && (args.ldh & 3) == 0;
    const float nw[4] = {ahead.norm_w.x, ahead.norm_w.y, ahead.norm_w.z, ahead.norm_w.w};
#pragma unroll
    for (int it = 0; it < EpilogueAhead<MPAD>::ROUNDS; ++it) {
      const int m = (etid + it * 128) >> 5;
      if (m >= args.M) break;  // the same for the whole warp
      const float4 v = *reinterpret_cast<const float4*>(tile + m * TILE_N + nl);
      const float vals[4] = {v.x, v.y, v.z, v.w};
      const float old[4] = {ahead.hidden[it].x, ahead.hidden[it].y, ahead.hidden[it].z, ahead.hidden[it].w};
      float h[4];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        h[i] = old[i] + vals[i] * rstd[m];
        if (n0 + i < args.N) ss += h[i] * h[i];
      }
      float* hp = args.hidden + (size_t)m * args.ldh + n0;
      __nv_bfloat16* xp = args.xprime + (size_t)m * args.ldh + n0;
      if (whole) {
        *reinterpret_cast<float4*>(hp) = make_float4(h[0], h[1], h[2], h[3]);
        __nv_bfloat162 lo = __floats2bfloat162_rn(h[0] * nw[0], h[1] * nw[1]), hi = __floats2bfloat162_rn(h[2] * nw[2], h[3] * nw[3]);
        uint2 packed;
        packed.x = *reinterpret_cast<unsigned*>(&lo);
        packed.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(xp) = packed;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (n0 + i < args.N) {
            hp[i] = h[i];
            xp[i] = __float2bfloat16_rn(h[i] * nw[i]);
          }
        }
      }
      ss = ts_warp_sum(ss);
      if (lane == 0) args.ssq_out[(size_t)t * args.M + m] = ss;
    }
  } else if (args.mode == EPI_QK_ROPE) {
    // Tile t is head t: per-head RMS norm over the tile's 128 columns, rotate-half rotation of
    // the pairs (j, j + 64) (the partner sits 16 lanes away), then queries to q_out, keys and
    // values to their cache slot (engine/nn/attention.py:171-188 of the reference; angles and
    // trigonometry in float32).
    const bool is_q = t < args.nq, is_k = !is_q && t < args.nq + args.nkv;
    const float* w = is_q ? args.q_norm_w : (is_k ? args.k_norm_w : nullptr);
    for (int idx = etid; idx < args.M * 32; idx += 128) {
      const int m = idx >> 5, nl = (idx & 31) * 4;  // the 32 lanes of a warp share m
      const float4 v4 = *reinterpret_cast<const float4*>(tile + m * TILE_N + nl);
      float v[4] = {v4.x * rstd[m], v4.y * rstd[m], v4.z * rstd[m], v4.w * rstd[m]};
      if (is_q || is_k) {
        if (w != nullptr) {
          const float ss = ts_warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
          const float r = rsqrtf(ss / (float)TILE_N + args.qk_eps);
#pragma unroll
          for (int i = 0; i < 4; ++i) v[i] *= r * w[nl + i];
        }
        if (args.inv_freq != nullptr) {
          const float pos = (float)args.positions[m];
          const bool upper = nl >= 64;
          float sn[4], cs[4];
          if (args.rope_cs != nullptr) {
            // the step's table: the same float32 values that sincosf gives here, computed once for all layers
            const float4 a = *reinterpret_cast<const float4*>(args.rope_cs + (size_t)m * 64 + (nl & 63));
            const float4 b = *reinterpret_cast<const float4*>(args.rope_cs + (size_t)m * 64 + (nl & 63) + 2);
            cs[0] = a.x; sn[0] = a.y; cs[1] = a.z; sn[1] = a.w;
            cs[2] = b.x; sn[2] = b.y; cs[3] = b.z; sn[3] = b.w;
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) sincosf(pos * args.inv_freq[(nl & 63) + i], &sn[i], &cs[i]);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float partner = __shfl_xor_sync(0xffffffffu, v[i], 16);
            v[i] = upper ? v[i] * cs[i] + partner * sn[i] : v[i] * cs[i] - partner * sn[i];
          }
        }
      }
      const int slot = is_q ? 0 : args.slot_mapping[m];
      if (slot < 0) continue;
      __nv_bfloat16* dst = is_q ? args.q_out + ((size_t)m * args.nq + t) * TILE_N
                                : (is_k ? args.k_cache + ((size_t)slot * args.nkv + (t - args.nq)) * TILE_N
                                        : args.v_cache + ((size_t)slot * args.nkv + (t - args.nq - args.nkv)) * TILE_N);
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
      uint2 packed;
      packed.x = *reinterpret_cast<unsigned*>(&lo);
      packed.y = *reinterpret_cast<unsigned*>(&hi);
      *reinterpret_cast<uint2*>(dst + nl) = packed;
    }
  } else {
    for (int idx = etid; idx < args.M * 32; idx += 128) {
      const int m = idx >> 5, nl = (idx & 31) * 4;
      const float4 v = *reinterpret_cast<const float4*>(tile + m * TILE_N + nl);
      const float vals[4] = {v.x * rstd[m], v.y * rstd[m], v.z * rstd[m], v.w * rstd[m]};
      const int n0 = t * TILE_N + nl;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (n0 + i < args.N) {
          if (args.out_f32)
            reinterpret_cast<float*>(args.out)[(size_t)m * args.ldo + n0 + i] = vals[i];
          else
            reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)m * args.ldo + n0 + i] = __float2bfloat16_rn(vals[i]);
        }
      }
    }
  }
}

template <int MPAD, int NPH>
__global__ void __launch_bounds__(NUM_THREADS) gemm_skinny_kernel(const __grid_constant__ ChainMapsT<NPH> maps,
                                                                  const __grid_constant__ ChainArgsT<NPH> chain) {
  using C = Cfg<MPAD>;
  constexpr int STAGES = C::STAGES;
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MPAD >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24);

  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int last_s;
  __shared__ int go_s;
  __shared__ int ready_s;  // the last phase whose inputs the producer thread has seen ready
  __shared__ int arrived_s;  // how many phases this CTA's epilogue warps have stored and reported
  __shared__ __align__(16) float tile_s[(MPAD <= FUSED_MAX_ROWS ? MPAD : 1) * TILE_N];  // a finished tile, for the fused epilogues
  __shared__ float rstd_s[FUSED_MAX_ROWS];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int phases = NPH == 1 ? 1 : chain.n;
  const unsigned int ctas = gridDim.x;
  ts_pdl_launch_dependents();  // the next kernel may begin its own set-up now
  {
    const GemmArgs& args = chain.g[0];
    (void)args;
    if (tid == 0) TS_PROBE(0);
  }

  if (tid == 0) {
    abort_s = 0;
    last_s = 0;
    ready_s = 0;
    arrived_s = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(C::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort_flag = &abort_s;
  volatile int* ready_flag = &ready_s;
  volatile int* arrived_flag = &arrived_s;
  {
    const GemmArgs& args = chain.g[0];
    (void)args;
    if (tid == 0) TS_PROBE(1);
  }

  if (warp == 0) {
    if (lane == 0) {
      // Producer: TMA loads into the ring, unit after unit, across tile and phase boundaries.  The
      // weights are written by no kernel, so a phase's W tiles are requested before its inputs are
      // ready (the kernels ahead in the stream for the first phase, the phase before for the others):
      // up to a whole ring of them.  X, which is those inputs, follows when the wait is over.
      uint64_t w_policy;
      asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(w_policy));
      int it = 0;  // units requested so far, over all phases: the ring's clock
      bool ok = true;
      for (int p = 0; p < phases && ok; ++p) {
        const GemmArgs& args = chain.g[p];
        const Range range = cta_range(args, blockIdx.x);
        const int chunks = args.chunks;
        const int n_units = range.u1 - range.u0;
        const CUtensorMap* map_w = &maps.w[p];
        const CUtensorMap* map_x = &maps.x[p];
        const int first = it;   // ring clock of this phase's first unit
        int x_next = it;        // this phase's units before x_next have their X copy requested
        bool ready = false;     // the phase's inputs may be read
        // waits for the phase's inputs and requests the X copies that were held back
        auto inputs_ready = [&]() -> bool {
          if (p == 0) {
            ts_pdl_wait();
            TS_PROBE(6);
          } else {
            if (chain.ahead > 0) {
              // the ring is full and stands still until the inputs are there: meanwhile ask the L2 for
              // the W tiles of the units that come after the ring
              const int from = it - first, upto = min(n_units, from + chain.ahead);
              for (int j = from; j < upto; ++j) {
                const int u = range.u0 + j;
                const int t = u / chunks, kc = u - t * chunks;
                asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map_w), "r"(kc * TILE_K), "r"(t * TILE_N) : "memory");
              }
            }
            if (!grid_wait(chain.sync, p - 1, abort_flag)) return false;
            __threadfence();
            asm volatile("fence.proxy.async;" ::: "memory");  // what other SMs stored is read by this SM's copy engine
            ready_s = p;  // the epilogue warps of this CTA wait for this word, not for the device's
          }
          { const GemmArgs& args = chain.g[0]; (void)args; TS_PROBE(8 + 8 * p + 0); }
          ready = true;
          for (; x_next < it; ++x_next) {
            const int kc = (range.u0 + (x_next - first)) % chunks;
            const int s = x_next % STAGES;
#pragma unroll
            for (int a = 0; a < KATOMS; ++a)
              tma_load_2d(smem_u32(smem + (size_t)s * C::STAGE_BYTES) + C::A_BYTES + a * C::B_ATOM, map_x, smem_u32(&full_bar[s]),
                          kc * TILE_K + a * ATOM_K, 0);
          }
          return true;
        };
        if (p == 0 && n_units == 0) ts_pdl_wait();
        if (p > 0 && chain.hold) {
          // not before this CTA has stored its own share of the phase before: its last trips to the L2
          // (partial sums, ticket, the finished tile) would queue behind the copies asked for here
          for (uint32_t i = 0; i < GRID_SPIN_LIMIT && *arrived_flag < p && !*abort_flag; ++i) __nanosleep(40);
        }
        for (int i = 0; i < n_units; ++i, ++it) {
          const int u = range.u0 + i;
          const int t = u / chunks, kc = u - t * chunks;
          const int s = it % STAGES;
          const uint32_t round = (uint32_t)(it / STAGES);
          if (round > 0) {
            // the stage's last user may be a unit of this phase that still lacks its X: then nothing
            // frees the stage before the inputs are there
            if (!ready && it - STAGES >= first && !inputs_ready()) { ok = false; break; }
            if (!mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1, abort_flag)) { ok = false; break; }
          }
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t dst = smem_u32(smem + (size_t)s * C::STAGE_BYTES);
          mbar_expect_tx(bar, C::A_BYTES + C::B_BYTES);
#pragma unroll
          for (int a = 0; a < KATOMS; ++a) tma_load_2d_hint(dst + a * C::A_ATOM, map_w, bar, kc * TILE_K + a * ATOM_K, t * TILE_N, w_policy);
          if (ready) {
#pragma unroll
            for (int a = 0; a < KATOMS; ++a) tma_load_2d(dst + C::A_BYTES + a * C::B_ATOM, map_x, bar, kc * TILE_K + a * ATOM_K, 0);
            x_next = it + 1;
          }
        }
        if (ok && !ready && n_units > 0 && !inputs_ready()) ok = false;
      }
      // All loads of this launch are on their way.  While its last tiles are multiplied and stored
      // (and while the small kernels after it run) HBM would idle: ask for this CTA's share of the
      // next GEMM's weights to be brought into L2.
      const GemmArgs& tail = chain.g[phases - 1];
      if (tail.prefetch != nullptr && !*abort_flag) {
        constexpr unsigned long long PIECE = 32 * 1024;
        const unsigned long long pieces = (tail.prefetch_bytes + PIECE - 1) / PIECE;
        for (unsigned long long i = blockIdx.x; i < pieces; i += gridDim.x) {
          const unsigned long long off = i * PIECE;
          const unsigned bytes = (unsigned)min(PIECE, tail.prefetch_bytes - off) & ~15u;
          if (bytes) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(tail.prefetch + off), "r"(bytes) : "memory");
        }
      }
      if (*abort_flag) {
        // Let the copies that are still in flight land before shared memory is given up.  (A stage
        // whose X copy was never requested cannot complete; its wait runs out, bounded like the others.)
        for (int i = max(0, it - STAGES); i < it; ++i)
          mbar_wait(smem_u32(&full_bar[i % STAGES]), (uint32_t)(i / STAGES) & 1, abort_flag, 1u << 16);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // MMA issuer.
      int it = 0, item = 0;
      bool ok = true;
      for (int p = 0; p < phases && ok; ++p) {
        const GemmArgs& args = chain.g[p];
        const Range range = cta_range(args, blockIdx.x);
        const int chunks = args.chunks;
        const int t_first = range.u0 / chunks;
        const int t_last = range.u1 > range.u0 ? (range.u1 - 1) / chunks : t_first - 1;
        for (int t = t_first; t <= t_last && ok; ++t, ++item) {
          const int k0 = max(range.u0, t * chunks) - t * chunks;
          const int k1 = min(range.u1, (t + 1) * chunks) - t * chunks;
          const int acc = item & 1;
          const uint32_t use = (uint32_t)(item >> 1);
          if (use > 0 && !mbar_wait(smem_u32(&acc_empty[acc]), (use - 1) & 1, abort_flag)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t tmem_d = tmem_base + (uint32_t)(acc * MPAD);
          for (int kc = k0; kc < k1; ++kc, ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(smem_u32(&full_bar[s]), (uint32_t)(it / STAGES) & 1, abort_flag)) {
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (it == 0) TS_PROBE(2);
            if (t == t_first && kc == k0) { const GemmArgs& args = chain.g[0]; (void)args; TS_PROBE(8 + 8 * p + 1); }
            const uint32_t a_addr = smem_u32(smem + (size_t)s * C::STAGE_BYTES);
            const uint64_t adesc = umma_desc_sw128(a_addr);
            const uint64_t bdesc = umma_desc_sw128(a_addr + C::A_BYTES);
#pragma unroll
            for (int k = 0; k < TILE_K / UMMA_K; ++k) {
              // 16 bf16 = 32 bytes further along K inside the swizzle atom: +2 in the address field;
              // the next atom (box) of the stage starts A_ATOM / B_ATOM bytes further
              const int atom = k / (ATOM_K / UMMA_K), kk = k % (ATOM_K / UMMA_K);
              umma_bf16(tmem_d, adesc + (uint64_t)(atom * (C::A_ATOM >> 4) + 2 * kk), bdesc + (uint64_t)(atom * (C::B_ATOM >> 4) + 2 * kk), IDESC,
                        (kc > k0 || k > 0) ? 1u : 0u);
            }
            umma_commit(smem_u32(&empty_bar[s]));  // arrives when these MMAs have read the stage
          }
          if (ok) umma_commit(smem_u32(&acc_full[acc]));  // arrives when this accumulator is complete
        }
        { const GemmArgs& args = chain.g[0]; (void)args; TS_PROBE(8 + 8 * p + 2); }
      }
      {
        const GemmArgs& args = chain.g[0];
        (void)args;
        TS_PROBE(3);
      }
    }
  } else {
    // Epilogue warps 2..5: TMEM lanes 32 * (warp % 4) .. + 31.
    const int quarter = warp & 3;
    const int etid = (warp - 2) * 32 + lane;  // 0..127 among the epilogue threads
    int item = 0;
    bool alive = true;
    for (int p = 0; p < phases && alive; ++p) {
      const GemmArgs& args = chain.g[p];
      const Range range = cta_range(args, blockIdx.x);
      const int chunks = args.chunks;
      const int t_first = range.u0 / chunks;
      const int t_last = range.u1 > range.u0 ? (range.u1 - 1) / chunks : t_first - 1;
      if (MPAD <= FUSED_MAX_ROWS && args.mode == EPI_QK_ROPE && t_last >= t_first) {
        // the step's positions and cache slots and the small weight vectors of the rotation epilogue
        // (none of them written by a kernel of the step) go to the L1 ahead of their use
        if (etid < args.M) {
          asm volatile("prefetch.global.L1 [%0];" ::"l"(args.positions + etid));
          asm volatile("prefetch.global.L1 [%0];" ::"l"(args.slot_mapping + etid));
        } else if (etid < 64) {
          if (args.inv_freq != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(args.inv_freq + (etid & 7) * 8));
        } else if (etid < 96) {
          if (args.q_norm_w != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(args.q_norm_w + (etid & 15) * 8));
        } else {
          if (args.k_norm_w != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(args.k_norm_w + (etid & 15) * 8));
        }
      }
      if (p == 0) {
        ts_pdl_wait();  // nothing is stored before the kernels ahead in the stream are done
      } else if (t_last >= t_first) {
        // this phase reads what every CTA stored in the phase before (row sums, the residual stream)
        // (the producer thread polls the device-wide flag for the CTA and says so in shared memory)
        if (etid == 0) {
          bool there = false;
          for (uint32_t i = 0; i < GRID_SPIN_LIMIT && !there && !*abort_flag; ++i) {
            there = *ready_flag >= p;
            if (!there) __nanosleep(40);
          }
          if (there) there = grid_wait(chain.sync, p - 1, abort_flag);  // set by now: one load, and the ordering that goes with it
          if (there) __threadfence();
          else *abort_flag = 1;
          go_s = there ? 1 : 0;
        }
        epilogue_sync();
        if (go_s == 0) break;  // the same for all epilogue threads
        if (etid == 0) { const GemmArgs& args = chain.g[0]; (void)args; TS_PROBE(8 + 8 * p + 5); }
      }
      const bool fused = MPAD <= FUSED_MAX_ROWS && (args.mode != EPI_PLAIN || args.scale_ssq != nullptr);
      if (fused && t_last >= t_first) {
        // rstd of every row of x's source, from the per-tile sums of squares the kernel before left
        if (etid < args.M) {
          float sum = 0.f;
          if (args.scale_ssq != nullptr)
            for (int j = 0; j < args.scale_tiles; ++j) sum += __ldcg(args.scale_ssq + (size_t)j * args.M + etid);
          rstd_s[etid] = args.scale_ssq != nullptr ? rsqrtf(sum / args.scale_width + args.scale_eps) : 1.f;
        }
        epilogue_sync();
      }
      for (int t = t_first; t <= t_last; ++t, ++item) {
        const int k0 = max(range.u0, t * chunks) - t * chunks;
        const int k1 = min(range.u1, (t + 1) * chunks) - t * chunks;
        const bool whole = (k0 == 0 && k1 == chunks);
        const int acc = item & 1;
        if (!mbar_wait(smem_u32(&acc_full[acc]), (uint32_t)(item >> 1) & 1, abort_flag)) { alive = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        __syncwarp();
        if (etid == 0 && t == t_last && p == phases - 1) TS_PROBE(4);
        if (etid == 0 && t == t_last) { const GemmArgs& args = chain.g[0]; (void)args; TS_PROBE(8 + 8 * p + 3); }
        EpilogueAhead<MPAD <= FUSED_MAX_ROWS ? MPAD : 4> ahead;
        if (MPAD <= FUSED_MAX_ROWS && fused && args.mode == EPI_RESIDUAL_NORM) {
          // whoever finishes this tile adds it to the residual stream: ask for those values now (into
          // registers), so that they are here when the partial sums and the ticket have made their
          // trips.  Nobody else writes them before this tile is finished: a tile's columns are
          // written by the CTA that finishes it, and by kernels that are over.
          load_ahead<MPAD <= FUSED_MAX_ROWS ? MPAD : 4>(args, t, etid, ahead);
        }
        const int n_local = quarter * 32 + lane;
        const int n = t * TILE_N + n_local;
        const int slot = (t == t_first) ? 0 : 1;
        float* part = args.partial + ((size_t)(blockIdx.x * 2 + slot) * args.M) * TILE_N;
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * MPAD);
        uint32_t r[MPAD / 16][16];
#pragma unroll
        for (int c = 0; c < MPAD / 16; ++c) {
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
              : "=r"(r[c][0]), "=r"(r[c][1]), "=r"(r[c][2]), "=r"(r[c][3]), "=r"(r[c][4]), "=r"(r[c][5]), "=r"(r[c][6]),
                "=r"(r[c][7]), "=r"(r[c][8]), "=r"(r[c][9]), "=r"(r[c][10]), "=r"(r[c][11]), "=r"(r[c][12]), "=r"(r[c][13]),
                "=r"(r[c][14]), "=r"(r[c][15])
              : "r"(taddr + c * 16));
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // The accumulator is in registers: hand it back to the MMA warp before storing.
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
#pragma unroll
        for (int c = 0; c < MPAD / 16; ++c) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = c * 16 + i;
            if (m < args.M) {
              const float v = __uint_as_float(r[c][i]);
              if (!whole)
                part[(size_t)m * TILE_N + n_local] = v;
              else if (fused)
                tile_s[(MPAD <= FUSED_MAX_ROWS ? m : 0) * TILE_N + n_local] = v;
              else if (n < args.N) {
                if (args.out_f32)
                  reinterpret_cast<float*>(args.out)[(size_t)m * args.ldo + n] = v;
                else
                  reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)m * args.ldo + n] = __float2bfloat16_rn(v);
              }
            }
          }
        }
        bool last = false;
        if (!whole) {
          // Ticket: whoever arrives last for this tile adds the slots, in contributor order.
          // (units are counted in 32 bits: the host refuses a weight with more than 2^31 of them)
          const int c_first = (int)(((unsigned)t * (unsigned)chunks) / (unsigned)args.units_per);
          const int c_last = (int)((((unsigned)t + 1u) * (unsigned)chunks - 1u) / (unsigned)args.units_per);
          // Slot of every contributor for this tile (0: it is that CTA's first tile, else 1): worked out
          // while the partial sums are on their way, whoever will need it.
          const float* src[MAX_CONTRIB];
          const int nc = min(c_last - c_first + 1, MAX_CONTRIB);
#pragma unroll
          for (int j = 0; j < MAX_CONTRIB; ++j) {
            const int c = c_first + min(j, nc - 1);
            const int c_t_first = (int)(((unsigned)c * (unsigned)args.units_per) / (unsigned)chunks);
            src[j] = args.partial + (size_t)(c * 2 + ((t == c_t_first) ? 0 : 1)) * args.M * TILE_N;
          }
          __threadfence();
          epilogue_sync();
          if (etid == 0 && t == t_last) TS_PROBE(40);
          if (etid == 0) {
            const int ticket = atomicAdd(&args.counters[t], 1);
            last_s = (ticket == c_last - c_first) ? 1 : 0;
          }
          epilogue_sync();
          last = last_s != 0;
          if (etid == 0 && t == t_last) TS_PROBE(41);
          epilogue_sync();  // everyone has read the flag before the next tile may rewrite it
          if (last) {
            __threadfence();
            // Two pieces of four columns per thread and pass, all their loads first (they are
            // independent: one trip to the L2 per pass, not one per piece), then the sums in contributor order.
            constexpr int PIECES = 2;
            const int total = args.M * (TILE_N / 4);
            for (int base = etid; base < total; base += 128 * PIECES) {
              float4 v[PIECES][MAX_CONTRIB];
#pragma unroll
              for (int u = 0; u < PIECES; ++u) {
                const int idx = base + u * 128;
                if (idx < total) {
                  const size_t off = (size_t)(idx / (TILE_N / 4)) * TILE_N + (idx % (TILE_N / 4)) * 4;
#pragma unroll
                  for (int j = 0; j < MAX_CONTRIB; ++j)
                    if (j < nc) v[u][j] = __ldcg(reinterpret_cast<const float4*>(src[j] + off));
                }
              }
#pragma unroll
              for (int u = 0; u < PIECES; ++u) {
                const int idx = base + u * 128;
                if (idx >= total) continue;
                const int m = idx / (TILE_N / 4), nl = (idx % (TILE_N / 4)) * 4;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < MAX_CONTRIB; ++j)
                  if (j < nc) { sum.x += v[u][j].x; sum.y += v[u][j].y; sum.z += v[u][j].z; sum.w += v[u][j].w; }
                const int nn = t * TILE_N + nl;
                const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
                if (fused) {
                  *reinterpret_cast<float4*>(&tile_s[(MPAD <= FUSED_MAX_ROWS ? m : 0) * TILE_N + nl]) = sum;
                  continue;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (nn + j < args.N) {
                    if (args.out_f32)
                      reinterpret_cast<float*>(args.out)[(size_t)m * args.ldo + nn + j] = vals[j];
                    else
                      reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)m * args.ldo + nn + j] = __float2bfloat16_rn(vals[j]);
                  }
                }
              }
            }
            if (etid == 0) args.counters[t] = 0;
            if (etid == 0 && t == t_last) TS_PROBE(42);
          }
        }
        if (fused && (whole || last)) {  // the same for all epilogue threads
          epilogue_sync();  // tile_s holds the tile's final sums
          fused_epilogue<MPAD <= FUSED_MAX_ROWS ? MPAD : 4>(args, t, etid, lane, tile_s, rstd_s, ahead);
          epilogue_sync();  // before the next tile overwrites tile_s
          if (etid == 0 && t == t_last) TS_PROBE(43);
        }
      }
      if (alive && p + 1 < phases) {
        // this CTA's share of the phase is stored: say so to the grid (the next phase's copy engines
        // read it, hence the proxy fence)
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
        epilogue_sync();
        if (etid == 0) {
          grid_arrive(chain.sync, p, ctas);
          arrived_s = p + 1;
        }
        if (etid == 0) { const GemmArgs& args = chain.g[0]; (void)args; TS_PROBE(8 + 8 * p + 4); }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  {
    const GemmArgs& args = chain.g[0];
    (void)args;
    if (tid == 0) TS_PROBE(5);
  }
  if (abort_s != 0 && tid == 0) *chain.g[0].error = 1;
  if (phases > 1 && tid == 0) {
    // the last CTA to leave zeroes the barrier's counters: by then everyone has passed every wait
    __threadfence();
    if (atomicAdd(sync_departed(chain.sync), 1u) == ctas - 1) {
      for (int i = 0; i < MAX_PHASES; ++i) {
        *sync_counter(chain.sync, i) = 0;
        *sync_flag(chain.sync, i) = 0;
      }
      *sync_departed(chain.sync) = 0;
      __threadfence();
    }
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
}

// The give-up path of the bounded waits, alone: one CTA waits, with a small limit, on an mbarrier
// that nothing feeds, and then does what the GEMM's CTAs do when a wait ran out: it records the
// fact in the error word and returns.  Nothing traps, nothing hangs; the context stays usable.
__global__ void wait_gives_up_kernel(int* error, uint32_t limit) {
  __shared__ __align__(8) uint64_t nobody_arrives;
  __shared__ int abort_s;
  if (threadIdx.x == 0) {
    abort_s = 0;
    mbar_init(smem_u32(&nobody_arrives), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(smem_u32(&nobody_arrives), 0, &abort_s, limit);
  __syncthreads();
  if (abort_s != 0 && threadIdx.x == 0) *error = 1;
}

// ---------------------------------------------------------------------------
// host side: tensor maps (cached) and launch

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, cols, ld;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h = h * 1000003u ^ std::hash<long long>()(k.rows * 131 + k.cols);
    h = h * 1000003u ^ std::hash<long long>()(k.ld * 31 + k.box_rows);
    return h;
  }
};

std::mutex map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> map_cache;

// A [rows, cols] bf16 matrix with row stride `ld` elements, boxes of [box_rows x 64], 128-byte swizzle.
int tensor_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
  MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lock(map_mutex);
  auto it = map_cache.find(key);
  if (it != map_cache.end()) {
    *out = it->second;
    return 0;
  }
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return TS_ERR_UNSUPPORTED_SIZE;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)ATOM_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return TS_ERR_BAD_ARGUMENT;
  if (map_cache.size() > 4096) map_cache.clear();
  map_cache.emplace(key, *out);
  return 0;
}

template <int MPAD, int NPH>
int launch_phases(const ChainMapsT<NPH>& maps, const ChainArgsT<NPH>& chain, int ctas, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<MPAD, NPH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<MPAD>::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return ts_launch(gemm_skinny_kernel<MPAD, NPH>, dim3(ctas), dim3(NUM_THREADS), Cfg<MPAD>::SMEM, stream, maps, chain);
}

template <int MPAD>
int launch_skinny(const ChainMaps& maps, const ChainArgs& chain, int ctas, cudaStream_t stream) {
  if (chain.n > 1) return launch_phases<MPAD, MAX_PHASES>(maps, chain, ctas, stream);
  ChainMapsT<1> one_map;
  ChainArgsT<1> one;
  one_map.w[0] = maps.w[0];
  one_map.x[0] = maps.x[0];
  one.g[0] = chain.g[0];
  one.n = 1;
  one.hold = 0;
  one.ahead = 0;
  one.sync = nullptr;
  return launch_phases<MPAD, 1>(one_map, one, ctas, stream);
}

// Products waiting to be launched together (see ts_gemm_chain_begin).  One list for the process:
// the engine records and launches from one thread, on one stream at a time.
struct PendingChain {
  ChainMaps maps;
  ChainArgs args;
  int mpad = 0;
  int ctas = 0;
  cudaStream_t stream = nullptr;
  bool recording = false;
  unsigned int* sync = nullptr;
  int launches = 0;  // kernels launched by the flushes since the last ts_gemm_chain_begin
};
PendingChain pending;

int launch_pending() {
  if (pending.args.n == 0) return 0;
  ChainArgs& c = pending.args;
  for (int i = 0; i + 1 < c.n; ++i) {  // the next phase streams its weights itself: nothing to ask ahead
    c.g[i].prefetch = nullptr;
    c.g[i].prefetch_bytes = 0;
  }
  c.sync = pending.sync;
  static int hold = -1, ahead = -1;
  if (hold < 0) {
    const char* v = getenv("TS_GEMM_HOLD");
    hold = v ? atoi(v) : 1;
    v = getenv("TS_GEMM_AHEAD");
    ahead = v ? atoi(v) : 0;
  }
  c.hold = hold;
  c.ahead = ahead;
  int st;
  switch (pending.mpad) {
    case 16: st = launch_skinny<16>(pending.maps, c, pending.ctas, pending.stream); break;
    case 32: st = launch_skinny<32>(pending.maps, c, pending.ctas, pending.stream); break;
    case 64: st = launch_skinny<64>(pending.maps, c, pending.ctas, pending.stream); break;
    default: st = launch_skinny<128>(pending.maps, c, pending.ctas, pending.stream); break;
  }
  c.n = 0;
  pending.ctas = 0;
  pending.launches += 1;
  return st;
}

int sm_count() {
  static int count = 0;
#ifdef TS_GEMM_PROBE
  if (getenv("TS_GEMM_CTAS")) return atoi(getenv("TS_GEMM_CTAS"));
#endif
  if (count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count <= 0)
      count = 148;
  }
  return count;
}

// Units (tile x chunk) per CTA for an [N, K] weight: the work is spread over all SMs, but no
// tile is shared by more than MAX_CONTRIB CTAs.
void plan(int N, int K, int* tiles, int* chunks, int* units_per, int* ctas) {
  *tiles = (N + TILE_N - 1) / TILE_N;
  *chunks = (K + TILE_K - 1) / TILE_K;
  const long long total = (long long)*tiles * *chunks;
  long long per = (total + sm_count() - 1) / sm_count();
  const long long least = (*chunks + MAX_CONTRIB - 2) / (MAX_CONTRIB - 1);
  if (per < least) per = least;
  if (per < 1) per = 1;
  *units_per = (int)per;
  *ctas = (int)((total + per - 1) / per);
}

}  // namespace

#ifdef TS_GEMM_PROBE
unsigned long long* ts_gemm_probe_buffer = nullptr;
TS_EXPORT void ts_gemm_set_probe(unsigned long long* buffer) { ts_gemm_probe_buffer = buffer; }
#endif

// Floats of scratch the caller brings for an [N, K] weight and M rows: two shared-tile slots
// per CTA.
TS_EXPORT long long ts_gemm_skinny_scratch_floats(int M, int N, int K) {
  int tiles, chunks, units_per, ctas;
  plan(N, K, &tiles, &chunks, &units_per, &ctas);
  return (long long)ctas * 2 * M * TILE_N;
}

TS_EXPORT int ts_gemm_skinny_max_rows() { return 128; }

// For tests of the error path: a kernel whose one bounded wait (at most `limit` tries, capped at
// 65536) runs out by construction and sets `error` as the GEMM does.  It faults and hangs nothing.
TS_EXPORT int ts_wait_gives_up_probe(int* error, int limit, void* stream_) {
  if (error == nullptr || limit < 1) return TS_ERR_BAD_ARGUMENT;
  if (limit > 65536) limit = 65536;
  return ts_launch(wait_gives_up_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream_, error, (uint32_t)limit);
}

// out[M, ldo] (bf16, or f32 when out_f32) = x[M, K] (row stride ldx) * w[N, K]^T (row stride ldw).
// `partial`: ts_gemm_skinny_scratch_floats(M, N, K) floats.  `counters`: ints, one per 128-row
// tile of W, zero before the first call (the kernel leaves them zero).  `error`: one int the
// kernel sets to 1 if one of its waits gave up.
// `prefetch` / `prefetch_bytes`: optionally the start of the weights the next GEMM will read (16-byte
// aligned); the kernel asks for them to be brought into L2 once its own loads are issued.
// The same product with work that would otherwise be kernels of their own done where the tile
// is finished (M <= 32 rows):
//   scale_ssq [scale_tiles, M] (or null): x holds rows of a source that still lack their
//     norm's 1/rms; the sums of squares of the source rows, per 128 columns, come from the kernel
//     that wrote it; every product row m is multiplied by rsqrt(sum_m / scale_width + scale_eps).
//   mode 0: out as in ts_gemm_skinny_bf16.
//   mode 1 (N even, rows of w in blocks of 128: 64 gate rows, then the 64 up rows of the same
//     outputs): out [M, ldo] bf16 = silu(gate) * up, N / 2 columns.
//   mode 2: hidden [M, ldh] float32 += product; xprime [M, ldh] bf16 = hidden * norm_w;
//     ssq_out [ceil(N / 128), M] = sums of squares of the new hidden rows per 128 columns.
TS_EXPORT int ts_gemm_skinny_fused(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
                                   long long ldw, long long ldo, int out_f32, int mode, const float* scale_ssq,
                                   int scale_tiles, float scale_width, float scale_eps, float* hidden, long long ldh,
                                   const float* norm_w, void* xprime, float* ssq_out, float* partial, int* counters,
                                   int* error, const void* prefetch, long long prefetch_bytes, void* stream_);

// The q/k/v projection of an attention layer with head size 128 (w: nq query heads, then nkv key
// heads, then nkv value heads, 128 rows each), with what follows it done where each head's tile is
// finished: per-head RMS norm of queries and keys (weights [128] or null), rotate-half rotation
// with angle = position * inv_freq[j] (inv_freq [64] or null; rope_cos_sin [M, 64, 2] or null: the
// cosines and sines of those angles if the caller has them, as ts_rope_cos_sin leaves them),
// queries to q_out [M, nq * 128], keys
// and values to slot slot_mapping[m] of the caches [slots, nkv, 128] (-1: not stored).
// scale_ssq as in ts_gemm_skinny_fused.
TS_EXPORT int ts_gemm_skinny_qk_rope(const void* x, const void* w, int M, int K, long long ldx, long long ldw, int nq, int nkv,
                                     void* q_out, void* k_cache, void* v_cache, const int* slot_mapping, const int* positions,
                                     const float* q_norm_w, const float* k_norm_w, float qk_eps, const float* inv_freq,
                                     const float* rope_cos_sin, const float* scale_ssq, int scale_tiles, float scale_width, float scale_eps,
                                     float* partial, int* counters, int* error, const void* prefetch, long long prefetch_bytes,
                                     void* stream_);

TS_EXPORT int ts_gemm_skinny_bf16(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
                                  long long ldw, long long ldo, int out_f32, float* partial, int* counters,
                                  int* error, const void* prefetch, long long prefetch_bytes, void* stream_) {
  return ts_gemm_skinny_fused(x, w, out, M, N, K, ldx, ldw, ldo, out_f32, 0, nullptr, 0, 1.f, 0.f, nullptr, 0, nullptr,
                              nullptr, nullptr, partial, counters, error, prefetch, prefetch_bytes, stream_);
}

// What every entry point shares: checks, the split of the work, tensor maps, launch.  `a` comes
// with its epilogue fields set.
static int run_gemm(const void* x, const void* w, int M, int N, int K, long long ldx, long long ldw, GemmArgs& a, float* partial,
                    int* counters, int* error, const void* prefetch, long long prefetch_bytes, void* stream_) {
  if (K <= 0 || ldx < K || ldw < K || counters == nullptr || error == nullptr || partial == nullptr)
    return TS_ERR_BAD_ARGUMENT;
  if (M > 128 || (K % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)partial % 16))
    return TS_ERR_UNSUPPORTED_SIZE;
  if ((a.mode != EPI_PLAIN || a.scale_ssq != nullptr) && M > FUSED_MAX_ROWS) return TS_ERR_UNSUPPORTED_SIZE;
  if (a.scale_ssq != nullptr && (a.scale_tiles <= 0 || !(a.scale_width > 0.f))) return TS_ERR_BAD_ARGUMENT;
  const int mpad = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  int ctas;
  plan(N, K, &a.tiles, &a.chunks, &a.units_per, &ctas);
  if ((long long)a.tiles * a.chunks + a.units_per >= (1ll << 31)) return TS_ERR_UNSUPPORTED_SIZE;  // the kernel counts units in 32 bits
  CUtensorMap mw, mx;
  int st = tensor_map(w, N, K, ldw, TILE_N, &mw);
  if (st != 0) return st;
  st = tensor_map(x, M, K, ldx, mpad, &mx);
  if (st != 0) return st;
  a.partial = partial;
  a.counters = counters;
  a.error = error;
  a.M = M;
  a.N = N;
  a.K = K;
  a.prefetch = (prefetch_bytes > 0 && ((uintptr_t)prefetch % 16) == 0) ? (const char*)prefetch : nullptr;
  a.prefetch_bytes = prefetch_bytes > 0 ? (unsigned long long)prefetch_bytes : 0ull;
#ifdef TS_GEMM_PROBE
  // every product writes a region of its own (256 CTAs x 64 stamps), 64 regions in turn; the stamps of a chain land in its first product's region
  static int probe_launch = 0;
  a.probe = ts_gemm_probe_buffer ? ts_gemm_probe_buffer + (size_t)(probe_launch++ % 64) * 16384 : nullptr;
#endif
  cudaStream_t stream = (cudaStream_t)stream_;
  // While a chain is being recorded the product joins it (same row count and stream, and room
  // left; otherwise what is pending is launched first); else it is a launch of its own.
  if (pending.args.n > 0 && (!pending.recording || pending.mpad != mpad || pending.args.g[0].M != M || pending.stream != stream ||
                             pending.args.n == MAX_PHASES)) {
    st = launch_pending();
    if (st != 0) return st;
  }
  const int i = pending.args.n;
  pending.args.g[i] = a;
  pending.maps.w[i] = mw;
  pending.maps.x[i] = mx;
  pending.args.n = i + 1;
  pending.mpad = mpad;
  pending.stream = stream;
  if (ctas > pending.ctas) pending.ctas = ctas;
  if (pending.recording && pending.sync != nullptr) return 0;
  return launch_pending();
}

// Chains.  Between ts_gemm_chain_begin and ts_gemm_chain_end the products of this file are not
// launched when they are called but collected, up to MAX_PHASES of them, and launched as ONE kernel
// by ts_gemm_chain_flush (or when the list is full, or when a product with another row count or
// stream arrives): each reads what the one before it wrote.  The caller flushes before anything
// else reads a collected product's output, and keeps every buffer alive until then.  `sync`:
// ts_gemm_chain_sync_words() unsigned ints in device memory, zero before the first chain (the
// kernel leaves them zero); chains that share them must not run at the same time (one stream).
TS_EXPORT void ts_gemm_chain_begin(unsigned int* sync) {
  pending.recording = true;
  pending.sync = sync;
  pending.launches = 0;
}
TS_EXPORT int ts_gemm_chain_flush(void) { return launch_pending(); }
TS_EXPORT int ts_gemm_chain_end(void) {
  const int st = launch_pending();
  pending.recording = false;
  return st;
}
// Kernels that the flushes launched since ts_gemm_chain_begin.
TS_EXPORT int ts_gemm_chain_launches(void) { return pending.launches; }
TS_EXPORT int ts_gemm_chain_max_phases(void) { return MAX_PHASES; }
TS_EXPORT int ts_gemm_chain_sync_words(void) { return (2 * MAX_PHASES + 1) * SYNC_LINE; }

TS_EXPORT int ts_gemm_skinny_fused(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
                                   long long ldw, long long ldo, int out_f32, int mode, const float* scale_ssq,
                                   int scale_tiles, float scale_width, float scale_eps, float* hidden, long long ldh,
                                   const float* norm_w, void* xprime, float* ssq_out, float* partial, int* counters,
                                   int* error, const void* prefetch, long long prefetch_bytes, void* stream_) {
  if (M <= 0 || N <= 0) return 0;
  if (mode < 0 || mode > EPI_RESIDUAL_NORM) return TS_ERR_BAD_ARGUMENT;
  if (mode == EPI_SWIGLU && ((N & 1) || out_f32 || ldo < N / 2)) return TS_ERR_BAD_ARGUMENT;
  if (mode == EPI_RESIDUAL_NORM && (hidden == nullptr || norm_w == nullptr || xprime == nullptr || ssq_out == nullptr || ldh < N))
    return TS_ERR_BAD_ARGUMENT;
  if (mode == EPI_PLAIN && ldo < N) return TS_ERR_BAD_ARGUMENT;
  GemmArgs a = {};
  a.out = out;
  a.ldo = (int)ldo;
  a.out_f32 = out_f32;
  a.mode = mode;
  a.scale_ssq = scale_ssq;
  a.scale_tiles = scale_tiles;
  a.scale_width = scale_width;
  a.scale_eps = scale_eps;
  a.hidden = hidden;
  a.norm_w = norm_w;
  a.xprime = (__nv_bfloat16*)xprime;
  a.ssq_out = ssq_out;
  a.ldh = ldh;
  return run_gemm(x, w, M, N, K, ldx, ldw, a, partial, counters, error, prefetch, prefetch_bytes, stream_);
}

TS_EXPORT int ts_gemm_skinny_qk_rope(const void* x, const void* w, int M, int K, long long ldx, long long ldw, int nq, int nkv,
                                     void* q_out, void* k_cache, void* v_cache, const int* slot_mapping, const int* positions,
                                     const float* q_norm_w, const float* k_norm_w, float qk_eps, const float* inv_freq,
                                     const float* rope_cos_sin, const float* scale_ssq, int scale_tiles, float scale_width, float scale_eps,
                                     float* partial, int* counters, int* error, const void* prefetch, long long prefetch_bytes,
                                     void* stream_) {
  if (M <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || q_out == nullptr || k_cache == nullptr || v_cache == nullptr || slot_mapping == nullptr ||
      (inv_freq != nullptr && positions == nullptr))
    return TS_ERR_BAD_ARGUMENT;
  if (((uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) % 8 || (uintptr_t)rope_cos_sin % 16) return TS_ERR_UNSUPPORTED_SIZE;
  GemmArgs a = {};
  a.mode = EPI_QK_ROPE;
  a.scale_ssq = scale_ssq;
  a.scale_tiles = scale_tiles;
  a.scale_width = scale_width;
  a.scale_eps = scale_eps;
  a.q_out = (__nv_bfloat16*)q_out;
  a.k_cache = (__nv_bfloat16*)k_cache;
  a.v_cache = (__nv_bfloat16*)v_cache;
  a.slot_mapping = slot_mapping;
  a.positions = positions;
  a.q_norm_w = q_norm_w;
  a.k_norm_w = k_norm_w;
  a.inv_freq = inv_freq;
  a.rope_cs = inv_freq != nullptr ? reinterpret_cast<const float2*>(rope_cos_sin) : nullptr;
  a.qk_eps = qk_eps;
  a.nq = nq;
  a.nkv = nkv;
  return run_gemm(x, w, M, (nq + 2 * nkv) * TILE_N, K, ldx, ldw, a, partial, counters, error, prefetch, prefetch_bytes, stream_);
}
