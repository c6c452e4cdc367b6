// Paged causal attention for prompt portions on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory, operands brought by TMA): head size 128.
//
// What it computes is what attention_simple.cu computes (engine/nn/sdpa.py:56,85-102 of the
// reference).  How: one CTA per (sequence, KV head, tile of 128 rows), a row being a (query
// token, query head of the group) pair, so the heads that share a KV head share every key/value
// block.  Keys are walked in blocks of 64:
//   S = Q K^T      tcgen05.mma M=128 N=64 K=16 x 8, Q and K in shared memory (128-byte swizzle,
//                  K-major), S in tensor memory;
//   softmax        thread r owns row r: it reads its 64 scores from tensor memory, keeps the
//                  running max and sum in registers (no shuffles), and writes P as bfloat16
//                  into shared memory in the swizzled layout the next MMA reads;
//   O_blk = P V    tcgen05.mma M=128 N=128 K=16 x 4, V read in its natural [key][dim] order
//                  (an MN-major operand), O_blk in tensor memory;
//   O = O c + O_blk in registers (c rescales to the new running max).
// Q comes by one 4-d TMA box per half head; every page of K and V by one box per half head,
// into a ring of two stages, one block ahead.  The S product of the next block is issued
// before the rows of this block are folded into O, so the tensor core works while the
// threads do.  One thread issues all TMA and MMA instructions.
//
// Every wait is on an mbarrier fed by this CTA's own copies and MMAs, bounded; a wait that
// gives up raises the error word and the CTA frees its tensor memory and returns.
//
// Limits (the caller falls back to the mma.sync kernel otherwise): head size 128; at most 128
// query heads per KV head; the page size is at least 8 and divides 64 or is a multiple of 128.
#include "../common.cuh"
#include "kv_tensor_map.cuh"

#if TS_HEAD_DIM != 128
#error "attention_tcgen05.cu is written for TS_HEAD_DIM=128"
#endif

namespace {

constexpr int D = 128;
constexpr int BM = 128;  // rows per tile
constexpr int BN = 64;   // keys per block
constexpr int STAGES = 2;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

constexpr uint32_t Q_BYTES = 2 * BM * 128;        // two half-head atoms of [128 rows x 128 B]
constexpr uint32_t KV_HALF = BN * 128;            // [64 keys x 128 B]
constexpr uint32_t KV_STAGE = 2 * KV_HALF;        // both halves of the head
constexpr uint32_t P_BYTES = BM * 128;            // [128 rows x 64 keys] bfloat16
constexpr uint32_t OFF_Q = 0;
constexpr uint32_t OFF_K = OFF_Q + Q_BYTES;
constexpr uint32_t OFF_V = OFF_K + STAGES * KV_STAGE;
// P of a block lies where that block's K lay: K is dead once S is computed, P is dead once
// O_blk is, and only then is the stage filled again.
static_assert(P_BYTES == KV_STAGE, "P takes the place of one K stage");
constexpr uint32_t SMEM_TILES = OFF_V + STAGES * KV_STAGE;  // 98,304 bytes: two CTAs per SM
constexpr int MAX_TABLE = 1024;                   // block-table entries kept in shared memory
constexpr uint32_t TMEM_COLS = 256;               // S: 64 columns, O_blk: 128 columns
constexpr uint32_t TMEM_S = 0, TMEM_O = 64;

struct Params {
  __nv_bfloat16* out;     // [T, nq, D]
  const int* cu_q;        // [B + 1]
  const int* ctx_len;     // [B]
  const int* block_table; // [B, max_blocks]
  int* error;
  int max_blocks, page, nq, nkv, window, total_slots, num_seqs;
  float scale_log2;
  long long* probe;  // TS_ATT_PROBE builds: clock stamps of CTA 0's first softmax warp and of its MMA thread
};

#ifdef TS_ATT_PROBE
#define PROBE(slot, blk, k) \
  do { if (blockIdx.x == 0 && p.probe && (blk) < 64) p.probe[((slot) * 64 + (blk)) * 8 + (k)] = clock64(); } while (0)
#else
#define PROBE(slot, blk, k) do { } while (0)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
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
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// K-major operand, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand (V as [key][dim]), 128-byte swizzle: rows of 64 dims (128 B), 8-key groups
// 1024 bytes apart (stride offset), the second 64 dims `lbo` bytes further (leading offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// the same with the accumulate flag known when compiling: D = A B, and D += A B
__device__ __forceinline__ void umma_bf16_first(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}
__device__ __forceinline__ void umma_bf16_more(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}
// A (here P, [128 rows x 16 keys], two bfloat16 per column) from tensor memory
__device__ __forceinline__ void umma_bf16_tmem_a_first(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc) : "memory");
}
__device__ __forceinline__ void umma_bf16_tmem_a_more(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc) : "memory");
}
// one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
  uint32_t chosen;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(chosen));
  return chosen != 0;
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// idesc: float32 accumulate, bfloat16 operands, A K-major; B K-major or MN-major.
__host__ __device__ constexpr uint32_t idesc(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}

__global__ void __launch_bounds__(128, 2) attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                   const __grid_constant__ CUtensorMap map_k,
                                                                   const __grid_constant__ CUtensorMap map_v,
                                                                   const Params p) {
  // Tensor memory is taken only after the kernels ahead are done, and the kernel behind may
  // start only after every CTA of this one has its tensor memory: no CTA ever holds tensor
  // memory while it waits for a kernel whose CTAs still need some.
  ts_pdl_wait();
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t q_full, kv_full[STAGES], s_done, pv_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int table_s[MAX_TABLE];

  const int tid = threadIdx.x, warp = tid >> 5;
  // CTAs are numbered so that those launched first have the most keys to walk: the last tile
  // of every (sequence, KV head), then the tiles before them, and so on.
  const int hk = blockIdx.x % p.nkv, b = (blockIdx.x / p.nkv) % p.num_seqs;
  const int G = p.nq / p.nkv;
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int ctx = p.ctx_len[b];
  const int start_pos = ctx - q_len;
  const int rows_total = q_len * G;
  // A tile holds whole tokens: 128 / G of them, that is RT = (128 / G) * G rows; where G does not
  // divide 128 the tile's last rows (RT..127) belong to nobody and are masked like rows beyond the
  // sequence's end.
  const int RT = (BM / G) * G;
  const int seq_tiles = (rows_total + RT - 1) / RT;
  const int row_tile = seq_tiles - 1 - (int)(blockIdx.x / (p.nkv * p.num_seqs));
  if (q_len <= 0 || row_tile < 0) return;
  const int r0 = row_tile * RT;

  const int last_row = min(r0 + RT, rows_total) - 1;
  const int hi = start_pos + last_row / G;          // last key any row of the tile sees
  const int first_pos = start_pos + r0 / G;         // position of the tile's first row
  const int lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int kb0 = lo / BN, kb1 = hi / BN;
  const int nblocks = kb1 - kb0 + 1;
  const int box_rows = min(p.page, BN);  // keys per copy: a whole page, or 64 keys of a larger one
  const int copies_per_block = BN / box_rows;

  if (tid == 0) {
    abort_s = 0;
    mbar_init(smem_u32(&q_full), 1);
    for (int s = 0; s < STAGES; ++s) mbar_init(smem_u32(&kv_full[s]), 1);
    mbar_init(smem_u32(&s_done), 1);
    mbar_init(smem_u32(&pv_done), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  // The block-table entries of the keys this tile walks, once, into shared memory.
  const int first_entry = (kb0 * BN) / p.page;
  {
    const int n_entries = min(hi / p.page - first_entry + 1, MAX_TABLE);
    const int* table = p.block_table + (size_t)b * p.max_blocks;
    for (int i = tid; i < n_entries; i += 128) {
      const int e = first_entry + i;
      table_s[i] = e < p.max_blocks ? table[e] : -1;
    }
  }
  if (RT < BM) {
    // the rows of the Q tile that no copy fills (they belong to nobody): zeros, so that their scores are
    // numbers like any others
    for (int i = tid; i < 2 * (BM - RT) * 8; i += 128) {
      const int half = i / ((BM - RT) * 8), rest = i % ((BM - RT) * 8);
      *reinterpret_cast<uint4*>(smem + OFF_Q + half * (BM * 128) + (RT + rest / 8) * 128 + (rest % 8) * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  ts_pdl_launch_dependents();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort_flag = &abort_s;
  const uint32_t sm = smem_u32(smem);

  // One thread feeds the copy engine and the tensor core.
  auto load_kv = [&](int blk) {  // keys of block kb0 + blk into stage blk % 2
    const int stage = blk & 1;
    const uint32_t bar = smem_u32(&kv_full[stage]);
    mbar_expect_tx(bar, 2 * KV_STAGE);
    for (int c = 0; c < copies_per_block; ++c) {
      const int key0 = (kb0 + blk) * BN + c * box_rows;  // the first key of this copy
      const int e = key0 / p.page;
      int page_id = -1;
      if (key0 <= hi && e < p.max_blocks)
        page_id = e - first_entry < MAX_TABLE ? table_s[e - first_entry] : p.block_table[(size_t)b * p.max_blocks + e];
      // a page that is not held is read from beyond the tensor's end: the copy engine fills zeros
      const int slot = page_id >= 0 ? page_id * p.page + key0 % p.page : p.total_slots;
      const uint32_t row_off = (uint32_t)(c * box_rows) * 128u;
      for (int half = 0; half < 2; ++half) {
        tma_load_3d(sm + OFF_K + stage * KV_STAGE + half * KV_HALF + row_off, &map_k, bar, half * 64, hk, slot);
        tma_load_3d(sm + OFF_V + stage * KV_STAGE + half * KV_HALF + row_off, &map_v, bar, half * 64, hk, slot);
      }
    }
  };
  auto issue_s = [&](int blk) {  // S = Q K^T of block blk
    const int stage = blk & 1;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const uint32_t half = ks >> 2, inner = (ks & 3) * 32;
      umma_bf16(tmem_base + TMEM_S, desc_k_major(sm + OFF_Q + half * (BM * 128) + inner),
                desc_k_major(sm + OFF_K + stage * KV_STAGE + half * KV_HALF + inner), idesc(BN, false), ks > 0 ? 1u : 0u);
    }
    umma_commit(smem_u32(&s_done));
  };

  if (tid == 0) {
    mbar_expect_tx(smem_u32(&q_full), (uint32_t)(2 * RT * 128));  // two half-head boxes of RT rows
    for (int half = 0; half < 2; ++half)
      tma_load_4d(sm + OFF_Q + half * (BM * 128), &map_q, smem_u32(&q_full), half * 64, 0, hk, q_begin + r0 / G);
    load_kv(0);
    if (nblocks > 1) load_kv(1);
    bool ok = mbar_wait(smem_u32(&q_full), 0, abort_flag) && mbar_wait(smem_u32(&kv_full[0]), 0, abort_flag);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_s(0);
    }
  }

  // Row state of this thread.
  const int r = r0 + tid;
  const int row_pos = (tid < RT && r < rows_total) ? start_pos + r / G : -1;
  const int row_lo = (p.window > 0 && row_pos >= 0) ? max(0, row_pos - p.window + 1) : 0;
  float o[D];
#pragma unroll
  for (int i = 0; i < D; ++i) o[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);

  // A wait that gives up raises abort_s; the CTA leaves the loop together at the next barrier.

  for (int blk = 0; blk < nblocks; ++blk) {
    const int stage = blk & 1;
    const int kbase = (kb0 + blk) * BN;
    mbar_wait(smem_u32(&s_done), (uint32_t)blk & 1, abort_flag);
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    unsigned char* p_row = smem + OFF_K + stage * KV_STAGE + tid * 128;

    // scores of this row
    float s[BN];
#pragma unroll
    for (int c = 0; c < BN / 16; ++c) {
      uint32_t v[16];
      tmem_ld16(lane_addr + TMEM_S + c * 16, v);
#pragma unroll
      for (int i = 0; i < 16; ++i) s[c * 16 + i] = __uint_as_float(v[i]);
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");

    // every key of the block is seen by every row of the tile that belongs to a token (rows that belong
    // to nobody need no mask: a row's result depends on that row alone, and theirs is never stored)
    const bool unmasked = (kbase + BN - 1 <= first_pos) && (p.window <= 0 || kbase >= start_pos + last_row / G - p.window + 1);
    float m_new = m_run;
    if (unmasked) {
#pragma unroll
      for (int j = 0; j < BN; ++j) m_new = fmaxf(m_new, s[j]);
    } else {
#pragma unroll
      for (int j = 0; j < BN; ++j) {
        const int key = kbase + j;
        s[j] = (key <= row_pos && key >= row_lo) ? s[j] : -INFINITY;
        m_new = fmaxf(m_new, s[j]);
      }
    }
    const float m_off = m_new == -INFINITY ? 0.f : m_new * p.scale_log2;
    const float corr = fast_exp2(m_run * p.scale_log2 - m_off);
    m_run = m_new;
    float l_add = 0.f;
    uint32_t packed[BN / 2];
#pragma unroll
    for (int j = 0; j < BN; j += 2) {
      const float p0 = fast_exp2(fmaf(s[j], p.scale_log2, -m_off));
      const float p1 = fast_exp2(fmaf(s[j + 1], p.scale_log2, -m_off));
      l_add += p0 + p1;
      packed[j >> 1] = pack_bf16(p0, p1);
    }
    l_run = l_run * corr + l_add;
    // P row into shared memory, 16-byte chunk c at position c ^ (row % 8): the 128-byte swizzle
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 chunk = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      *reinterpret_cast<uint4*>(p_row + ((c ^ (tid & 7)) << 4)) = chunk;
    }
    // The last block of a sequence may hold rows of V that no request has written: make them
    // zeros (a masked key's weight is zero, but zero times garbage must stay zero).
    if (kbase + BN - 1 > hi) {
      mbar_wait(smem_u32(&kv_full[stage]), (uint32_t)(blk >> 1) & 1, abort_flag);
      const int first_bad = hi - kbase + 1;  // 1..63
      for (int i = tid; i < (BN - first_bad) * 16; i += 128) {
        const int row = first_bad + i / 16, piece = i % 16;  // 16 pieces of 16 bytes: both halves of the head
        *reinterpret_cast<uint4*>(smem + OFF_V + stage * KV_STAGE + (piece >> 3) * KV_HALF + row * 128 + ((piece & 7) << 4)) =
            make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if (__syncthreads_or(abort_s)) break;

    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      bool ok = mbar_wait(smem_u32(&kv_full[stage]), (uint32_t)(blk >> 1) & 1, abort_flag);
      if (ok) {
        // O_blk = P V: V is read in its natural [key][dim] order as an MN-major operand
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          umma_bf16(tmem_base + TMEM_O, desc_k_major(sm + OFF_K + stage * KV_STAGE + kk * 32),
                    desc_mn_major(sm + OFF_V + stage * KV_STAGE + kk * 2048, KV_HALF), idesc(D, true), kk > 0 ? 1u : 0u);
        umma_commit(smem_u32(&pv_done));
        // the next block's scores can be computed while the rows are folded into O
        if (blk + 1 < nblocks && mbar_wait(smem_u32(&kv_full[stage ^ 1]), (uint32_t)((blk + 1) >> 1) & 1, abort_flag)) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(blk + 1);
        }
      }
    }
    __syncwarp();

    const bool pv_ok = mbar_wait(smem_u32(&pv_done), (uint32_t)blk & 1, abort_flag);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // this stage is free now: fetch the block after next into it
    if (tid == 0 && pv_ok && blk + 2 < nblocks) load_kv(blk + 2);
    __syncwarp();
#pragma unroll
    for (int c = 0; c < D / 16; ++c) {
      uint32_t v[16];
      tmem_ld16(lane_addr + TMEM_O + c * 16, v);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int i = 0; i < 16; ++i) o[c * 16 + i] = fmaf(o[c * 16 + i], corr, __uint_as_float(v[i]));
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }

  __syncthreads();
  if (abort_s == 0 && tid < RT && r < rows_total) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* dst = p.out + ((size_t)(q_begin + r / G) * p.nq + hk * G + r % G) * D;
#pragma unroll
    for (int c = 0; c < D / 8; ++c) {
      uint4 chunk;
      chunk.x = pack_bf16(o[8 * c] * inv, o[8 * c + 1] * inv);
      chunk.y = pack_bf16(o[8 * c + 2] * inv, o[8 * c + 3] * inv);
      chunk.z = pack_bf16(o[8 * c + 4] * inv, o[8 * c + 5] * inv);
      chunk.w = pack_bf16(o[8 * c + 6] * inv, o[8 * c + 7] * inv);
      *reinterpret_cast<uint4*>(dst + 8 * c) = chunk;
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (abort_s != 0 && tid == 0) *p.error = 1;
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------
// Two tiles per CTA, roles in warps of their own (long prompt portions).
//
// A CTA owns 256 consecutive rows as two tiles of 128 and walks the keys once for both, in blocks
// of 128 keys: an S product of 128 keys reads as many bytes of shared memory per clock of tensor
// work as the tensor core takes (a product of 64 keys reads half as much again as it can use).
//   warps 0-7, 8-15 softmax of tile 0 and of tile 1: two threads per row, each with 64 of a
//                   block's 128 keys (a tile's turn is as long as its threads take, so the row
//                   is cut in two);
//   warp 16         TMA loads (Q once, then K and V blocks into rings of 2 stages);
//   warp 17         one elected lane: every tcgen05.mma;
//   warp 18         a messenger between the copies and warp 17 (see there).
// Tensor memory holds S of both tiles (128 columns each) and O of both tiles (128 columns each):
// all 512 columns.  P (bfloat16, two keys per column) is written over the first half of the scores
// it came from (keys 0..63 at column 0, keys 64..127 at column 64 of the tile's S), and the tensor
// core reads it from there.  The two tiles take turns: while the threads
// of one tile work on their scores, the tensor core runs P V and the next S of the other.  O stays
// in tensor memory and P V accumulates into it.  The running max of a row is only raised when the
// new max exceeds it by more than 2^8 (the weights then stay below 2^8, well inside bfloat16 and
// float32 range, and the final division by the row sum, taken with the same max, cancels it);
// only then is the row of O rescaled in tensor memory.
// Synchronisation is by mbarriers alone; every wait is bounded.

constexpr int PBN = 128;                          // keys per block of this kernel
constexpr uint32_t PKV_HALF = PBN * 128;          // [128 keys x 128 B]: half a head
constexpr uint32_t PKV_STAGE = 2 * PKV_HALF;      // both halves of the head
constexpr int KV_RING = 2;
constexpr uint32_t P2_OFF_Q = 0;                                   // 2 tiles x 32 KB
constexpr uint32_t P2_OFF_K = P2_OFF_Q + 2 * Q_BYTES;
constexpr uint32_t P2_OFF_V = P2_OFF_K + KV_RING * PKV_STAGE;
constexpr uint32_t P2_SMEM = P2_OFF_V + KV_RING * PKV_STAGE;       // 196,608 bytes
constexpr uint32_t P2_TMEM_COLS = 512;
// columns: S[tile] at tile * 128; O[tile] at 256 + tile * 128.  P of a block takes the first 64
// columns of its tile's S.
constexpr float RESCALE_THRESHOLD = 8.f;
// of every four pairs of weights, how many take their exponentials on the FMA pipe (the rest on the special-function unit)
#ifndef TS_ATT_FMA_PAIRS
#define TS_ATT_FMA_PAIRS 1
#endif

// two float32 in one 64-bit register, and the packed arithmetic on them
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^x for two values without the special-function unit: x = j + f with j the nearest integer
// (adding 1.5 * 2^23 leaves j in the low mantissa bits), 2^f by a cubic fitted to [-0.5, 0.5]
// (relative error below 8e-5, far below bfloat16's 4e-3), and j added into the exponent field.
// Inputs are clamped at -120: smaller ones give about 2^-120 instead of 0.
__device__ __forceinline__ void exp2_pair_fma(uint64_t x, float& r0, float& r1) {
  float x0, x1;
  unpack2(x, x0, x1);
  x = pack2(fmaxf(x0, -120.f), fmaxf(x1, -120.f));
  const uint64_t magic = pack2(12582912.f, 12582912.f);
  const uint64_t t = add2(x, magic);
  const uint64_t f = sub2(x, sub2(t, magic));
  uint64_t q = fma2(f, pack2(0.05508868396282196f, 0.05508868396282196f), pack2(0.24260404706001282f, 0.24260404706001282f));
  q = fma2(q, f, pack2(0.6932762265205383f, 0.6932762265205383f));
  q = fma2(q, f, pack2(0.9999289512634277f, 0.9999289512634277f));
  float q0, q1, t0, t1;
  unpack2(q, q0, q1);
  unpack2(t, t0, t1);
  r0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
  r1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__global__ void __launch_bounds__(608, 1) attention_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                        const __grid_constant__ CUtensorMap map_k,
                                                                        const __grid_constant__ CUtensorMap map_v,
                                                                        const Params p) {
  ts_pdl_wait();  // see the other kernel: tensor memory is never held while waiting for another kernel
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t q_full, k_full[KV_RING], k_empty[KV_RING], v_full[KV_RING], v_empty[KV_RING];
  __shared__ __align__(8) uint64_t s_done[2], p_ready[2], all_done;  // per tile
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int table_s[MAX_TABLE];
  __shared__ int quit_s[2][4][2];   // [tile][quarter of the rows][block parity]: see the softmax warps
  __shared__ float sum_s[2][2][BM];  // [tile][half of the keys][row]: what the two threads of a row tell each other (a block's largest score; at the end their sums)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // the CTAs with the most keys to walk are launched first (see the other kernel)
  const int hk = blockIdx.x % p.nkv, b = (blockIdx.x / p.nkv) % p.num_seqs;
  const int G = p.nq / p.nkv;
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int ctx = p.ctx_len[b];
  const int start_pos = ctx - q_len;
  const int rows_total = q_len * G;
  const int RT = (BM / G) * G;  // rows of a tile that belong to tokens (see the other kernel)
  const int seq_pairs = (rows_total + 2 * RT - 1) / (2 * RT);
  const int pair = seq_pairs - 1 - (int)(blockIdx.x / (p.nkv * p.num_seqs));
  if (q_len <= 0 || pair < 0) return;
  const int r0 = pair * 2 * RT;
  const int ntiles = rows_total - r0 > RT ? 2 : 1;

  // the last key any row of the pair sees, and how many key blocks the pair walks
  const int first_pos = start_pos + r0 / G;
  const int lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int kb0 = lo / PBN;
  const int hi = start_pos + (min(r0 + ntiles * RT, rows_total) - 1) / G;
  // Both tiles walk all blocks of the later one (its last block may be fully masked for the
  // earlier tile): the two tiles stay in step.
  const int nblocks = hi / PBN - kb0 + 1;
  const int box_rows = min(p.page, PBN);
  const int copies_per_block = PBN / box_rows;

  if (tid == 0) {
    abort_s = 0;
    mbar_init(smem_u32(&q_full), 1);
    mbar_init(smem_u32(&all_done), 1);
    for (int s = 0; s < KV_RING; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&k_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&s_done[t]), 1);
      mbar_init(smem_u32(&p_ready[t]), t == 0 ? 9 : 8);  // one arrival per softmax warp; tile 0's also one from the messenger warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  const int first_entry = (kb0 * PBN) / p.page;
  {
    const int n_entries = min(hi / p.page - first_entry + 1, MAX_TABLE);
    const int* table = p.block_table + (size_t)b * p.max_blocks;
    for (int i = tid; i < n_entries; i += blockDim.x) {
      const int e = first_entry + i;
      table_s[i] = e < p.max_blocks ? table[e] : -1;
    }
  }
  if (RT < BM) {
    // the rows of the Q tiles that no copy fills (they belong to nobody): zeros, so that their scores are
    // numbers like any others
    for (int i = tid; i < 4 * (BM - RT) * 8; i += blockDim.x) {
      const int part = i / ((BM - RT) * 8), rest = i % ((BM - RT) * 8);  // part: tile * 2 + half of the head
      *reinterpret_cast<uint4*>(smem + P2_OFF_Q + (part >> 1) * Q_BYTES + (part & 1) * (BM * 128) + (RT + rest / 8) * 128 + (rest % 8) * 16) =
          make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(P2_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  ts_pdl_launch_dependents();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort_flag = &abort_s;
  const uint32_t sm = smem_u32(smem);

  if (warp == 16) {
    // ---------------- copies: lane 0 announces the bytes, lanes 0..2*copies-1 each ask for one box ----------------
    if (lane == 0) {
      mbar_expect_tx(smem_u32(&q_full), (uint32_t)(ntiles * 2 * RT * 128));  // per tile two half-head boxes of RT rows
      for (int t = 0; t < ntiles; ++t)
        for (int half = 0; half < 2; ++half)
          tma_load_4d(sm + P2_OFF_Q + t * Q_BYTES + half * (BM * 128), &map_q, smem_u32(&q_full), half * 64, 0, hk,
                      q_begin + (r0 + t * RT) / G);
    }
    const int c = lane >> 1, half = lane & 1;  // this lane's copy within a block, and its half of the head
    const bool copies = c < copies_per_block;
    const uint32_t lane_off = (uint32_t)half * PKV_HALF + (uint32_t)(c * box_rows) * 128u;
    int issued[2] = {0, 0};  // K and V blocks asked for
    bool ok = true;
    for (int blk = 0; ok && blk < nblocks; ++blk) {
      const int st = blk % KV_RING;
      const uint32_t use = (uint32_t)(blk / KV_RING);
      // where this lane's box starts in the cache
      int slot = p.total_slots;  // beyond the end: the copy engine fills zeros (a page that is not held)
      if (copies) {
        const int key0 = (kb0 + blk) * PBN + c * box_rows;
        const int e = p.page < PBN ? (kb0 + blk) * copies_per_block + c : key0 / p.page;
        if (key0 <= hi && e < p.max_blocks) {
          const int page_id = e - first_entry < MAX_TABLE ? table_s[e - first_entry] : p.block_table[(size_t)b * p.max_blocks + e];
          if (page_id >= 0) slot = page_id * p.page + (key0 - e * p.page);
        }
      }
#pragma unroll
      for (int which = 0; which < 2; ++which) {  // K first: S needs it first
        const uint32_t full = smem_u32(which == 0 ? &k_full[st] : &v_full[st]);
        const uint32_t empty = smem_u32(which == 0 ? &k_empty[st] : &v_empty[st]);
        if (blk >= KV_RING) ok = mbar_wait(empty, (use - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(full, PKV_STAGE);
        __syncwarp();
        if (copies)
          tma_load_3d(sm + (which == 0 ? P2_OFF_K : P2_OFF_V) + st * PKV_STAGE + lane_off, which == 0 ? &map_k : &map_v, full,
                      half * 64, hk, slot);
        issued[which] = blk + 1;
      }
    }
    if (*abort_flag) {
      // leave nothing in flight: wait (bounded, on a count of its own) for the copies already asked for
      int patience = 0;
      volatile int* own = &patience;
      for (int which = 0; which < 2; ++which)
        for (int blk = max(0, issued[which] - KV_RING); blk < issued[which]; ++blk)
          mbar_wait(smem_u32(which == 0 ? &k_full[blk % KV_RING] : &v_full[blk % KV_RING]), (uint32_t)(blk / KV_RING) & 1, own);
    }
  } else if (warp == 18) {
    // ---------------- messenger: tells the MMA warp that what a round needs has landed ----------------
    // It arrives on tile 0's p_ready for block j (beside that tile's softmax warps) once V of j and
    // K of j + 1 are there.  An arrival counts for the barrier's current phase, so it waits until
    // the phase of block j - 1 is over; the copies it looks at landed long before that as a rule.
    bool ok = true;
    for (int j = 0; ok && j < nblocks; ++j) {
      ok = mbar_wait(smem_u32(&v_full[j % KV_RING]), (uint32_t)(j / KV_RING) & 1, abort_flag);
      if (ok && j + 1 < nblocks) ok = mbar_wait(smem_u32(&k_full[(j + 1) % KV_RING]), (uint32_t)((j + 1) / KV_RING) & 1, abort_flag);
      if (ok && j >= 1) ok = mbar_wait(smem_u32(&p_ready[0]), (uint32_t)(j - 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (ok && lane == 0) mbar_arrive(smem_u32(&p_ready[0]));
    }
  } else if (warp == 17) {
    // ---------------- tensor core: the warp runs together, one elected lane issues ----------------
    // Order of issue: S of block 0 for both tiles, then for every block j and tile t in turn: P V
    // of (t, j), S of (t, j + 1).  S(t, j + 1) goes where S and then P of (t, j) lay; the tensor
    // core runs what one thread issues in order, so P V has read P before the next S overwrites it.
    // While the threads of tile t work on S(t, j + 1), the tensor core runs tile 1 - t.  p_ready
    // of tile 0 for block j also gathers the messenger warp (V of j and K of j + 1 have landed),
    // so that one wait per tile and block is all this warp needs: each of its instructions is slow
    // beside eight busy warps.
    const uint64_t q_desc = desc_k_major(sm + P2_OFF_Q), k_desc = desc_k_major(sm + P2_OFF_K);
    const uint64_t v_desc = desc_mn_major(sm + P2_OFF_V, PKV_HALF);
    auto issue_s = [&](int t, int blk) {  // S of block blk for tile t; the block's K is free again after the last tile's
      const int st = blk % KV_RING;
      const uint64_t kd = k_desc + (uint64_t)((st * PKV_STAGE) >> 4);
      const uint64_t qd = q_desc + (uint64_t)((t * Q_BYTES) >> 4);
      const uint32_t s_addr = tmem_base + t * 128;
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off_q = ((ks >> 2) * (BM * 128) + (ks & 3) * 32) >> 4, off_k = ((ks >> 2) * PKV_HALF + (ks & 3) * 32) >> 4;
          if (ks == 0)
            umma_bf16_first(s_addr, qd + off_q, kd + off_k, idesc(PBN, false));
          else
            umma_bf16_more(s_addr, qd + off_q, kd + off_k, idesc(PBN, false));
        }
        umma_commit(smem_u32(&s_done[t]));
        if (t == ntiles - 1) umma_commit(smem_u32(&k_empty[st]));
      }
      __syncwarp();
    };
    bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&q_full), 0, abort_flag));
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&k_full[0]), 0, abort_flag));
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int t = 0; t < ntiles; ++t) issue_s(t, 0);
    }
    for (int j = 0; ok && j < nblocks; ++j) {
      const int st = j % KV_RING;
      const uint64_t vd = v_desc + (uint64_t)((st * PKV_STAGE) >> 4);
      for (int t = 0; ok && t < ntiles; ++t) {
        if (lane == 0) PROBE(1, j, t * 3);
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&p_ready[t]), (uint32_t)j & 1, abort_flag));
        if (!ok) break;
        if (lane == 0) PROBE(1, j, t * 3 + 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t o_addr = tmem_base + 256 + t * 128;
        const uint32_t p_addr = tmem_base + t * 128;  // 16 keys of P: 8 columns; keys 0..63 from column 0, keys 64..127 from column 64
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < PBN / 16; ++kk) {
            if (kk == 0 && j == 0)
              umma_bf16_tmem_a_first(o_addr, p_addr, vd, idesc(D, true));
            else
              umma_bf16_tmem_a_more(o_addr, p_addr + (kk >> 2) * 64 + (kk & 3) * 8, vd + ((kk * 2048) >> 4), idesc(D, true));
          }
          if (t == ntiles - 1) umma_commit(smem_u32(&v_empty[st]));
        }
        __syncwarp();
        if (j + 1 < nblocks) issue_s(t, j + 1);
        if (lane == 0) PROBE(1, j, t * 3 + 2);
      }
    }
    // Everything this CTA asked of the tensor core is done when this arrives, the arrivals of
    // the commits above included: nobody leaves before (an arrival after the CTA's end would
    // land in the barriers of the next CTA on this SM).
    if (elect_one()) umma_commit(smem_u32(&all_done));
    __syncwarp();
  } else if (warp < 8 * ntiles) {
    // ---------------- softmax: two threads per row, 64 of a block's 128 keys each ----------------
    // Warps 8 t .. 8 t + 7 belong to tile t; warp 8 t + 4 h + quad takes keys 64 h .. 64 h + 63 of
    // rows 32 quad .. 32 quad + 31 (a warp reaches the tensor-memory lanes of its number modulo 4).
    const int t = warp >> 3;
    const int h = (warp >> 2) & 1;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int r = r0 + t * RT + row;
    const int row_pos = (row < RT && r < rows_total) ? start_pos + r / G : -1;
    const int row_lo = (p.window > 0 && row_pos >= 0) ? max(0, row_pos - p.window + 1) : 0;
    const int tile_first_pos = start_pos + (r0 + t * RT) / G;
    const int tile_last_pos = start_pos + (min(r0 + t * RT + RT, rows_total) - 1) / G;  // of the tile's rows that belong to a token
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + t * 128 + h * 64;        // this thread's 64 scores; its P goes over the first 32 of them
    const int pair_bar = 3 + t * 4 + quad;                       // hardware barrier of the two warps that share rows
    const uint32_t o_addr = lane_addr + 256 + t * 128 + h * 64;  // its half of the row of O
    float m_run = -INFINITY, l_run = 0.f;  // l_run: the sum over this thread's keys only
    bool ok = true;

    for (int blk = 0; blk < nblocks; ++blk) {
      const int kbase = (kb0 + blk) * PBN + h * 64;
      if (h == 0 && row == 0) PROBE(t * 2, blk, 0);
      mbar_wait(smem_u32(&s_done[t]), (uint32_t)blk & 1, abort_flag);  // if it gives up: on to the barrier below, and out there
      __syncwarp();
      if (h == 0 && row == 0) PROBE(t * 2, blk, 1);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // every one of these 64 keys is seen by every row of the tile that belongs to a token (rows that
      // belong to nobody need no mask: a row's result depends on that row alone, and theirs is never stored)
      const bool unmasked = (kbase + 63 <= tile_first_pos) && (p.window <= 0 || kbase >= tile_last_pos - p.window + 1);
      // First walk over this thread's 64 scores: their largest.
      float m_blk;
      {
        uint32_t v0[32], v1[32];
        tmem_ld32(s_addr, v0);
        tmem_ld32(s_addr + 32, v1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains: the warp has few others to hide latency behind
        if (unmasked) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
#pragma unroll
            for (int u = 0; u < 4; ++u) mx[u] = fmaxf(mx[u], fmaxf(__uint_as_float(v0[i + u]), __uint_as_float(v1[i + u])));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key0 = kbase + i, key1 = key0 + 32;
            if (key0 <= row_pos && key0 >= row_lo) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(v0[i]));
            if (key1 <= row_pos && key1 >= row_lo) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(v1[i]));
          }
        }
        m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      }
      if (h == 0 && row == 0) PROBE(t * 2, blk, 2);
      // The row's largest score of the block is the larger of the two halves'.  The two warps that
      // share rows meet at a hardware barrier once per block, and it is the only place where they
      // leave the loop, both or neither: a wait that gave up has raised abort_s; the first warp of
      // the two looks at it before the barrier and leaves what it saw where both read it after the
      // barrier (in turns in two places, so that the next block's word never overtakes this one's).
      // So neither is ever left waiting for the other.
      sum_s[t][h][row] = m_blk;
      if (h == 0 && lane == 0) quit_s[t][quad][blk & 1] = *abort_flag;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      if (quit_s[t][quad][blk & 1] != 0) break;
      m_blk = fmaxf(m_blk, sum_s[t][h ^ 1][row]);
      if (h == 0 && row == 0) PROBE(t * 2, blk, 3);
      // raise the running max only when it is far behind (both threads of a row decide alike)
      const bool raise = (m_blk - m_run) * p.scale_log2 > RESCALE_THRESHOLD;  // also true when m_run is -inf and m_blk is not
      if (__any_sync(0xffffffffu, raise)) {
        const float m_new = raise ? m_blk : m_run;
        const float corr = m_new == -INFINITY ? 1.f : fast_exp2((m_run - m_new) * p.scale_log2);
        m_run = m_new;
        l_run *= corr;
        if (blk > 0) {
          // (P V of the block before is complete: the tensor core finishes what one thread issues in
          // order, and S of this block, issued after it, is)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t v[32];
            tmem_ld32(o_addr + c * 32, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
            tmem_st32(o_addr + c * 32, v);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      const float m_off = m_run == -INFINITY ? 0.f : m_run * p.scale_log2;
      // Weights p = 2^(s * scale - m * scale), two at a time.  The special-function unit does 16
      // exponentials a clock per SM; one pair in four is computed on the FMA pipe instead
      // (exp2_pair_fma).  (Measured at 8,192 tokens: none 543 us, one 524, two 525, three 566.)
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};  // four chains of two float32 sums each (0 is +0.0 twice)
      const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), off2 = pack2(-m_off, -m_off);
      // Second walk, 32 scores at a time.  P goes over the first half of the scores it came from
      // (this thread's own lane and columns): P of keys 32 g .. 32 g + 31 to columns 16 g .. 16 g + 15,
      // over scores that have been read.
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        uint32_t v[32];
        tmem_ld32(s_addr + g * 32, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (!unmasked) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = kbase + g * 32 + i;
            if (!(key <= row_pos && key >= row_lo)) v[i] = __float_as_uint(-INFINITY);
          }
        }
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float p0, p1;
            if (i < TS_ATT_FMA_PAIRS) {
              const uint64_t x = fma2(pack2(__uint_as_float(v[j + 2 * i]), __uint_as_float(v[j + 2 * i + 1])), scale2, off2);
              exp2_pair_fma(x, p0, p1);
            } else {
              p0 = fast_exp2(fmaf(__uint_as_float(v[j + 2 * i]), p.scale_log2, -m_off));
              p1 = fast_exp2(fmaf(__uint_as_float(v[j + 2 * i + 1]), p.scale_log2, -m_off));
            }
            sum2[i] = add2(sum2[i], pack2(p0, p1));
            packed[(j >> 1) + i] = pack_bf16(p0, p1);
          }
        }
        tmem_st16(s_addr + g * 16, packed);
      }
      {
        float even, odd;
        unpack2(add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3])), even, odd);
        l_run += even + odd;
      }
      if (h == 0 && row == 0) PROBE(t * 2, blk, 4);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      if (h == 0 && row == 0) PROBE(t * 2, blk, 5);
      // Rows of V that no request has written (beyond the last key): zeros (a masked key's weight
      // is zero, but zero times garbage must stay zero).  Both tiles write them: each tile's P V
      // waits for its own threads only.
      if ((kb0 + blk) * PBN + PBN - 1 > hi) {
        const int st = blk % KV_RING;
        mbar_wait(smem_u32(&v_full[st]), (uint32_t)(blk / KV_RING) & 1, abort_flag);  // if it gives up: the next barrier ends the loop
        __syncwarp();
        const int first_bad = hi - (kb0 + blk) * PBN + 1;
        for (int i = h * BM + row; i < (PBN - first_bad) * 16; i += 2 * BM) {
          const int vrow = first_bad + i / 16, piece = i % 16;
          *reinterpret_cast<uint4*>(smem + P2_OFF_V + st * PKV_STAGE + (piece >> 3) * PKV_HALF + vrow * 128 + ((piece & 7) << 4)) =
              make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      if (h == 0 && row == 0) PROBE(t * 2, blk, 6);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_ready[t]));
      if (h == 0 && row == 0) PROBE(t * 2, blk, 7);
    }

    ok = mbar_wait(smem_u32(&all_done), 0, abort_flag);
    const bool good = __all_sync(0xffffffffu, ok) && *abort_flag == 0;
    // the row's sum: both halves'.  (The eight warps of the tile meet whatever happened before.)
    sum_s[t][h][row] = l_run;
    asm volatile("bar.sync %0, 256;" ::"r"(1 + t) : "memory");
    l_run += sum_s[t][h ^ 1][row];
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    unsigned char* o_tile = smem + P2_OFF_Q + t * Q_BYTES;
    if (good) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // The tile goes through shared memory (where its Q lay: the tensor core is done with it), so
      // that rows leave as whole 256-byte lines: row `row` at row * 256, its 16-byte piece c at
      // position c ^ (row % 16), which spreads both the writes and the reads over the banks.
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld32(o_addr + c * 32, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 chunk;
          chunk.x = pack_bf16(__uint_as_float(v[8 * i]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
          chunk.y = pack_bf16(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
          chunk.z = pack_bf16(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
          chunk.w = pack_bf16(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
          *reinterpret_cast<uint4*>(o_tile + row * 256 + (((h * 8 + c * 4 + i) ^ (row & 15)) << 4)) = chunk;
        }
      }
    }
    asm volatile("bar.sync %0, 256;" ::"r"(1 + t) : "memory");
    if (good) {
      const int me = h * BM + row;  // 0..255 among the tile's threads
#pragma unroll 4
      for (int it = 0; it < 8; ++it) {
        const int idx = it * 2 * BM + me;
        const int rr = idx >> 4, piece = idx & 15;
        const int rg = r0 + t * RT + rr;
        if (rr < RT && rg < rows_total) {
          const uint4 chunk = *reinterpret_cast<const uint4*>(o_tile + rr * 256 + ((piece ^ (rr & 15)) << 4));
          __nv_bfloat16* dst = p.out + ((size_t)(q_begin + rg / G) * p.nq + hk * G + rg % G) * D + piece * 8;
          *reinterpret_cast<uint4*>(dst) = chunk;
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (abort_s != 0 && tid == 0) *p.error = 1;
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P2_TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------
// host side

// q [T, nq, D] as a 4-d tensor {D, G, nkv, T}; boxes of {64, G, 1, 128 / G}: the rows of a box
// come out ordered (token, head of the group), which is the tile's row order.
int query_map(const void* ptr, long long T, int nq, int nkv, CUtensorMap* out) {
  TsMapKey key{ptr, T, nq, -(long long)nkv};
  std::lock_guard<std::mutex> lock(ts_map_mutex());
  auto& map_cache = ts_map_cache();
  auto it = map_cache.find(key);
  if (it != map_cache.end()) {
    *out = it->second;
    return 0;
  }
  TsEncodeTiledFn fn = ts_encode_tiled();
  if (!fn) return TS_ERR_UNSUPPORTED_SIZE;
  const int G = nq / nkv;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)G, (cuuint64_t)nkv, (cuuint64_t)T};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)G * D * 2, (cuuint64_t)nq * D * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)G, 1, (cuuint32_t)(BM / G)};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return TS_ERR_BAD_ARGUMENT;
  if (map_cache.size() > 4096) map_cache.clear();
  map_cache.emplace(key, *out);
  return 0;
}

}  // namespace

// TS_ATT_PROBE builds only: where the next launches write their clock stamps (2 x 64 x 8 values).
static long long* probe_buffer = nullptr;
TS_EXPORT void ts_attention_tcgen05_set_probe(long long* buffer) { probe_buffer = buffer; }

// Whether this kernel takes the sizes (the caller uses the mma.sync kernel otherwise).
TS_EXPORT int ts_attention_tcgen05_supported(int nq, int nkv, int page) {
  if (nq <= 0 || nkv <= 0 || nq % nkv) return 0;
  const int G = nq / nkv;
  if (G > BM) return 0;
  if (page < 8 || (BN % page && page % PBN)) return 0;  // a page divides 64, or is a multiple of 128
  return 1;
}

// q/out [T, nq, 128] bf16; caches [pages, page, nkv, 128] bf16 (`total_slots` = pages * page);
// cu_q [B+1]; ctx_len [B]; block_table [B, max_blocks]; max_q: the most tokens of any sequence.
// `mode`: 0 chooses by the longest portion (two tiles per CTA when a sequence has more than 128
// rows), 1 one tile per CTA, 2 two tiles per CTA.
// `error`: one int the kernel sets to 1 if one of its waits gave up.
TS_EXPORT int ts_attention_prefill_tcgen05(const void* q, const void* kcache, const void* vcache, void* out,
                                           const int* cu_q, const int* ctx_len, const int* block_table,
                                           int max_blocks, int page, long long total_slots, int T, int B, int max_q,
                                           int nq, int nkv, float scale, int window, int mode, int* error, void* stream_) {
  if (T <= 0 || B <= 0) return 0;
  if (!ts_attention_tcgen05_supported(nq, nkv, page) || max_blocks <= 0 || max_q <= 0 || error == nullptr)
    return TS_ERR_BAD_ARGUMENT;
  if (total_slots > 0x7fffffffLL - page || ((long long)max_q * (nq / nkv) / ((BM / (nq / nkv)) * (nq / nkv)) + 1) * nkv * B > 0x7fffffffLL) return TS_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)q | (uintptr_t)kcache | (uintptr_t)vcache | (uintptr_t)out) % 16) return TS_ERR_UNSUPPORTED_SIZE;
  Params p;
  p.out = (__nv_bfloat16*)out;
  p.cu_q = cu_q;
  p.ctx_len = ctx_len;
  p.block_table = block_table;
  p.error = error;
  p.max_blocks = max_blocks;
  p.page = page;
  p.nq = nq;
  p.nkv = nkv;
  p.window = window;
  p.total_slots = (int)total_slots;
  p.num_seqs = B;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.probe = probe_buffer;
  const int G = nq / nkv;
  const int RT = (BM / G) * G;  // rows of a tile that belong to tokens
  const long long rows = (long long)max_q * G;
  const bool pairs = mode == 2 || (mode == 0 && rows > RT);
  const int block_keys = pairs ? PBN : BN;  // keys per copy: a whole page, or a block's worth of a larger one
  CUtensorMap mq, mk, mv;
  int st = query_map(q, T, nq, nkv, &mq);
  if (st) return st;
  st = ts_kv_cache_map(kcache, total_slots, nkv, D, page < block_keys ? page : block_keys, &mk);
  if (st) return st;
  st = ts_kv_cache_map(vcache, total_slots, nkv, D, page < block_keys ? page : block_keys, &mv);
  if (st) return st;
  if (pairs) {
    const size_t smem = P2_SMEM + 1024;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    return ts_launch(attention_tcgen05_pair_kernel, dim3((unsigned)(((rows + 2 * RT - 1) / (2 * RT)) * nkv * B)), dim3(608), smem,
                     (cudaStream_t)stream_, mq, mk, mv, p);
  }
  const size_t smem = SMEM_TILES + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return ts_launch(attention_tcgen05_kernel, dim3((unsigned)(((rows + RT - 1) / RT) * nkv * B)), dim3(128), smem, (cudaStream_t)stream_, mq, mk,
                   mv, p);
}
