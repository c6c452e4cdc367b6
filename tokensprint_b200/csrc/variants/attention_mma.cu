// Paged causal attention on tensor cores (bfloat16 in, float32 softmax and accumulation).
//
// Compiled once per head size: -DTS_HEAD_DIM=<multiple of 16, at most 256>.
//
// What it computes is what attention_simple.cu computes (engine/nn/sdpa.py:56,85-102 of the
// reference: scale, causal mask, GQA by head ratio, keys and values through the block
// table; a sliding window where the layer has one).  How: for one sequence and one KV
// head, the rows of the work tile are (query token, query head of the group) pairs, so
// all heads that share a KV head share each loaded key/value tile.  Keys are walked in
// blocks of BN with an online softmax; K and V blocks arrive by cp.async (16-byte
// chunks, zero-filled where a key does not exist) two blocks ahead of the math.
// Prefill uses 8 warps x 16 rows per CTA.  Decode (at most 16 rows per sequence and KV head)
// uses 4 warps that share the rows and take 16 keys each of every block, and splits the keys
// of a sequence over several CTAs, whose partial results (running max, sum, unnormalised
// output, float32) go to a scratch buffer and are merged by attention_combine_kernel.
//
// The order of the sums for one query row depends on its own keys and on the number of
// splits only, never on what else is in the batch.
#include <string.h>

#include "../common.cuh"
#include "kv_tensor_map.cuh"

#ifndef TS_HEAD_DIM
#error "compile with -DTS_HEAD_DIM=<head size>"
#endif
#if (TS_HEAD_DIM % 16) != 0 || TS_HEAD_DIM > 256 || TS_HEAD_DIM < 16
#error "TS_HEAD_DIM must be a multiple of 16 between 16 and 256"
#endif

namespace {

constexpr int D = TS_HEAD_DIM;
constexpr int BN = 64;            // keys per block
constexpr int LD = D + 8;         // padded row of a shared-memory tile (odd count of 16-byte chunks)
constexpr int CH = D / 8;         // 16-byte chunks per row
constexpr int STAGES = 2;
constexpr bool Q_IN_REGS = D <= 128;
// Decode with the copy engine (TMA): head sizes that are multiples of 64 (a box is 64 wide).
constexpr bool TMA_HEAD = (D % 64) == 0;
constexpr int HALVES = TMA_HEAD ? D / 64 : 1;           // 64-wide boxes per head row
constexpr unsigned KV_TILE = HALVES * BN * 128;         // bytes of the K (or V) rows of one block: [HALVES][64 keys][128 B], swizzled
constexpr long long SLOT_BOUND = 1ll << 30;             // slots the maps declare; coordinate SLOT_BOUND is out of bounds: zeros, no access
constexpr unsigned TMA_SPIN_LIMIT = 1u << 22;
#ifndef TS_DECODE_TMA_STAGES
#define TS_DECODE_TMA_STAGES 2
#endif
constexpr int TSTAGES = TS_DECODE_TMA_STAGES;           // key blocks in flight per CTA on the copy-engine path

struct AttnParams {
  const __nv_bfloat16* q;         // [T, nq, D]
  const __nv_bfloat16* kcache;    // [slots, nkv, D]
  const __nv_bfloat16* vcache;
  __nv_bfloat16* out;             // [T, nq, D]
  float* part_o;                  // [T * nq, splits, D]   (splits > 1)
  float* part_ml;                 // [T * nq, splits, 2]
  const int* cu_q;                // [B + 1]
  const int* ctx_len;             // [B] keys in the cache after this step
  const int* block_table;         // [B, max_blocks]
  int max_blocks, page, nq, nkv, window, splits, row_tiles;
  int* counters;                  // [B * nkv] tickets of the key splits (zero between launches), or null: merge in a kernel of its own
  int keys_per_split;             // > 0: split s covers this many keys (a multiple of BN); 0: the range is divided evenly
  int cluster;                    // 1: the key splits of a (sequence, KV head) pair are one thread-block cluster and merge through its shared memory
  long long* probe;               // TS_ATT_PROBE builds: clock stamps of a few CTAs of the decode kernel
  int* error;                     // set to 1 when a bounded wait of the copy-engine path gave up
  float scale_log2;               // scale * log2(e)
  int num_seqs;                   // B
  int* flat_prefix;               // even-share kernel: [B + 1] key blocks of the sequences before each one, left for its combine kernel
};

#ifdef TS_ATT_PROBE
#define APROBE(k) do { if (p.probe && threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) p.probe[blockIdx.x * 16 + (k)] = clock64(); } while (0)
#else
#define APROBE(k) do { } while (0)
#endif

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded: gives up after TMA_SPIN_LIMIT tries or when another thread of the CTA has.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag) {
  for (unsigned i = 0; i < TMA_SPIN_LIMIT; ++i) {
    unsigned done;
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
// In a decode step every key and value is read once: the copies say "evict first", which leaves
// the L2 to what is read again (activations, the next weights asked ahead).
__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap* map, unsigned bar, int c0, int c1, int c2) {
  unsigned long long policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy) : "memory");
}
// Address of the 16-byte piece that holds elements [col, col + 8) of row `row` in a swizzled tile
// [HALVES][64 rows][128 B]: piece c of a row sits at position c ^ (row % 8).
__device__ __forceinline__ const unsigned char* swizzled(const unsigned char* tile, int row, int col) {
  return tile + (col >> 6) * (BN * 128) + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4);
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {  // one MUFU op; -inf gives 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// NT / BN threads share a row of a key block and interleave its 16-byte chunks, so a thread
// needs one page of the block table per block, and neighbouring lanes fetch neighbouring chunks.
// The page is looked up one block ahead of its use, so the dependent load hides behind the math.
template <int NT>
__device__ __forceinline__ int lookup_page(const int* table, int page, int kbase, int kend, int tid) {
  const int j = kbase + tid / (NT / BN);
  return j <= kend ? table[j / page] : -1;
}

// Copies keys [kbase, kbase + BN) of one KV head into [BN][LD] tiles of K and V; keys that do
// not exist (beyond the sequence, or in a page that is not held: pg < 0) become zeros.
template <int NT>
__device__ __forceinline__ void load_kv_tiles(__nv_bfloat16* k_tile, __nv_bfloat16* v_tile, const __nv_bfloat16* kcache,
                                              const __nv_bfloat16* vcache, int pg, int page, int nkv, int hk, int kbase,
                                              int tid, bool k_and_v_in_one_group) {
  constexpr int TPR = NT / BN;  // threads per row
  static_assert(NT % BN == 0 && TPR >= 1, "thread count must be a multiple of the key block");
  const int row = tid / TPR;
  const int j = kbase + row;
  const bool valid = pg >= 0;
  const size_t off = valid ? (((size_t)pg * page + (j % page)) * nkv + hk) * D : 0;
#pragma unroll
  for (int ch = tid % TPR; ch < CH; ch += TPR) cp_async16(k_tile + row * LD + ch * 8, kcache + off + ch * 8, valid);
  if (!k_and_v_in_one_group) cp_async_commit();
#pragma unroll
  for (int ch = tid % TPR; ch < CH; ch += TPR) cp_async16(v_tile + row * LD + ch * 8, vcache + off + ch * 8, valid);
  cp_async_commit();
}

// The key splits of one (sequence, KV head) pair meet here when the caller gave ticket counters:
// every split CTA has written its partial rows, takes a ticket, and the one that arrives last
// merges all splits of the pair (in split order) and writes the output rows.  No CTA waits.
template <int NT>
__device__ __forceinline__ void merge_splits_by_last_arriver(const AttnParams& p, int b, int hk, int q_begin, int rows_total,
                                                             int G, int* last_flag) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(&p.counters[b * p.nkv + hk], 1);
    *last_flag = (ticket == p.splits - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!*last_flag) return;
  __threadfence();
  for (int row = warp; row < rows_total; row += NT / 32) {
    const size_t qrow = (size_t)(q_begin + row / G) * p.nq + hk * G + row % G;
    const float* ml = p.part_ml + qrow * p.splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < p.splits; ++s) {
      const float ls = __ldcg(ml + 2 * s + 1);
      if (ls > 0.f) m = fmaxf(m, __ldcg(ml + 2 * s));
    }
    float l = 0.f;
    float acc[(D + 31) / 32];
#pragma unroll
    for (int i = 0; i < (D + 31) / 32; ++i) acc[i] = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float ls = __ldcg(ml + 2 * s + 1);
      if (!(ls > 0.f)) continue;
      const float w = exp2f(__ldcg(ml + 2 * s) - m);
      l += w * ls;
      const float* src = p.part_o + (qrow * p.splits + s) * D;
#pragma unroll
      for (int i = 0; i < (D + 31) / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] += w * __ldcg(src + d);
      }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* dst = p.out + qrow * D;
#pragma unroll
    for (int i = 0; i < (D + 31) / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < D) dst[d] = __float2bfloat16_rn(acc[i] * inv);
    }
  }
  if (tid == 0) p.counters[b * p.nkv + hk] = 0;
}

// SPLIT_KEYS = false (prefill): the CTA's warps own 16 query rows each and all walk every key.
// SPLIT_KEYS = true (decode, at most 16 rows): the warps share the rows and own 16 keys each of
// every 64-key block, with running max/sum/output of their own, merged when the keys are done.
// USE_TMA (decode only): the copy engine brings whole pages into swizzled tiles, one instruction
// per box of [page rows x 64 elements] instead of one 16-byte copy per thread and piece (at
// large batches the 16-byte copies, not the memory, bound the kernel); warp 0 asks, a pair of
// mbarriers per stage says "landed" and "all four warps are done with it".
template <int NWARPS, bool SPLIT_KEYS, bool USE_TMA>
__global__ void __launch_bounds__(NWARPS * 32) attention_mma_kernel(const AttnParams p, const __grid_constant__ CUtensorMap map_k,
                                                                    const __grid_constant__ CUtensorMap map_v) {
  static_assert(!USE_TMA || (SPLIT_KEYS && TMA_HEAD), "the copy-engine path is the decode path, for head sizes that are multiples of 64");
  constexpr int NT = NWARPS * 32;
  constexpr int BM = SPLIT_KEYS ? 16 : NWARPS * 16;
  constexpr int NTILES = SPLIT_KEYS ? 2 : BN / 8;  // 8-key score tiles per warp and block
  APROBE(0);
  // Decode (key-split mode): everything that does not depend on the kernel before is done before
  // waiting for it: the step's index arrays (copied from the host before the step's first kernel)
  // and the keys and values of earlier steps.  Only the queries and the keys and values of
  // this step's own tokens (written by the projection just before) are fetched after the wait.
  ts_pdl_launch_dependents();
  if constexpr (!SPLIT_KEYS) ts_pdl_wait();
  static_assert(!SPLIT_KEYS || NWARPS * 16 == BN, "key-split mode: the warps must cover one key block");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [BM][LD]
  __nv_bfloat16* k_s = q_s + BM * LD;                                        // [STAGES][BN][LD]
  __nv_bfloat16* v_s = k_s + STAGES * BN * LD;                               // [STAGES][BN][LD]
  // copy-engine path: swizzled tiles on a 1,024-byte boundary, K of both stages, then V of both stages
  unsigned char* kv_tma = reinterpret_cast<unsigned char*>(((uintptr_t)(q_s + BM * LD) + 1023) & ~(uintptr_t)1023);
  if constexpr (USE_TMA) {
    k_s = reinterpret_cast<__nv_bfloat16*>(kv_tma);  // the merge at the end reuses this region through k_s
    v_s = reinterpret_cast<__nv_bfloat16*>(kv_tma + TSTAGES * KV_TILE);
  }
  __shared__ int last_flag;
  __shared__ __align__(8) unsigned long long full_bar[TSTAGES], empty_bar[TSTAGES];
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int b = blockIdx.z, hk = blockIdx.y;
  const int row_tile = blockIdx.x % p.row_tiles, split = blockIdx.x / p.row_tiles;
  const int G = p.nq / p.nkv;
  // In key-split mode a warp copies exactly the 16 rows of each key block that it then reads
  // (thread t fills row t / 2), so the warps never wait for one another inside the loop.
  auto tile_sync = [] {
    if constexpr (SPLIT_KEYS) __syncwarp(); else __syncthreads();
  };

  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int ctx = p.ctx_len[b];
  const int start_pos = ctx - q_len;
  const int rows_total = q_len * G;
  const int r0 = row_tile * BM;
  if (q_len <= 0 || r0 >= rows_total) return;

  // Keys this tile can see at all.
  const int last_row = min(r0 + BM, rows_total) - 1;
  const int hi = start_pos + last_row / G;
  const int lo = p.window > 0 ? max(0, start_pos + r0 / G - p.window + 1) : 0;
  int kb0 = lo / BN, kb1 = hi / BN;
  if (p.splits > 1) {
    const int per = p.keys_per_split > 0 ? p.keys_per_split / BN : (kb1 - kb0 + p.splits) / p.splits;
    kb0 = kb0 + split * per;
    kb1 = min(kb1, kb0 + per - 1);
  }
  const int nblocks = kb1 - kb0 + 1;  // may be <= 0 for a split without work
  const int* table = p.block_table + (size_t)b * p.max_blocks;
  if (nblocks <= 0 && p.splits > 1 && !p.cluster) {
    // A split beyond this sequence's keys: mark its partial as empty and leave.  (In a cluster it
    // stays for the barriers and brings an empty partial: no key seen, sum 0.)  Nothing is written
    // before the kernels ahead are done: the scratch may be memory they still read.
    if constexpr (SPLIT_KEYS) ts_pdl_wait();
    for (int r = tid; r < min(BM, rows_total - r0); r += NT) {
      const int row = r0 + r;
      const size_t qrow = (size_t)(q_begin + row / G) * p.nq + hk * G + row % G;
      float* ml = p.part_ml + (qrow * p.splits + split) * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
    if (SPLIT_KEYS && p.counters != nullptr) merge_splits_by_last_arriver<NT>(p, b, hk, q_begin, rows_total, G, &last_flag);
    return;
  }

  // Rows of this thread: g and g + 8 of the warp's 16-row tile.
  const int warp_row0 = SPLIT_KEYS ? 0 : warp * 16;
  const int key0 = SPLIT_KEYS ? warp * 16 : 0;  // first key of the block this warp scores
  int row_pos[2], row_lo[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = r0 + warp_row0 + g + 8 * h;
    row_pos[h] = r < rows_total ? start_pos + r / G : -1;
    row_lo[h] = (p.window > 0 && row_pos[h] >= 0) ? max(0, row_pos[h] - p.window + 1) : 0;
  }
  // Smallest position and largest window start among this warp's rows that exist: key blocks
  // between them are seen in full by every such row.  (Rows that do not exist are never
  // stored, so what an unmasked block leaves in them does not matter.)
  const int warp_first_row = r0 + warp_row0;
  const int warp_last_row = min(warp_first_row + 15, rows_total - 1);
  const int warp_min_pos = warp_first_row < rows_total ? start_pos + warp_first_row / G : -1;
  const int warp_max_lo = (p.window > 0 && warp_first_row < rows_total) ? max(0, start_pos + warp_last_row / G - p.window + 1) : 0;

  // Copy-engine path: warp 0 asks for block `blk` (all its lanes together: every lane one box of
  // [page rows x 64 elements] of K or V), waiting first until the four warps are done with what
  // the stage held.  A page that is not held is asked for at a coordinate beyond the declared
  // pool: the copy engine then writes zeros and touches no memory.
  const int box_rows = min(p.page, BN), copies = BN / box_rows;
  // where box `item` of block `blk` starts in the pool (the block table is read here)
  auto slot_of = [&](int blk, int item) -> int {
    const int key0 = (kb0 + blk) * BN + (item / (2 * HALVES)) * box_rows;
    const int e = key0 / p.page;
    int page_id = -1;
    if (key0 <= hi && e < p.max_blocks) page_id = table[e];
    return page_id >= 0 ? (int)((long long)page_id * p.page + key0 % p.page) : (int)SLOT_BOUND;
  };
  // The first blocks' places are looked up once, before the wait (the block table is the step's own,
  // written before its first kernel): a trip to the table while a stage waits to be filled again
  // cost the walk more than a microsecond after the wait.  (A lane keeps the place of its own box;
  // blocks of more than 32 boxes, and later blocks, are looked up when they are asked for.)
  constexpr int PLACES = 4;
  const bool places_kept = USE_TMA && copies * 2 * HALVES <= 32;
  int place[PLACES];
#pragma unroll
  for (int i = 0; i < PLACES; ++i)
    place[i] = (places_kept && warp == 0 && i < nblocks && lane < copies * 2 * HALVES) ? slot_of(i, lane) : (int)SLOT_BOUND;
  auto tma_ask = [&](int blk) -> bool {
    const int stage = blk % TSTAGES;
    bool ok = true;
    if (blk >= TSTAGES) ok = mbar_wait(smem_u32(&empty_bar[stage]), (unsigned)(blk / TSTAGES - 1) & 1, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return false;
    if (lane == 0) mbar_expect_tx(smem_u32(&full_bar[stage]), 2 * KV_TILE);
    __syncwarp();
    for (int item = lane; item < copies * 2 * HALVES; item += 32) {
      const int c = item / (2 * HALVES), which = (item / HALVES) & 1, half = item % HALVES;
      int slot;
      if (places_kept && blk < PLACES)
        slot = blk == 0 ? place[0] : (blk == 1 ? place[1] : (blk == 2 ? place[2] : place[3]));
      else
        slot = slot_of(blk, item);
      unsigned char* dst = kv_tma + (which * TSTAGES + stage) * KV_TILE + half * (BN * 128) + c * box_rows * 128;
      tma_load_3d(smem_u32(dst), which ? &map_v : &map_k, smem_u32(&full_bar[stage]), half * 64, hk, slot);
    }
    return true;
  };
  // decode: where this thread's pieces of the queries lie (nothing of it depends on the kernel ahead;
  // the copies themselves are asked for after the wait)
  constexpr int Q_COPIES = SPLIT_KEYS ? (BM * CH + NT - 1) / NT : 1;
  const __nv_bfloat16* q_src[Q_COPIES];
#pragma unroll
  for (int i = 0; i < Q_COPIES; ++i) {
    q_src[i] = nullptr;
    if constexpr (SPLIT_KEYS) {
      const int c = tid + i * NT, row = c / CH, r = r0 + row;
      if (c < BM * CH && r < rows_total) q_src[i] = p.q + ((size_t)(q_begin + r / G) * p.nq + hk * G + r % G) * D + (c % CH) * 8;
    }
  }
  int asked = 0;  // blocks asked for so far (warp 0 keeps count; the other warps do not use it)
  if constexpr (USE_TMA) {
    if (tid == 0) {
      abort_s = 0;
      for (int i = 0; i < TSTAGES; ++i) {
        mbar_init(smem_u32(&full_bar[i]), 1);
        mbar_init(smem_u32(&empty_bar[i]), NWARPS);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // before the wait: blocks that hold only keys of earlier steps
    if (warp == 0)
      while (asked < min(nblocks, TSTAGES) && (kb0 + asked) * BN + BN - 1 < start_pos && tma_ask(asked)) ++asked;
    ts_pdl_wait();
    APROBE(1);
    if (warp == 0)
      while (asked < min(nblocks, TSTAGES) && tma_ask(asked)) ++asked;
  }

  // Keys and values of the first two blocks (in decode: before the wait, see above).
  int pg_first[2] = {-1, -1}, pg_next = -1;
  if (nblocks > 0 && !USE_TMA) {
    pg_first[0] = lookup_page<NT>(table, p.page, kb0 * BN, hi, tid);
    if (nblocks > 1) pg_first[1] = lookup_page<NT>(table, p.page, (kb0 + 1) * BN, hi, tid);
    if constexpr (SPLIT_KEYS) {
      load_kv_tiles<NT>(k_s, v_s, p.kcache, p.vcache, pg_first[0], p.page, p.nkv, hk, kb0 * BN, tid, false);
      if (nblocks > 1)
        load_kv_tiles<NT>(k_s + BN * LD, v_s + BN * LD, p.kcache, p.vcache, pg_first[1], p.page, p.nkv, hk, (kb0 + 1) * BN, tid, false);
      if (nblocks > 2) pg_next = lookup_page<NT>(table, p.page, (kb0 + 2) * BN, hi, tid);
    }
  }
  if constexpr (SPLIT_KEYS && !USE_TMA) {
    ts_pdl_wait();
    APROBE(1);
    // what was asked for above has landed before rows of it are fetched again
    cp_async_wait<0>();
    __syncwarp();
  }

  // Queries of the tile (in decode from addresses worked out before the wait).
  if constexpr (SPLIT_KEYS) {
#pragma unroll
    for (int i = 0; i < Q_COPIES; ++i) {
      const int c = tid + i * NT;
      if (c < BM * CH) cp_async16(q_s + (c / CH) * LD + (c % CH) * 8, q_src[i] != nullptr ? q_src[i] : p.q, q_src[i] != nullptr);
    }
  } else {
    for (int c = tid; c < BM * CH; c += NT) {
      const int row = c / CH, ch = c - row * CH;
      const int r = r0 + row;
      const bool valid = r < rows_total;
      const __nv_bfloat16* src = p.q;
      if (valid) src = p.q + ((size_t)(q_begin + r / G) * p.nq + hk * G + r % G) * D + ch * 8;
      cp_async16(q_s + row * LD + ch * 8, src, valid);
    }
  }
  if constexpr (USE_TMA) {
    cp_async_commit();  // the queries
  } else if constexpr (SPLIT_KEYS) {
    // this step's own keys and values (positions from start_pos on), where they lie in the two blocks already fetched
    constexpr int TPR = NT / BN;
    const int row = tid / TPR;
#pragma unroll
    for (int sblk = 0; sblk < 2; ++sblk) {
      const int j = (kb0 + sblk) * BN + row;
      if (sblk < nblocks && j >= start_pos && j <= hi && pg_first[sblk] >= 0) {
        const size_t off = (((size_t)pg_first[sblk] * p.page + (j % p.page)) * p.nkv + hk) * D;
#pragma unroll
        for (int ch = tid % TPR; ch < CH; ch += TPR) {
          cp_async16(k_s + (sblk * BN + row) * LD + ch * 8, p.kcache + off + ch * 8, true);
          cp_async16(v_s + (sblk * BN + row) * LD + ch * 8, p.vcache + off + ch * 8, true);
        }
      }
    }
    cp_async_commit();
  } else {
    cp_async_commit();
    if (nblocks > 0) {
      if (nblocks > 1) pg_next = pg_first[1];
      load_kv_tiles<NT>(k_s, v_s, p.kcache, p.vcache, pg_first[0], p.page, p.nkv, hk, kb0 * BN, tid, false);
    }
  }

  APROBE(2);
  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  unsigned q_frag[Q_IN_REGS ? D / 16 : 1][4];
  const __nv_bfloat16* q_warp = q_s + warp_row0 * LD;
  if (nblocks > 0 && !SPLIT_KEYS) {
    cp_async_wait<2>();  // the queries have landed (K and V of block 0 may still fly)
  } else {
    cp_async_wait<0>();  // decode: the queries and this step's own keys and values; the rest landed before
  }
  __syncthreads();
  if constexpr (Q_IN_REGS) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldmatrix_x4(q_frag[ks][0], q_frag[ks][1], q_frag[ks][2], q_frag[ks][3],
                  q_warp + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
  }

  for (int it = 0; it < nblocks; ++it) {
    const int stage = USE_TMA ? it % TSTAGES : (it & 1);
    const int kbase = (kb0 + it) * BN;
    const bool more = it + 1 < nblocks;
    // decode: blocks 0 and 1 are there already, so the first round has nothing to ask or wait for
    const bool ask = !USE_TMA && more && !(SPLIT_KEYS && it == 0);
    if constexpr (USE_TMA) {
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[stage]), (unsigned)(it / TSTAGES) & 1, abort_flag))) break;
      // rows of V beyond the last key hold whatever was in the cache: zeros instead (their weights
      // are zero, but zero times garbage must stay zero); each warp clears its own 16 rows
      if (kbase + BN - 1 > hi) {
        unsigned char* v_tile = kv_tma + (TSTAGES + stage) * KV_TILE;
        for (int i = lane; i < 16 * HALVES * 8; i += 32) {
          const int row = warp * 16 + i / (HALVES * 8), piece = i % (HALVES * 8);
          if (kbase + row > hi)
            *reinterpret_cast<uint4*>(v_tile + (piece >> 3) * (BN * 128) + row * 128 + ((piece & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
      }
    } else if (ask) {
      load_kv_tiles<NT>(k_s + (stage ^ 1) * BN * LD, v_s + (stage ^ 1) * BN * LD, p.kcache, p.vcache, pg_next, p.page,
                        p.nkv, hk, kbase + BN, tid, false);
      if (it + 2 < nblocks) pg_next = lookup_page<NT>(table, p.page, kbase + 2 * BN, hi, tid);
      if constexpr (SPLIT_KEYS) cp_async_wait<2>(); else cp_async_wait<3>();
    } else if (!more) {
      if constexpr (SPLIT_KEYS) cp_async_wait<0>(); else cp_async_wait<1>();
    }
    if constexpr (!USE_TMA) tile_sync();
    APROBE(3 + min(it, 3) * 2);

    // S = Q K^T over this warp's keys of the block
    float s[NTILES][4];
#pragma unroll
    for (int i = 0; i < NTILES; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    const __nv_bfloat16* k_tile = k_s + stage * BN * LD + key0 * LD;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      unsigned a[4];
      if constexpr (Q_IN_REGS) {
#pragma unroll
        for (int j = 0; j < 4; ++j) a[j] = q_frag[ks][j];
      } else {
        ldmatrix_x4(a[0], a[1], a[2], a[3],
                    q_warp + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
      }
#pragma unroll
      for (int np = 0; np < NTILES / 2; ++np) {
        unsigned b0, b1, b2, b3;
        if constexpr (USE_TMA)
          ldmatrix_x4(b0, b1, b2, b3, swizzled(kv_tma + stage * KV_TILE, key0 + np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8,
                                               ks * 16 + ((lane >> 3) & 1) * 8));
        else
          ldmatrix_x4(b0, b1, b2, b3,
                      k_tile + (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], a, b0, b1);
        mma_bf16(s[2 * np + 1], a, b2, b3);
      }
    }

    // mask, online softmax.  The running max is kept in raw score units (the scale is positive,
    // so it commutes with max) and the scale is folded into the exponent's multiply-add:
    // p = 2^(s * scale - max * scale).  Blocks that every valid row of this warp sees in full
    // skip the mask; the output is rescaled only when some row's max moved.
    float m_new[2] = {m_run[0], m_run[1]};
    const int wk0 = kbase + key0;  // first key this warp scores in this block
    const bool unmasked = (wk0 + NTILES * 8 - 1 <= warp_min_pos) && (wk0 >= warp_max_lo);
    if (unmasked) {
#pragma unroll
      for (int nt = 0; nt < NTILES; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nt][e]);
    } else {
#pragma unroll
      for (int nt = 0; nt < NTILES; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const int j = wk0 + nt * 8 + tq * 2 + (e & 1);
          const bool ok = j <= row_pos[h] && j >= row_lo[h];
          const float v = ok ? s[nt][e] : -INFINITY;
          s[nt][e] = v;
          m_new[h] = fmaxf(m_new[h], v);
        }
      }
    }
    float corr[2], m_off[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
      m_off[h] = m_new[h] == -INFINITY ? 0.f : m_new[h] * p.scale_log2;  // a row that has seen no key yet
      corr[h] = fast_exp2(m_run[h] * p.scale_log2 - m_off[h]);           // m_run = -inf gives 0
      m_run[h] = m_new[h];
    }
    float l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NTILES; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = fast_exp2(fmaf(s[nt][e], p.scale_log2, -m_off[e >> 1]));
        s[nt][e] = pv;
        l_add[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + l_add[h];
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o_acc[i][0] *= corr[0];
        o_acc[i][1] *= corr[0];
        o_acc[i][2] *= corr[1];
        o_acc[i][3] *= corr[1];
      }
    }

    if constexpr (!USE_TMA) {
      if (ask) {
        cp_async_wait<2>();
      } else if (!more) {
        cp_async_wait<0>();
      }
      tile_sync();
    }

    // O += P V
    const __nv_bfloat16* v_tile = v_s + stage * BN * LD + key0 * LD;
#pragma unroll
    for (int kk = 0; kk < NTILES / 2; ++kk) {
      unsigned a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
        unsigned b0, b1, b2, b3;
        if constexpr (USE_TMA)
          ldmatrix_x4_trans(b0, b1, b2, b3, swizzled(kv_tma + (TSTAGES + stage) * KV_TILE, key0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                     np * 16 + ((lane >> 4) & 1) * 8));
        else
          ldmatrix_x4_trans(b0, b1, b2, b3,
                            v_tile + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + np * 16 + ((lane >> 4) & 1) * 8);
        mma_bf16(o_acc[2 * np], a, b0, b1);
        mma_bf16(o_acc[2 * np + 1], a, b2, b3);
      }
    }
    if constexpr (USE_TMA) {
      // this warp is done with the stage; warp 0 asks for the block after next once all are
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
      if (warp == 0 && asked < nblocks && asked == it + TSTAGES) {
        if (!tma_ask(asked)) break;
        ++asked;
      }
    } else {
      tile_sync();  // the next round's prefetch overwrites this stage
    }
    APROBE(4 + min(it, 3) * 2);
  }
  if constexpr (USE_TMA) {
    if (abort_s != 0 && tid == 0 && p.error != nullptr) *p.error = 1;
  }
  APROBE(11);

  // Row sums live spread over the four threads of a quad.
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }

  if constexpr (SPLIT_KEYS) {
    // Merge the warps (each saw its own quarter of the keys) through shared memory, which
    // is free once every warp has left the loop and no copy is in flight.
    __syncthreads();
    float* m_s = reinterpret_cast<float*>(k_s);        // [NWARPS][16]
    float* l_s = m_s + NWARPS * 16;                    // [NWARPS][16]
    float* o_s = l_s + NWARPS * 16;                    // [NWARPS][16][D]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g + 8 * h;
      if (r0 + r >= rows_total) continue;  // a row of the tile that belongs to nobody is not merged either
      if (tq == 0) {
        m_s[warp * 16 + r] = m_run[h] * p.scale_log2;  // log2 units from here on (-inf stays -inf)
        l_s[warp * 16 + r] = l_run[h];
      }
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<float2*>(o_s + (warp * 16 + r) * D + i * 8 + tq * 2) = make_float2(o_acc[i][2 * h], o_acc[i][2 * h + 1]);
    }
    __syncthreads();
    for (int r = warp; r < 16; r += NWARPS) {  // a warp per row, lanes over the head dims
      const int row = r0 + r;
      if (row >= rows_total) continue;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < NWARPS; ++w)
        if (l_s[w * 16 + r] > 0.f) m = fmaxf(m, m_s[w * 16 + r]);
      float l = 0.f, wgt[NWARPS];
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) {
        wgt[w] = l_s[w * 16 + r] > 0.f ? exp2f(m_s[w * 16 + r] - m) : 0.f;
        l += wgt[w] * l_s[w * 16 + r];
      }
      const size_t qrow = (size_t)(q_begin + row / G) * p.nq + hk * G + row % G;
      const float inv = (p.splits == 1) ? (l > 0.f ? 1.f / l : 0.f) : 1.f;
      float* cta_part = o_s + NWARPS * 16 * D + r * (D + 2);  // cluster mode: this CTA's partial of row r
      for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) acc += wgt[w] * o_s[(w * 16 + r) * D + d];
        if (p.splits == 1)
          p.out[qrow * D + d] = __float2bfloat16_rn(acc * inv);
        else if (p.cluster)
          cta_part[d] = acc;
        else
          p.part_o[(qrow * p.splits + split) * D + d] = acc;
      }
      if (p.splits > 1 && lane == 0) {
        float* ml = p.cluster ? cta_part + D : p.part_ml + (qrow * p.splits + split) * 2;
        ml[0] = m;
        ml[1] = l;
      }
    }
    APROBE(12);
    if (p.splits > 1 && p.cluster) {
      // The splits of this (sequence, KV head) pair are the CTAs of one cluster: each has left its
      // partial (weighted sum, max, sum of weights per row) in its own shared memory; after a
      // cluster barrier CTA r % splits merges row r from all of them through distributed shared
      // memory, in rank order, and a second barrier keeps every CTA's memory alive until then.
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
      APROBE(13);
      unsigned rank, nranks;
      asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
      asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(nranks));
      const int rows_here = min(16, rows_total - r0);
      for (int r = (int)rank + (int)nranks * warp; r < rows_here; r += (int)nranks * NWARPS) {  // a warp per row
        const int row = r0 + r;
        const unsigned local = (unsigned)__cvta_generic_to_shared(o_s + NWARPS * 16 * D + r * (D + 2));
        // all loads of a kind are issued before the first is used: two round trips through the
        // cluster's shared memory instead of two per rank
        constexpr int MAXR = 8;  // a cluster has at most 8 CTAs
        unsigned remote[MAXR];
        float mc[MAXR], lc[MAXR];
#pragma unroll
        for (unsigned c = 0; c < MAXR; ++c) {
          remote[c] = 0;
          mc[c] = -INFINITY;
          lc[c] = 0.f;
          if (c < nranks) {
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[c]) : "r"(local), "r"(c));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(mc[c]) : "r"(remote[c] + D * 4));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(lc[c]) : "r"(remote[c] + D * 4 + 4));
          }
        }
        float v[MAXR][(D + 31) / 32];
#pragma unroll
        for (unsigned c = 0; c < MAXR; ++c) {
#pragma unroll
          for (int i = 0; i < (D + 31) / 32; ++i) {
            const int d = lane + 32 * i;
            v[c][i] = 0.f;
            if (c < nranks && d < D) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[c][i]) : "r"(remote[c] + d * 4));
          }
        }
        float m = -INFINITY;
#pragma unroll
        for (unsigned c = 0; c < MAXR; ++c)
          if (lc[c] > 0.f) m = fmaxf(m, mc[c]);
        float l = 0.f, acc[(D + 31) / 32];
#pragma unroll
        for (int i = 0; i < (D + 31) / 32; ++i) acc[i] = 0.f;
#pragma unroll
        for (unsigned c = 0; c < MAXR; ++c) {  // in rank order
          const float wgt = lc[c] > 0.f ? exp2f(mc[c] - m) : 0.f;
          l += wgt * lc[c];
#pragma unroll
          for (int i = 0; i < (D + 31) / 32; ++i) acc[i] += wgt * v[c][i];
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const size_t qrow = (size_t)(q_begin + row / G) * p.nq + hk * G + row % G;
#pragma unroll
        for (int i = 0; i < (D + 31) / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < D) p.out[qrow * D + d] = __float2bfloat16_rn(acc[i] * inv);
        }
      }
      APROBE(14);
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
      APROBE(15);
    }
    if (p.splits > 1 && !p.cluster && p.counters != nullptr) merge_splits_by_last_arriver<NT>(p, b, hk, q_begin, rows_total, G, &last_flag);
  } else {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = r0 + warp_row0 + g + 8 * h;
    if (r >= rows_total) continue;
    const size_t qrow = (size_t)(q_begin + r / G) * p.nq + hk * G + r % G;
    if (p.splits == 1) {
      const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
      __nv_bfloat16* dst = p.out + qrow * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        __nv_bfloat162 v = __floats2bfloat162_rn(o_acc[i][2 * h] * inv, o_acc[i][2 * h + 1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + tq * 2) = v;
      }
    } else {
      float* dst = p.part_o + (qrow * p.splits + split) * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + tq * 2) = make_float2(o_acc[i][2 * h], o_acc[i][2 * h + 1]);
      if (tq == 0) {
        float* ml = p.part_ml + (qrow * p.splits + split) * 2;
        ml[0] = m_run[h] * p.scale_log2;  // log2 units, as the merge expects
        ml[1] = l_run[h];
      }
    }
  }
  }
}

// Prefill for head sizes up to 128: 4 warps, each with 32 query rows (two 16-row MMA tiles), so
// every key/value fragment fetched from shared memory feeds two MMAs.  128 rows per tile.  A
// causal tile's work grows with its position, so a CTA takes two tiles: number x from the end
// and number x from the start of its sequence; every CTA then walks about the same number of
// keys and one wave of CTAs ends together.  Blocks of keys that lie wholly below the diagonal
// (and inside the window) skip the mask.
constexpr int PF_WARPS = 4;
constexpr int PF_MT = 2;                      // 16-row tiles per warp
constexpr int PF_BM = PF_WARPS * 16 * PF_MT;  // 128

__global__ void __launch_bounds__(PF_WARPS * 32, 2) attention_prefill_kernel(const AttnParams p) {
  constexpr int NT = PF_WARPS * 32;
  ts_pdl_prologue();
  constexpr int NTILES = BN / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [PF_BM][LD]
  __nv_bfloat16* k_s = q_s + PF_BM * LD;                                     // [STAGES][BN][LD]
  __nv_bfloat16* v_s = k_s + STAGES * BN * LD;                               // [STAGES][BN][LD]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int b = blockIdx.z, hk = blockIdx.y;
  const int G = p.nq / p.nkv;

  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  const int ctx = p.ctx_len[b];
  const int start_pos = ctx - q_len;
  const int rows_total = q_len * G;
  if (q_len <= 0) return;
  const int seq_tiles = (rows_total + PF_BM - 1) / PF_BM;  // tiles of this sequence
  if ((int)blockIdx.x * 2 >= seq_tiles) return;

  for (int pass = 0; pass < 2; ++pass) {
  const int row_tile = pass == 0 ? seq_tiles - 1 - (int)blockIdx.x : (int)blockIdx.x;
  if (pass == 1 && row_tile >= seq_tiles - 1 - (int)blockIdx.x) break;  // the middle tile was done in pass 0
  if (pass == 1) __syncthreads();  // every warp is done with the first tile's shared memory
  const int r0 = row_tile * PF_BM;

  const int last_row = min(r0 + PF_BM, rows_total) - 1;
  const int hi = start_pos + last_row / G;
  const int first_pos = start_pos + r0 / G;  // position of the tile's first row
  const int lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int kb0 = lo / BN, kb1 = hi / BN;
  const int nblocks = kb1 - kb0 + 1;
  const int* table = p.block_table + (size_t)b * p.max_blocks;

  const int warp_row0 = warp * 16 * PF_MT;
  int row_pos[PF_MT][2], row_lo[PF_MT][2];
#pragma unroll
  for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = r0 + warp_row0 + mt * 16 + g + 8 * h;
      row_pos[mt][h] = r < rows_total ? start_pos + r / G : -1;
      row_lo[mt][h] = (p.window > 0 && row_pos[mt][h] >= 0) ? max(0, row_pos[mt][h] - p.window + 1) : 0;
    }
  // Positions of this warp's first and last row: blocks of keys between them need no mask.
  const int warp_first_pos = start_pos + min(r0 + warp_row0, rows_total - 1) / G;
  const int warp_rows_valid = (r0 + warp_row0 + 16 * PF_MT <= rows_total);

  for (int c = tid; c < PF_BM * CH; c += NT) {
    const int row = c / CH, ch = c - row * CH;
    const int r = r0 + row;
    const bool valid = r < rows_total;
    const __nv_bfloat16* src = p.q;
    if (valid) src = p.q + ((size_t)(q_begin + r / G) * p.nq + hk * G + r % G) * D + ch * 8;
    cp_async16(q_s + row * LD + ch * 8, src, valid);
  }
  int pg_next = -1;
  {
    const int pg0 = lookup_page<NT>(table, p.page, kb0 * BN, hi, tid);
    if (nblocks > 1) pg_next = lookup_page<NT>(table, p.page, (kb0 + 1) * BN, hi, tid);
    load_kv_tiles<NT>(k_s, v_s, p.kcache, p.vcache, pg0, p.page, p.nkv, hk, kb0 * BN, tid, true);
  }

  float o_acc[PF_MT][D / 8][4];
#pragma unroll
  for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o_acc[mt][i][j] = 0.f;
  float m_run[PF_MT][2], l_run[PF_MT][2];
#pragma unroll
  for (int mt = 0; mt < PF_MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
  }
  const __nv_bfloat16* q_warp = q_s + warp_row0 * LD;

  for (int it = 0; it < nblocks; ++it) {
    const int stage = it & 1;
    const int kbase = (kb0 + it) * BN;
    if (it + 1 < nblocks) {
      load_kv_tiles<NT>(k_s + (stage ^ 1) * BN * LD, v_s + (stage ^ 1) * BN * LD, p.kcache, p.vcache, pg_next, p.page,
                        p.nkv, hk, kbase + BN, tid, true);
      if (it + 2 < nblocks) pg_next = lookup_page<NT>(table, p.page, kbase + 2 * BN, hi, tid);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    float s[PF_MT][NTILES][4];
#pragma unroll
    for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
      for (int i = 0; i < NTILES; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[mt][i][j] = 0.f;
    const __nv_bfloat16* k_tile = k_s + stage * BN * LD;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      unsigned a[PF_MT][4];
#pragma unroll
      for (int mt = 0; mt < PF_MT; ++mt)
        ldmatrix_x4(a[mt][0], a[mt][1], a[mt][2], a[mt][3],
                    q_warp + (mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < NTILES / 2; ++np) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3,
                    k_tile + (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int mt = 0; mt < PF_MT; ++mt) {
          mma_bf16(s[mt][2 * np], a[mt], b0, b1);
          mma_bf16(s[mt][2 * np + 1], a[mt], b2, b3);
        }
      }
    }

    // A block whose last key is at or before the warp's first position, whose first key is
    // inside every row's window, and whose rows all exist needs no mask.
    const bool unmasked = warp_rows_valid && (kbase + BN - 1 <= warp_first_pos) &&
                          (p.window <= 0 || kbase >= start_pos + (r0 + warp_row0 + 16 * PF_MT - 1) / G - p.window + 1);
#pragma unroll
    for (int mt = 0; mt < PF_MT; ++mt) {
      // Running max in raw score units (the scale is positive, so it commutes with max); the
      // scale is folded into the exponent's multiply-add: p = 2^(s * scale - max * scale).
      float m_new[2] = {m_run[mt][0], m_run[mt][1]};
      if (unmasked) {
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) m_new[e >> 1] = fmaxf(m_new[e >> 1], s[mt][nt][e]);
      } else {
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int h = e >> 1;
            const int j = kbase + nt * 8 + tq * 2 + (e & 1);
            const bool ok = j <= row_pos[mt][h] && j >= row_lo[mt][h];
            const float v = ok ? s[mt][nt][e] : -INFINITY;
            s[mt][nt][e] = v;
            m_new[h] = fmaxf(m_new[h], v);
          }
      }
      float corr[2], m_off[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
        m_off[h] = m_new[h] == -INFINITY ? 0.f : m_new[h] * p.scale_log2;  // a row that has seen no key yet
        corr[h] = fast_exp2(m_run[mt][h] * p.scale_log2 - m_off[h]);       // m_run = -inf gives 0
        m_run[mt][h] = m_new[h];
      }
      float l_add[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < NTILES; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = fast_exp2(fmaf(s[mt][nt][e], p.scale_log2, -m_off[e >> 1]));
          s[mt][nt][e] = pv;
          l_add[e >> 1] += pv;
        }
#pragma unroll
      for (int h = 0; h < 2; ++h) l_run[mt][h] = l_run[mt][h] * corr[h] + l_add[h];
      // The output only needs rescaling when some row's max moved in this block.
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          o_acc[mt][i][0] *= corr[0];
          o_acc[mt][i][1] *= corr[0];
          o_acc[mt][i][2] *= corr[1];
          o_acc[mt][i][3] *= corr[1];
        }
      }
    }

    const __nv_bfloat16* v_tile = v_s + stage * BN * LD;
#pragma unroll
    for (int kk = 0; kk < NTILES / 2; ++kk) {
      unsigned a[PF_MT][4];
#pragma unroll
      for (int mt = 0; mt < PF_MT; ++mt) {
        a[mt][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
        a[mt][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
        a[mt][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
        a[mt][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
      }
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3,
                          v_tile + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + np * 16 + ((lane >> 4) & 1) * 8);
#pragma unroll
        for (int mt = 0; mt < PF_MT; ++mt) {
          mma_bf16(o_acc[mt][2 * np], a[mt], b0, b1);
          mma_bf16(o_acc[mt][2 * np + 1], a[mt], b2, b3);
        }
      }
    }
    __syncthreads();  // the next round's prefetch overwrites this stage
  }

#pragma unroll
  for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float l = l_run[mt][h];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int r = r0 + warp_row0 + mt * 16 + g + 8 * h;
      if (r >= rows_total) continue;
      const size_t qrow = (size_t)(q_begin + r / G) * p.nq + hk * G + r % G;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + qrow * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        __nv_bfloat162 v = __floats2bfloat162_rn(o_acc[mt][i][2 * h] * inv, o_acc[mt][i][2 * h + 1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + tq * 2) = v;
      }
    }
  }  // pass
}

int launch_prefill(const AttnParams& p, int B, cudaStream_t stream) {
  const size_t smem = (size_t)(PF_BM + 2 * STAGES * BN) * LD * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((p.row_tiles + 1) / 2, p.nkv, B);
  return ts_launch(attention_prefill_kernel, grid, dim3(PF_WARPS * 32), smem, stream, p);
}

// Merges the partial results of the key splits of one (token, head): one warp each.
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         __nv_bfloat16* __restrict__ out, const int* __restrict__ seq_index,
                                         int rows, int nq, int splits) {
  ts_pdl_prologue();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  __nv_bfloat16* dst = out + (size_t)row * D;
  if (seq_index && seq_index[row / nq] < 0) {  // a padded lane of a fixed-size batch
    for (int d = lane; d < D; d += 32) dst[d] = __float2bfloat16_rn(0.f);
    return;
  }
  const float* ml = part_ml + (size_t)row * splits * 2;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s)
    if (ml[2 * s + 1] > 0.f) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  float acc[(D + 31) / 32];
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) acc[i] = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ls = ml[2 * s + 1];
    if (!(ls > 0.f)) continue;  // a split without keys wrote nothing worth reading
    const float w = exp2f(ml[2 * s] - m);
    l += w * ls;
    const float* src = part_o + ((size_t)row * splits + s) * D;
#pragma unroll
    for (int i = 0; i < (D + 31) / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < D) acc[i] += w * src[d];
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) dst[d] = __float2bfloat16_rn(acc[i] * inv);
  }
}

#if (TS_HEAD_DIM % 64) == 0
// ---------------------------------------------------------------------------
// Decode with an even share of key blocks per CTA.
//
// The kernel above gives every (sequence, KV head) pair the same number of CTAs, chosen before the
// launch; with many pairs the CTAs queue in waves whose last is nearly empty, and with few pairs
// and long contexts the fixed count is too small.  Here the key blocks of all pairs form one list
// (sequence-major, then KV head, then block), and CTA c of C takes blocks [c * total / C,
// (c + 1) * total / C) of it, whatever the lengths are: every CTA walks the same number of blocks
// (to within one), through as many pairs as its range meets.  The copy engine runs ahead across
// the pairs, so the start of a pair costs no memory latency.  A pair that lies inside one CTA's
// range gets its output from that CTA; a pair that several CTAs share gets partial results (a CTA
// has at most two such pairs: its first and its last) and attention_flat_combine_kernel, which
// derives the same ranges, merges them.  All of it is computed on the device from the step's
// lengths, so one captured launch serves every step.
constexpr int FLAT_MAX_SEQS = 512;   // sequences whose block counts fit the shared-memory prefix
constexpr int FLAT_ROWS = 16;        // rows of a pair (tokens x heads of the group) at most

struct FlatSeq {
  int q_begin, rows_total, start_pos, hi, kb0, n;  // n: key blocks of each of its pairs
};

__device__ __forceinline__ FlatSeq flat_seq(const AttnParams& p, int b, int G) {
  FlatSeq s;
  s.q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - s.q_begin;
  const int ctx = p.ctx_len[b];
  s.start_pos = ctx - q_len;
  s.rows_total = min(q_len * G, FLAT_ROWS);
  s.hi = ctx - 1;
  const int lo = p.window > 0 ? max(0, s.start_pos - p.window + 1) : 0;
  s.kb0 = lo / BN;
  s.n = (q_len > 0 && ctx > 0 && s.start_pos >= 0) ? s.hi / BN - s.kb0 + 1 : 0;
  return s;
}

struct FlatCursor {
  int b, hk, blk;
  FlatSeq s;
};

// The cursor of block f of the list (f < total).
__device__ __forceinline__ void flat_seek(const AttnParams& p, const int* prefix, int G, int f, FlatCursor& c) {
  int lo = 0, hi = p.num_seqs - 1;
  while (lo < hi) {  // the last sequence whose first block is at or before f (sequences without blocks share their successor's start)
    const int mid = (lo + hi + 1) >> 1;
    if (p.nkv * prefix[mid] <= f) lo = mid; else hi = mid - 1;
  }
  c.b = lo;
  c.s = flat_seq(p, lo, G);
  const int rem = f - p.nkv * prefix[lo];
  const int n = max(c.s.n, 1);
  c.hk = rem / n;
  c.blk = rem - c.hk * n;
}

__device__ __forceinline__ void flat_next(const AttnParams& p, int G, FlatCursor& c) {
  if (++c.blk < c.s.n) return;
  c.blk = 0;
  if (++c.hk < p.nkv) return;
  c.hk = 0;
  do {
    if (++c.b >= p.num_seqs) {
      c.b = p.num_seqs - 1;
      c.s.n = 0;
      return;
    }
    c.s = flat_seq(p, c.b, G);
  } while (c.s.n == 0);
}

// CTAs that take part: all that run at once, but no more than leaves each FLAT_MIN_BLOCKS blocks
// (a CTA that walks one block costs more in starting and merging than it saves).
constexpr int FLAT_MIN_BLOCKS = 2;
__device__ __forceinline__ int flat_ctas_used(int total, int grid) { return max(1, min(grid, total / FLAT_MIN_BLOCKS)); }

// First block of CTA c: floor(c * total / ctas), in 32-bit steps (total < 2^31, ctas < 2^15).
__device__ __forceinline__ int flat_start(int total, int ctas, int c) {
  const int per = total / ctas, rest = total - per * ctas;
  return c * per + (c * rest) / ctas;
}

// The CTA whose range holds block f.
__device__ __forceinline__ int flat_owner(int total, int ctas, int f) {
  int c = (int)((long long)f * ctas / total);
  while (c + 1 < ctas && flat_start(total, ctas, c + 1) <= f) ++c;
  return c;
}

__global__ void __launch_bounds__(128) attention_decode_flat_kernel(const AttnParams p, const __grid_constant__ CUtensorMap map_k,
                                                                    const __grid_constant__ CUtensorMap map_v) {
  constexpr int NWARPS = 4, NT = 128, NTILES = 2;
  static_assert(2 * 4 * D * sizeof(float) <= FLAT_ROWS * LD * sizeof(__nv_bfloat16), "the merge buffer is the query tile");
  ts_pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [16][LD]
  // swizzled tiles on a 1,024-byte boundary: per stage the K tile, then the V tile
  unsigned char* kv = reinterpret_cast<unsigned char*>(((uintptr_t)(q_s + FLAT_ROWS * LD) + 1023) & ~(uintptr_t)1023);
  __shared__ int prefix_s[FLAT_MAX_SEQS + 1];
  __shared__ float mb_s[8], lb_s[8];
  __shared__ __align__(8) unsigned long long full_bar[TSTAGES], empty_bar[TSTAGES];
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int G = p.nq / p.nkv;
  const int key0 = warp * 16;  // first key of every block that this warp scores

  // Before the wait for the kernel ahead: what depends only on the step's index arrays (copied
  // from the host before the step's first kernel) and on keys and values of earlier steps.
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < p.num_seqs; base += 32) {
      const int b = base + lane;
      const int n = b < p.num_seqs ? flat_seq(p, b, G).n : 0;
      int incl = n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      if (b < p.num_seqs) prefix_s[b] = carry + incl - n;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      prefix_s[p.num_seqs] = carry;
      abort_s = 0;
      for (int i = 0; i < TSTAGES; ++i) {
        mbar_init(smem_u32(&full_bar[i]), 1);
        mbar_init(smem_u32(&empty_bar[i]), NWARPS);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
  }
  __syncthreads();
  const int total = p.nkv * prefix_s[p.num_seqs];
  const int ctas = flat_ctas_used(total, (int)gridDim.x), cta = (int)blockIdx.x;
  const int f0 = cta < ctas ? flat_start(total, ctas, cta) : 0, f1 = cta < ctas ? flat_start(total, ctas, cta + 1) : 0;
  const int nblk = f1 - f0;  // blocks of this CTA

  // Warp 0 asks for the blocks, all its lanes together (every lane one box of [page rows x 64
  // elements] of K or V), in list order, each into the stage that its number names, waiting first
  // until the four warps are done with what the stage held.  A page that is not held is asked for
  // at a coordinate beyond the declared pool: the copy engine then writes zeros and touches no memory.
  const int box_rows = min(p.page, BN), copies = BN / box_rows;
  FlatCursor pc;  // the next block to ask for (warp 0 only)
  int asked = 0;
  auto ask = [&]() -> bool {
    const int stage = asked % TSTAGES;
    bool ok = true;
    if (asked >= TSTAGES) ok = mbar_wait(smem_u32(&empty_bar[stage]), (unsigned)(asked / TSTAGES - 1) & 1, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      if (lane == 0) mbar_expect_tx(smem_u32(&full_bar[stage]), 2 * KV_TILE);
      __syncwarp();
      const int* table = p.block_table + (size_t)pc.b * p.max_blocks;
      for (int item = lane; item < copies * 2 * HALVES; item += 32) {
        const int c = item / (2 * HALVES), which = (item / HALVES) & 1, half = item % HALVES;
        const int k0 = (pc.s.kb0 + pc.blk) * BN + c * box_rows;
        const int e = k0 / p.page;
        int page_id = -1;
        if (k0 <= pc.s.hi && e < p.max_blocks) page_id = table[e];
        const long long slot = page_id >= 0 ? (long long)page_id * p.page + k0 % p.page : SLOT_BOUND;
        unsigned char* dst = kv + (stage * 2 + which) * KV_TILE + half * (BN * 128) + c * box_rows * 128;
        tma_load_3d(smem_u32(dst), which ? &map_v : &map_k, smem_u32(&full_bar[stage]), half * 64, pc.hk, (int)slot);
      }
    }
    // after a wait that gave up nothing more is asked for; the count goes on so that every warp
    // leaves the loops at the same place (their waits give up at once)
    ++asked;
    flat_next(p, G, pc);
    return ok;
  };
  if (warp == 0 && nblk > 0) {
    flat_seek(p, prefix_s, G, f0, pc);
    while (asked < min(nblk, TSTAGES) && (pc.s.kb0 + pc.blk) * BN + BN - 1 < pc.s.start_pos) ask();
  }
  ts_pdl_wait();
  if (cta == 0 && p.flat_prefix != nullptr)
    for (int i = tid; i <= p.num_seqs; i += NT) p.flat_prefix[i] = prefix_s[i];
  if (nblk <= 0) return;
  if (warp == 0)
    while (asked < min(nblk, TSTAGES)) ask();

  auto load_queries = [&](const FlatSeq& s, int hk) {
    for (int c = tid; c < FLAT_ROWS * CH; c += NT) {
      const int row = c / CH, ch = c - row * CH;
      const bool valid = row < s.rows_total;
      const __nv_bfloat16* src = p.q;
      if (valid) src = p.q + ((size_t)(s.q_begin + row / G) * p.nq + hk * G + row % G) * D + ch * 8;
      cp_async16(q_s + row * LD + ch * 8, src, valid);
    }
    cp_async_commit();
  };
  FlatCursor cc;
  flat_seek(p, prefix_s, G, f0, cc);
  int done = 0;  // blocks walked so far
  for (int seg = 0; done < nblk; ++seg) {
    // One pair: blocks [blk0, blk0 + cnt) of sequence b, KV head hk.
    const FlatSeq s = cc.s;
    const int b = cc.b, hk = cc.hk, blk0 = cc.blk;
    const int cnt = min(s.n - blk0, nblk - done);
    const bool whole = blk0 == 0 && cnt == s.n;
    (void)b;

    // The pair after this one: its queries are asked for while this pair's warps merge.
    FlatCursor nc = cc;
    nc.blk = blk0 + cnt - 1;
    flat_next(p, G, nc);
    if (seg == 0) load_queries(s, hk);  // the first pair's queries: nothing could ask for them earlier
    int row_pos[2], row_lo[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g + 8 * h;
      row_pos[h] = r < s.rows_total ? s.start_pos + r / G : -1;
      row_lo[h] = (p.window > 0 && row_pos[h] >= 0) ? max(0, row_pos[h] - p.window + 1) : 0;
    }
    const int warp_min_pos = s.start_pos;
    const int warp_max_lo = p.window > 0 ? max(0, s.start_pos + (s.rows_total - 1) / G - p.window + 1) : 0;

    float o_acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    cp_async_wait<0>();
    __syncthreads();
    unsigned q_frag[Q_IN_REGS ? D / 16 : 1][4];
    if constexpr (Q_IN_REGS) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        ldmatrix_x4(q_frag[ks][0], q_frag[ks][1], q_frag[ks][2], q_frag[ks][3],
                    q_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
    }

    for (int it = 0; it < cnt; ++it, ++done) {
      const int stage = done % TSTAGES;
      const int kbase = (s.kb0 + blk0 + it) * BN;
      unsigned char* k_tile = kv + (stage * 2) * KV_TILE;
      unsigned char* v_tile = k_tile + KV_TILE;
      mbar_wait(smem_u32(&full_bar[stage]), (unsigned)(done / TSTAGES) & 1, abort_flag);
      __syncwarp();
      // rows of V beyond the last key hold whatever was in the cache: zeros instead (their weights
      // are zero, but zero times garbage must stay zero); each warp clears its own 16 rows
      if (kbase + BN - 1 > s.hi) {
        for (int i = lane; i < 16 * HALVES * 8; i += 32) {
          const int row = key0 + i / (HALVES * 8), piece = i % (HALVES * 8);
          if (kbase + row > s.hi)
            *reinterpret_cast<uint4*>(v_tile + (piece >> 3) * (BN * 128) + row * 128 + ((piece & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
      }

      // S = Q K^T over this warp's 16 keys of the block
      float sc[NTILES][4];
#pragma unroll
      for (int i = 0; i < NTILES; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        unsigned a[4];
        if constexpr (Q_IN_REGS) {
#pragma unroll
          for (int j = 0; j < 4; ++j) a[j] = q_frag[ks][j];
        } else {
          ldmatrix_x4(a[0], a[1], a[2], a[3], q_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
        }
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, swizzled(k_tile, key0 + (lane & 7) + ((lane >> 4) & 1) * 8, ks * 16 + ((lane >> 3) & 1) * 8));
        mma_bf16(sc[0], a, b0, b1);
        mma_bf16(sc[1], a, b2, b3);
      }

      // mask and online softmax, as in the kernel above
      float m_new[2] = {m_run[0], m_run[1]};
      const int wk0 = kbase + key0;
      const bool unmasked = (wk0 + NTILES * 8 - 1 <= warp_min_pos) && (wk0 >= warp_max_lo);
      if (unmasked) {
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) m_new[e >> 1] = fmaxf(m_new[e >> 1], sc[nt][e]);
      } else {
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int h = e >> 1;
            const int j = wk0 + nt * 8 + tq * 2 + (e & 1);
            const bool ok = j <= row_pos[h] && j >= row_lo[h];
            const float v = ok ? sc[nt][e] : -INFINITY;
            sc[nt][e] = v;
            m_new[h] = fmaxf(m_new[h], v);
          }
        }
      }
      float corr[2], m_off[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
        m_off[h] = m_new[h] == -INFINITY ? 0.f : m_new[h] * p.scale_log2;
        corr[h] = fast_exp2(m_run[h] * p.scale_log2 - m_off[h]);
        m_run[h] = m_new[h];
      }
      float l_add[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < NTILES; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = fast_exp2(fmaf(sc[nt][e], p.scale_log2, -m_off[e >> 1]));
          sc[nt][e] = pv;
          l_add[e >> 1] += pv;
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + l_add[h];
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          o_acc[i][0] *= corr[0];
          o_acc[i][1] *= corr[0];
          o_acc[i][2] *= corr[1];
          o_acc[i][3] *= corr[1];
        }
      }

      // O += P V
      {
        unsigned a[4];
        a[0] = pack_bf16(sc[0][0], sc[0][1]);
        a[1] = pack_bf16(sc[0][2], sc[0][3]);
        a[2] = pack_bf16(sc[1][0], sc[1][1]);
        a[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
        for (int np = 0; np < D / 16; ++np) {
          unsigned b0, b1, b2, b3;
          ldmatrix_x4_trans(b0, b1, b2, b3, swizzled(v_tile, key0 + (lane & 7) + ((lane >> 3) & 1) * 8, np * 16 + ((lane >> 4) & 1) * 8));
          mma_bf16(o_acc[2 * np], a, b0, b1);
          mma_bf16(o_acc[2 * np + 1], a, b2, b3);
        }
      }

      // this warp is done with the stage; warp 0 asks for the block that takes it next once all are
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
      if (warp == 0 && asked < nblk && asked == done + TSTAGES) ask();
    }

    // The pair's blocks of this CTA are walked: the four warps (each saw a quarter of the keys)
    // merge.  No stage of the pipeline is held for it (the copy engine goes on fetching the next
    // pair's blocks): the warps fold in pairs through the small tile that held the queries, four
    // rows at a time, each thread merging the elements it holds itself with the same elements of
    // its partner (warps 2 and 3 into 0 and 1, then 1 into 0), and warp 0 writes the rows.
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float* buf = reinterpret_cast<float*>(q_s);  // [2][4][D]
    __syncthreads();  // the queries are in registers (or read for the last time) in every warp
#pragma unroll
    for (int chunk = 0; chunk < 4; ++chunk) {
      if (chunk * 4 >= s.rows_total) continue;  // the same for every thread
      // rows g + 8 * hs with g / 4 == gs: 0..3, 4..7, 8..11, 12..15
      constexpr int hs_of[4] = {0, 0, 1, 1};
      const int hs = hs_of[chunk], gs = chunk & 1;
      const bool mine = (g >> 2) == gs;
      const int slot = g & 3;
      auto put = [&](int which) {
        if (tq == 0) {
          mb_s[which * 4 + slot] = m_run[hs];
          lb_s[which * 4 + slot] = l_run[hs];
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
          *reinterpret_cast<float2*>(buf + (which * 4 + slot) * D + i * 8 + tq * 2) = make_float2(o_acc[i][2 * hs], o_acc[i][2 * hs + 1]);
      };
      auto fold = [&](int which) {
        const float m_b = mb_s[which * 4 + slot], l_b = lb_s[which * 4 + slot];
        const float m = fmaxf(m_run[hs], m_b);
        const float m_off = m == -INFINITY ? 0.f : m * p.scale_log2;
        const float wa = fast_exp2(m_run[hs] * p.scale_log2 - m_off), wb = fast_exp2(m_b * p.scale_log2 - m_off);
        m_run[hs] = m;
        l_run[hs] = wa * l_run[hs] + wb * l_b;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          const float2 o_b = *reinterpret_cast<const float2*>(buf + (which * 4 + slot) * D + i * 8 + tq * 2);
          o_acc[i][2 * hs] = wa * o_acc[i][2 * hs] + wb * o_b.x;
          o_acc[i][2 * hs + 1] = wa * o_acc[i][2 * hs + 1] + wb * o_b.y;
        }
      };
      if (warp >= 2 && mine) put(warp - 2);
      __syncthreads();
      if (warp < 2 && mine) fold(warp);
      if (warp == 1) {
        __syncwarp();  // the quad has read the partner's max and sum before one of it overwrites them
        if (mine) put(1);  // of the rows, every thread overwrites only what it has just read itself
      }
      __syncthreads();
      if (warp == 0 && mine) {
        fold(1);
        const int r = g + 8 * hs;
        if (r < s.rows_total) {
          const size_t qrow = (size_t)(s.q_begin + r / G) * p.nq + hk * G + r % G;
          if (whole) {
            const float inv = l_run[hs] > 0.f ? 1.f / l_run[hs] : 0.f;
            __nv_bfloat16* dst = p.out + qrow * D;
#pragma unroll
            for (int i = 0; i < D / 8; ++i)
              *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + tq * 2) = __floats2bfloat162_rn(o_acc[i][2 * hs] * inv, o_acc[i][2 * hs + 1] * inv);
          } else {
            // a shared pair: slot 0 of this CTA if the pair is its first, else slot 1 (then it is its last)
            float* part = p.part_o + ((size_t)(cta * 2 + (seg == 0 ? 0 : 1)) * FLAT_ROWS + r) * (D + 2);
#pragma unroll
            for (int i = 0; i < D / 8; ++i)
              *reinterpret_cast<float2*>(part + i * 8 + tq * 2) = make_float2(o_acc[i][2 * hs], o_acc[i][2 * hs + 1]);
            if (tq == 0) {
              part[D] = m_run[hs] * p.scale_log2;  // log2 units, as the combine kernel expects (-inf stays -inf)
              part[D + 1] = l_run[hs];
            }
          }
        }
      }
      __syncthreads();
    }
    if (done < nblk) load_queries(nc.s, nc.hk);
    cc = nc;
  }
  if (abort_s != 0) {
    // A wait gave up: say so, and let the copies that were asked for land before the CTA leaves
    // (bounded again), so that none writes into the shared memory of the CTA that comes next.
    if (tid == 0) {
      if (p.error != nullptr) *p.error = 1;
      volatile int never = 0;
      for (int i = max(0, asked - TSTAGES); i < asked; ++i) mbar_wait(smem_u32(&full_bar[i % TSTAGES]), (unsigned)(i / TSTAGES) & 1, &never);
    }
    __syncthreads();
  }
}

// Merges the partial results of the pairs that several CTAs of attention_decode_flat_kernel shared:
// one warp per (token, head); pairs that one CTA held whole already have their output.  The lanes
// fetch the maxima and sums of up to 32 CTAs at once; the weighted sum then runs over the CTAs
// in list order, a few rows in flight at a time.
__global__ void attention_flat_combine_kernel(const float* __restrict__ part, const int* __restrict__ prefix,
                                              __nv_bfloat16* __restrict__ out, const int* __restrict__ seq_index,
                                              const int* __restrict__ cu_q, int rows, int nq, int nkv, int num_seqs, int grid) {
  ts_pdl_prologue();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int t = row / nq, h = row - t * nq;
  __nv_bfloat16* dst = out + (size_t)row * D;
  const int b = seq_index[t];
  if (b < 0) {  // a padded lane of a fixed-size batch
    for (int d = lane; d < D; d += 32) dst[d] = __float2bfloat16_rn(0.f);
    return;
  }
  const int G = nq / nkv, hk = h / G;
  const int n = prefix[b + 1] - prefix[b];
  const int total = nkv * prefix[num_seqs];
  if (n <= 0 || total <= 0) return;
  const int ctas = flat_ctas_used(total, grid);
  const int off = nkv * prefix[b] + hk * n;
  const int c_first = flat_owner(total, ctas, off), c_last = flat_owner(total, ctas, off + n - 1);
  if (c_first == c_last) return;  // held whole by one CTA
  const int r = (t - cu_q[b]) * G + h % G;
  if (r >= FLAT_ROWS) return;
  // Only the first CTA can have begun before the pair (the pair is then its last, slot 1); every
  // other one begins inside it (the pair is its first, slot 0).
  const int first_slot = flat_start(total, ctas, c_first) < off ? 1 : 0;
  auto rows_of = [&](int c) { return part + ((size_t)(c * 2 + (c == c_first ? first_slot : 0)) * FLAT_ROWS + r) * (D + 2); };
  float m = -INFINITY;
  for (int c = c_first + lane; c <= c_last; c += 32) {
    const float* src = rows_of(c);
    if (src[D + 1] > 0.f) m = fmaxf(m, src[D]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float l = 0.f;
  float acc[(D + 31) / 32];
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) acc[i] = 0.f;
  for (int base = c_first; base <= c_last; base += 32) {
    const int mine = base + lane;
    float w_mine = 0.f;
    if (mine <= c_last) {
      const float* src = rows_of(mine);
      const float ls = src[D + 1];
      if (ls > 0.f) {
        w_mine = exp2f(src[D] - m);
        l += w_mine * ls;
      }
    }
    const int here = min(32, c_last - base + 1);
#pragma unroll 4
    for (int j = 0; j < here; ++j) {  // in list order
      const float w = __shfl_sync(0xffffffffu, w_mine, j);
      const float* src = rows_of(base + j);
#pragma unroll
      for (int i = 0; i < (D + 31) / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] += w * src[d];
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) dst[d] = __float2bfloat16_rn(acc[i] * inv);
  }
}

#endif  // head sizes that the copy engine takes

template <int NWARPS, bool SPLIT_KEYS>
int launch(const AttnParams& p, int B, cudaStream_t stream) {
  constexpr int BM = SPLIT_KEYS ? 16 : NWARPS * 16;
  const size_t smem = (size_t)(BM + 2 * STAGES * BN) * LD * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<NWARPS, SPLIT_KEYS, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap none;
  memset(&none, 0, sizeof(none));
  dim3 grid(p.row_tiles * p.splits, p.nkv, B);
  if (p.cluster)  // the grid's x dimension is the key splits of one pair: one cluster
    return ts_launch_cluster(attention_mma_kernel<NWARPS, SPLIT_KEYS, false>, grid, dim3(NWARPS * 32), smem, stream, p.splits, p, none, none);
  return ts_launch(attention_mma_kernel<NWARPS, SPLIT_KEYS, false>, grid, dim3(NWARPS * 32), smem, stream, p, none, none);
}

// Whether the decode kernel's copy-engine path takes these sizes.
bool decode_tma_ok(const AttnParams& p) {
  return TMA_HEAD && p.page >= 8 && (BN % p.page == 0 || p.page % BN == 0) &&
         ((uintptr_t)p.kcache | (uintptr_t)p.vcache) % 16 == 0 && ((long long)p.nkv * D * 2) % 16 == 0;
}

// Decode with the copy engine: the same kernel, its K/V tiles swizzled and brought by TMA.
int launch_decode_tma(const AttnParams& p, int B, cudaStream_t stream) {
  if constexpr (!TMA_HEAD) {
    return TS_ERR_UNSUPPORTED_SIZE;
  } else {
    const size_t smem = (size_t)16 * LD * sizeof(__nv_bfloat16) + 1024 + (size_t)2 * TSTAGES * KV_TILE;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<4, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    CUtensorMap mk, mv;
    const int box_rows = p.page < BN ? p.page : BN;
    int st = ts_kv_cache_map(p.kcache, SLOT_BOUND, p.nkv, D, box_rows, &mk);
    if (st != 0) return st;
    st = ts_kv_cache_map(p.vcache, SLOT_BOUND, p.nkv, D, box_rows, &mv);
    if (st != 0) return st;
    dim3 grid(p.row_tiles * p.splits, p.nkv, B);
    if (p.cluster)
      return ts_launch_cluster(attention_mma_kernel<4, true, true>, grid, dim3(128), smem, stream, p.splits, p, mk, mv);
    return ts_launch(attention_mma_kernel<4, true, true>, grid, dim3(128), smem, stream, p, mk, mv);
  }
}


#if (TS_HEAD_DIM % 64) == 0
size_t flat_smem() { return (size_t)FLAT_ROWS * LD * sizeof(__nv_bfloat16) + 1024 + (size_t)2 * TSTAGES * KV_TILE; }

// How many CTAs of the even-share decode kernel the GPU runs at once: its grid.
int flat_ctas() {
  static int ctas = 0;
  if (ctas == 0) {
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
    cudaFuncSetAttribute(attention_decode_flat_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)flat_smem());
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_flat_kernel, 128, flat_smem()) != cudaSuccess || per_sm <= 0) per_sm = 1;
    ctas = sms * per_sm;
  }
  return ctas;
}
#endif

}  // namespace

// Scratch floats needed for `rows` = tokens * query heads and `splits` key splits.
TS_EXPORT long long ts_attention_mma_scratch_floats(long long rows, int splits) {
  return splits > 1 ? rows * splits * (long long)(D + 2) : 0;
}

TS_EXPORT int ts_attention_mma_head_dim() { return D; }

// q/out [T, nq, D] bf16; caches [slots, nkv, D] bf16; cu_q [B+1]; ctx_len [B]; block_table
// [B, max_blocks].  max_q: the most tokens any sequence brings in this step.  splits > 1
// needs `scratch` of ts_attention_mma_scratch_floats(T * nq, splits) floats; seq_index
// ([T], -1 marks padding) is only read when splits > 1.
// As ts_attention_paged_mma, with the keys of a sequence cut into fixed chunks of
// `keys_per_split` keys (a multiple of 64; split s takes chunk s, splits beyond the sequence do
// nothing), so that sequences of different lengths give CTAs of equal work.  0 divides each
// sequence's keys evenly over the splits.
// `counters` (B * nkv ints, zero before the first call; the kernel leaves them zero): with it the
// last CTA of every (sequence, KV head) pair merges the pair's splits itself and no second kernel
// runs; only for decode steps (at most 16 query rows per pair).  Null: the merge is a kernel of
// its own.
// How many CTAs of the decode kernel the GPU runs at once.
static long long decode_slots() {
  static long long slots = 0;
  if (slots == 0) {
    int dev = 0, sms = 0, per_sm = 0;
    const size_t smem = (size_t)(16 + 2 * STAGES * BN) * LD * sizeof(__nv_bfloat16);
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
    cudaFuncSetAttribute(attention_mma_kernel<4, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_mma_kernel<4, true, false>, 128, smem) != cudaSuccess || per_sm <= 0) per_sm = 1;
    slots = (long long)sms * per_sm;
  }
  return slots;
}

// TS_ATT_PROBE builds: where the decode kernel's first CTAs leave their clock stamps (16 per CTA).
static long long* ts_attention_probe = nullptr;
TS_EXPORT void ts_attention_mma_set_probe(long long* buffer) { ts_attention_probe = buffer; }

// Whether decode steps fetch keys and values with the copy engine where the sizes allow it, and the
// word (in memory the host can read) that a kernel sets when one of its bounded waits gave up.
static int ts_attention_decode_tma = 1;
static int* ts_attention_error_word = nullptr;
TS_EXPORT void ts_attention_mma_set_decode_tma(int on) { ts_attention_decode_tma = on ? 1 : 0; }
TS_EXPORT void ts_attention_mma_set_error_word(int* word) { ts_attention_error_word = word; }

// Whether decode steps with 2..8 key splits merge the splits inside a thread-block cluster
// (through distributed shared memory) instead of through scratch and a second kernel.
static int ts_attention_cluster_merge = 1;
TS_EXPORT void ts_attention_mma_set_cluster_merge(int on) { ts_attention_cluster_merge = on ? 1 : 0; }
TS_EXPORT int ts_attention_mma_cluster_merge(void) { return ts_attention_cluster_merge; }

// What the Python side plans with: CTAs of the decode kernel that run at once, the most query
// rows (tokens x heads of a group) a sequence may bring to be served by the decode kernels, and
// how many kernels the last call of ts_attention_paged_mma_fused launched (1, or 2 with the merge).
TS_EXPORT long long ts_attention_mma_decode_slots(void) { return decode_slots(); }
TS_EXPORT int ts_attention_mma_decode_rows(void) { return 16; }
static int ts_attention_last_launches = 0;
TS_EXPORT int ts_attention_mma_last_launches(void) { return ts_attention_last_launches; }

TS_EXPORT int ts_attention_paged_mma_fused(const void* q, const void* kcache, const void* vcache, void* out,
                                           float* scratch, const int* cu_q, const int* ctx_len,
                                           const int* block_table, const int* seq_index, int max_blocks,
                                           int page, int T, int B, int max_q, int nq, int nkv, float scale,
                                           int window, int splits, int keys_per_split, int* counters, void* stream_) {
  if (T <= 0 || B <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page <= 0 || max_blocks <= 0 || max_q <= 0 || splits < 1 ||
      keys_per_split < 0 || keys_per_split % BN != 0)
    return TS_ERR_BAD_ARGUMENT;
  if (splits > 1 && scratch == nullptr) return TS_ERR_BAD_ARGUMENT;
  if (nkv > 65535 || B > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  cudaStream_t stream = (cudaStream_t)stream_;
  const int G = nq / nkv;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q;
  p.kcache = (const __nv_bfloat16*)kcache;
  p.vcache = (const __nv_bfloat16*)vcache;
  p.out = (__nv_bfloat16*)out;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + (size_t)T * nq * splits * D : nullptr;
  p.cu_q = cu_q;
  p.ctx_len = ctx_len;
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.page = page;
  p.nq = nq;
  p.nkv = nkv;
  p.window = window;
  p.splits = splits;
  p.keys_per_split = keys_per_split;
  p.counters = (counters != nullptr && splits > 1 && (long long)max_q * (nq / nkv) <= 16) ? counters : nullptr;
  // merge inside a cluster: decode steps (one row tile) with 2..8 splits, the splits dividing each sequence's keys evenly
  // (and only while all CTAs run at once: clusters are placed as wholes, which costs occupancy as soon as CTAs queue)
  p.cluster = (ts_attention_cluster_merge && splits > 1 && splits <= 8 && (long long)max_q * (nq / nkv) <= 16 && keys_per_split == 0 &&
               (long long)B * nkv * splits <= decode_slots()) ? 1 : 0;
  if (p.cluster) p.counters = nullptr;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_seqs = B;
  p.flat_prefix = nullptr;
  p.probe = ts_attention_probe;
  p.error = ts_attention_error_word;
  const long long rows = (long long)max_q * G;
  int status;
  if (rows <= 16) {
    p.row_tiles = 1;
    status = (ts_attention_decode_tma && decode_tma_ok(p)) ? launch_decode_tma(p, B, stream) : launch<4, true>(p, B, stream);
  } else {
    p.row_tiles = (int)((rows + 127) / 128);
    if (D <= 128 && splits == 1)
      status = launch_prefill(p, B, stream);
    else
      status = launch<8, false>(p, B, stream);
  }
  if (status != 0) return status;
  ts_attention_last_launches = 1;
  if (splits > 1 && p.counters == nullptr && !p.cluster) {
    const int total = T * nq;
    ts_attention_last_launches = 2;
    status = ts_launch(attention_combine_kernel, dim3((total + 3) / 4), dim3(128), 0, stream, (const float*)p.part_o, (const float*)p.part_ml, p.out, seq_index, total, nq, splits);
  }
  return status;
}

TS_EXPORT int ts_attention_paged_mma_chunked(const void* q, const void* kcache, const void* vcache, void* out,
                                             float* scratch, const int* cu_q, const int* ctx_len,
                                             const int* block_table, const int* seq_index, int max_blocks,
                                             int page, int T, int B, int max_q, int nq, int nkv, float scale,
                                             int window, int splits, int keys_per_split, void* stream_) {
  return ts_attention_paged_mma_fused(q, kcache, vcache, out, scratch, cu_q, ctx_len, block_table, seq_index,
                                      max_blocks, page, T, B, max_q, nq, nkv, scale, window, splits, keys_per_split,
                                      nullptr, stream_);
}

TS_EXPORT int ts_attention_paged_mma(const void* q, const void* kcache, const void* vcache, void* out,
                                     float* scratch, const int* cu_q, const int* ctx_len,
                                     const int* block_table, const int* seq_index, int max_blocks,
                                     int page, int T, int B, int max_q, int nq, int nkv, float scale,
                                     int window, int splits, void* stream_) {
  return ts_attention_paged_mma_fused(q, kcache, vcache, out, scratch, cu_q, ctx_len, block_table, seq_index,
                                      max_blocks, page, T, B, max_q, nq, nkv, scale, window, splits, 0, nullptr, stream_);
}

// ---------------------------------------------------------------------------
// Decode with an even share of key blocks per CTA (see attention_decode_flat_kernel): decode steps
// only (at most 16 rows per sequence and KV head), head sizes that are multiples of 64, at most 512
// sequences, pages the copy engine takes.  `ctas`: the grid, at most ts_attention_decode_flat_ctas();
// `scratch`: ts_attention_decode_flat_scratch_floats(B, ctas) floats.
TS_EXPORT int ts_attention_decode_flat_ctas(void) {
#if (TS_HEAD_DIM % 64) == 0
  return flat_ctas();
#else
  return 0;
#endif
}

TS_EXPORT long long ts_attention_decode_flat_scratch_floats(int B, int ctas) {
#if (TS_HEAD_DIM % 64) == 0
  return (long long)ctas * 2 * FLAT_ROWS * (D + 2) + B + 1;
#else
  (void)B;
  (void)ctas;
  return 0;
#endif
}

TS_EXPORT int ts_attention_decode_flat(const void* q, const void* kcache, const void* vcache, void* out, float* scratch,
                                       const int* cu_q, const int* ctx_len, const int* block_table, const int* seq_index,
                                       int max_blocks, int page, int T, int B, int max_q, int nq, int nkv, float scale,
                                       int window, int ctas, void* stream_) {
#if (TS_HEAD_DIM % 64) == 0
  if (T <= 0 || B <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page <= 0 || max_blocks <= 0 || max_q <= 0 || scratch == nullptr || seq_index == nullptr)
    return TS_ERR_BAD_ARGUMENT;
  if ((long long)max_q * (nq / nkv) > FLAT_ROWS || B > FLAT_MAX_SEQS || ctas < 1 || ctas > flat_ctas()) return TS_ERR_UNSUPPORTED_SIZE;
  cudaStream_t stream = (cudaStream_t)stream_;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.q = (const __nv_bfloat16*)q;
  p.kcache = (const __nv_bfloat16*)kcache;
  p.vcache = (const __nv_bfloat16*)vcache;
  p.out = (__nv_bfloat16*)out;
  p.part_o = scratch;
  p.flat_prefix = reinterpret_cast<int*>(scratch + (size_t)ctas * 2 * FLAT_ROWS * (D + 2));
  p.cu_q = cu_q;
  p.ctx_len = ctx_len;
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.page = page;
  p.nq = nq;
  p.nkv = nkv;
  p.window = window;
  p.splits = 1;
  p.row_tiles = 1;
  p.num_seqs = B;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.probe = ts_attention_probe;
  p.error = ts_attention_error_word;
  if (!decode_tma_ok(p)) return TS_ERR_UNSUPPORTED_SIZE;
  CUtensorMap mk, mv;
  const int box_rows = page < BN ? page : BN;
  int st = ts_kv_cache_map(p.kcache, SLOT_BOUND, nkv, D, box_rows, &mk);
  if (st != 0) return st;
  st = ts_kv_cache_map(p.vcache, SLOT_BOUND, nkv, D, box_rows, &mv);
  if (st != 0) return st;
  (void)flat_ctas();  // sets the kernel's shared-memory limit
  st = ts_launch(attention_decode_flat_kernel, dim3(ctas), dim3(128), flat_smem(), stream, p, mk, mv);
  if (st != 0) return st;
  const int total = T * nq;
  return ts_launch(attention_flat_combine_kernel, dim3((total + 3) / 4), dim3(128), 0, stream, (const float*)p.part_o,
                   (const int*)p.flat_prefix, p.out, seq_index, cu_q, total, nq, nkv, B, ctas);
#else
  return TS_ERR_UNSUPPORTED_SIZE;
#endif
}

// ---------------------------------------------------------------------------
// The entry point that allocates nothing (see attention_mma_noalloc.h for who needs it,
// the limit and the rules of use).  It changes nothing above: it looks up the address of
// a scratch array that lives in this library and calls ts_attention_paged_mma with it.
#include "attention_mma_noalloc.h"

// File-scope scratch: in host code this name is only a handle for cudaGetSymbolAddress,
// never a pointer a kernel may be given.
static __device__ __align__(256) float ts_attention_noalloc_scratch[TS_ATTENTION_NOALLOC_SCRATCH_FLOATS];

#define TS_NOALLOC_MAX_DEVICES 64
static float* ts_noalloc_scratch_address[TS_NOALLOC_MAX_DEVICES];  // per device, filled at its first call

TS_EXPORT long long ts_attention_noalloc_scratch_floats(void) { return TS_ATTENTION_NOALLOC_SCRATCH_FLOATS; }

TS_EXPORT const char* ts_attention_noalloc_error_text(int code) {
  switch (code) {
    case 0: return "ok";
    case TS_ERR_BAD_ARGUMENT: return "bad argument (sizes must be positive, heads a multiple of kv heads)";
    case TS_ERR_UNSUPPORTED_SIZE: return "size not supported by this kernel";
    case TS_ERR_SCRATCH_LIMIT:
      return "tokens * query_heads * splits * (head_dim + 2) exceeds the library's built-in scratch "
             "(TS_ATTENTION_NOALLOC_SCRATCH_FLOATS floats): use fewer splits or tokens, or the entry "
             "point that takes scratch from the caller";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
  }
}

TS_EXPORT int ts_attention_paged_mma_noalloc(const void* q, const void* kcache, const void* vcache, void* out,
                                             const int* cu_q, const int* ctx_len, const int* block_table,
                                             const int* seq_index, int max_blocks, int page, int T, int B,
                                             int max_q, int nq, int nkv, float scale, int window, int splits,
                                             void* stream) {
  if (T <= 0 || B <= 0) return 0;
  if (nq <= 0 || splits < 1) return TS_ERR_BAD_ARGUMENT;
  float* scratch = nullptr;
  if (splits > 1) {
    if (ts_attention_mma_scratch_floats((long long)T * nq, splits) > (long long)TS_ATTENTION_NOALLOC_SCRATCH_FLOATS)
      return TS_ERR_SCRATCH_LIMIT;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= TS_NOALLOC_MAX_DEVICES) return TS_ERR_UNSUPPORTED_SIZE;
    if (ts_noalloc_scratch_address[device] == nullptr) {
      // First call on this device: turn the symbol into the address the kernels can use.
      float* address = nullptr;
      e = cudaGetSymbolAddress((void**)&address, ts_attention_noalloc_scratch);
      if (e != cudaSuccess) return (int)e;
      if (address == nullptr) return (int)cudaErrorInvalidSymbol;
      ts_noalloc_scratch_address[device] = address;
    }
    scratch = ts_noalloc_scratch_address[device];
  }
  return ts_attention_paged_mma(q, kcache, vcache, out, scratch, cu_q, ctx_len, block_table, seq_index,
                                max_blocks, page, T, B, max_q, nq, nkv, scale, window, splits, stream);
}
