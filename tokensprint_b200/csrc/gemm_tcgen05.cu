// Skinny bfloat16 GEMM for decode steps on the 5th-generation tensor cores:
//   out[M, N] = X[M, K] * W[N, K]^T,  M <= 128 tokens, float32 accumulation in tensor memory.
//
// A decode step reads every weight once and does little math with it, so the kernel is built
// to stream W at HBM speed.  The roles are swapped against the usual picture: the 128 rows
// of a W tile are the MMA's M dimension, the (padded) tokens its N dimension, so even one
// token fills the tensor core's rows.  Per CTA: one 128-row tile of W and one slice of K.
//   * thread 0 of warp 0 issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of
//     [128 x 64] W tiles and [MPAD x 64] X tiles into a ring of shared-memory stages;
//   * thread 0 of warp 1 issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=MPAD, K=16)
//     from those stages into a TMEM accumulator and frees each stage with tcgen05.commit;
//   * all four warps read the accumulator back with tcgen05.ld and store it.
// Layers with few rows (o_proj, down_proj) would leave most SMs idle, so K is cut into
// `splits` slices; each CTA writes its float32 partial tile to scratch, takes a ticket, and
// the CTA that arrives last adds the slices in their fixed order and writes the result.
// Nobody waits for anybody there; the only waits are on mbarriers fed by this CTA's own
// copies and MMAs, and each of them gives up after a bounded number of tries, raises the
// error word and lets the CTA free its tensor memory and return.
//
// The reference runs these products through nn.Linear (engine/nn/attention.py:122-135,
// engine/nn/layers.py:61-66); W is row-major [out, in] as there.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int TILE_N = 128;   // W rows per CTA (the MMA's M)
constexpr int TILE_K = 64;    // bf16 per stage and row: one 128-byte swizzle atom
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

struct GemmArgs {
  void* out;             // [M, ldo] bf16 or f32
  float* partial;        // [splits, M, N] f32 (splits > 1)
  int* counters;         // [n_tiles] zero before the first launch, zero again after each
  int* error;            // set to 1 when a wait gave up
  int M, N, K, ldo, splits, out_f32;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for a phase of an mbarrier.  False: gave up (or another role already did).
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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
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

template <int MPAD>
__global__ void __launch_bounds__(128) gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w,
                                                          const __grid_constant__ CUtensorMap map_x,
                                                          const GemmArgs args) {
  constexpr uint32_t A_BYTES = TILE_N * TILE_K * 2;
  constexpr uint32_t B_BYTES = MPAD * TILE_K * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + ((B_BYTES + 1023) / 1024) * 1024;
  constexpr uint32_t TMEM_COLS = MPAD < 32 ? 32 : MPAD;
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MPAD >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24);

  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int last_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * TILE_N;
  const int split = blockIdx.y;
  const int chunks = (args.K + TILE_K - 1) / TILE_K;
  const int per = (chunks + args.splits - 1) / args.splits;
  const int kc0 = split * per;
  const int nk = max(0, min(chunks, kc0 + per) - kc0);

  if (tid == 0) {
    abort_s = 0;
    last_s = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&acc_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort_flag = &abort_s;

  if (nk > 0) {
    if (warp == 0 && lane == 0) {
      // Producer: TMA loads into the ring.
      int issued = 0;
      for (int i = 0; i < nk; ++i) {
        const int s = i % STAGES;
        const uint32_t round = (uint32_t)(i / STAGES);
        if (i >= STAGES && !mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1, abort_flag)) break;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t dst = smem_u32(smem + (size_t)s * STAGE_BYTES);
        mbar_expect_tx(bar, A_BYTES + B_BYTES);
        tma_load_2d(dst, &map_w, bar, (kc0 + i) * TILE_K, n0);
        tma_load_2d(dst + A_BYTES, &map_x, bar, (kc0 + i) * TILE_K, 0);
        issued = i + 1;
      }
      if (*abort_flag) {
        // Let the copies that are still in flight land before shared memory is given up.
        for (int i = max(0, issued - STAGES); i < issued; ++i)
          mbar_wait(smem_u32(&full_bar[i % STAGES]), (uint32_t)(i / STAGES) & 1, abort_flag);
      }
    } else if (warp == 1 && lane == 0) {
      // MMA issuer.
      bool ok = true;
      for (int i = 0; i < nk && ok; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(smem_u32(&full_bar[s]), (uint32_t)(i / STAGES) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
        const uint64_t adesc = umma_desc_sw128(a_addr);
        const uint64_t bdesc = umma_desc_sw128(a_addr + A_BYTES);
#pragma unroll
        for (int k = 0; k < TILE_K / UMMA_K; ++k) {
          // 16 bf16 = 32 bytes further along K inside the swizzle atom: +2 in the address field
          umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, IDESC, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&empty_bar[s]));  // arrives when these MMAs have read the stage
      }
      if (ok) umma_commit(smem_u32(&acc_bar));  // arrives when the accumulator is complete
    }
    __syncwarp();
    // Everybody: wait for the accumulator.
    mbar_wait(smem_u32(&acc_bar), 0, abort_flag);
  }
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  __syncthreads();
  const bool aborted = abort_s != 0;

  if (!aborted) {
    const int n = n0 + warp * 32 + lane;  // this thread's W row = output column
    const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll
    for (int c = 0; c < MPAD / 16; ++c) {
      uint32_t r[16];
      if (nk > 0) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr + c * 16));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = 0u;
      }
      if (n < args.N) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int m = c * 16 + i;
          if (m >= args.M) break;
          const float v = __uint_as_float(r[i]);
          if (args.splits > 1)
            args.partial[((size_t)split * args.M + m) * args.N + n] = v;
          else if (args.out_f32)
            reinterpret_cast<float*>(args.out)[(size_t)m * args.ldo + n] = v;
          else
            reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)m * args.ldo + n] = __float2bfloat16_rn(v);
        }
      }
    }
    if (args.splits > 1) {
      // Ticket: whoever arrives last for this tile adds the slices, in slice order.
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int ticket = atomicAdd(&args.counters[blockIdx.x], 1);
        last_s = (ticket == args.splits - 1) ? 1 : 0;
      }
      __syncthreads();
      if (last_s) {
        __threadfence();
        const int nn = n0 + tid;
        if (nn < args.N) {
          for (int m = 0; m < args.M; ++m) {
            float acc = 0.f;
            for (int s = 0; s < args.splits; ++s) acc += __ldcg(&args.partial[((size_t)s * args.M + m) * args.N + nn]);
            if (args.out_f32)
              reinterpret_cast<float*>(args.out)[(size_t)m * args.ldo + nn] = acc;
            else
              reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)m * args.ldo + nn] = __float2bfloat16_rn(acc);
          }
        }
        if (tid == 0) args.counters[blockIdx.x] = 0;
      }
    }
  } else if (tid == 0) {
    *args.error = 1;
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
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
  cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return TS_ERR_BAD_ARGUMENT;
  if (map_cache.size() > 4096) map_cache.clear();
  map_cache.emplace(key, *out);
  return 0;
}

template <int MPAD>
int launch_skinny(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& a, int n_tiles, cudaStream_t stream) {
  constexpr size_t A_BYTES = TILE_N * TILE_K * 2;
  constexpr size_t B_BYTES = MPAD * TILE_K * 2;
  constexpr size_t STAGE_BYTES = A_BYTES + ((B_BYTES + 1023) / 1024) * 1024;
  const size_t smem = STAGES * STAGE_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<MPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  gemm_skinny_kernel<MPAD><<<dim3(n_tiles, a.splits), 128, smem, stream>>>(mw, mx, a);
  return ts_launch_status();
}

}  // namespace

// How many K slices the kernel would use for an [N, K] weight (depends on the shape only,
// so a token's result never depends on the batch around it).
TS_EXPORT int ts_gemm_skinny_splits(int N, int K) {
  const int tiles = (N + TILE_N - 1) / TILE_N;
  const int chunks = (K + TILE_K - 1) / TILE_K;
  int s = 1;
  while (s < 8 && tiles * s < 148 && chunks / (s * 2) >= 8) s *= 2;
  return s;
}

// Scratch the caller brings: floats for the partial tiles (splits * M * N when splits > 1).
TS_EXPORT long long ts_gemm_skinny_scratch_floats(int M, int N, int K) {
  const int s = ts_gemm_skinny_splits(N, K);
  return s > 1 ? (long long)s * M * N : 0;
}

TS_EXPORT int ts_gemm_skinny_max_rows() { return 128; }

// out[M, ldo] (bf16, or f32 when out_f32) = x[M, K] (row stride ldx) * w[N, K]^T (row stride ldw).
// `counters`: ints, one per 128-row tile of W, zero before the first call (the kernel leaves
// them zero).  `error`: one int the kernel sets to 1 if one of its waits gave up.
TS_EXPORT int ts_gemm_skinny_bf16(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
                                  long long ldw, long long ldo, int out_f32, float* partial, int* counters,
                                  int* error, void* stream_) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || ldx < K || ldw < K || ldo < N || counters == nullptr || error == nullptr) return TS_ERR_BAD_ARGUMENT;
  if (M > 128 || (K % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)x % 16) || ((uintptr_t)w % 16))
    return TS_ERR_UNSUPPORTED_SIZE;
  const int splits = ts_gemm_skinny_splits(N, K);
  if (splits > 1 && partial == nullptr) return TS_ERR_BAD_ARGUMENT;
  const int mpad = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  const int n_tiles = (N + TILE_N - 1) / TILE_N;
  CUtensorMap mw, mx;
  int st = tensor_map(w, N, K, ldw, TILE_N, &mw);
  if (st != 0) return st;
  st = tensor_map(x, M, K, ldx, mpad, &mx);
  if (st != 0) return st;
  GemmArgs a;
  a.out = out;
  a.partial = partial;
  a.counters = counters;
  a.error = error;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldo = (int)ldo;
  a.splits = splits;
  a.out_f32 = out_f32;
  cudaStream_t stream = (cudaStream_t)stream_;
  switch (mpad) {
    case 16: return launch_skinny<16>(mw, mx, a, n_tiles, stream);
    case 32: return launch_skinny<32>(mw, mx, a, n_tiles, stream);
    case 64: return launch_skinny<64>(mw, mx, a, n_tiles, stream);
    default: return launch_skinny<128>(mw, mx, a, n_tiles, stream);
  }
}
