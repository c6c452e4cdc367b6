// Shared helpers of the sm_100a kernels: element types, conversions, reductions.
//
// Every exported entry point is `extern "C"`, takes raw device pointers, sizes and a
// CUDA stream, launches asynchronously on that stream and returns 0 or a cudaError_t
// as int (negative values: an argument this kernel does not take).  Element types are
// passed as codes: 0 = float32, 1 = bfloat16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TS_DTYPE_F32 0
#define TS_DTYPE_BF16 1

#define TS_ERR_BAD_ARGUMENT (-1)
#define TS_ERR_UNSUPPORTED_SIZE (-2)

#define TS_EXPORT extern "C" __attribute__((visibility("default")))

// Programmatic dependent launch: every kernel of this library is launched with the attribute
// that lets it start while the kernel before it in the stream is still running, and begins with
// ts_pdl_prologue(): it first lets its own successor start launching, then waits until the
// kernels before it have completed and their writes are visible.  What a kernel does before that
// wait (set-up, loads of weights that no kernel writes) overlaps with its predecessor; launch
// latency overlaps in any case.  TS_PDL=0 in the environment turns the attribute off.
#include <stdlib.h>

__device__ __forceinline__ void ts_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void ts_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ts_pdl_prologue() {
  ts_pdl_launch_dependents();
  ts_pdl_wait();
}

static inline bool ts_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* v = getenv("TS_PDL");
    enabled = (v && v[0] == '0') ? 0 : 1;
  }
  return enabled == 1;
}

template <typename... KArgs, typename... Args>
static inline int ts_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = ts_pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

// The same with the grid's x dimension cut into thread-block clusters of `cluster_x` CTAs.
template <typename... KArgs, typename... Args>
static inline int ts_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                                    Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = ts_pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = (unsigned)cluster_x;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

static inline int ts_launch_status() {
  cudaError_t e = cudaGetLastError();
  return (int)e;
}

__device__ __forceinline__ float ts_to_float(float x) { return x; }
__device__ __forceinline__ float ts_to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T ts_from_float(float x);
template <>
__device__ __forceinline__ float ts_from_float<float>(float x) {
  return x;
}
template <>
__device__ __forceinline__ __nv_bfloat16 ts_from_float<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float ts_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float ts_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float ts_block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = ts_warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = ts_warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  float r = scratch[32];
  __syncthreads();
  return r;
}
