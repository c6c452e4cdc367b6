// Sampling from float32 logits: greedy argmax, or the reference's exponential race.
//
// Reference (engine/generation/sampler.py:11-16): probs = softmax(logits / T);
// token = argmax(probs / max(E, 1e-10)) with E ~ Exp(1) drawn per entry.  Dividing by
// the softmax's sum and taking a log change no argmax, so the kernel compares
// logits / T - log(max(E, 1e-10)) and never forms the softmax.  E comes from a counter
// hash of (key, vocabulary index); the host makes `key` from (seed, request, position),
// so a request draws the same noise however it was batched, cut or recomputed.
// Temperature 0 is greedy.  Ties go to the lowest index.
#include "common.cuh"

__device__ __forceinline__ uint64_t ts_mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// Exp(1) noise for (key, index): u in (0, 1) from 24 bits, E = -log(u).
__device__ __forceinline__ float ts_exp_noise(uint64_t key, int index) {
  const uint64_t h = ts_mix64(key ^ ts_mix64((uint64_t)(uint32_t)index));
  const float u = ((float)(uint32_t)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
  return -logf(u);
}

__global__ void sample_kernel(const float* __restrict__ logits, int V, long long row_stride,
                              const float* __restrict__ temperature,
                              const unsigned long long* __restrict__ keys, int* __restrict__ out) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const float temp = temperature[r];
  const bool greedy = !(temp > 1e-10f);
  const uint64_t key = keys ? keys[r] : 0ull;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = row[i];
    if (!greedy) v = v / temp - logf(fmaxf(ts_exp_noise(key, i), 1e-10f));
    if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) {
      bv = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
      bv = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    best_v[warp] = bv;
    best_i[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (blockDim.x + 31) >> 5;
    bv = lane < nwarps ? best_v[lane] : -INFINITY;
    bi = lane < nwarps ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) out[r] = bi;
  }
}

TS_EXPORT int ts_sample(const float* logits, int V, long long row_stride, const float* temperature,
                        const unsigned long long* keys, int* out, int R, void* stream) {
  if (R <= 0) return 0;
  if (V <= 0 || row_stride < V) return TS_ERR_BAD_ARGUMENT;
  int threads = V >= 8192 ? 1024 : (V >= 1024 ? 256 : 64);
  sample_kernel<<<R, threads, 0, (cudaStream_t)stream>>>(logits, V, row_stride, temperature, keys, out);
  return ts_launch_status();
}
