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

#define SAMPLE_CHUNK 2048
#define SAMPLE_THREADS 256

struct Best {
  float v;
  int i;
};

__device__ __forceinline__ Best better(Best a, Best b) {
  // the larger value wins; on equal values the lower index; i = INT_MAX marks "nothing yet"
  if (b.i != 0x7fffffff && (a.i == 0x7fffffff || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
  return a;
}

__device__ __forceinline__ Best block_best(Best x, Best* shared /* [32] */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) shared[warp] = x;
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (blockDim.x + 31) >> 5;
    Best none;
    none.v = -INFINITY;
    none.i = 0x7fffffff;
    x = lane < nwarps ? shared[lane] : none;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best y;
      y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
      y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
      x = better(x, y);
    }
  }
  return x;  // valid in warp 0
}

// Stage 1: one CTA per (chunk of the vocabulary, row) finds the best entry of its chunk.
__global__ void sample_partial_kernel(const float* __restrict__ logits, int V, long long row_stride,
                                      const float* __restrict__ temperature,
                                      const unsigned long long* __restrict__ keys, Best* __restrict__ partial) {
  ts_pdl_prologue();
  __shared__ Best shared[32];
  const int r = blockIdx.y, chunk = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const float temp = temperature[r];
  const bool greedy = !(temp > 1e-10f);
  const uint64_t key = keys ? keys[r] : 0ull;
  Best best;
  best.v = -INFINITY;
  best.i = 0x7fffffff;
  const int end = min(V, (chunk + 1) * SAMPLE_CHUNK);
  for (int i = chunk * SAMPLE_CHUNK + threadIdx.x; i < end; i += SAMPLE_THREADS) {
    float v = row[i];
    if (!greedy) v = v / temp - logf(fmaxf(ts_exp_noise(key, i), 1e-10f));
    Best cand;
    cand.v = v;
    cand.i = i;
    best = better(best, cand);
  }
  best = block_best(best, shared);
  if (threadIdx.x == 0) partial[(size_t)r * gridDim.x + chunk] = best;
}

// Stage 2: one CTA per row picks among the chunk winners.
__global__ void sample_final_kernel(const Best* __restrict__ partial, int chunks, int* __restrict__ out) {
  ts_pdl_prologue();
  __shared__ Best shared[32];
  const int r = blockIdx.x;
  Best best;
  best.v = -INFINITY;
  best.i = 0x7fffffff;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) best = better(best, partial[(size_t)r * chunks + c]);
  best = block_best(best, shared);
  if (threadIdx.x == 0) out[r] = best.i;
}

TS_EXPORT long long ts_sample_scratch_bytes(int R, int V) {
  const long long chunks = (V + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
  return (long long)R * chunks * (long long)sizeof(Best);
}

TS_EXPORT int ts_sample(const float* logits, int V, long long row_stride, const float* temperature,
                        const unsigned long long* keys, int* out, int R, void* scratch, void* stream) {
  if (R <= 0) return 0;
  if (V <= 0 || row_stride < V || scratch == nullptr) return TS_ERR_BAD_ARGUMENT;
  if (R > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  const int chunks = (V + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
  cudaStream_t s = (cudaStream_t)stream;
  int status = ts_launch(sample_partial_kernel, dim3(chunks, R), dim3(SAMPLE_THREADS), 0, s, logits, V, row_stride, temperature, keys, (Best*)scratch);
  if (status != 0) return status;
  return ts_launch(sample_final_kernel, dim3(R), dim3(128), 0, s, (const Best*)scratch, chunks, out);
}
