// Sampling from float32 logits: greedy argmax, or the reference's exponential race.
//
// Reference (engine/generation/sampler.py:11-16): probs = softmax(logits / T);
// token = argmax(probs / max(E, 1e-10)) with E ~ Exp(1) drawn per entry.  Dividing by
// the softmax's sum and taking a log change no argmax, so the kernel compares
// logits / T - ln(E) and never forms the softmax.  E = -ln(u) comes from a counter hash:
// one 64-bit hash of (key, index / 2) gives the 24-bit uniforms of the entries 2k (its top
// bits) and 2k + 1 (the 24 bits below).  u <= 1 - 2^-25 keeps E above 2.9e-8, so the
// reference's floor of 1e-10 never acts.  With ln = ln2 * lg2 the score is
// logits / T - ln2 * lg2(-lg2(u)) up to a constant that no argmax sees: two hardware
// logarithms and one hash per two entries.  The host makes `key` from (seed, request,
// position), so a request draws the same noise however it was batched, cut or recomputed.
// Temperature 0 is greedy.  Ties go to the lowest index.
#include "common.cuh"

__device__ __forceinline__ uint64_t ts_mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// The hash that the entries 2 * pair and 2 * pair + 1 of a row with this key share.  The key is a
// full hash of (seed, request, position) already (the host makes it); per pair one multiply and two
// shifts spread the pair's index over the 48 bits that are used.
__device__ __forceinline__ uint64_t ts_pair_hash(uint64_t key, uint32_t pair) {
  uint64_t z = key ^ ((uint64_t)pair * 0xD1342543DE82EF95ull);
  z ^= z >> 32;
  z *= 0x94D049BB133111EBull;
  return z ^ (z >> 29);
}

// What the race subtracts from logit / T for a 24-bit uniform number: ln2 * lg2(-lg2(u)),
// u = (bits + 0.5) / 2^24, which is ln(E) for E = -ln(u) less a constant.
__device__ __forceinline__ float ts_race_penalty(uint32_t bits24) {
  const float u = ((float)bits24 + 0.5f) * (1.0f / 16777216.0f);
  return 0.69314718056f * __log2f(-__log2f(u));
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

// Stage 1: one CTA per (chunk of the vocabulary, row) finds the best entry of its chunk.  A thread
// takes four neighbouring entries at a time (two hashes); rows whose start is 16-byte aligned are
// read four floats at once.
__global__ void sample_partial_kernel(const float* __restrict__ logits, int V, long long row_stride,
                                      const float* __restrict__ temperature,
                                      const unsigned long long* __restrict__ keys, Best* __restrict__ partial) {
  ts_pdl_prologue();
  __shared__ Best shared[32];
  const int r = blockIdx.y, chunk = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const float temp = temperature[r];
  const bool greedy = !(temp > 1e-10f);
  const float inv_temp = greedy ? 1.f : 1.f / temp;
  const uint64_t key = keys ? keys[r] : 0ull;
  const bool vector = ((uintptr_t)row & 15) == 0;
  Best best;
  best.v = -INFINITY;
  best.i = 0x7fffffff;
  const int end = min(V, (chunk + 1) * SAMPLE_CHUNK);
  for (int i0 = chunk * SAMPLE_CHUNK + threadIdx.x * 4; i0 < end; i0 += SAMPLE_THREADS * 4) {
    float v[4];
    if (vector && i0 + 3 < end) {
      const float4 f = *reinterpret_cast<const float4*>(row + i0);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = i0 + j < end ? row[i0 + j] : -INFINITY;
    }
    if (!greedy) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint64_t h = ts_pair_hash(key, (uint32_t)(i0 >> 1) + half);
        v[2 * half] = v[2 * half] * inv_temp - ts_race_penalty((uint32_t)(h >> 40));
        v[2 * half + 1] = v[2 * half + 1] * inv_temp - ts_race_penalty((uint32_t)(h >> 16) & 0xFFFFFFu);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (i0 + j < end) {
        Best cand;
        cand.v = v[j];
        cand.i = i0 + j;
        best = better(best, cand);
      }
    }
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
