// True float32 matrix product on CUDA cores: C[M, N] = A[M, K] * W[N, K]^T.
//
// This is the float32 path's GEMM: FFMA only, no tensor cores and no reduced-precision
// mode.  Each output element is one dot product summed over k in increasing order inside
// fixed tiles, so a row's result does not depend on which other rows share the launch.
// W is row-major [out, in] as the reference's Linear weights are (engine/nn/attention.py:
// 122-135).
#include "common.cuh"

#define SG_BM 64
#define SG_BN 64
#define SG_BK 16

__global__ void __launch_bounds__(256) sgemm_nt_kernel(const float* __restrict__ A,
                                                       const float* __restrict__ W,
                                                       float* __restrict__ C, int M, int N, int K,
                                                       long long lda, long long ldw, long long ldc) {
  ts_pdl_prologue();
  __shared__ float As[SG_BK][SG_BM + 1];
  __shared__ float Ws[SG_BK][SG_BN + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += SG_BK) {
    for (int i = threadIdx.x; i < SG_BM * SG_BK; i += 256) {
      const int r = i / SG_BK, c = i % SG_BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SG_BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
    }
  }
}

TS_EXPORT int ts_sgemm_nt(const float* A, const float* W, float* C, int M, int N, int K,
                          long long lda, long long ldw, long long ldc, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || lda < K || ldw < K || ldc < N) return TS_ERR_BAD_ARGUMENT;
  dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
  if (grid.y > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  return ts_launch(sgemm_nt_kernel, grid, dim3(256), 0, (cudaStream_t)stream, A, W, C, M, N, K, lda, ldw, ldc);
}
