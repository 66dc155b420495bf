// True 32-bit matrix product  C[M,N] = A[M,K] * W[N,K]^T  on the CUDA cores: fp32 operands,
// fp32 fused multiply-adds, no tensor-core (TF32) mode.  It stands where hari495/dryft calls
// F.linear with TF32 switched off (engine/engine.py:32-33; engine/dryft_qwen3/model.py:153),
// and is the matrix product of the library's 32-bit path.
//
// Each output element is accumulated over k = 0..K-1 in that order by one thread, so a row's
// result does not depend on how many other rows are in the batch: in the 32-bit path the same
// token gives bit-identical projections whether it is run alone, in a prompt or in a batch.
// Any M, N, K >= 1; lda/ldc are row strides in elements.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256) gemm_nt_f32_kernel(const float* __restrict__ A, int lda,
                                                          const float* __restrict__ W, float* __restrict__ C, int ldc,
                                                          int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, each a 4 x 4 block of C
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 x 16 tile of A and of W: 1024 elements each, 4 per thread; k is the fast index in memory
    for (int i = tid; i < BM * BK; i += 256) {
      const int r = i / BK, c = i % BK;
      const int m = m0 + r, n = n0 + r, k = k0 + c;
      As[c][r] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
      Ws[c][r] = (n < N && k < K) ? W[(size_t)n * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}
}  // namespace

DRYFT_API int dryft_gemm_nt_f32(const float* A, int lda, const float* W, float* C, int ldc, int M, int N, int K,
                                cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return DRYFT_ERR_UNSUPPORTED;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return DRYFT_ERR_UNSUPPORTED;
  gemm_nt_f32_kernel<<<grid, 256, 0, st>>>(A, lda, W, C, ldc, M, N, K);
  return launch_status();
}
