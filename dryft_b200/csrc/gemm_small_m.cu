// Decode matrix product  C[M,N] = A[M,K] * W[N,K]^T  for a handful of rows (M <= 64): bfloat16
// operands, 32-bit accumulation on the tensor cores, every weight byte read from HBM exactly once.
// It stands where hari495/dryft calls cuBLAS through F.linear in its decode step
// (engine/dryft_qwen3/model.py:237,258,260,261); at these M the product is bound by streaming W.
//
// One block of 8 warps owns 16 rows of W (16 outputs per batch row).  The warps split K into 8
// contiguous ranges; each streams its part of the 16 weight rows with 16-byte loads, four 32-wide k
// steps in flight and the next four prefetched, and feeds mma.sync.m16n8k16 with W as the 16 x 16
// operand and the batch rows as the 16 x 8 operand (8 batch rows per instruction, M padded to a
// multiple of 8).  The k index is permuted identically in both operands so that every thread's
// fragment is one contiguous 16-byte load.  The 8 partial sums are added in warp order through
// shared memory, so a row's result depends neither on the other rows nor on M.
//
// Requires K % 8 == 0 and 16-byte aligned rows (checked by the launcher).  No block waits on
// another; there is no spin in this file.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;
constexpr int ROWS = 16;   // weight rows (outputs) per block
constexpr int U = 4;       // k steps of 32 per prefetch group

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MB, bool OUT_F32>
__global__ void __launch_bounds__(WARPS * 32) gemm_small_m_kernel(const __nv_bfloat16* __restrict__ A, int lda,
                                                                  const __nv_bfloat16* __restrict__ W, void* __restrict__ C,
                                                                  int ldc, int M, int N, int K) {
  __shared__ float red[WARPS][ROWS][8 * MB + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * ROWS;
  const int r0 = n0 + g, r1 = n0 + g + 8;
  const __nv_bfloat16* w0 = W + (size_t)min(r0, N - 1) * K;
  const __nv_bfloat16* w1 = W + (size_t)min(r1, N - 1) * K;
  const bool ok0 = r0 < N, ok1 = r1 < N;

  float acc[MB][4];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[mb][i] = 0.f;

  const int steps = (K + 31) / 32;
  const int s_begin = (int)(((long long)steps * warp) / WARPS);
  const int s_end = (int)(((long long)steps * (warp + 1)) / WARPS);

  uint4 wa[U], wb[U], na[U], nb[U];
  const uint4 zero = make_uint4(0, 0, 0, 0);
  auto load_group = [&](int s, uint4 (&ra)[U], uint4 (&rb)[U]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (s + u) * 32 + t * 8;
      const bool in = (s + u) < s_end && k < K;
      ra[u] = (in && ok0) ? ld_stream(w0 + k) : zero;
      rb[u] = (in && ok1) ? ld_stream(w1 + k) : zero;
    }
  };
  if (s_begin < s_end) load_group(s_begin, wa, wb);
  for (int s = s_begin; s < s_end; s += U) {
    if (s + U < s_end) load_group(s + U, na, nb);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (s + u) * 32 + t * 8;
      const bool in = (s + u) < s_end && k < K;
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        const int m = mb * 8 + g;
        uint4 a = zero;
        if (in && m < M) a = __ldg(reinterpret_cast<const uint4*>(A + (size_t)m * lda + k));
        mma16816(acc[mb], wa[u].x, wb[u].x, wa[u].y, wb[u].y, a.x, a.y);
        mma16816(acc[mb], wa[u].z, wb[u].z, wa[u].w, wb[u].w, a.z, a.w);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) { wa[u] = na[u]; wb[u] = nb[u]; }
  }

  // accumulator (row g | g+8 of the 16 weight rows, batch column mb*8 + 2t | 2t+1)
#pragma unroll
  for (int mb = 0; mb < MB; ++mb) {
    red[warp][g][mb * 8 + 2 * t] = acc[mb][0];
    red[warp][g][mb * 8 + 2 * t + 1] = acc[mb][1];
    red[warp][g + 8][mb * 8 + 2 * t] = acc[mb][2];
    red[warp][g + 8][mb * 8 + 2 * t + 1] = acc[mb][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < ROWS * 8 * MB; i += WARPS * 32) {
    const int row = i % ROWS, m = i / ROWS;  // consecutive threads -> consecutive n: contiguous stores
    const int n = n0 + row;
    if (m >= M || n >= N) continue;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) s += red[w][row][m];
    if (OUT_F32) reinterpret_cast<float*>(C)[(size_t)m * ldc + n] = s;
    else reinterpret_cast<__nv_bfloat16*>(C)[(size_t)m * ldc + n] = __float2bfloat16_rn(s);
  }
}

template <int MB>
int launch_mb(const void* A, int lda, const void* W, void* C, int ldc, int out_f32, int M, int N, int K, cudaStream_t st) {
  const unsigned blocks = (unsigned)((N + ROWS - 1) / ROWS);
  if (out_f32)
    gemm_small_m_kernel<MB, true><<<blocks, WARPS * 32, 0, st>>>((const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, C, ldc, M, N, K);
  else
    gemm_small_m_kernel<MB, false><<<blocks, WARPS * 32, 0, st>>>((const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, C, ldc, M, N, K);
  return launch_status();
}
}  // namespace

DRYFT_API int dryft_gemm_small_m(const void* A, int lda, const void* W, void* C, int ldc, int out_f32, int M, int N, int K,
                                 cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (lda & 7) || M > 64) return DRYFT_ERR_UNSUPPORTED;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return DRYFT_ERR_UNSUPPORTED;
  if (M <= 8) return launch_mb<1>(A, lda, W, C, ldc, out_f32, M, N, K, st);
  if (M <= 16) return launch_mb<2>(A, lda, W, C, ldc, out_f32, M, N, K, st);
  if (M <= 32) return launch_mb<4>(A, lda, W, C, ldc, out_f32, M, N, K, st);
  return launch_mb<8>(A, lda, W, C, ldc, out_f32, M, N, K, st);
}
