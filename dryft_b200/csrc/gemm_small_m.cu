// Decode matrix product  C[M,N] = A[M,K] * W[N,K]^T  for a handful of rows (M <= 16): bfloat16
// operands, 32-bit accumulation on the tensor cores, every weight byte read from HBM exactly once.
// It stands where hari495/dryft calls cuBLAS through F.linear in its decode step
// (engine/dryft_qwen3/model.py:237,258,260,261); at these M the product is bound by streaming W,
// and what surrounds it in the layer is fused into it so that a decode layer is five launches:
//
//   norm prologue   A is the residual stream x; the kernel applies RMSNorm to it on the fly,
//                   a[m,k] = T(T(x[m,k] * inv[m]) * w[k]) (model.py:28-32), with inv[m] from per-row sums
//                   of squares that the PREVIOUS product's epilogue left behind (ss_in, summed in a
//                   fixed order).  Replaces the separate (add+)RMSNorm launch (kernels/rmsnorm.py:21-39).
//   residual epilogue   x[m,n] = T(x[m,n] + T(sum)) in place (rmsnorm.py:34), and the sum of squares of
//                   the new x over this block's 16 columns goes to ss_out[block][m] for the next norm.
//   SiLU*mul epilogue   W holds gate rows then up rows (weights.py:98-100); a block takes 8 gate rows and
//                   the 8 matching up rows, and writes act = T(T(silu(g)) * u) (kernels/silu_mul.py:29-32).
//
// A block of 8 warps takes 16 rows of W at a time (blocks are persistent: at most two per SM, each
// walking over every grid-th tile, so the norm prologue is paid once per block and the weight stream
// runs on across tiles).  The warps split K into 8 contiguous ranges; each streams
// its part of the 16 weight rows straight into registers with 16-byte loads that bypass L1, four
// 32-wide k steps in flight and the next four already requested, and feeds mma.sync.m16n8k16 with W
// as the 16 x 16 operand and 8 batch rows as the 16 x 8 operand.  The k index is permuted identically
// in both operands so that every thread's fragment is one contiguous 16-byte piece.  With the norm
// prologue the normalised activations are made once per block and stay in shared memory (padded so
// that the fragment reads are conflict-free); otherwise they are read through L1.  The 8 partial sums
// are added in warp order through shared memory, so a row's result depends neither on the other rows
// nor on M.
//
// Launch overlap: the kernel may be launched as a programmatic dependent of the launch before it.  It
// requests its first weights, which depend on nothing, and only then waits for the earlier grid
// (griddepcontrol.wait) before it touches activations; it lets its own dependents launch at once.
//
// Requires K % 16 == 0, M <= 16 (checked by the launcher, which otherwise refuses).  No block waits on
// another block of its grid; there is no spin in this file.
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int ROWS = 16;            // weight rows per block
constexpr int U = 4;                // k steps of 32 per request group
constexpr int SS_STRIDE = 64;       // floats per block of ss_in / ss_out

enum Mode { STORE_BF16 = 0, STORE_F32 = 1, RESIDUAL = 2, SILU = 3 };

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
__device__ __forceinline__ float bfr(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// row stride (elements) of the resident activations: bytes = 64 mod 128, so that the eight 16-byte
// fragment reads of a quarter-warp (rows g, g+1; pieces t = 0..3) fall into distinct banks
__host__ __device__ inline int resident_stride(int K) { return K + ((64 - (K * 2) % 128 + 128) % 128) / 2; }

template <int MB, int MODE, bool NORM>
__global__ void __launch_bounds__(THREADS) gemm_small_m_kernel(
    const bf16* __restrict__ A, int lda, const bf16* __restrict__ W, void* C, int ldc, int M, int N, int K,
    const float* __restrict__ norm_w, const float* __restrict__ ss_in, int ss_parts, float eps, float* __restrict__ ss_out) {
  constexpr int MP = 8 * MB;
  constexpr int RED = WARPS * ROWS * (MP + 1);
  extern __shared__ __align__(16) unsigned char smem[];
  // two buffers of [WARPS][ROWS][MP + 1] partial sums, 64 floats of inv, then the resident activations
  float* red_base = reinterpret_cast<float*>(smem);
  float* inv_s = red_base + 2 * RED;
  bf16* a_res = reinterpret_cast<bf16*>(inv_s + SS_STRIDE);
  const int KA = resident_stride(K);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int g = lane >> 2, t = lane & 3;
  constexpr int TILE_N = MODE == SILU ? 8 : ROWS;   // outputs per tile
  const int n_tiles = (N + TILE_N - 1) / TILE_N;

  pdl_launch_dependents();

  const int steps = (K + 31) / 32;
  const int s_begin = (int)(((long long)steps * warp) / WARPS);
  const int s_end = (int)(((long long)steps * (warp + 1)) / WARPS);

  uint4 wa[U], wb[U], na[U], nb[U];
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // this thread's two weight rows of a tile (tile rows g and g+8; SILU: gate row and matching up row)
  auto load_group = [&](int tile, int s, uint4 (&ra)[U], uint4 (&rb)[U]) {
    const int n0 = tile * TILE_N;
    int r0, r1;
    bool ok0, ok1;
    if (MODE == SILU) { r0 = n0 + g; r1 = N + n0 + g; ok0 = ok1 = n0 + g < N; }
    else { r0 = n0 + g; r1 = n0 + g + 8; ok0 = r0 < N; ok1 = r1 < N; }
    const bf16* w0 = W + (size_t)(ok0 ? r0 : 0) * K;
    const bf16* w1 = W + (size_t)(ok1 ? r1 : 0) * K;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (s + u) * 32 + t * 8;
      const bool in = (s + u) < s_end && k < K;
      ra[u] = (in && ok0) ? ld_stream(w0 + k) : zero;
      rb[u] = (in && ok1) ? ld_stream(w1 + k) : zero;
    }
  };
  int tile = blockIdx.x;
  if (tile < n_tiles && s_begin < s_end) load_group(tile, s_begin, wa, wb);  // weights depend on no earlier launch

  pdl_wait();  // from here on, what earlier launches wrote (activations, sums of squares) is visible

  if (NORM) {
    // inv[m] = rsqrt(mean(x[m]^2) + eps), sums of squares added in block order; then the normalised
    // rows a[m,k] = T(T(x[m,k] * inv[m]) * w[k]) go to shared memory once per block (rows >= M are zero)
    if (tid < MP) {
      float s = 0.f;
      if (tid < M)
        for (int p = 0; p < ss_parts; ++p) s += ld_prev(ss_in + p * SS_STRIDE + tid);
      inv_s[tid] = rsqrtf(s / (float)K + eps);
    }
    __syncthreads();
    const int chunks = K / 8;
    for (int i = tid; i < MP * chunks; i += THREADS) {
      const int m = i / chunks, c = i - m * chunks;
      uint4 out = zero;
      if (m < M) {
        const uint4 raw = ld_prev(reinterpret_cast<const uint4*>(A + (size_t)m * lda + c * 8));
        const float4 wv0 = __ldg(reinterpret_cast<const float4*>(norm_w + c * 8));
        const float4 wv1 = __ldg(reinterpret_cast<const float4*>(norm_w + c * 8 + 4));
        const float wv[8] = {wv0.x, wv0.y, wv0.z, wv0.w, wv1.x, wv1.y, wv1.z, wv1.w};
        const bf16* e = reinterpret_cast<const bf16*>(&raw);
        const float inv = inv_s[m];
        __align__(16) bf16 o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(bfr(__bfloat162float(e[j]) * inv) * wv[j]);
        out = *reinterpret_cast<const uint4*>(o);
      }
      *reinterpret_cast<uint4*>(a_res + (size_t)m * KA + c * 8) = out;
    }
    __syncthreads();
  }

  int buf = 0;
  for (; tile < n_tiles; tile += gridDim.x) {
    float acc[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mb][i] = 0.f;

    for (int s = s_begin; s < s_end; s += U) {
      // request what comes next: the rest of this tile, else the start of this block's next tile
      if (s + U < s_end) load_group(tile, s + U, na, nb);
      else if (tile + (int)gridDim.x < n_tiles) load_group(tile + gridDim.x, s_begin, na, nb);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = (s + u) * 32 + t * 8;
        const bool in = (s + u) < s_end && k < K;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const int m = mb * 8 + g;
          uint4 a = zero;
          if (in) {
            if (NORM) a = *reinterpret_cast<const uint4*>(a_res + (size_t)m * KA + k);
            else if (m < M) a = ld_prev(reinterpret_cast<const uint4*>(A + (size_t)m * lda + k));
          }
          mma16816(acc[mb], wa[u].x, wb[u].x, wa[u].y, wb[u].y, a.x, a.y);
          mma16816(acc[mb], wa[u].z, wb[u].z, wa[u].w, wb[u].w, a.z, a.w);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) { wa[u] = na[u]; wb[u] = nb[u]; }
    }

    // partial sums -> shared memory (two buffers, so one barrier per tile is enough)
    float* red = red_base + buf * RED;
    buf ^= 1;
    auto red_at = [&](int w, int row, int m) -> float& { return red[(w * ROWS + row) * (MP + 1) + m]; };
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      red_at(warp, g, mb * 8 + 2 * t) = acc[mb][0];
      red_at(warp, g, mb * 8 + 2 * t + 1) = acc[mb][1];
      red_at(warp, g + 8, mb * 8 + 2 * t) = acc[mb][2];
      red_at(warp, g + 8, mb * 8 + 2 * t + 1) = acc[mb][3];
    }
    __syncthreads();
    auto total = [&](int row, int m) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) s += red_at(w, row, m);
      return s;
    };
    const int n0 = tile * TILE_N;
    if (MODE == SILU) {
      bf16* out = reinterpret_cast<bf16*>(C);
      for (int i = tid; i < 8 * MP; i += THREADS) {
        const int j = i & 7, m = i >> 3;
        if (m >= M || n0 + j >= N) continue;
        const float gt = bfr(total(j, m)), up = bfr(total(j + 8, m));
        const float s = bfr(gt / (1.f + expf(-gt)));
        out[(size_t)m * ldc + n0 + j] = __float2bfloat16_rn(s * up);
      }
    } else if (MODE == RESIDUAL) {
      bf16* x = reinterpret_cast<bf16*>(C);
      // thread -> (row = i % 16, m = i / 16): a half-warp covers the 16 columns of one batch row
      for (int i = tid; i < ROWS * MP; i += THREADS) {
        const int row = i & 15, m = i >> 4;
        const int n = n0 + row;
        float sq = 0.f;
        if (m < M && n < N) {
          const float v = bfr(ld_prev_bf16(x + (size_t)m * ldc + n) + bfr(total(row, m)));
          x[(size_t)m * ldc + n] = __float2bfloat16_rn(v);
          sq = v * v;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (ss_out && row == 0 && m < M) ss_out[(size_t)tile * SS_STRIDE + m] = sq;
      }
    } else {
      for (int i = tid; i < ROWS * MP; i += THREADS) {
        const int row = i & 15, m = i >> 4;
        const int n = n0 + row;
        if (m >= M || n >= N) continue;
        const float s = total(row, m);
        if (MODE == STORE_F32) reinterpret_cast<float*>(C)[(size_t)m * ldc + n] = s;
        else reinterpret_cast<bf16*>(C)[(size_t)m * ldc + n] = __float2bfloat16_rn(s);
      }
    }
  }
}

template <int MB, int MODE, bool NORM>
int launch3(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K, const float* norm_w,
            const float* ss_in, int ss_parts, float eps, float* ss_out, int pdl, cudaStream_t st) {
  constexpr int MP = 8 * MB;
  size_t smem = (size_t)2 * WARPS * ROWS * (MP + 1) * 4 + SS_STRIDE * 4;
  if (NORM) smem += (size_t)MP * resident_stride(K) * 2;
  if (smem > 200 * 1024) return DRYFT_ERR_UNSUPPORTED;
  static size_t attr_bytes = 48 * 1024;  // per instantiation; raised by an eager launch before any capture
  if (smem > attr_bytes) {
    cudaError_t e = cudaFuncSetAttribute(gemm_small_m_kernel<MB, MODE, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_bytes = smem;
  }
  // persistent blocks: two per SM at most, each taking every grid-th tile; the grid is chosen so
  // that the tiles divide as evenly as they can
  static int max_blocks = 0;
  if (max_blocks == 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    max_blocks = 2 * (sms > 0 ? sms : 148);
  }
  const int n_tiles = MODE == SILU ? (N + 7) / 8 : (N + ROWS - 1) / ROWS;
  const int rounds = (n_tiles + max_blocks - 1) / max_blocks;
  const unsigned blocks = (unsigned)((n_tiles + rounds - 1) / rounds);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_small_m_kernel<MB, MODE, NORM>, (const bf16*)A, lda, (const bf16*)W, C, ldc, M,
                                     N, K, norm_w, ss_in, ss_parts, eps, ss_out);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}
template <int MB, int MODE>
int launch2(bool norm, const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K, const float* norm_w,
            const float* ss_in, int ss_parts, float eps, float* ss_out, int pdl, cudaStream_t st) {
  return norm ? launch3<MB, MODE, true>(A, lda, W, C, ldc, M, N, K, norm_w, ss_in, ss_parts, eps, ss_out, pdl, st)
              : launch3<MB, MODE, false>(A, lda, W, C, ldc, M, N, K, norm_w, ss_in, ss_parts, eps, ss_out, pdl, st);
}
template <int MB>
int launch1(int mode, bool norm, const void* A, int lda, const void* W, void* C, int ldc, int M, int N, int K,
            const float* norm_w, const float* ss_in, int ss_parts, float eps, float* ss_out, int pdl, cudaStream_t st) {
  switch (mode) {
    case STORE_BF16: return launch2<MB, STORE_BF16>(norm, A, lda, W, C, ldc, M, N, K, norm_w, ss_in, ss_parts, eps, ss_out, pdl, st);
    case STORE_F32: return launch2<MB, STORE_F32>(norm, A, lda, W, C, ldc, M, N, K, norm_w, ss_in, ss_parts, eps, ss_out, pdl, st);
    case RESIDUAL: return launch2<MB, RESIDUAL>(norm, A, lda, W, C, ldc, M, N, K, norm_w, ss_in, ss_parts, eps, ss_out, pdl, st);
    case SILU: return launch2<MB, SILU>(norm, A, lda, W, C, ldc, M, N, K, norm_w, ss_in, ss_parts, eps, ss_out, pdl, st);
  }
  return DRYFT_ERR_UNSUPPORTED;
}
}  // namespace

// mode: 0 store bf16, 1 store f32, 2 residual (C is x, updated in place; ss_out optional),
//       3 SiLU*mul (W has 2N rows: N gate rows then N up rows; C is [M, N] bf16).
// norm_w != null selects the norm prologue: A is the residual stream, ss_in [ss_parts][64] its
// per-row sums of squares split over ss_parts blocks, eps the norm's epsilon.
// pdl != 0 launches the kernel as a programmatic dependent of the launch before it in the stream.
DRYFT_API int dryft_gemm_small_m(const void* A, int lda, const void* W, void* C, int ldc, int mode, int M, int N, int K,
                                 const float* norm_w, const float* ss_in, int ss_parts, float eps, float* ss_out,
                                 int pdl, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 15) || (lda & 7) || M > 16) return DRYFT_ERR_UNSUPPORTED;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return DRYFT_ERR_UNSUPPORTED;
  const bool norm = norm_w != nullptr;
  if (norm && (!ss_in || ss_parts <= 0 || ((uintptr_t)norm_w & 15))) return DRYFT_ERR_UNSUPPORTED;
  if (M <= 8) return launch1<1>(mode, norm, A, lda, W, C, ldc, M, N, K, norm_w, ss_in, ss_parts, eps, ss_out, pdl, st);
  return launch1<2>(mode, norm, A, lda, W, C, ldc, M, N, K, norm_w, ss_in, ss_parts, eps, ss_out, pdl, st);
}

// Sum of squares of each row of x [M, H] (bf16) -> ss[0][m]: the entry point of the chain of norm
// prologues (the embedding's output has no product before it).  With a norm weight w [H] it also leaves
// the weighted activations xw = T(x * w) for a product that scales by the norm's factor in its epilogue.
__global__ void row_sumsq_kernel(const bf16* __restrict__ x, int hidden, float* __restrict__ ss, const float* __restrict__ w,
                                 bf16* __restrict__ xw) {
  __shared__ float scratch[33];
  const int m = blockIdx.x;
  float s = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = __bfloat162float(x[(size_t)m * hidden + i]);
    s += v * v;
    if (xw) xw[(size_t)m * hidden + i] = __float2bfloat16_rn(v * w[i]);
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) ss[m] = s;
}
DRYFT_API int dryft_row_sumsq(const void* x, int rows, int hidden, float* ss, const float* w, void* xw, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (rows > SS_STRIDE || ((w != nullptr) != (xw != nullptr))) return DRYFT_ERR_UNSUPPORTED;
  row_sumsq_kernel<<<rows, 256, 0, st>>>((const bf16*)x, hidden, ss, w, (bf16*)xw);
  return launch_status();
}
