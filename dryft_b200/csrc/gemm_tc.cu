// Prefill matrix product on the 5th-generation tensor cores:  C[M,N] = A[M,K] * W[N,K]^T, bfloat16
// operands, 32-bit accumulation in tensor memory, with the layer's element-wise work fused into the
// epilogue.  It stands where hari495/dryft calls cuBLAS through F.linear in its prefill
// (engine/dryft_qwen3/model.py:153,179,180) followed by separate kernels for the residual add
// (kernels/rmsnorm.py:34) and SiLU*mul (kernels/silu_mul.py:23-32).
//
// One block computes a 128 x 256 tile of C.  Six warps, three roles:
//   warp 4, one thread   producer: TMA (cp.async.bulk.tensor.2d) brings 128 x 64 of A and 256 x 64 of W per
//                        k block into a ring of shared-memory stages, 128-byte swizzled, completion
//                        counted on the stage's "full" mbarrier;
//   warp 5, one thread   issues tcgen05.mma (cta_group::1, M 128, N 256, K 16; four per k block) reading
//                        the stages through shared-memory descriptors and accumulating into 256 columns
//                        of tensor memory; tcgen05.commit frees a stage ("empty" mbarrier) when the MMAs
//                        that read it are done, and at the end signals the accumulator ("done" mbarrier);
//   warps 0-3            epilogue: tcgen05.ld brings the accumulator rows to registers (warp w owns TMEM
//                        lanes 32w..32w+31 = tile rows), which are rounded and stored, or added into the
//                        residual stream in place, or — with gate rows and the matching up rows of W
//                        loaded side by side as the tile's two halves — turned into silu(gate) * up.
//
// Every mbarrier wait is bounded: after about a second the waiter raises *err, and every role leaves
// its loop; the block then waits (bounded) for copies it may still have in flight, frees its tensor
// memory and returns.  No block waits on another block.  TMA loads use no cluster multicast.
//
// Requires K % 64 == 0 and 16-byte aligned rows.  M and N are arbitrary (TMA zero-fills out-of-range
// rows; stores are guarded).
#include "common.cuh"
#include <cuda.h>

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;            // 16 KB
constexpr int B_BYTES = BN * BK * 2;            // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 48 KB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 256;
constexpr long long WAIT_CYCLES = 2000000000LL;  // about a second: the bound of every mbarrier wait

enum Mode { STORE_BF16 = 0, RESIDUAL = 2, SILU = 3 };

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(void* bar, unsigned parity) {
  unsigned ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false (and *err raised) when the phase did not complete within WAIT_CYCLES.
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, int* err) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > WAIT_CYCLES) {
      if (err) atomicExch(err, 1);
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// K-major operand tile in shared memory, 128-byte swizzle: rows of 64 bf16 (128 bytes), 8-row groups
// 1024 bytes apart.  Descriptor fields: start address >> 4, leading byte offset 1 (unused for swizzled
// K-major), stride byte offset 1024 >> 4, version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ unsigned long long umma_desc(const void* smem_tile) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_u32(smem_tile) & 0x3FFFF) >> 4);
  d |= (unsigned long long)1 << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
// Instruction descriptor of kind::f16: D fp32, A and B bf16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);

__device__ __forceinline__ void umma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
               "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float bfr(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                             const __grid_constant__ CUtensorMap map_w, bf16* C, int ldc,
                                                             int M, int N, int K, int* err) {
  extern __shared__ unsigned char smem_raw[];
  // stages must sit on a 1024-byte boundary (the swizzle pattern repeats every 1024 bytes)
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned long long* full = reinterpret_cast<unsigned long long*>(stages + STAGES * STAGE_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* done = empty + STAGES;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(done + 1);
  __shared__ int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM;
  // SILU: the tile's output columns are j0..j0+127; its W rows are gate rows j0.. and up rows N + j0..
  const int n0 = MODE == SILU ? blockIdx.x * (BN / 2) : blockIdx.x * BN;
  const int n_k = K / BK;

  if (threadIdx.x == 0) {
    failed = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {  // the MMA warp owns the tensor-memory allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      // ---- producer ----
      for (int kb = 0; kb < n_k; ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES && !mbar_wait(&empty[s], (unsigned)(((kb / STAGES) - 1) & 1), err)) { failed = 1; break; }
        if (*(volatile int*)&failed) break;
        unsigned char* st = stages + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        tma_load_2d(st, &map_a, kb * BK, m0, &full[s]);
        if (MODE == SILU) {
          tma_load_2d(st + A_BYTES, &map_w, kb * BK, n0, &full[s]);                    // 128 gate rows
          tma_load_2d(st + A_BYTES + B_BYTES / 2, &map_w, kb * BK, N + n0, &full[s]);  // the matching up rows
        } else {
          tma_load_2d(st + A_BYTES, &map_w, kb * BK, n0, &full[s]);
          tma_load_2d(st + A_BYTES + B_BYTES / 2, &map_w, kb * BK, n0 + BN / 2, &full[s]);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ---- MMA issuer ----
      for (int kb = 0; kb < n_k; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(&full[s], (unsigned)((kb / STAGES) & 1), err)) { failed = 1; break; }
        if (*(volatile int*)&failed) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned char* st = stages + (size_t)s * STAGE_BYTES;
        const unsigned long long a_desc = umma_desc(st), b_desc = umma_desc(st + A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)  // advance 16 elements = 32 bytes = 2 descriptor units inside the swizzle row
          umma(tmem, a_desc + 2 * k, b_desc + 2 * k, (kb | k) != 0);
        umma_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
      }
      umma_commit(done);         // the accumulator is complete once every MMA issued so far is
    }
  } else {
    // ---- epilogue: warp w owns tile rows 32w .. 32w+31 ----
    const bool ok = mbar_wait(done, 0, err);
    if (!ok) failed = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int row = m0 + warp * 32 + lane;
    const unsigned lane_base = tmem + ((unsigned)(warp * 32) << 16);
    if (ok) {
      if (MODE == SILU) {
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          float gt[32], up[32];
          tmem_ld32(lane_base + c, gt);
          tmem_ld32(lane_base + BN / 2 + c, up);
          if (row < M) {
            bf16* dst = C + (size_t)row * ldc + n0 + c;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              if (n0 + c + i < N) {  // N (the intermediate size) is even: pairs never straddle the edge
                const float g0 = bfr(gt[i]), g1 = bfr(gt[i + 1]);
                const float s0 = bfr(g0 / (1.f + expf(-g0))), s1 = bfr(g1 / (1.f + expf(-g1)));
                *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(s0 * bfr(up[i]), s1 * bfr(up[i + 1]));
              }
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          float v[32];
          tmem_ld32(lane_base + c, v);
          if (row < M && n0 + c < N) {
            bf16* dst = C + (size_t)row * ldc + n0 + c;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              if (n0 + c + i < N) {
                float a = v[i], b = v[i + 1];
                if (MODE == RESIDUAL) {
                  const __nv_bfloat162 old = *reinterpret_cast<const __nv_bfloat162*>(dst + i);
                  a = __bfloat162float(old.x) + bfr(a);
                  b = __bfloat162float(old.y) + bfr(b);
                }
                *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(a, b);
              }
            }
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }

  __syncthreads();
  if (failed) {
    // a wait ran out: copies may still be in flight into this block's shared memory; give them a
    // bounded time to land before the block (and its shared memory) goes away
    if (threadIdx.x == 0) {
      const long long t0 = clock64();
      for (int s = 0; s < STAGES; ++s)
        while (!mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1) && clock64() - t0 < WAIT_CYCLES) {}
    }
    __syncthreads();
  }
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}
// [rows, K] bf16 row-major, boxes of 64 (k) x box_rows, 128-byte swizzle, zero fill outside
int make_map(CUtensorMap* map, const void* base, unsigned long long rows, unsigned long long K, unsigned box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return DRYFT_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K * 2};
  cuuint32_t box[2] = {BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : DRYFT_ERR_UNSUPPORTED;
}

template <int MODE>
int launch(const void* A, const void* W, void* C, int ldc, int M, int N, int K, int* err, cudaStream_t st) {
  CUtensorMap map_a, map_w;
  const unsigned long long w_rows = MODE == SILU ? 2ull * N : (unsigned long long)N;
  int rc = make_map(&map_a, A, M, K, BM);
  if (rc) return rc;
  rc = make_map(&map_w, W, w_rows, K, BN / 2);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int tile_n = MODE == SILU ? BN / 2 : BN;
  dim3 grid((N + tile_n - 1) / tile_n, (M + BM - 1) / BM);
  gemm_tc_kernel<MODE><<<grid, THREADS, SMEM_BYTES, st>>>(map_a, map_w, (bf16*)C, ldc, M, N, K, err);
  return launch_status();
}
}  // namespace

// mode: 0 store bf16 (C[M,N]); 2 residual (C is the stream x[M,N], updated in place x += A W^T);
//       3 SiLU*mul (W has 2N rows: N gate rows then N up rows; C[M,N] = silu(gate) * up).
// err: device int raised to 1 if a bounded wait inside the kernel ran out.
DRYFT_API int dryft_gemm_tc(const void* A, const void* W, void* C, int ldc, int mode, int M, int N, int K, int* err,
                            cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % BK || (ldc & 1) || (N & 1)) return DRYFT_ERR_UNSUPPORTED;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)C & 3)) return DRYFT_ERR_UNSUPPORTED;
  switch (mode) {
    case STORE_BF16: return launch<STORE_BF16>(A, W, C, ldc, M, N, K, err, st);
    case RESIDUAL: return launch<RESIDUAL>(A, W, C, ldc, M, N, K, err, st);
    case SILU: return launch<SILU>(A, W, C, ldc, M, N, K, err, st);
  }
  return DRYFT_ERR_UNSUPPORTED;
}
