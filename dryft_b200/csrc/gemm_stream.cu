// Decode matrix product on the 5th-generation tensor cores, built to stream weights:
//
//   C[M,N] = A[M,K] * W[N,K]^T,  M <= 64 rows of activations, bfloat16 operands, 32-bit accumulation,
//   every weight byte read from HBM exactly once (hari495/dryft: cuBLAS via F.linear,
//   engine/dryft_qwen3/model.py:237,258,260,261), with the layer's element-wise work fused in:
//   norm prologue (kernels/rmsnorm.py:21-39), residual epilogue with sums of squares for the next
//   norm (rmsnorm.py:34), SiLU*mul epilogue (kernels/silu_mul.py:29-32; weights.py:98-100).
//
// The product is computed transposed: a tile is 128 rows of W (the M = 128 operand of tcgen05.mma,
// K-major, 128-byte swizzle, brought in by TMA) against the NB = 16 / 32 / 64 padded activation rows
// (the N operand, K-major, also by TMA; rows beyond M are zero-filled), accumulating a 128 x NB tile in
// tensor memory.  What is in flight lives in a ring of shared-memory stages, not in registers, so
// several blocks, also of consecutive launches, sit on an SM with their rings full: a launch may be a
// programmatic dependent of the one before it, requests its first weights at once and only then waits.
//
// Few tiles of 128 rows cover a product (20 for 2,560 outputs), so K is split over the blocks of a
// thread-block cluster (1, 2, 4 or 8): each block leaves its partial tile in its own shared memory,
// and after a cluster barrier every block adds one slice of the tile's rows over all ranks, in rank
// order (through distributed shared memory), and finishes that slice: rounds and stores it, or adds it
// into the residual stream and leaves its sums of squares, or turns gate and up rows into
// silu(gate) * up.  A result depends neither on the other rows nor on M.
//
// Six warps: warp 0 (one thread) TMA producer; warp 1 (one thread) issues tcgen05.mma; warps 2-5 the
// 128 threads that normalise the activation stages in place (norm prologue) and run the epilogue.
// Every mbarrier wait is bounded by a clock (about a second): a waiter that gives up raises *err and
// every role leaves its loop; the block still passes both cluster barriers (so no block of the cluster
// waits for it), lets its own copies land, frees its tensor memory and returns.  Blocks of different
// clusters never wait on one another.  No TMA load uses cluster multicast.
//
// Requires K % 64 == 0 and 16-byte aligned rows; N and M are arbitrary (M <= 64).
#include "common.cuh"
#include <cuda.h>
#include <math.h>

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BM = 128;                 // rows of W per tile
constexpr int BK = 64;                  // k per stage (128 bytes: one swizzle atom)
constexpr int W_BYTES = BM * BK * 2;    // 16 KB
constexpr int THREADS = 192;
constexpr int SS_STRIDE = 64;
constexpr long long WAIT_CYCLES = 2000000000LL;

enum Mode { STORE_BF16 = 0, STORE_F32 = 1, RESIDUAL = 2, SILU = 3 };

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(void* bar, unsigned parity) {
  unsigned ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, int* err, volatile int* failed) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*failed) return false;
    if (clock64() - t0 > WAIT_CYCLES) {
      if (err) atomicExch(err, 1);
      *failed = 1;
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// K-major operand tile, 128-byte swizzle: rows of 64 bf16 (128 bytes), 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc(const void* smem_tile) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_u32(smem_tile) & 0x3FFFF) >> 4);
  d |= (unsigned long long)1 << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
// kind::f16 instruction descriptor: D fp32, A and B bf16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr unsigned idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned id, unsigned accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float bfr(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned cluster_size() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a float of block `rank`'s shared memory at the same offset as `local`
__device__ __forceinline__ float ld_remote(const float* local, unsigned rank) {
  unsigned raddr;
  float v;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(raddr));   // ordered by the cluster barriers around it
  return v;
}
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // warps 2-5 only

struct Params {
  void* C; int ldc; int M; int N; int n_kb;
  const float* norm_w; const float* ss_in; int ss_parts; float eps; float* ss_out;
  int* err;
};

template <int NB, int STAGES> struct Layout {
  static constexpr int X_BYTES = NB * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + (X_BYTES < 1024 ? 1024 : X_BYTES);   // stages stay 1024-aligned
  static constexpr int PART_BYTES = BM * NB * 4;
  static constexpr int N_BARS = 4 * STAGES + 1;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + PART_BYTES + 8 * N_BARS + 4 * NB + 4 * 4 * NB + 64;
  static constexpr int TMEM_COLS = NB < 32 ? 32 : NB;
};

template <int NB, int MODE, bool NORM, int STAGES>
__global__ void __launch_bounds__(THREADS) gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w,
                                                              const __grid_constant__ CUtensorMap map_x, const Params p) {
  typedef Layout<NB, STAGES> L;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* part_s = reinterpret_cast<float*>(stages + STAGES * L::STAGE_BYTES);          // [128][NB] this block's partial tile
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(part_s + BM * NB);
  unsigned long long* w_full = bars;                 // [S] TMA (weights) -> MMA
  unsigned long long* x_full = w_full + STAGES;      // [S] TMA (activations) -> MMA, or -> the normalising warps
  unsigned long long* x_ready = x_full + STAGES;     // [S] normalising warps (128 arrivals) -> MMA
  unsigned long long* empty = x_ready + STAGES;      // [S] MMA done -> TMA
  unsigned long long* done = empty + STAGES;         // all MMAs done -> epilogue
  float* inv_s = reinterpret_cast<float*>(done + 1);  // [NB]
  float* ssw_s = inv_s + NB;                          // [4][NB] sums of squares per epilogue warp
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(ssw_s + 4 * NB);
  __shared__ int failed_s;
  volatile int* failed = &failed_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned ks = cluster_size(), rank = cluster_rank();
  const int tile = blockIdx.x / ks;
  // SILU: the tile's outputs are j0 .. j0+63; its W rows are gate rows j0.. (tile rows 0-63) and up rows N + j0.. (64-127)
  const int n0 = MODE == SILU ? tile * (BM / 2) : tile * BM;
  const int kb0 = (int)((long long)p.n_kb * rank / ks), kb1 = (int)((long long)p.n_kb * (rank + 1) / ks);
  const int n_kb = kb1 - kb0;

  if (threadIdx.x == 0) {
    failed_s = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&w_full[s], 1); mbar_init(&x_full[s], 1); mbar_init(&x_ready[s], 128); mbar_init(&empty[s], 1);
    }
    mbar_init(done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(L::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = *tmem_slot;
  DRYFT_TRACE_NOW(tr0);
  pdl_launch_dependents();
#ifdef DRYFT_TRACE
  unsigned long long tr1 = 0, tr2 = 0;
#endif

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: the ring's first weights depend on no earlier launch; activations do ----
      auto load_w = [&](int i) {
        const int s = i % STAGES;
        unsigned char* ws = stages + (size_t)s * L::STAGE_BYTES;
        mbar_expect_tx(&w_full[s], W_BYTES);
        if (MODE == SILU) {
          tma_load_2d(ws, &map_w, (kb0 + i) * BK, n0, &w_full[s]);
          tma_load_2d(ws + W_BYTES / 2, &map_w, (kb0 + i) * BK, p.N + n0, &w_full[s]);
        } else {
          tma_load_2d(ws, &map_w, (kb0 + i) * BK, n0, &w_full[s]);
        }
      };
      auto load_x = [&](int i) {
        const int s = i % STAGES;
        unsigned char* xs = stages + (size_t)s * L::STAGE_BYTES + W_BYTES;
        mbar_expect_tx(&x_full[s], L::X_BYTES);
        tma_load_2d(xs, &map_x, (kb0 + i) * BK, 0, &x_full[s]);
      };
      const int pre = n_kb < STAGES ? n_kb : STAGES;
      for (int i = 0; i < pre; ++i) load_w(i);
      pdl_wait();
#ifdef DRYFT_TRACE
      tr1 = dryft_now();
#endif
      for (int i = 0; i < pre; ++i) load_x(i);
      for (int i = pre; i < n_kb; ++i) {
        if (!mbar_wait(&empty[i % STAGES], (unsigned)(((i / STAGES) - 1) & 1), p.err, failed)) break;
        load_w(i);
        load_x(i);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- tcgen05.mma: D[128 x NB] += W stage [128 x 64] * X stage [NB x 64]^T, four k steps of 16 ----
      constexpr unsigned ID = idesc(BM, NB);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % STAGES;
        const unsigned par = (unsigned)((i / STAGES) & 1);
        ok = mbar_wait(&w_full[s], par, p.err, failed);
        if (ok) ok = mbar_wait(NORM ? &x_ready[s] : &x_full[s], par, p.err, failed);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned char* ws = stages + (size_t)s * L::STAGE_BYTES;
        const unsigned char* xs = ws + W_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk)
          umma(tmem, umma_desc(ws + kk * 32), umma_desc(xs + kk * 32), ID, (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&empty[s]);
      }
      umma_commit(done);   // also when the loop was left early: the epilogue warps must not wait a second for nothing
    }
  } else {
    // ---- warps 2-5: norm prologue over the activation stages, then this block's partial tile ----
    const int et = threadIdx.x - 64;             // 0..127
    const int q = warp & 3;                      // the quarter of tensor memory this warp may read
    pdl_wait();
    bool ok = true;
    if (NORM) {
      // inv[m] = rsqrt(mean(x[m]^2) + eps): a warp adds a row's blocks of sums of squares in a fixed order
      for (int m = warp - 2; m < NB; m += 4) {
        float s = 0.f;
        if (m < p.M)
          for (int i = lane; i < p.ss_parts; i += 32) s += ld_prev(p.ss_in + (size_t)i * SS_STRIDE + m);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) inv_s[m] = rsqrtf(s / (float)(p.n_kb * BK) + p.eps);
      }
      epi_bar();
      // a stage's activations [NB rows][64 k] become T(T(x * inv[m]) * w[k]) in place: thread -> row
      // et / 8 (+16, ...), 16-byte chunk et % 8, which the swizzle keeps at chunk (c ^ (row & 7))
      const int c = et & 7;
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(&x_full[s], (unsigned)((i / STAGES) & 1), p.err, failed);
        if (!ok) break;
        unsigned char* xs = stages + (size_t)s * L::STAGE_BYTES + W_BYTES;
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(p.norm_w + (size_t)(kb0 + i) * BK + c * 8));
        const float4 w1 = __ldg(reinterpret_cast<const float4*>(p.norm_w + (size_t)(kb0 + i) * BK + c * 8 + 4));
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int m = et >> 3; m < NB; m += 16) {
          uint4* cell = reinterpret_cast<uint4*>(xs + m * 128 + ((c ^ (m & 7)) << 4));
          uint4 raw = *cell;
          bf16* e = reinterpret_cast<bf16*>(&raw);
          const float inv = inv_s[m];
#pragma unroll
          for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16_rn(bfr(__bfloat162float(e[j]) * inv) * wv[j]);
          *cell = raw;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads through the async proxy
        mbar_arrive(&x_ready[s]);
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      ok = mbar_wait(done, 0, p.err, failed);
      ok = __all_sync(0xffffffffu, ok);
    }
    // this block's partial tile: tile row = TMEM lane, NB columns; zeros if it computed nothing or gave up
    const int row = q * 32 + lane;
    if (ok && n_kb > 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < NB; c0 += 16) {
        float v[16];
        tmem_ld16(tmem + ((unsigned)(q * 32) << 16) + c0, v);
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<float4*>(part_s + row * NB + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    } else {
#pragma unroll
      for (int c0 = 0; c0 < NB; c0 += 4) *reinterpret_cast<float4*>(part_s + row * NB + c0) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }

  // ---- every block of the cluster has left its partial: each finishes one slice of the tile's rows ----
  __syncwarp();
#ifdef DRYFT_TRACE
  if (threadIdx.x == 0) tr2 = dryft_now();
#endif   // the one-thread roles rejoin their warps: the cluster barrier is a warp-wide instruction
  cluster_sync_all();
  if (warp >= 2) {
    const int et = threadIdx.x - 64;
    constexpr int ROWS_T = MODE == SILU ? BM / 2 : BM;     // output rows of a tile
    const int rows_per = ROWS_T / (int)ks;                 // this block's slice (ks is 1, 2, 4 or 8)
    const int r_begin = (int)rank * rows_per;
    // item = m * rows_per + r: consecutive threads take consecutive outputs of one activation row
    for (int base = 0; base < NB * rows_per; base += 128) {
      const int item = base + et;
      const int m = item / rows_per, r = r_begin + item % rows_per;
      const int n = n0 + r;
      const bool live = item < NB * rows_per && m < p.M && n < p.N;
      float sq = 0.f;
      if (live) {
        // rank order: the sum does not depend on who arrived first; the loads are issued together
        float pv[8], pu[8];
#pragma unroll
        for (unsigned qk = 0; qk < 8; ++qk) {
          pv[qk] = qk < ks ? ld_remote(part_s + r * NB + m, qk) : 0.f;
          pu[qk] = (MODE == SILU && qk < ks) ? ld_remote(part_s + (r + BM / 2) * NB + m, qk) : 0.f;
        }
        float acc = 0.f, acc_up = 0.f;
#pragma unroll
        for (unsigned qk = 0; qk < 8; ++qk) { acc += pv[qk]; acc_up += pu[qk]; }
        if (MODE == SILU) {
          const float gt = bfr(acc), up = bfr(acc_up);
          const float sg = bfr(gt / (1.f + expf(-gt)));
          reinterpret_cast<bf16*>(p.C)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(sg * up);
        } else if (MODE == RESIDUAL) {
          bf16* x = reinterpret_cast<bf16*>(p.C);
          const float v = bfr(ld_prev_bf16(x + (size_t)m * p.ldc + n) + bfr(acc));
          x[(size_t)m * p.ldc + n] = __float2bfloat16_rn(v);
          sq = v * v;
        } else if (MODE == STORE_F32) {
          reinterpret_cast<float*>(p.C)[(size_t)m * p.ldc + n] = acc;
        } else {
          reinterpret_cast<bf16*>(p.C)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(acc);
        }
      }
      if (MODE == RESIDUAL && p.ss_out) {
        // sums of squares of this slice, per activation row, added in a fixed order: lanes that share m
        // (rows_per of them if rows_per < 32, else the whole warp), then the warps' parts
        const int span = rows_per < 32 ? rows_per : 32;
        for (int o = span >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (rows_per >= 32) {
          // a warp holds 32 rows of one m; rows_per / 32 warps share that m
          const int w_in_m = (item % rows_per) / 32;
          if (lane == 0 && item < NB * rows_per) ssw_s[w_in_m * NB + m] = sq;
          epi_bar();
          if (item < NB * rows_per && item % rows_per == 0 && m < p.M) {
            float t = 0.f;
            for (int w = 0; w < rows_per / 32; ++w) t += ssw_s[w * NB + m];
            p.ss_out[((size_t)tile * ks + rank) * SS_STRIDE + m] = t;
          }
          epi_bar();
        } else if (item < NB * rows_per && item % rows_per == 0 && m < p.M) {
          p.ss_out[((size_t)tile * ks + rank) * SS_STRIDE + m] = sq;
        }
      }
    }
  }
  __syncwarp();
  cluster_sync_all();   // nobody leaves while another block may still read its partial tile

  if (*failed) {
    // a wait ran out: give copies that may still be in flight a bounded time to land
    if (threadIdx.x == 0) {
      const long long t0 = clock64();
      for (int s = 0; s < STAGES; ++s) {
        while (!mbar_try_wait(&w_full[s], 0) && !mbar_try_wait(&w_full[s], 1) && clock64() - t0 < WAIT_CYCLES) {}
        while (!mbar_try_wait(&x_full[s], 0) && !mbar_try_wait(&x_full[s], 1) && clock64() - t0 < WAIT_CYCLES) {}
      }
    }
    __syncthreads();
  }
  DRYFT_TRACE_PUT((unsigned)(MODE * 2 + (NORM ? 1 : 0) + 100 * ks), tr0, tr1, tr2);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(L::TMEM_COLS) : "memory");
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
// [rows, K] bfloat16 row-major, box 64 k x box_rows rows, 128-byte swizzle, zero fill out of range
bool encode(CUtensorMap* map, const void* base, long long rows, int K, int ld, int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  return sms;
}
// K splits (= cluster size): enough blocks for two per SM, a power of two up to 8, at least two k blocks each
int k_splits(int n_tiles, int n_kb) {
  int ks = 1;
  while (ks < 8 && n_tiles * ks * 2 <= 2 * sm_count() && n_kb / (ks * 2) >= 2) ks *= 2;
  return ks;
}

template <int NB, int MODE, bool NORM>
int launch3(const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, int n_tiles, int ks, int pdl, cudaStream_t st) {
  constexpr int STAGES = NB <= 16 ? 5 : (NB <= 32 ? 4 : 4);
  typedef Layout<NB, STAGES> L;
  static bool attr_set = false;  // per instantiation; set by an eager launch before any capture
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<NB, MODE, NORM, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(n_tiles * ks));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = L::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)ks;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel<NB, MODE, NORM, STAGES>, map_w, map_x, p);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}
template <int NB, int MODE>
int launch2(bool norm, const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, int n_tiles, int ks, int pdl, cudaStream_t st) {
  return norm ? launch3<NB, MODE, true>(map_w, map_x, p, n_tiles, ks, pdl, st) : launch3<NB, MODE, false>(map_w, map_x, p, n_tiles, ks, pdl, st);
}
template <int NB>
int launch1(int mode, bool norm, const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, int n_tiles, int ks, int pdl,
            cudaStream_t st) {
  switch (mode) {
    case STORE_BF16: return launch2<NB, STORE_BF16>(norm, map_w, map_x, p, n_tiles, ks, pdl, st);
    case STORE_F32: return launch2<NB, STORE_F32>(norm, map_w, map_x, p, n_tiles, ks, pdl, st);
    case RESIDUAL: return launch2<NB, RESIDUAL>(norm, map_w, map_x, p, n_tiles, ks, pdl, st);
    case SILU: return launch2<NB, SILU>(norm, map_w, map_x, p, n_tiles, ks, pdl, st);
  }
  return DRYFT_ERR_UNSUPPORTED;
}

int tiles_of(int N, int mode) { return mode == SILU ? (N + BM / 2 - 1) / (BM / 2) : (N + BM - 1) / BM; }
}  // namespace
DRYFT_TRACE_EXPORT(dryft_gemm_stream_trace)

// Blocks of sums of squares that a residual product of N outputs over K inputs leaves in ss_out.
DRYFT_API int dryft_gemm_stream_ss_parts(int N, int K) {
  if (K <= 0 || K % BK) return 0;
  const int t = tiles_of(N, RESIDUAL);
  return t * k_splits(t, K / BK);
}

// Same contract as dryft_gemm_small_m (csrc/gemm_small_m.cu) with M <= 64:
//   mode 0 store bf16, 1 store f32, 2 residual add in place (C = x [M, ldc]; ss_out gets
//   dryft_gemm_stream_ss_parts(N, K) blocks of 64 floats), 3 SiLU*mul (W holds N gate rows then N up rows).
//   norm_w != null: A is normalised first, ss_in [ss_parts][64] holding the rows' sums of squares.
// Activations must be contiguous rows of K (lda = K).
DRYFT_API int dryft_gemm_stream(const void* A, int lda, const void* W, void* C, int ldc, int mode, int M, int N, int K,
                                const float* norm_w, const float* ss_in, int ss_parts, float eps, float* ss_out, int pdl,
                                int* err, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || K % BK || lda % 8 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return DRYFT_ERR_UNSUPPORTED;
  if (norm_w && (!ss_in || ss_parts <= 0)) return DRYFT_ERR_UNSUPPORTED;
  if (mode != RESIDUAL && ss_out) return DRYFT_ERR_UNSUPPORTED;
  const int NB = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  CUtensorMap map_w, map_x;
  const long long w_rows = mode == SILU ? 2LL * N : N;
  if (!encode(&map_w, W, w_rows, K, K, mode == SILU ? BM / 2 : BM)) return DRYFT_ERR_UNSUPPORTED;
  if (!encode(&map_x, A, M, K, lda, NB)) return DRYFT_ERR_UNSUPPORTED;
  const int n_tiles = tiles_of(N, mode);
  const int ks = k_splits(n_tiles, K / BK);
  Params p;
  p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.n_kb = K / BK;
  p.norm_w = norm_w; p.ss_in = ss_in; p.ss_parts = ss_parts; p.eps = eps; p.ss_out = ss_out; p.err = err;
  const bool norm = norm_w != nullptr;
  switch (NB) {
    case 16: return launch1<16>(mode, norm, map_w, map_x, p, n_tiles, ks, pdl, st);
    case 32: return launch1<32>(mode, norm, map_w, map_x, p, n_tiles, ks, pdl, st);
    default: return launch1<64>(mode, norm, map_w, map_x, p, n_tiles, ks, pdl, st);
  }
}
