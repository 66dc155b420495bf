// Decode matrix product for up to 64 rows of activations on the 5th-generation tensor cores, built to
// stream weights at the speed of memory:
//
//   C[M,N] = A[M,K] * W[N,K]^T,  M <= 64, bfloat16 operands, 32-bit accumulation, every weight byte read
//   from HBM exactly once (hari495/dryft: cuBLAS via F.linear, engine/dryft_qwen3/model.py:237,258,260,261),
//   with the layer's element-wise work fused in: RMSNorm of the activations on their way in
//   (kernels/rmsnorm.py:21-39; model.py:28-32, both roundings kept), residual add with the sums of squares
//   for the next norm on the way out (rmsnorm.py:34), SiLU*mul on the way out (kernels/silu_mul.py:29-32;
//   weights.py:98-100).
//
// The product is computed transposed: a tile is 128 rows of W (the M = 128 operand of tcgen05.mma, K-major,
// 128-byte swizzle, brought in by TMA) against the NB = 16 / 32 / 64 padded activation rows (the N operand,
// K-major, also by TMA; rows beyond M are zero-filled), accumulating a 128 x NB tile in tensor memory.
//
// Work is cut evenly, not by tiles.  A unit is one (tile, 64-wide k block) pair: 16 KB of weights.  The
// grid is one block per SM (or fewer), and block c takes the units [c U / G, (c + 1) U / G) in (tile, k)
// order, so every block streams the same number of bytes, whatever the number of tiles (20 tiles of 2,560
// outputs and 1,187 tiles of a vocabulary alike), through one ring of shared-memory stages that never
// drains between tiles.  A block's run of units covers whole tiles, finished straight from tensor memory,
// and at most two pieces of tiles shared with its neighbours.  A piece goes to a slot of a workspace in
// global memory; the block then draws a ticket of that tile, and the block that draws the last one adds
// the tile's pieces in block order (so a result does not depend on who arrived first) and finishes the tile.
// No block waits for another block: there is no spin on global memory in this file.
//
// Warps: 0 (one thread) TMA producer; 1 (one thread) issues tcgen05.mma; 2-5 the 128 threads that read the
// accumulator (one W row each) and finish tiles; with a norm, 6-9 normalise each activation stage in place
// before the tensor core reads it.  The kernel may be a programmatic dependent of the launch before it: its
// ring fills with weights, which depend on nothing, before it waits for that launch.
// Every mbarrier wait is bounded by a clock (about a second): a waiter that gives up raises *err, every role
// leaves its loop, the block lets its own copies land, frees its tensor memory and returns.
// No TMA load uses cluster multicast; the kernel does not use clusters.
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
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, int* err, volatile int* failed, int site) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*failed) return false;
    if (clock64() - t0 > WAIT_CYCLES) {
      if (err) atomicCAS(err, 0, 100 + site);   // the first wait that gave up names its place
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
__device__ __forceinline__ void tmem_ld16_issue(unsigned taddr, unsigned (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float bfr(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // warps 2-5 only

struct Params {
  void* C; int ldc; int M; int N; int n_kb; int n_tiles;
  const float* norm_w; const float* ss_in; int ss_parts; float eps; float* ss_out;
  int* err; float* ws; int* tickets;
};

template <int NB, int MODE, int STAGES> struct Layout {
  static constexpr int X_BYTES = NB * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + (X_BYTES < 1024 ? 1024 : X_BYTES);   // stages stay 1024-aligned
  static constexpr int XCH_BYTES = MODE == SILU ? (BM / 2) * NB * 2 : 0;            // up rows on their way to the gate rows
  static constexpr int N_BARS = 4 * STAGES + 4;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + XCH_BYTES + 8 * N_BARS + 4 * 64 + 4 * 4 * 64 + 64;
  static constexpr int TMEM_COLS = 2 * NB;   // two accumulators: a run is read while the next one is multiplied
};

// first unit of block c when U units are cut evenly over G blocks
__device__ __forceinline__ long long first_unit(long long U, int G, int c) { return U * c / G; }
// the block that holds unit u
__device__ __forceinline__ int block_of(long long U, int G, long long u) {
  int c = (int)(u * G / U);
  while (c + 1 < G && first_unit(U, G, c + 1) <= u) ++c;
  while (c > 0 && first_unit(U, G, c) > u) --c;
  return c;
}

template <int NB, int MODE, bool NORM, int STAGES>
__global__ void __launch_bounds__(NORM ? 320 : 192) gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                         const __grid_constant__ CUtensorMap map_x, const Params p) {
  typedef Layout<NB, MODE, STAGES> L;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  bf16* xch = reinterpret_cast<bf16*>(stages + STAGES * L::STAGE_BYTES);               // [NB][64] (SILU only)
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(stages + STAGES * L::STAGE_BYTES + L::XCH_BYTES);
  unsigned long long* w_full = bars;                 // [S] TMA (weights) -> MMA
  unsigned long long* x_full = w_full + STAGES;      // [S] TMA (activations) -> MMA, or -> the normalising warps
  unsigned long long* x_ready = x_full + STAGES;     // [S] normalising warps (128 arrivals) -> MMA
  unsigned long long* empty = x_ready + STAGES;      // [S] MMA done -> TMA
  unsigned long long* acc_full = empty + STAGES;     // [2] a run of one tile's units is in tensor memory -> finishing warps
  unsigned long long* acc_empty = acc_full + 2;      // [2] finishing warps have read it (128 arrivals) -> MMA
  float* inv_s = reinterpret_cast<float*>(acc_empty + 2);   // [64]
  float* ssw_s = inv_s + 64;                                // [4][64] sums of squares per finishing warp
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(ssw_s + 4 * 64);
  int* last_s = reinterpret_cast<int*>(tmem_slot + 1);
  __shared__ int failed_s;
  volatile int* failed = &failed_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = p.n_kb;
  const long long U = (long long)p.n_tiles * KB;
  const int G = (int)gridDim.x, c = (int)blockIdx.x;
  const long long u0 = first_unit(U, G, c), u1 = first_unit(U, G, c + 1);
  const int n_units = (int)(u1 - u0);

  if (threadIdx.x == 0) {
    failed_s = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&w_full[s], 1); mbar_init(&x_full[s], 1); mbar_init(&x_ready[s], 128); mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
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
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: the ring's first weights depend on no earlier launch; activations do ----
      auto load_w = [&](int i) {
        const int s = i % STAGES;
        const long long u = u0 + i;
        const int tile = (int)(u / KB), kb = (int)(u - (long long)tile * KB);
        unsigned char* ws = stages + (size_t)s * L::STAGE_BYTES;
        mbar_expect_tx(&w_full[s], W_BYTES);
        if (MODE == SILU) {   // a tile's outputs are j0 .. j0+63: gate rows j0.. (tile rows 0-63), up rows N + j0.. (64-127)
          tma_load_2d(ws, &map_w, kb * BK, tile * (BM / 2), &w_full[s]);
          tma_load_2d(ws + W_BYTES / 2, &map_w, kb * BK, p.N + tile * (BM / 2), &w_full[s]);
        } else {
          tma_load_2d(ws, &map_w, kb * BK, tile * BM, &w_full[s]);
        }
      };
      auto load_x = [&](int i) {
        const int s = i % STAGES;
        const int kb = (int)((u0 + i) % KB);
        unsigned char* xs = stages + (size_t)s * L::STAGE_BYTES + W_BYTES;
        mbar_expect_tx(&x_full[s], L::X_BYTES);
        tma_load_2d(xs, &map_x, kb * BK, 0, &x_full[s]);
      };
      const int pre = n_units < STAGES ? n_units : STAGES;
      for (int i = 0; i < pre; ++i) load_w(i);
      pdl_wait();
      for (int i = 0; i < pre; ++i) load_x(i);
      for (int i = pre; i < n_units; ++i) {
        if (!mbar_wait(&empty[i % STAGES], (unsigned)(((i / STAGES) - 1) & 1), p.err, failed, 1)) break;
        load_w(i);
        load_x(i);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- tcgen05.mma: D[128 x NB] (+)= W stage [128 x 64] * X stage [NB x 64]^T, four k steps of 16 ----
      constexpr unsigned ID = idesc(BM, NB);
      bool ok = true;
      int seg = 0;   // runs of one tile's units this block has started
      for (int i = 0; i < n_units && ok; ++i) {
        const int s = i % STAGES;
        const unsigned par = (unsigned)((i / STAGES) & 1);
        const long long u = u0 + i;
        const int kb = (int)(u % KB);
        const bool first = (i == 0) || kb == 0;
        const bool last = (i == n_units - 1) || kb == KB - 1;
        ok = mbar_wait(&w_full[s], par, p.err, failed, 2);
        if (ok) ok = mbar_wait(NORM ? &x_ready[s] : &x_full[s], par, p.err, failed, 3);
        // run `seg` accumulates in buffer seg & 1, which the finishing warps must have read two runs ago
        if (ok && first && seg >= 2) ok = mbar_wait(&acc_empty[seg & 1], (unsigned)(((seg >> 1) - 1) & 1), p.err, failed, 4);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned char* ws = stages + (size_t)s * L::STAGE_BYTES;
        const unsigned char* xs = ws + W_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk)
          umma(tmem + (unsigned)((seg & 1) * NB), umma_desc(ws + kk * 32), umma_desc(xs + kk * 32), ID, (!first || kk > 0) ? 1u : 0u);
        umma_commit(&empty[s]);
        if (last) { umma_commit(&acc_full[seg & 1]); ++seg; }
      }
    }
  } else if (warp < 6) {
    // ---- warps 2-5: read each run's accumulator 16 activation rows at a time, finish whole tiles, hand pieces over ----
    const int q = warp & 3;                      // the quarter of tensor memory this warp may read
    const int row = q * 32 + lane;               // W row of the tile = TMEM lane
    const int et = (warp - 2) * 32 + lane;       // 0..127, for work shared out by index
    pdl_wait();                                  // the residual stream and earlier tickets are visible from here on

    // finish 16 activation rows m0 .. m0+15 of W row `row` of `tile`
    auto finish16 = [&](int tile, int m0, const float (&v)[16]) {
      if (MODE == SILU) {
        const int n0 = tile * (BM / 2);
        if (row >= BM / 2) {
#pragma unroll
          for (int j = 0; j < 16; ++j) xch[(m0 + j) * (BM / 2) + row - BM / 2] = __float2bfloat16_rn(v[j]);
        }
        epi_bar();
        if (row < BM / 2 && n0 + row < p.N) {
          bf16* out = reinterpret_cast<bf16*>(p.C) + n0 + row;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + j;
            if (m < p.M) {
              const float gt = bfr(v[j]), up = __bfloat162float(xch[m * (BM / 2) + row]);
              const float sg = bfr(gt / (1.f + expf(-gt)));
              out[(size_t)m * p.ldc] = __float2bfloat16_rn(sg * up);
            }
          }
        }
      } else if (MODE == RESIDUAL) {
        const int n = tile * BM + row;
        bf16* x = reinterpret_cast<bf16*>(p.C) + n;
        float xv[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) xv[j] = (m0 + j < p.M && n < p.N) ? ld_prev_bf16(x + (size_t)(m0 + j) * p.ldc) : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + j;
          float sq = 0.f;
          if (m < p.M && n < p.N) {
            const float nv = bfr(xv[j] + bfr(v[j]));
            x[(size_t)m * p.ldc] = __float2bfloat16_rn(nv);
            sq = nv * nv;
          }
          if (p.ss_out) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) ssw_s[(warp - 2) * 64 + m] = sq;
          }
        }
      } else {
        const int n = tile * BM + row;
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + j;
            if (m < p.M) {
              if (MODE == STORE_F32) reinterpret_cast<float*>(p.C)[(size_t)m * p.ldc + n] = v[j];
              else reinterpret_cast<bf16*>(p.C)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(v[j]);
            }
          }
        }
      }
    };
    // after the last 16 rows of a tile: the tile's sums of squares (RESIDUAL); buffers shared by tiles are free again
    auto finish_tile = [&](int tile) {
      if (MODE == RESIDUAL && p.ss_out) {
        epi_bar();
        // the four warps' parts in the order of the tile's rows (0-31, 32-63, 64-95, 96-127): warps 4, 5, 2, 3
        if (et < p.M) p.ss_out[(size_t)tile * SS_STRIDE + et] = ssw_s[2 * 64 + et] + ssw_s[3 * 64 + et] + ssw_s[0 * 64 + et] + ssw_s[1 * 64 + et];
      }
      if (MODE == SILU || (MODE == RESIDUAL && p.ss_out)) epi_bar();
    };

    bool ok = true;
    int seg = 0;
    for (long long u = u0; u < u1 && ok; ++seg) {
      const int tile = (int)(u / KB);
      const long long t_begin = (long long)tile * KB, t_end = t_begin + KB;
      const long long seg_end = u1 < t_end ? u1 : t_end;
      const bool whole = (u == t_begin) && (seg_end == t_end);
      u = seg_end;
      const int b = seg & 1;
      ok = mbar_wait(&acc_full[b], (unsigned)((seg >> 1) & 1), p.err, failed, 5);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const unsigned t_addr = tmem + ((unsigned)(q * 32) << 16) + (unsigned)(b * NB);
      if (whole) {
#pragma unroll 1
        for (int m0 = 0; m0 < NB; m0 += 16) {
          unsigned r[16];
          tmem_ld16_issue(t_addr + m0, r);
          tmem_ld_wait();
          if (m0 + 16 >= NB) {   // the whole run is in registers or stored: the tensor core may reuse this buffer
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&acc_empty[b]);
          }
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
          finish16(tile, m0, v);
          if (MODE == SILU && m0 + 16 < NB) epi_bar();   // xch is rewritten by the next 16 rows
        }
        finish_tile(tile);
        continue;
      }
      // this block's piece of the tile -> its slot of the workspace
      const int slot = 2 * c + (u0 < t_begin ? 1 : 0);
      float* dst = p.ws + ((size_t)slot * BM + row) * NB;
#pragma unroll 1
      for (int m0 = 0; m0 < NB; m0 += 16) {
        unsigned r[16];
        tmem_ld16_issue(t_addr + m0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          __stcg(reinterpret_cast<float4*>(dst + m0 + j), make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                      __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])));
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&acc_empty[b]);
      // a ticket of the tile; whoever draws the last one adds all pieces in block order and finishes the tile
      __threadfence();
      epi_bar();
      const int c_first = block_of(U, G, t_begin), c_last = block_of(U, G, t_end - 1);
      if (et == 0) *last_s = (atomicAdd(&p.tickets[tile], 1) == c_last - c_first) ? 1 : 0;
      epi_bar();
      const bool finish = *last_s != 0;
      epi_bar();   // last_s may be rewritten by the next run
      if (!finish) continue;
      __threadfence();
      if (et == 0) p.tickets[tile] = 0;   // ready for the next launch
#pragma unroll 1
      for (int m0 = 0; m0 < NB; m0 += 16) {
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
        for (int cc = c_first; cc <= c_last; ++cc) {
          const int sl = 2 * cc + (first_unit(U, G, cc) < t_begin ? 1 : 0);
          const float* src = p.ws + ((size_t)sl * BM + row) * NB + m0;
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 a = __ldcg(reinterpret_cast<const float4*>(src + j));
            v[j] += a.x; v[j + 1] += a.y; v[j + 2] += a.z; v[j + 3] += a.w;
          }
        }
        finish16(tile, m0, v);
        if (MODE == SILU && m0 + 16 < NB) epi_bar();
      }
      finish_tile(tile);
    }
  } else if (NORM) {
    // ---- warps 6-9: every activation stage [NB rows][64 k] becomes T(T(x * inv[m]) * w[k]) in place ----
    const int nt = threadIdx.x - 192;            // 0..127
    pdl_wait();
    // inv[m] = rsqrt(mean(x[m]^2) + eps): a warp adds a row's blocks of sums of squares in a fixed order
    for (int m = warp - 6; m < NB; m += 4) {
      float s = 0.f;
      if (m < p.M)
        for (int i = lane; i < p.ss_parts; i += 32) s += ld_prev(p.ss_in + (size_t)i * SS_STRIDE + m);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) inv_s[m] = rsqrtf(s / (float)(KB * BK) + p.eps);
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");
    // thread -> row nt / 8 (+16, ...), 16-byte chunk nt % 8, which the swizzle keeps at chunk (c ^ (row & 7))
    const int ch = nt & 7;
    for (int i = 0; i < n_units; ++i) {
      const int s = i % STAGES;
      if (!mbar_wait(&x_full[s], (unsigned)((i / STAGES) & 1), p.err, failed, 6)) break;
      const int kb = (int)((u0 + i) % KB);
      unsigned char* xs = stages + (size_t)s * L::STAGE_BYTES + W_BYTES;
      const float4 w0 = __ldg(reinterpret_cast<const float4*>(p.norm_w + (size_t)kb * BK + ch * 8));
      const float4 w1 = __ldg(reinterpret_cast<const float4*>(p.norm_w + (size_t)kb * BK + ch * 8 + 4));
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int m = nt >> 3; m < NB; m += 16) {
        uint4* cell = reinterpret_cast<uint4*>(xs + m * 128 + ((ch ^ (m & 7)) << 4));
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

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
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

int tiles_of(int N, int mode) { return mode == SILU ? (N + BM / 2 - 1) / (BM / 2) : (N + BM - 1) / BM; }
// one block per SM, or one per unit if there are fewer units than SMs
int blocks_of(long long units) { return (int)(units < (long long)sm_count() ? units : (long long)sm_count()); }

template <int NB, int MODE, bool NORM>
int launch3(const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, int blocks, int pdl, cudaStream_t st) {
  constexpr int STAGES = NB <= 16 ? 5 : (NB <= 32 ? 5 : 4);
  typedef Layout<NB, MODE, STAGES> L;
  static bool attr_set[64] = {false};  // per instantiation and device; set by an eager launch before any capture
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DRYFT_ERR_UNSUPPORTED;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<NB, MODE, NORM, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(NORM ? 320 : 192);
  cfg.dynamicSmemBytes = L::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel<NB, MODE, NORM, STAGES>, map_w, map_x, p);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}
template <int NB>
int launch1(int mode, bool norm, const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, int blocks, int pdl, cudaStream_t st) {
  switch (mode) {
    case STORE_BF16: return norm ? launch3<NB, STORE_BF16, true>(map_w, map_x, p, blocks, pdl, st) : launch3<NB, STORE_BF16, false>(map_w, map_x, p, blocks, pdl, st);
    case STORE_F32: return norm ? launch3<NB, STORE_F32, true>(map_w, map_x, p, blocks, pdl, st) : launch3<NB, STORE_F32, false>(map_w, map_x, p, blocks, pdl, st);
    case RESIDUAL: return norm ? DRYFT_ERR_UNSUPPORTED : launch3<NB, RESIDUAL, false>(map_w, map_x, p, blocks, pdl, st);
    case SILU: return norm ? launch3<NB, SILU, true>(map_w, map_x, p, blocks, pdl, st) : launch3<NB, SILU, false>(map_w, map_x, p, blocks, pdl, st);
  }
  return DRYFT_ERR_UNSUPPORTED;
}
}  // namespace

// Blocks of sums of squares that a residual product of N outputs leaves in ss_out: one per tile of 128 outputs.
DRYFT_API int dryft_gemm_stream_ss_parts(int N, int K) {
  if (K <= 0 || K % BK) return 0;
  return tiles_of(N, RESIDUAL);
}

// What a launch needs beside its operands: floats of workspace for the pieces of shared tiles (two slots of
// 128 x 64 per block) and ints of tickets (one per tile), both owned by the caller, one set per device and
// stream; the tickets start at zero and every launch leaves them at zero.
DRYFT_API long long dryft_gemm_stream_workspace_floats() { return (long long)2 * sm_count() * BM * 64; }
DRYFT_API int dryft_gemm_stream_tickets(int N, int mode) { return tiles_of(N, mode); }

// Same contract as dryft_gemm_small_m (csrc/gemm_small_m.cu) with M <= 64:
//   mode 0 store bf16, 1 store f32, 2 residual add in place (C = x [M, ldc]; ss_out gets
//   dryft_gemm_stream_ss_parts(N, K) blocks of 64 floats), 3 SiLU*mul (W holds N gate rows then N up rows).
//   norm_w != null: A is normalised first, ss_in [ss_parts][64] holding the rows' sums of squares.
// Activations are rows of K elements, lda apart.
DRYFT_API int dryft_gemm_stream(const void* A, int lda, const void* W, void* C, int ldc, int mode, int M, int N, int K,
                                const float* norm_w, const float* ss_in, int ss_parts, float eps, float* ss_out, int pdl,
                                int* err, float* workspace, int* tickets, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || K % BK || lda % 8 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return DRYFT_ERR_UNSUPPORTED;
  if (norm_w && (!ss_in || ss_parts <= 0 || ((uintptr_t)norm_w & 15))) return DRYFT_ERR_UNSUPPORTED;
  if (mode != RESIDUAL && ss_out) return DRYFT_ERR_UNSUPPORTED;
  if (!workspace || !tickets) return DRYFT_ERR_UNSUPPORTED;
  const int NB = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  CUtensorMap map_w, map_x;
  const long long w_rows = mode == SILU ? 2LL * N : N;
  if (!encode(&map_w, W, w_rows, K, K, mode == SILU ? BM / 2 : BM)) return DRYFT_ERR_UNSUPPORTED;
  if (!encode(&map_x, A, M, K, lda, NB)) return DRYFT_ERR_UNSUPPORTED;
  Params p;
  p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.n_kb = K / BK; p.n_tiles = tiles_of(N, mode);
  p.norm_w = norm_w; p.ss_in = ss_in; p.ss_parts = ss_parts; p.eps = eps; p.ss_out = ss_out; p.err = err;
  p.ws = workspace; p.tickets = tickets;
  const int blocks = blocks_of((long long)p.n_tiles * p.n_kb);
  const bool norm = norm_w != nullptr;
  switch (NB) {
    case 16: return launch1<16>(mode, norm, map_w, map_x, p, blocks, pdl, st);
    case 32: return launch1<32>(mode, norm, map_w, map_x, p, blocks, pdl, st);
    default: return launch1<64>(mode, norm, map_w, map_x, p, blocks, pdl, st);
  }
}
