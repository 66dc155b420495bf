// Prefill attention on the 5th-generation tensor cores (bfloat16): causal grouped-query attention of
// packed prompts of unequal lengths over the paged cache, with Q K^T and P V issued as tcgen05.mma,
// S, P and O in tensor memory, and Q, K and V brought in by TMA.  Same operation and same masks as
// csrc/attn_prefill.cu (which stays as the general form); compiled per model with -DDRYFT_HEAD_DIM
// (64 or 128), -DDRYFT_GROUP, -DDRYFT_PAGE (64).
//
// Grid (query tiles, query heads); two blocks share an SM, so that one block's softmax runs under the
// other's products.  A tile is up to 128 consecutive query tokens of ONE sequence.
//   warp 4, one thread   TMA: the Q tile once (3-D map over [token, head, d]), then page after page of K
//       and of V (2-D maps over the page pool, 64 keys x 64 d boxes, 128-byte swizzle) into two rings of
//       their own: a K stage is free again as soon as its S product is done, a V stage after its P V.
//   warp 5, one thread   tcgen05.mma: S_j = Q K_j^T (M 128, N 64, K = head size; both operands K-major
//       in shared memory) into one of two 64-column buffers of tensor memory, one tile ahead of the
//       softmax; then, once P_j is in tensor memory, O += P_j V_j (M 128, N = head size, K 64; P is the
//       operand read from tensor memory, V the MN-major operand in shared memory).
//   warps 0-3, one thread per query row   tcgen05.ld S, mask (key <= query position, window) on the
//       tiles that need one, running maximum and sum in 32-bit (log2 domain), P rounded to bfloat16 and
//       stored over the first 32 columns of its own S buffer (two keys a column).  The running maximum
//       moves only when it grows by more than 8 (a factor of 256 in P, exact in 32-bit and harmless in
//       bfloat16); only then is O in tensor memory rescaled (tcgen05.ld / st), after the P V product
//       before it has finished.  At the end O / l is rounded and stored.
// hari495/dryft uses SDPA's flash kernel here (engine/dryft_qwen3/model.py:172-177).
//
// Every mbarrier wait is bounded by a clock (about a second); a waiter that gives up raises *err and
// every role leaves its loop; the block then gives its own copies a bounded time to land, frees its
// tensor memory and returns.  No block waits on another block.  No TMA load uses cluster multicast.
#include "common.cuh"
#include <cuda.h>
#include <math.h>

#if !defined(DRYFT_HEAD_DIM) || !defined(DRYFT_GROUP) || !defined(DRYFT_PAGE)
#error "compile with -DDRYFT_HEAD_DIM=.. -DDRYFT_GROUP=.. -DDRYFT_PAGE=.."
#endif

namespace {
typedef __nv_bfloat16 bf16;
constexpr int D = DRYFT_HEAD_DIM;
constexpr int G = DRYFT_GROUP;
constexpr int BN = DRYFT_PAGE;      // keys per tile = one cache page
constexpr int BM = 128;             // query rows per block
static_assert(D == 64 || D == 128, "this kernel takes head sizes 64 and 128");
static_assert(BN == 64, "written for 64-token pages");
constexpr int DA = D / 64;          // 64-wide (128-byte) atoms along the head size
constexpr int Q_ATOM = BM * 128;    // bytes of one Q atom [128 rows][64 d]
constexpr int KV_ATOM = BN * 128;   // bytes of one K or V atom [64 keys][64 d]
constexpr int Q_BYTES = DA * Q_ATOM;
constexpr int K_BYTES = DA * KV_ATOM;
constexpr int V_BYTES = DA * KV_ATOM;
// Stages of the K ring and of the V ring.  Two blocks of 256 tensor-memory columns fill an SM's 512, and
// the shared memory asked for keeps a third block off the SM, so that no allocation ever has to wait.
constexpr int STAGES = D == 128 ? 2 : 4;
constexpr int N_BARS = 1 + 4 * STAGES + 2 + 2 + 1;
constexpr int SMEM_BYTES = Q_BYTES + STAGES * (K_BYTES + V_BYTES) + 1024 + 8 * N_BARS + 16;
static_assert(3 * (SMEM_BYTES + 1024) > 227 * 1024 && 2 * (SMEM_BYTES + 1024) <= 227 * 1024, "two blocks an SM");
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 256;      // S buffers at columns 0 and 64 (P over the first 32 of each), O from 128 on
constexpr int S_COL = 64;           // columns of one S buffer
constexpr int O_COL = 128;
constexpr float GROW = 8.f;         // the running maximum moves when it grows by more than this (log2)
constexpr long long WAIT_CYCLES = 2000000000LL;

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
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, int* err, volatile int* failed, int site = 1) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*failed) return false;
    if (clock64() - t0 > WAIT_CYCLES) {
      if (err) atomicCAS(err, 0, site);   // the first wait that gave up names its place
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
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, void* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle, version 1; offsets in bytes.
__device__ __forceinline__ unsigned long long umma_desc(const void* p, unsigned lbo_bytes, unsigned sbo_bytes) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_u32(p) & 0x3FFFF) >> 4);
  d |= (unsigned long long)(lbo_bytes >> 4) << 16;
  d |= (unsigned long long)(sbo_bytes >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
// kind::f16 instruction descriptor: D fp32, A/B bf16; b_major = 1 makes B the MN-major operand
__host__ __device__ constexpr unsigned idesc(int m, int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)b_mn_major << 16) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned id, unsigned accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// A from tensor memory (row = lane, two bfloat16 a column), B from shared memory
__device__ __forceinline__ void umma_ts(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc, unsigned id, unsigned accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32_issue(unsigned taddr, unsigned (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
               "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
               "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
               ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                 "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                 "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
                 "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&pk);
}

__global__ void __launch_bounds__(THREADS, 2) attn_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q,   // [tokens, heads, D], box 64 x 1 x 128
    const __grid_constant__ CUtensorMap map_k,   // [pages * kv heads * 64, D], box 64 x 64
    const __grid_constant__ CUtensorMap map_v,
    const int* __restrict__ page_table, int max_pages, const int* __restrict__ tile_tok0, const int* __restrict__ tile_rows,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, bf16* __restrict__ out, int nH, int nKV,
    float scale_log2, int window, int* err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = base;                        // [DA][128][64]
  unsigned char* k_s = q_s + Q_BYTES;               // [stages][DA][64][64]
  unsigned char* v_s = k_s + STAGES * K_BYTES;      // [stages][DA][64][64]
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(v_s + STAGES * V_BYTES);
  unsigned long long* q_full = bars;                    // TMA -> MMA
  unsigned long long* k_full = bars + 1;                // [stages] TMA -> MMA
  unsigned long long* k_free = k_full + STAGES;         // [stages] S product done -> TMA
  unsigned long long* v_full = k_free + STAGES;         // [stages] TMA -> MMA
  unsigned long long* v_free = v_full + STAGES;         // [stages] P V product done -> TMA
  unsigned long long* s_full = v_free + STAGES;         // [2] S product done -> softmax warps
  unsigned long long* p_ready = s_full + 2;             // [2] softmax warps (128 arrivals) -> MMA
  unsigned long long* o_done = p_ready + 2;             // P V product done -> softmax warps
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(o_done + 1);
  __shared__ int failed_s;
  volatile int* failed = &failed_s;

  // Heads run fastest: the host lists the tiles with the most keys first, so all heads of the longest
  // tiles start first and the short ones fill the gaps at the end (with tiles fastest, every head's
  // longest tile would be spread over the launch and the last of them would finish alone).
  const int tile = blockIdx.x / nH, h = blockIdx.x % nH, kvh = h / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok0 = tile_tok0[tile], rows = tile_rows[tile];
  const int slot = tok_slot[tok0];
  if (slot < 0 || rows <= 0) return;  // padding tile (uniform for the block; nothing allocated yet)
  const int pos0 = tok_pos[tok0];
  const int pg_first = window > 0 ? max(0, pos0 + 1 - window) / BN : 0;
  const int pg_last = (pos0 + rows - 1) / BN;
  const int n_tiles = pg_last - pg_first + 1;
  const int* pt = page_table + (size_t)slot * max_pages;

  if (threadIdx.x == 0) {
    failed_s = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_free[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_free[s], 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_full[b], 1); mbar_init(&p_ready[b], BM); }
    mbar_init(o_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      // ---- TMA: Q, then K one tile ahead of V, in the order the products use them ----
      auto load_k = [&](int j) {
        const int s = j % STAGES;
        unsigned char* ks = k_s + (size_t)s * K_BYTES;
        const int row0 = (pt[pg_first + j] * nKV + kvh) * BN;
        mbar_expect_tx(&k_full[s], K_BYTES);
#pragma unroll
        for (int a = 0; a < DA; ++a) tma_load_2d(ks + a * KV_ATOM, &map_k, a * 64, row0, &k_full[s]);
      };
      auto load_v = [&](int j) {
        const int s = j % STAGES;
        unsigned char* vs = v_s + (size_t)s * V_BYTES;
        const int row0 = (pt[pg_first + j] * nKV + kvh) * BN;
        mbar_expect_tx(&v_full[s], V_BYTES);
#pragma unroll
        for (int a = 0; a < DA; ++a) tma_load_2d(vs + a * KV_ATOM, &map_v, a * 64, row0, &v_full[s]);
      };
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int a = 0; a < DA; ++a) tma_load_3d(q_s + a * Q_ATOM, &map_q, a * 64, h, tok0, q_full);
      load_k(0);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          if (j + 1 >= STAGES) ok = mbar_wait(&k_free[(j + 1) % STAGES], (unsigned)((((j + 1) / STAGES) - 1) & 1), err, failed, 2);
          if (!ok) break;
          load_k(j + 1);
        }
        if (j >= STAGES) ok = mbar_wait(&v_free[j % STAGES], (unsigned)(((j / STAGES) - 1) & 1), err, failed, 3);
        if (!ok) break;
        load_v(j);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ---- tcgen05.mma: S one tile ahead, O += P V behind the softmax ----
      constexpr unsigned ID_S = idesc(BM, BN, 0);   // S[128 x 64]  = Q (K-major) x K (K-major)
      constexpr unsigned ID_O = idesc(BM, D, 1);    // O[128 x D]  += P (tensor memory) x V (MN-major)
      auto issue_s = [&](int j) {
        const unsigned char* ks = k_s + (size_t)(j % STAGES) * K_BYTES;
        // k steps of 16 along the head size; 4 steps per 64-wide atom, 32 bytes apart
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const unsigned long long a_desc = umma_desc(q_s + (kk / 4) * Q_ATOM + (kk % 4) * 32, 16, 1024);
          const unsigned long long b_desc = umma_desc(ks + (kk / 4) * KV_ATOM + (kk % 4) * 32, 16, 1024);
          umma(tmem + (unsigned)((j & 1) * S_COL), a_desc, b_desc, ID_S, kk != 0);
        }
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_free[j % STAGES]);
      };
      bool ok = mbar_wait(q_full, 0, err, failed, 4);
      if (ok) ok = mbar_wait(&k_full[0], 0, err, failed, 5);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_s(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          // S of the next tile goes into the other buffer: the P V product that read it was issued before
          ok = mbar_wait(&k_full[(j + 1) % STAGES], (unsigned)(((j + 1) / STAGES) & 1), err, failed, 6);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(j + 1);
        }
        ok = mbar_wait(&v_full[j % STAGES], (unsigned)((j / STAGES) & 1), err, failed, 7);
        if (ok) ok = mbar_wait(&p_ready[j & 1], (unsigned)((j >> 1) & 1), err, failed, 8);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned char* vs = v_s + (size_t)(j % STAGES) * V_BYTES;
        // k steps of 16 keys: 8 columns of P; in V two 8-row swizzle groups = 2048 bytes; V is MN-major:
        // 64 d contiguous per key, the next 64-wide atom KV_ATOM bytes on (leading offset)
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const unsigned long long b_desc = umma_desc(vs + kk * 2048, KV_ATOM, 1024);
          umma_ts(tmem + O_COL, tmem + (unsigned)((j & 1) * S_COL + kk * 8), b_desc, ID_O, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&v_free[j % STAGES]);
        umma_commit(o_done);
      }
    }
  } else {
    // ---- softmax: one thread per query row ----
    const int r = warp * 32 + lane;                       // tile row = TMEM lane
    const int qpos = pos0 + r;
    const unsigned lane_base = tmem + ((unsigned)(warp * 32) << 16);
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = mbar_wait(&s_full[j & 1], (unsigned)((j >> 1) & 1), err, failed, 9);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const unsigned s_addr = lane_base + (unsigned)((j & 1) * S_COL);
      const int key0 = (pg_first + j) * BN;
      float sc[BN];
      {
        unsigned r0[32], r1[32];
        tmem_ld32_issue(s_addr, r0);
        tmem_ld32_issue(s_addr + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sc[i] = __uint_as_float(r0[i]); sc[32 + i] = __uint_as_float(r1[i]); }
      }
      // only tiles that reach the diagonal or the window's far edge need a mask (uniform for the block)
      const bool masked = (key0 + BN - 1 > pos0) || (window > 0 && pos0 + BM - 1 - key0 >= window);
      float mx = -INFINITY;
      if (masked) {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int kp = key0 + i;
          bool vis = kp <= qpos;
          if (window > 0) vis = vis && (qpos - kp < window);
          sc[i] = vis ? sc[i] : -INFINITY;
          mx = fmaxf(mx, sc[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < BN; ++i) mx = fmaxf(mx, sc[i]);
      }
      const float m_new = fmaxf(m_run, mx * scale_log2);
      float alpha = 1.f;
      if (__any_sync(0xffffffffu, m_new - m_run > GROW)) {
        // some row's maximum grew by much: every row of the warp takes its exact maximum and rescales
        alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_run - m_new);
        m_run = m_new;
        if (j > 0) {
          // S of tile j is done, hence every product issued before it, the P V of tile j-2 among them: the
          // barrier is in phase j-1 or j, which one parity bit tells apart
          ok = mbar_wait(o_done, (unsigned)((j - 1) & 1), err, failed, 10);   // O holds tiles 0 .. j-1
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int c = 0; c < D; c += 32) {
            unsigned v[32];
            tmem_ld32_issue(lane_base + O_COL + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st32(lane_base + O_COL + c, v);
          }
        }
      }
      const float m_use = m_run == -INFINITY ? 0.f : m_run;
      float sum = 0.f;
      unsigned pk[32];
#pragma unroll
      for (int i = 0; i < BN / 2; ++i) {
        const float p0 = fast_exp2(fmaf(sc[2 * i], scale_log2, -m_use));
        const float p1 = fast_exp2(fmaf(sc[2 * i + 1], scale_log2, -m_use));
        sum += p0 + p1;
        pk[i] = pack_bf16(p0, p1);
      }
      tmem_st32(s_addr, pk);   // P over the first half of its own S buffer
      tmem_st_wait();
      l_run = l_run * alpha + sum;
      if (j > 0 && j == n_tiles - 1) {
        // A parity wait tells two phases apart, not three.  Having seen S of the last tile only proves the
        // P V product of tile n-3 done.  The one of tile n-2 is awaited here, while the last one cannot have
        // run (it needs this thread's arrival below): the barrier is in phase n-2 or n-1.  After the arrival
        // it is in phase n-1 or n, which the wait behind the loop tells apart.  (Waiting for both behind the
        // loop would hang a thread that slept through phase n-1.)
        ok = mbar_wait(o_done, (unsigned)((j - 1) & 1), err, failed, 20);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&p_ready[j & 1]);
    }
    if (ok) {
      ok = mbar_wait(o_done, (unsigned)((n_tiles - 1) & 1), err, failed, 12);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* dst = out + ((size_t)(tok0 + r) * nH + h) * D;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        unsigned v[32];
        tmem_ld32_issue(lane_base + O_COL + c, v);
        tmem_ld_wait();
        if (r < rows) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c + i) = w;
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*failed) {
    // a wait ran out: give copies that may still be in flight a bounded time to land
    if (threadIdx.x == 0) {
      const long long t0 = clock64();
      for (int s = 0; s < STAGES; ++s) {
        while (!mbar_try_wait(&k_full[s], 0) && !mbar_try_wait(&k_full[s], 1) && clock64() - t0 < WAIT_CYCLES) {}
        while (!mbar_try_wait(&v_full[s], 0) && !mbar_try_wait(&v_full[s], 1) && clock64() - t0 < WAIT_CYCLES) {}
      }
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
}  // namespace

DRYFT_API int dryft_attn_prefill_tc_head_dim() { return D; }

// q [n_tokens, nH, D]; k_pages / v_pages [n_pages, nKV, 64, D]; out [n_tokens, nH * D]; all bfloat16.
DRYFT_API int dryft_attn_prefill_tc(const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                                    int max_pages, const int* tile_tok0, const int* tile_rows, const int* tok_slot,
                                    const int* tok_pos, void* out, int n_tiles, int n_tokens, int n_pages, int nH, int nKV,
                                    float scale, int window, int* err, cudaStream_t st) {
  if (n_tiles <= 0) return 0;
  if (nH != nKV * G || nH > 65535) return DRYFT_ERR_UNSUPPORTED;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return DRYFT_ERR_UNSUPPORTED;
  CUtensorMap map_q, map_k, map_v;
  {
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)nH, (cuuint64_t)n_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)nH * D * 2};
    cuuint32_t box[3] = {64, 1, BM};
    cuuint32_t estr[3] = {1, 1, 1};
    if (enc(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return DRYFT_ERR_UNSUPPORTED;
  }
  for (int which = 0; which < 2; ++which) {
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)n_pages * nKV * BN};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, BN};
    cuuint32_t estr[2] = {1, 1};
    if (enc(which ? &map_v : &map_k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(which ? v_pages : k_pages), dims,
            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return DRYFT_ERR_UNSUPPORTED;
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if ((long long)n_tiles * nH > 2147483647LL) return DRYFT_ERR_UNSUPPORTED;
  dim3 grid((unsigned)(n_tiles * nH));
  attn_prefill_tc_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(map_q, map_k, map_v, page_table, max_pages, tile_tok0, tile_rows,
                                                           tok_slot, tok_pos, (bf16*)out, nH, nKV,
                                                           scale * 1.4426950408889634f, window, err);
  return launch_status();
}
