// Decode attention in one launch (bfloat16): per-head q/k RMSNorm + rotate-half RoPE of the new
// token, write of its K and V into the paged cache, attention of its GROUP query heads over the
// cache split across blocks, and the combination of the splits — what hari495/dryft does in three
// kernels (kernels/rope_qknorm.py:50-99 decode mapping; kernels/attn_decode.py:36-99 split-KV;
// kernels/attn_decode.py:102-118 reduce).  Compiled per model with -DDRYFT_HEAD_DIM, -DDRYFT_GROUP,
// -DDRYFT_PAGE.
//
// Grid (rows, kv heads, splits); a row is one sequence's new token.  Every block rebuilds the row's
// GROUP rotated queries (cheap, and it saves a launch and a round trip through memory); the one block
// whose page range holds the token's own position also makes the new key and value and writes them
// into the cache before anyone in the block reads that page.  Both products run on the tensor cores
// (mma.sync.m16n8k16) with a slice's 16 keys as the 16-row operand and the token's GROUP query heads as
// the 8 columns (two column tiles above 8 heads): S^T = K Q^T, then O^T = V^T P^T with P transposed in
// registers (movmatrix).  A group of four heads fills half of that operand; as the rows of a 16-row
// operand it would fill a quarter, at twice the products, exponentials and accumulators.
// Inside a block each warp walks over 16-key slices of its own (no block-wide barrier in the loop):
// it requests the slice's K and V rows with cp.async into its own ring of shared-memory buffers, the
// next slice in flight while one is used, the first requests going out before the queries are rebuilt (the
// new token's own row is patched into the staged slice from shared memory, so the early request need
// not wait for the cache write); scores, running maximum and sums are 32-bit
// (attn_decode.py:77-90), P is rounded to bfloat16 for the second product (attn_decode.py:12-14,89).
// The warps' partial (m, l, acc) are combined through shared memory.  With several splits each block
// leaves its partial in global memory and takes a ticket; the block that draws the last ticket of a
// (row, kv head) combines all partials in split order, so the result does not depend on arrival
// order, and puts the ticket counter back to zero.  No block waits for another: there is no spin.
//
// Formulas and rounding points are those of csrc/rope_kv.cu and csrc/attn_prefill.cu.
#include "common.cuh"
#include <math.h>

#if !defined(DRYFT_HEAD_DIM) || !defined(DRYFT_GROUP) || !defined(DRYFT_PAGE)
#error "compile with -DDRYFT_HEAD_DIM=.. -DDRYFT_GROUP=.. -DDRYFT_PAGE=.."
#endif

namespace {
typedef __nv_bfloat16 bf16;
constexpr int D = DRYFT_HEAD_DIM;
constexpr int G = DRYFT_GROUP;
constexpr int PAGE = DRYFT_PAGE;
constexpr int SLICE = 16;                   // keys a warp handles at a time
constexpr int SPP = PAGE / SLICE;           // slices per page
constexpr int KS = D + 8;                   // padded row (elements): conflict-free ldmatrix
constexpr int KSTEPS = D / 16;
constexpr int MT = D / 16;                  // 16-wide tiles of the head size
constexpr int NT = (G + 7) / 8;             // 8-wide tiles of the query heads
static_assert(D % 16 == 0 && D <= 256, "head size 16..256 in steps of 16");
static_assert(G >= 1 && G <= 16, "1..16 query heads per kv head");
static_assert(PAGE % SLICE == 0, "page size must be a multiple of 16");
// shared memory: Q [8 or 16][KS] bf16 (rows from GROUP on zero) and the new token's K and V rows, then per warp STAGES stages of
// (K slice, V slice) [16][KS] bf16 each.
// The combine buffers (m, l: [NWARP][16]; acc: [NWARP][G][D] floats) overlay the stages at the end.
// The block's shape is a template: NWARP warps with STAGES slices staged per warp (STAGES - 1 in flight
// while one is used).  Few (row, kv head) pairs: wide blocks, one per SM, so that one sequence's keys
// are walked by many warps.  Many pairs: narrow blocks with deeper rings, several per SM, so that no SM
// waits on the one block it holds and the grid is not cut into a few coarse waves.
constexpr int PT_CACHE = 64;                // page numbers of a block kept in shared memory (more are read from global)
constexpr int Q_ROWS = (G + 7) / 8 * 8;                     // the query heads, padded with zero rows to whole column tiles
constexpr size_t Q_BYTES = (size_t)(Q_ROWS + 2) * KS * 2;  // then the new key and the new value
template <int NWARP, int STAGES> struct Shape {
  static constexpr int THREADS = NWARP * 32;
  static constexpr size_t WARP_STAGE_BYTES = (size_t)STAGES * 2 * SLICE * KS * 2;
  static constexpr size_t COMBINE_BYTES = (size_t)NWARP * 16 * 2 * 4 + (size_t)NWARP * G * D * 4 + (size_t)G * D * 4 + (size_t)G * 2 * 4;
  static constexpr size_t PIPE_BYTES = NWARP * WARP_STAGE_BYTES;
  static constexpr size_t SMEM_BYTES = Q_BYTES + (PIPE_BYTES > COMBINE_BYTES ? PIPE_BYTES : COMBINE_BYTES);
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldsm_x2(unsigned& r0, unsigned& r1, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(s));
}
// an 8 x 8 block of 16-bit values held as an mma fragment (row lane / 4, columns 2 (lane mod 4) and + 1), transposed
__device__ __forceinline__ unsigned movmatrix_t(unsigned v) {
  unsigned r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ void ldsm_x4_t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float bfr(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a float of block `rank`'s shared memory at the same offset as `local` (between two cluster barriers)
__device__ __forceinline__ float ld_remote(const float* local, unsigned rank) {
  unsigned raddr;
  float v;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"((unsigned)__cvta_generic_to_shared(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(raddr));
  return v;
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Rotary constants of one token for a lane: pairs j = lane + 32 * jj.  They depend on the position only.
constexpr int MAXJ = (D / 2 + 31) / 32;
struct RopeConsts {
  float cs[MAXJ], sn[MAXJ];            // cos / sin, rounded to bfloat16
  float wq_a[MAXJ], wq_b[MAXJ];        // q norm weight at j and j + R/2
  float wk_a[MAXJ], wk_b[MAXJ];        // k norm weight
};
__device__ __forceinline__ void rope_consts(RopeConsts& c, const float* __restrict__ wq, const float* __restrict__ wk,
                                            const float* __restrict__ inv_freq, int pos, int R, int has_norm, int lane) {
  const int half = R >> 1;
#pragma unroll
  for (int jj = 0; jj < MAXJ; ++jj) {
    const int j = lane + 32 * jj;
    c.cs[jj] = 1.f; c.sn[jj] = 0.f;
    c.wq_a[jj] = c.wq_b[jj] = c.wk_a[jj] = c.wk_b[jj] = 1.f;
    if (j < half) {
      float sn, cs;
      sincosf((float)pos * inv_freq[j], &sn, &cs);
      c.cs[jj] = bfr(cs);
      c.sn[jj] = bfr(sn);
      if (has_norm) { c.wq_a[jj] = wq[j]; c.wq_b[jj] = wq[j + half]; c.wk_a[jj] = wk[j]; c.wk_b[jj] = wk[j + half]; }
    }
  }
}
// One warp: RMSNorm (optional) + RoPE of one head `src` [D] -> dst (bf16), with the token's constants
// already in registers: one read of the head, one reduction, one write.  Same arithmetic as
// qk_norm_rope_store_kernel.  `w` is only read for dims beyond the rotary part.
__device__ __forceinline__ void norm_rope_head(const bf16* __restrict__ src, const float* __restrict__ w, const RopeConsts& c,
                                               bool is_q, int R, float eps, int has_norm, bf16* dst, bf16* dst2, int lane) {
  const int half = R >> 1;
  float a[MAXJ], b[MAXJ];
  float ss = 0.f;
#pragma unroll
  for (int jj = 0; jj < MAXJ; ++jj) {
    const int j = lane + 32 * jj;
    a[jj] = b[jj] = 0.f;
    if (j < half) {
      a[jj] = ld_prev_bf16(src + j);   // the projection before this launch wrote it
      b[jj] = ld_prev_bf16(src + j + half);
      ss += a[jj] * a[jj] + b[jj] * b[jj];
    }
  }
  float inv = 1.f;
  if (has_norm) {
    for (int i = R + lane; i < D; i += 32) {
      const float v = ld_prev_bf16(src + i);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)D + eps);
  }
#pragma unroll
  for (int jj = 0; jj < MAXJ; ++jj) {
    const int j = lane + 32 * jj;
    if (j < half) {
      float x = a[jj], y = b[jj];
      if (has_norm) {
        x = bfr(bfr(x * inv) * (is_q ? c.wq_a[jj] : c.wk_a[jj]));
        y = bfr(bfr(y * inv) * (is_q ? c.wq_b[jj] : c.wk_b[jj]));
      }
      const bf16 o1 = __float2bfloat16_rn(__fadd_rn(bfr(__fmul_rn(x, c.cs[jj])), -bfr(__fmul_rn(y, c.sn[jj]))));
      const bf16 o2 = __float2bfloat16_rn(__fadd_rn(bfr(__fmul_rn(y, c.cs[jj])), bfr(__fmul_rn(x, c.sn[jj]))));
      dst[j] = o1;
      dst[j + half] = o2;
      if (dst2) { dst2[j] = o1; dst2[j + half] = o2; }
    }
  }
  for (int i = R + lane; i < D; i += 32) {
    float x = ld_prev_bf16(src + i);
    if (has_norm) x = bfr(bfr(x * inv) * w[i]);
    dst[i] = __float2bfloat16_rn(x);
    if (dst2) dst2[i] = __float2bfloat16_rn(x);
  }
}

struct Params {
  const bf16* qkv; int qkv_stride;            // [rows, q | k | v]
  const float* wq; const float* wk; const float* inv_freq;
  const int* tok_slot; const int* tok_pos;
  bf16* k_pages; bf16* v_pages;               // [pages, nKV, PAGE, D]
  const int* page_table; int max_pages;
  bf16* out;                                  // [rows, nH * D]
  float* part_o; float* part_ml; int* tickets;  // [rows, nKV, S, G, D], [rows, nKV, S, G, 2], [rows * nKV]
  int nKV; int n_splits; float scale; int window; int R; float eps; int has_norm; int write_kv;
  int cluster;   // the splits of a (row, kv head) are the blocks of one thread-block cluster
};

template <int NWARP, int STAGES>
__global__ void __launch_bounds__(NWARP * 32) attn_decode_kernel(const Params p) {
  constexpr int THREADS = Shape<NWARP, STAGES>::THREADS;
  constexpr size_t WARP_STAGE_BYTES = Shape<NWARP, STAGES>::WARP_STAGE_BYTES;
  extern __shared__ __align__(16) unsigned char smem[];
  bf16* qs = reinterpret_cast<bf16*>(smem);                        // [Q_ROWS][KS], rows >= G zero
  unsigned char* pipe = smem + Q_BYTES;
  __shared__ int is_last;

  const int n = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int nH = p.nKV * G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  pdl_launch_dependents();
  // What does not depend on the projection before this launch is done before waiting for it: the step's
  // token metadata and page table (complete before the step's first programmatic launch; the block's
  // page numbers go to shared memory), the token's rotary constants and norm weights, and, in a layer
  // that writes its own cache, the warps' first requests for keys and values of earlier tokens.
  const int slot = p.tok_slot[n];
  const int pos = p.tok_pos[n];
  const int kv_hi = pos + 1;
  const int kv_lo = p.window > 0 ? max(0, kv_hi - p.window) : 0;
  const int first_page = kv_lo / PAGE, last_page = pos / PAGE;
  const int n_pages = last_page - first_page + 1;
  const int per_split = (n_pages + p.n_splits - 1) / p.n_splits;
  const int pg_begin = first_page + split * per_split;
  const int pg_end = min(pg_begin + per_split, last_page + 1);
  const int* pt = p.page_table + (size_t)(slot < 0 ? 0 : slot) * p.max_pages;
  __shared__ int pt_s[PT_CACHE];
  if (slot >= 0)
    for (int i = tid; i < min(pg_end - pg_begin, PT_CACHE); i += THREADS) pt_s[i] = pt[pg_begin + i];
  RopeConsts rc;
  if (slot >= 0) rope_consts(rc, p.wq, p.wk, p.inv_freq, pos, p.R, p.has_norm, lane);
  __syncthreads();
  auto page_of = [&](int pg) { return pg - pg_begin < PT_CACHE ? pt_s[pg - pg_begin] : pt[pg]; };
  // ---- each warp's first slices are requested before anything else is computed ----
  bf16* stage = reinterpret_cast<bf16*>(pipe + (size_t)warp * WARP_STAGE_BYTES);  // [STAGES][K|V][SLICE][KS]
  // slices of this block, in key order: slice index sl covers keys sl*16 .. sl*16+15
  const int sl_begin = max(pg_begin * SPP, kv_lo / SLICE);
  const int sl_end = min(pg_end * SPP, (kv_hi + SLICE - 1) / SLICE);
  constexpr int CPR = D / 8;
  // a lane copies 16-byte chunk (lane % CPL) of rows lane / CPL, lane / CPL + RPI, ...: fixed offsets
  constexpr int CPL = CPR < 32 ? CPR : 32;        // chunks of one row handled side by side
  constexpr int RPI = 32 / CPL;                   // rows per instruction
  constexpr int CREP = CPR / CPL;                 // chunk repeats per row (head sizes above 256 elements: none)
  const int lr = lane / CPL, lc = lane % CPL;
  auto request = [&](int sl, int st) {
    if (sl < sl_end) {
      const int pg = sl / SPP;
      const size_t base = (((size_t)page_of(pg) * p.nKV + kvh) * PAGE + (size_t)(sl % SPP) * SLICE) * D;
      const bf16* ksrc = p.k_pages + base + (size_t)lr * D + lc * 8;
      const bf16* vsrc = p.v_pages + base + (size_t)lr * D + lc * 8;
      bf16* kd = stage + (size_t)st * 2 * SLICE * KS + lr * KS + lc * 8;
      bf16* vd = kd + SLICE * KS;
#pragma unroll
      for (int r = 0; r < SLICE; r += RPI)
#pragma unroll
        for (int c = 0; c < CREP; ++c) {
          if ((SLICE % RPI == 0 && 32 % CPL == 0) || (r + lr < SLICE && lane < RPI * CPL)) {
            cp_async16(kd + r * KS + c * CPL * 8, ksrc + (size_t)r * D + c * CPL * 8);
            cp_async16(vd + r * KS + c * CPL * 8, vsrc + (size_t)r * D + c * CPL * 8);
          }
        }
    }
    cp_async_commit();
  };
  // a layer that reads another layer's cache must see that layer's write of this step's token first
  const bool early = slot >= 0 && p.write_kv;
  if (early) {
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) request(sl_begin + warp + i * NWARP, i);
  }

  pdl_wait();  // the projection that made qkv is complete
  if (slot < 0) {  // padding row: defined zeros (written by split 0), no cache access, no ticket
    if (split == 0)
      for (int i = tid; i < G * D; i += THREADS) p.out[(size_t)n * nH * D + (size_t)kvh * G * D + i] = __float2bfloat16_rn(0.f);
    return;
  }
  const bf16* row = p.qkv + (size_t)n * p.qkv_stride;

  if (!early) {
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) request(sl_begin + warp + i * NWARP, i);
  }

  // ---- the row's queries; and, in the block that owns the last page, the new key and value ----
  bf16* new_k = qs + Q_ROWS * KS;
  bf16* new_v = new_k + KS;
  for (int i = tid; i < (Q_ROWS - G) * (D / 8); i += THREADS)  // zero the padding rows of Q
    *reinterpret_cast<uint4*>(qs + (G + i / (D / 8)) * KS + (i % (D / 8)) * 8) = make_uint4(0, 0, 0, 0);
  const bool owns_new = p.write_kv && last_page >= pg_begin && last_page < pg_end;
  const int n_items = G + (owns_new ? 2 : 0);
  for (int item = warp; item < n_items; item += NWARP) {
    if (item < G) {
      norm_rope_head(row + (size_t)(kvh * G + item) * D, p.wq, rc, true, p.R, p.eps, p.has_norm, qs + item * KS, nullptr, lane);
    } else {
      const size_t off = (((size_t)page_of(last_page) * p.nKV + kvh) * PAGE + (pos % PAGE)) * D;
      if (item == G) {
        norm_rope_head(row + (size_t)(nH + kvh) * D, p.wk, rc, false, p.R, p.eps, p.has_norm, p.k_pages + off, new_k, lane);
      } else {
        const bf16* vsrc = row + (size_t)(nH + p.nKV + kvh) * D;
        for (int i = lane; i < D; i += 32) {
          const bf16 v = __ushort_as_bfloat16(ld_prev(reinterpret_cast<const unsigned short*>(vsrc) + i));   // written by the projection before this launch
          p.v_pages[off + i] = v;
          new_v[i] = v;
        }
      }
    }
  }
  __syncthreads();  // queries (and the new key and value) are in shared memory

  // ---- each warp walks its own 16-key slices of the block's pages ----
  // The slice's 16 keys are the 16-row operand and the query heads the 8 columns (NT column tiles for more
  // than 8 heads): S^T = K Q^T and O^T = V^T P^T.  With the heads as the 16 rows, a group of four would
  // fill a quarter of the operand; this way it fills half, with half the products, exponentials and
  // accumulators.  A thread holds, of every tile, keys (or head dims) g and g + 8 for heads 2t and 2t + 1.
  float o_acc[NT][MT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) o_acc[nt][j][i] = 0.f;
  float m_run[NT][2], l_run[NT][2];   // heads nt*8 + 2t and + 1: running maximum (log2 units), this thread's share of the sum
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) { m_run[nt][0] = m_run[nt][1] = -INFINITY; l_run[nt][0] = l_run[nt][1] = 0.f; }
  // the queries' operand fragments are the same for every slice: read from shared memory once where they are few
  constexpr bool Q_IN_REGS = NT * KSTEPS * 2 <= 32;
  unsigned qb[Q_IN_REGS ? NT : 1][Q_IN_REGS ? KSTEPS : 1][2];
  const bf16* q_lane = qs + (lane & 7) * KS + ((lane >> 3) & 1) * 8;   // head (lane mod 8) of a column tile, low or high 8 of a k step
  if (Q_IN_REGS) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) ldsm_x2(qb[nt][kk][0], qb[nt][kk][1], q_lane + nt * 8 * KS + kk * 16);
  }
  const float scale_log2 = p.scale * 1.4426950408889634f;

  int it = 0;
  for (int sl = sl_begin + warp; sl < sl_end; sl += NWARP, ++it) {
    const int st = it % STAGES;
    request(sl + (STAGES - 1) * NWARP, (it + STAGES - 1) % STAGES);   // the next slice flies while this one is used
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    bf16* kst = stage + (size_t)st * 2 * SLICE * KS;
    bf16* vst = kst + SLICE * KS;
    if (sl == pos / SLICE) {
      const int r = pos % SLICE;
      if (owns_new) {  // the staged copy of the token's own row may predate its write
        for (int i = lane; i < CPR; i += 32) {
          *reinterpret_cast<uint4*>(kst + r * KS + i * 8) = *reinterpret_cast<const uint4*>(new_k + i * 8);
          *reinterpret_cast<uint4*>(vst + r * KS + i * 8) = *reinterpret_cast<const uint4*>(new_v + i * 8);
        }
      }
      // The rows behind the token's own hold what the page's last holder left.  Their keys are masked below
      // (probability exactly zero), but 0 * v is only 0 for a finite v: the staged values are zeroed
      // (the reference zeroes its whole cache once for the same reason, engine/dryft_qwen3/cache.py:43-47).
      for (int i = lane; i < (SLICE - 1 - r) * CPR; i += 32)
        *reinterpret_cast<uint4*>(vst + (r + 1 + i / CPR) * KS + (i % CPR) * 8) = make_uint4(0, 0, 0, 0);
      __syncwarp();
    }

    // S^T = K Q^T: 16 keys x 8 heads per column tile; the k steps go round two accumulators (chains of
    // dependent products half as long)
    constexpr int NCH = KSTEPS >= 2 ? 2 : 1;
    float sp[NCH][NT][4];
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) sp[c][nt][i] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      unsigned a0, a1, a2, a3;
      ldsm_x4(a0, a1, a2, a3, kst + (lane & 15) * KS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        unsigned b0, b1;
        if (Q_IN_REGS) { b0 = qb[nt][kk][0]; b1 = qb[nt][kk][1]; }
        else ldsm_x2(b0, b1, q_lane + nt * 8 * KS + kk * 16);
        mma16816(sp[kk % NCH][nt], a0, a1, a2, a3, b0, b1);
      }
    }
    // mask, online softmax (log2 domain); every slice visited holds at least one visible key
    const int key0 = sl * SLICE;
    const bool in0 = key0 + g >= kv_lo && key0 + g < kv_hi, in1 = key0 + g + 8 >= kv_lo && key0 + g + 8 < kv_hi;
    unsigned pb[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float t2 = sp[0][nt][i];
#pragma unroll
        for (int c = 1; c < NCH; ++c) t2 += sp[c][nt][i];
        v[i] = ((i < 2) ? in0 : in1) ? t2 * scale_log2 : -INFINITY;
      }
      float mx0 = fmaxf(v[0], v[2]), mx1 = fmaxf(v[1], v[3]);   // heads 2t and 2t + 1 over this thread's two keys
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {                          // ... and over the eight threads that hold the other keys
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
      }
      const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
      const float mu0 = (mn0 == -INFINITY) ? 0.f : mn0, mu1 = (mn1 == -INFINITY) ? 0.f : mn1;
      const float al0 = exp2f(m_run[nt][0] - mu0), al1 = exp2f(m_run[nt][1] - mu1);
      m_run[nt][0] = mn0;
      m_run[nt][1] = mn1;
      v[0] = exp2f(v[0] - mu0);
      v[1] = exp2f(v[1] - mu1);
      v[2] = exp2f(v[2] - mu0);
      v[3] = exp2f(v[3] - mu1);
      l_run[nt][0] = l_run[nt][0] * al0 + (v[0] + v[2]);
      l_run[nt][1] = l_run[nt][1] * al1 + (v[1] + v[3]);
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        o_acc[nt][j][0] *= al0;
        o_acc[nt][j][1] *= al1;
        o_acc[nt][j][2] *= al0;
        o_acc[nt][j][3] *= al1;
      }
      // P (bfloat16) as the second product's k x n operand: the 8 x 8 blocks (keys x heads) transposed in registers
      pb[nt][0] = movmatrix_t(pack_bf16(v[0], v[1]));
      pb[nt][1] = movmatrix_t(pack_bf16(v[2], v[3]));
    }
    // O^T += V^T P^T (one k16 step: the slice's 16 keys), 16 head dims a product
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      unsigned a0, a1, a2, a3;
      ldsm_x4_t(a0, a1, a2, a3, vst + ((lane & 7) + (lane >> 4) * 8) * KS + j * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) mma16816(o_acc[nt][j], a0, a1, a2, a3, pb[nt][0], pb[nt][1]);
    }
    __syncwarp();  // the stage may be refilled by the request two iterations on
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its stages: they become the combine buffers

  // ---- combine the warps of this block ----
  float* wm = reinterpret_cast<float*>(pipe);          // [NWARP][16]
  float* wl = wm + NWARP * 16;                         // [NWARP][16]
  float* wacc = wl + NWARP * 16;                       // [NWARP][G][D]
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    float l0 = l_run[nt][0], l1 = l_run[nt][1];
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, o);
      l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }
    const int h0 = nt * 8 + 2 * t;
    if (g == 0) {
      wm[warp * 16 + h0] = m_run[nt][0]; wl[warp * 16 + h0] = l0;
      wm[warp * 16 + h0 + 1] = m_run[nt][1]; wl[warp * 16 + h0 + 1] = l1;
    }
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int d = j * 16 + g;
      if (h0 < G) { wacc[(warp * G + h0) * D + d] = o_acc[nt][j][0]; wacc[(warp * G + h0) * D + d + 8] = o_acc[nt][j][2]; }
      if (h0 + 1 < G) { wacc[(warp * G + h0 + 1) * D + d] = o_acc[nt][j][1]; wacc[(warp * G + h0 + 1) * D + d + 8] = o_acc[nt][j][3]; }
    }
  }
  __syncthreads();
  float* bp_num = wacc + NWARP * G * D;   // [G][D] this block's partial (cluster mode)
  float* bp_ml = bp_num + G * D;          // [G][2] its maximum and sum
  const size_t pidx = ((size_t)n * p.nKV + kvh) * p.n_splits + split;
  for (int i = tid; i < G * D; i += THREADS) {
    const int h = i / D, d = i % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) mx = fmaxf(mx, wm[w * 16 + h]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) {
      const float m = wm[w * 16 + h];
      if (m == -INFINITY) continue;
      const float sc = exp2f(m - mx);
      num += sc * wacc[(w * G + h) * D + d];
      den += sc * wl[w * 16 + h];
    }
    if (p.n_splits == 1) {
      p.out[((size_t)n * nH + kvh * G + h) * D + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    } else if (p.cluster) {
      bp_num[i] = num;  // relative to mx
      if (d == 0) { bp_ml[h * 2] = mx; bp_ml[h * 2 + 1] = den; }
    } else {
      p.part_o[(pidx * G + h) * D + d] = num;  // relative to mx
      if (d == 0) { p.part_ml[(pidx * G + h) * 2] = mx; p.part_ml[(pidx * G + h) * 2 + 1] = den; }
    }
  }
  if (p.n_splits == 1) return;
  if (p.cluster) {
    // ---- the splits are the blocks of one cluster: every block combines a slice of the outputs over
    // all blocks' partials, in split order, reading them through distributed shared memory ----
    cluster_sync_all();
    const int per = (G * D + p.n_splits - 1) / p.n_splits;
    for (int i = split * per + tid; i < min((split + 1) * per, G * D); i += THREADS) {
      const int h = i / D, d = i % D;
      float mx = -INFINITY;
      for (int s2 = 0; s2 < p.n_splits; ++s2) mx = fmaxf(mx, ld_remote(bp_ml + h * 2, (unsigned)s2));
      float num = 0.f, den = 0.f;
      for (int s2 = 0; s2 < p.n_splits; ++s2) {
        const float m = ld_remote(bp_ml + h * 2, (unsigned)s2);
        if (m == -INFINITY) continue;
        const float sc = exp2f(m - mx);
        num += sc * ld_remote(bp_num + i, (unsigned)s2);
        den += sc * ld_remote(bp_ml + h * 2 + 1, (unsigned)s2);
      }
      p.out[((size_t)n * nH + kvh * G + h) * D + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    }
    cluster_sync_all();   // nobody leaves while another block may still read its partial
    return;
  }

  // ---- the block that draws the last ticket combines all splits, in split order ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int t = atomicAdd(&p.tickets[n * p.nKV + kvh], 1);
    is_last = (t == p.n_splits - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // The combine reads are independent of each other: all (m, l) pairs first, then one weight per
  // (split, head), then every output element sums its S partials with the loads in flight together.
  const size_t pbase = ((size_t)n * p.nKV + kvh) * p.n_splits;
  float* cm = reinterpret_cast<float*>(pipe);        // [S][G] maxima (the stages are free again)
  float* cl = cm + p.n_splits * G;                   // [S][G] sums
  float* cw = cl + p.n_splits * G;                   // [S][G] weights exp2(m - max) / total
  __syncthreads();
  for (int i = tid; i < p.n_splits * G; i += THREADS) {
    cm[i] = __ldcg(&p.part_ml[(pbase * G + i) * 2]);
    cl[i] = __ldcg(&p.part_ml[(pbase * G + i) * 2 + 1]);
  }
  __syncthreads();
  if (tid < G) {
    float mx = -INFINITY;
    for (int s2 = 0; s2 < p.n_splits; ++s2) mx = fmaxf(mx, cm[s2 * G + tid]);
    float den = 0.f;
    for (int s2 = 0; s2 < p.n_splits; ++s2) {
      const float m = cm[s2 * G + tid];
      const float sc = m == -INFINITY ? 0.f : exp2f(m - mx);  // maxima are kept in log2 units
      cw[s2 * G + tid] = sc;
      den += sc * cl[s2 * G + tid];
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    for (int s2 = 0; s2 < p.n_splits; ++s2) cw[s2 * G + tid] *= inv;
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += THREADS) {
    const int h = i / D, d = i % D;
    float num = 0.f;
#pragma unroll 8
    for (int s2 = 0; s2 < p.n_splits; ++s2) num += cw[s2 * G + h] * __ldcg(&p.part_o[((pbase + s2) * G + h) * D + d]);
    p.out[((size_t)n * nH + kvh * G + h) * D + d] = __float2bfloat16_rn(num);
  }
  if (tid == 0) p.tickets[n * p.nKV + kvh] = 0;  // ready for the next launch
}
template <int NWARP, int STAGES>
static int launch_shape(const Params& p, int n_rows, int nKV, int n_splits, int pdl, cudaStream_t st) {
  typedef Shape<NWARP, STAGES> S;
  if (S::SMEM_BYTES > 227 * 1024) return DRYFT_ERR_UNSUPPORTED;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_rows, nKV, n_splits);
  cfg.blockDim = dim3(S::THREADS);
  static bool attr_set = false;  // per shape; set by the first (eager) launch, outside any stream capture
  if (S::SMEM_BYTES > 48 * 1024 && !attr_set) {
    cudaError_t ea = cudaFuncSetAttribute(attn_decode_kernel<NWARP, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM_BYTES);
    if (ea != cudaSuccess) return (int)ea;
    attr_set = true;
  }
  cfg.dynamicSmemBytes = S::SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  if (p.cluster) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = (unsigned)n_splits;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, attn_decode_kernel<NWARP, STAGES>, p);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}
}  // namespace

DRYFT_API int dryft_attn_decode_head_dim() { return D; }
DRYFT_API int dryft_attn_decode_group() { return G; }

DRYFT_API int dryft_attn_decode(const void* qkv, int qkv_stride, const float* wq, const float* wk, const float* inv_freq,
                                const int* tok_slot, const int* tok_pos, void* k_pages, void* v_pages,
                                const int* page_table, int max_pages, void* out, float* part_o, float* part_ml,
                                int* tickets, int n_rows, int nKV, int n_splits, float scale, int window, int R, float eps,
                                int has_norm, int write_kv, int pdl, int shape, int cluster, cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (n_splits < 1 || nKV < 1 || nKV > 65535 || n_splits > 64 || (R & 1) || R > D || R < 0) return DRYFT_ERR_UNSUPPORTED;
  if (cluster && (n_splits < 2 || n_splits > 8)) cluster = 0;
  if (n_splits > 1 && !cluster && (!part_o || !part_ml || !tickets)) return DRYFT_ERR_UNSUPPORTED;
  Params p;
  p.qkv = (const bf16*)qkv; p.qkv_stride = qkv_stride; p.wq = wq; p.wk = wk; p.inv_freq = inv_freq;
  p.tok_slot = tok_slot; p.tok_pos = tok_pos; p.k_pages = (bf16*)k_pages; p.v_pages = (bf16*)v_pages;
  p.page_table = page_table; p.max_pages = max_pages; p.out = (bf16*)out; p.part_o = part_o; p.part_ml = part_ml;
  p.tickets = tickets; p.nKV = nKV; p.n_splits = n_splits; p.scale = scale; p.window = window; p.R = R; p.eps = eps;
  p.has_norm = has_norm; p.write_kv = write_kv; p.cluster = cluster;
  if (shape < 0) {
    // the widest block shape whose grid is resident at once (no second wave): 8, 4 or 2 warps
    static int sms = 0;
    if (sms == 0) {
      int dev = 0;
      if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        sms = 1;
    }
    const long long blocks = (long long)n_rows * nKV * n_splits;
    const long long usable = 227 * 1024;
    const long long per_sm_8 = usable / (long long)(Shape<8, 2>::SMEM_BYTES + 1024);   // 0: does not fit at all
    const long long per_sm_4 = usable / (long long)(Shape<4, 2>::SMEM_BYTES + 1024);
    shape = (per_sm_8 >= 1 && blocks <= sms * per_sm_8) ? 0 : ((per_sm_4 >= 1 && blocks <= sms * per_sm_4) ? 1 : 2);
    if (shape == 2 && (long long)(Shape<2, 2>::SMEM_BYTES + 1024) > usable) shape = per_sm_4 >= 1 ? 1 : 0;
  }
  return shape == 1 ? launch_shape<4, 2>(p, n_rows, nKV, n_splits, pdl, st)
       : shape == 2 ? launch_shape<2, 2>(p, n_rows, nKV, n_splits, pdl, st)
                    : launch_shape<8, 2>(p, n_rows, nKV, n_splits, pdl, st);
}
