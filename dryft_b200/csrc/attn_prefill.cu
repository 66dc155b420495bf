// Prefill attention (bfloat16): causal grouped-query attention of packed prompts of unequal lengths
// over the paged cache, flash style.  Compiled per model with -DDRYFT_HEAD_DIM, -DDRYFT_GROUP,
// -DDRYFT_PAGE (64).
//
// Grid (query tiles, query heads).  A tile is up to 64 consecutive query tokens of ONE sequence
// (tile_tok0 = first packed token, tile_rows = how many); its slot and first position are read from
// the step's token metadata.  The block's 4 warps own 16 query rows each.  It walks the sequence's
// cache pages from the first visible key to the tile's last position; each page is one K tile and
// one V tile [64, D], brought to shared memory with cp.async (two stages), so the keys written by
// this very step and those of earlier steps are read the same way — a prompt may therefore also be
// fed in chunks.  Q K^T and P V run on mma.sync.m16n8k16 (bf16 in, fp32 accumulate); scores, running
// maximum and sums are 32-bit; P is rounded to bfloat16 for the second product, as flash attention
// does (hari495/dryft relies on SDPA's flash kernel here, engine/dryft_qwen3/model.py:172-177, and
// rounds P the same way in its own decode kernel, kernels/attn_decode.py:12-14,89).
// Query at position p sees keys  max(0, p+1-window) .. p  (window <= 0: all), q head h reads kv head
// h / GROUP (model.py:65,172-178; config.py:99-101).
//
// No block waits on another block; the only waits are cp.async.wait_group and __syncthreads.
#include "common.cuh"
#include <math.h>

#if !defined(DRYFT_HEAD_DIM) || !defined(DRYFT_GROUP) || !defined(DRYFT_PAGE)
#error "compile with -DDRYFT_HEAD_DIM=.. -DDRYFT_GROUP=.. -DDRYFT_PAGE=.."
#endif

namespace {
constexpr int D = DRYFT_HEAD_DIM;
constexpr int G = DRYFT_GROUP;
constexpr int BN = DRYFT_PAGE;   // keys per tile = one cache page
constexpr int BM = 64;           // query rows per block
constexpr int NWARP = 4;
constexpr int THREADS = NWARP * 32;
constexpr int KS = D + 8;        // padded row stride (elements): conflict-free ldmatrix
constexpr int KSTEPS = D / 16;   // k16 steps of Q K^T
constexpr int NT = BN / 8;       // n8 tiles of the scores
constexpr int DT = D / 8;        // n8 tiles of the output
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size 16..256 in steps of 16");
static_assert(BN == 64, "the prefill kernel is written for 64-token pages");

typedef __nv_bfloat16 bf16;

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

constexpr size_t smem_bytes() { return sizeof(bf16) * (size_t)KS * (BM + 4 * BN); }

__device__ __forceinline__ void load_page(bf16* ks, bf16* vs, const bf16* kp, const bf16* vp, int tid) {
  constexpr int CPR = D / 8;  // 16-byte chunks per row
  for (int i = tid; i < BN * CPR; i += THREADS) {
    const int r = i / CPR, c = i % CPR;
    cp_async16(ks + r * KS + c * 8, kp + (size_t)r * D + c * 8);
    cp_async16(vs + r * KS + c * 8, vp + (size_t)r * D + c * 8);
  }
}

__global__ void __launch_bounds__(THREADS) attn_prefill_kernel(
    const bf16* __restrict__ q,                                      // [N, nH, D]
    const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,  // [pages, nKV, BN, D]
    const int* __restrict__ page_table, int max_pages,
    const int* __restrict__ tile_tok0, const int* __restrict__ tile_rows,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    bf16* __restrict__ out,                                          // [N, nH * D]
    int nH, int nKV, float scale_log2, int window) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);   // [BM][KS]
  bf16* ks = qs + BM * KS;                        // [2][BN][KS]
  bf16* vs = ks + 2 * BN * KS;                    // [2][BN][KS]

  // Heads run fastest: the host lists the tiles with the most keys first, so all heads of the longest
  // tiles start first and the short ones fill the gaps at the end (with tiles fastest, every head's
  // longest tile would be spread over the launch and the last of them would finish alone).
  const int tile = blockIdx.x / nH, h = blockIdx.x % nH, kvh = h / G;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tok0 = tile_tok0[tile], rows = tile_rows[tile];
  const int slot = tok_slot[tok0];
  if (slot < 0 || rows <= 0) return;  // padding tile (uniform for the block)
  const int pos0 = tok_pos[tok0];

  // ---- Q tile -> shared memory (rows beyond the tile are zero) ----
  {
    constexpr int CPR = D / 8;
    for (int i = tid; i < BM * CPR; i += THREADS) {
      const int r = i / CPR, c = i % CPR;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(tok0 + r) * nH + h) * D + c * 8);
      *reinterpret_cast<uint4*>(qs + r * KS + c * 8) = v;
    }
  }

  const int last_pos = pos0 + rows - 1;
  const int pg_first = window > 0 ? max(0, pos0 + 1 - window) / BN : 0;
  const int pg_last = last_pos / BN;
  const int* pt = page_table + (size_t)slot * max_pages;
  const size_t page_elems = (size_t)BN * D;

  auto page_ptr = [&](const bf16* base, int pg) { return base + ((size_t)pt[pg] * nKV + kvh) * page_elems; };

  load_page(ks, vs, page_ptr(k_pages, pg_first), page_ptr(v_pages, pg_first), tid);
  cp_async_commit();

  float o_acc[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[j][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};  // rows g and g+8 of this warp, in log2 units
  float l_run[2] = {0.f, 0.f};              // this thread's share of the row sums

  const int qrow0 = pos0 + warp * 16 + g;   // position of this thread's first row
  const int qrow1 = qrow0 + 8;

  for (int pg = pg_first; pg <= pg_last; ++pg) {
    const int stage = (pg - pg_first) & 1;
    if (pg + 1 <= pg_last) {
      load_page(ks + (stage ^ 1) * BN * KS, vs + (stage ^ 1) * BN * KS, page_ptr(k_pages, pg + 1),
                page_ptr(v_pages, pg + 1), tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* kst = ks + stage * BN * KS;
    const bf16* vst = vs + stage * BN * KS;

    // ---- S = Q K^T for this warp's 16 rows x 64 keys ----
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      unsigned a0, a1, a2, a3;
      ldsm_x4(a0, a1, a2, a3, qs + (warp * 16 + (lane & 15)) * KS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        unsigned b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, kst + (j * 8 + (lane & 7) + (lane >> 4) * 8) * KS + kk * 16 + ((lane >> 3) & 1) * 8);
        mma16816(s[j], a0, a1, a2, a3, b0, b1);
        mma16816(s[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }

    // ---- mask, online softmax (log2 domain) ----
    const int key0 = pg * BN;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kp = key0 + j * 8 + 2 * t + (i & 1);
        const int qp = (i < 2) ? qrow0 : qrow1;
        bool vis = kp <= qp;
        if (window > 0) vis = vis && (qp - kp < window);
        const float v = vis ? s[j][i] * scale_log2 : -INFINITY;
        s[j][i] = v;
        if (i < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
    const float mu0 = (mn0 == -INFINITY) ? 0.f : mn0, mu1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float al0 = exp2f(m_run[0] - mu0), al1 = exp2f(m_run[1] - mu1);  // exp2(-inf) = 0
    m_run[0] = mn0;
    m_run[1] = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      s[j][0] = exp2f(s[j][0] - mu0);
      s[j][1] = exp2f(s[j][1] - mu0);
      s[j][2] = exp2f(s[j][2] - mu1);
      s[j][3] = exp2f(s[j][3] - mu1);
      sum0 += s[j][0] + s[j][1];
      sum1 += s[j][2] + s[j][3];
    }
    l_run[0] = l_run[0] * al0 + sum0;
    l_run[1] = l_run[1] * al1 + sum1;
#pragma unroll
    for (int j = 0; j < DT; ++j) {
      o_acc[j][0] *= al0;
      o_acc[j][1] *= al0;
      o_acc[j][2] *= al1;
      o_acc[j][3] *= al1;
    }

    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      const unsigned a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      const unsigned a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const unsigned a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const unsigned a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int j = 0; j < DT; j += 2) {
        unsigned b0, b1, b2, b3;
        ldsm_x4_t(b0, b1, b2, b3, vst + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KS + j * 8 + (lane >> 4) * 8);
        mma16816(o_acc[j], a0, a1, a2, a3, b0, b1);
        mma16816(o_acc[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();  // both stages may be refilled only after every warp is done with this one
  }

  // ---- normalise and store ----
  float l0 = l_run[0], l1 = l_run[1];
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int r0 = warp * 16 + g, r1 = r0 + 8;
#pragma unroll
  for (int j = 0; j < DT; ++j) {
    const int d = j * 8 + 2 * t;
    if (r0 < rows)
      *reinterpret_cast<unsigned*>(out + ((size_t)(tok0 + r0) * nH + h) * D + d) = pack_bf16(o_acc[j][0] * inv0, o_acc[j][1] * inv0);
    if (r1 < rows)
      *reinterpret_cast<unsigned*>(out + ((size_t)(tok0 + r1) * nH + h) * D + d) = pack_bf16(o_acc[j][2] * inv1, o_acc[j][3] * inv1);
  }
}
}  // namespace

DRYFT_API int dryft_attn_prefill_head_dim() { return D; }

DRYFT_API int dryft_attn_prefill(const void* q, const void* k_pages, const void* v_pages, const int* page_table, int max_pages,
                                 const int* tile_tok0, const int* tile_rows, const int* tok_slot, const int* tok_pos,
                                 void* out, int n_tiles, int nH, int nKV, float scale, int window, cudaStream_t st) {
  if (n_tiles <= 0) return 0;
  if (nH != nKV * G || nH > 65535) return DRYFT_ERR_UNSUPPORTED;
  const size_t smem = smem_bytes();
  if (smem > 227 * 1024) return DRYFT_ERR_UNSUPPORTED;
  static bool attr_set = false;  // set by the first (eager) launch, outside any stream capture
  if (smem > 48 * 1024 && !attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if ((long long)n_tiles * nH > 2147483647LL) return DRYFT_ERR_UNSUPPORTED;
  dim3 grid((unsigned)(n_tiles * nH));
  attn_prefill_kernel<<<grid, THREADS, smem, st>>>((const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, page_table,
                                                  max_pages, tile_tok0, tile_rows, tok_slot, tok_pos, (bf16*)out, nH, nKV,
                                                  scale * 1.4426950408889634f, window);
  return launch_status();
}
