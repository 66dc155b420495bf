// Attention of independent query rows over the paged cache ("split-KV"): the decode kernel of both
// precisions, and the prefill kernel of the 32-bit path (a prompt token is just a row with its own
// position).  Compiled per model with -DDRYFT_HEAD_DIM, -DDRYFT_GROUP, -DDRYFT_PAGE.
//
// Grid (rows, kv heads, splits).  One block serves the GROUP query heads that share a kv head for
// one query row over one contiguous range of cache pages.  Row n at position p of slot s sees the
// keys j with  max(0, p+1-window) <= j <= p  (window <= 0: all keys) — the new token's own key is
// already in the cache (hari495/dryft, engine/dryft_qwen3/model.py:235,249-257;
// kernels/attn_decode.py:8-10,52-55).  Scores, the running maximum and the sums are 32-bit
// (attn_decode.py:77-90).  With one split the block writes the output; otherwise it writes an
// un-normalised partial (acc, m, l) and `attn_rows_reduce_kernel` combines them
// (attn_decode.py:102-118).
//
// No block waits on another block; there is no spin anywhere in this file.
#include "common.cuh"
#include "attn_rows_static.h"
#include <math.h>

#if !defined(DRYFT_HEAD_DIM) || !defined(DRYFT_GROUP) || !defined(DRYFT_PAGE)
#error "compile with -DDRYFT_HEAD_DIM=.. -DDRYFT_GROUP=.. -DDRYFT_PAGE=.."
#endif

namespace {
constexpr int D = DRYFT_HEAD_DIM;
constexpr int G = DRYFT_GROUP;
constexpr int PAGE = DRYFT_PAGE;
constexpr int THREADS = 128;
constexpr int NWARP = THREADS / 32;
constexpr int DIMS_PER_THREAD = (D + THREADS - 1) / THREADS;
static_assert(D % 16 == 0, "head size must be a multiple of 16");
static_assert(PAGE % 32 == 0, "page size must be a multiple of 32");

template <typename T> struct Smem {
  static constexpr int VEC = 16 / sizeof(T);       // elements per 16-byte vector
  static constexpr int KSTRIDE = D + VEC;          // padded K row: conflict-free row-per-thread reads
  static constexpr size_t bytes() {
    return sizeof(float) * (G * D + G * PAGE + 3 * G) + sizeof(T) * (size_t)(PAGE * KSTRIDE + PAGE * D) + 32;
  }
};

template <typename T>
__global__ void __launch_bounds__(THREADS) attn_rows_kernel(
    const T* __restrict__ q,                                   // [N, nH, D]
    const T* __restrict__ k_pages, const T* __restrict__ v_pages,  // [pages, nKV, PAGE, D]
    const int* __restrict__ page_table, int max_pages,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    T* __restrict__ out,                                       // [N, nH*D]
    float* __restrict__ part_o, float* __restrict__ part_ml,   // [N, nH, S, D], [N, nH, S, 2]
    int nKV, int n_splits, float scale, int window) {
  using L = Smem<T>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* kt = reinterpret_cast<T*>(smem_raw);                 // [PAGE][KSTRIDE]
  T* vt = kt + PAGE * L::KSTRIDE;                         // [PAGE][D]
  float* qs = reinterpret_cast<float*>(vt + PAGE * D);    // [G][D]
  float* sc = qs + G * D;                                 // [G][PAGE]
  float* m_s = sc + G * PAGE;                             // [G]
  float* l_s = m_s + G;
  float* a_s = l_s + G;

  const int n = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int nH = nKV * G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = tok_slot[n];

  if (slot < 0) {  // padding row: defined zeros, no cache access
    if (n_splits == 1) {
      for (int i = tid; i < G * D; i += THREADS) out[(size_t)n * nH * D + (size_t)kvh * G * D + i] = from_f32<T>(0.f);
    } else {
      for (int g = 0; g < G; ++g) {
        size_t pi = ((size_t)n * nH + kvh * G + g) * n_splits + split;
        for (int d = tid; d < D; d += THREADS) part_o[pi * D + d] = 0.f;
        if (tid == 0) { part_ml[pi * 2] = -INFINITY; part_ml[pi * 2 + 1] = 0.f; }
      }
    }
    return;
  }

  const int pos = tok_pos[n];
  const int kv_hi = pos + 1;                                        // exclusive
  const int kv_lo = window > 0 ? max(0, kv_hi - window) : 0;        // inclusive
  const int first_page = kv_lo / PAGE, last_page = (kv_hi - 1) / PAGE;
  const int n_pages = last_page - first_page + 1;
  const int per_split = (n_pages + n_splits - 1) / n_splits;
  const int pg_begin = first_page + split * per_split;
  const int pg_end = min(pg_begin + per_split, last_page + 1);

  for (int i = tid; i < G * D; i += THREADS) qs[i] = to_f32<T>(q[((size_t)n * nH + (size_t)kvh * G) * D + i]);
  if (tid < G) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; a_s[tid] = 1.f; }
  float acc[DIMS_PER_THREAD][G];
#pragma unroll
  for (int i = 0; i < DIMS_PER_THREAD; ++i)
#pragma unroll
    for (int g = 0; g < G; ++g) acc[i][g] = 0.f;

  const int* pt = page_table + (size_t)slot * max_pages;
  constexpr int VPR = D / L::VEC;  // 16-byte vectors per row
  for (int pg = pg_begin; pg < pg_end; ++pg) {
    const int page = pt[pg];
    const int p0 = pg * PAGE;
    const T* kp = k_pages + ((size_t)page * nKV + kvh) * PAGE * D;
    const T* vp = v_pages + ((size_t)page * nKV + kvh) * PAGE * D;
    __syncthreads();  // previous tile fully consumed
    for (int i = tid; i < PAGE * VPR; i += THREADS) {
      const int r = i / VPR, c = i % VPR;
      const int p = p0 + r;
      uint4 kv4 = make_uint4(0, 0, 0, 0), vv4 = make_uint4(0, 0, 0, 0);
      if (p >= kv_lo && p < kv_hi) {
        kv4 = reinterpret_cast<const uint4*>(kp + (size_t)r * D)[c];
        vv4 = reinterpret_cast<const uint4*>(vp + (size_t)r * D)[c];
      }
      *reinterpret_cast<uint4*>(kt + r * L::KSTRIDE + c * L::VEC) = kv4;
      *reinterpret_cast<uint4*>(vt + r * D + c * L::VEC) = vv4;
    }
    __syncthreads();
    // scores: item -> (head g, key r); consecutive threads take consecutive keys
    for (int item = tid; item < G * PAGE; item += THREADS) {
      const int g = item / PAGE, r = item % PAGE;
      const int p = p0 + r;
      float s = -INFINITY;
      if (p >= kv_lo && p < kv_hi) {
        const T* kr = kt + r * L::KSTRIDE;
        const float* qg = qs + g * D;
        float dot = 0.f;
#pragma unroll 4
        for (int c = 0; c < VPR; ++c) {
          uint4 raw = *reinterpret_cast<const uint4*>(kr + c * L::VEC);
          const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int t = 0; t < L::VEC; ++t) dot = fmaf(qg[c * L::VEC + t], to_f32<T>(e[t]), dot);
        }
        s = dot * scale;
      }
      sc[item] = s;
    }
    __syncthreads();
    // online softmax, one warp per head
    for (int g = warp; g < G; g += NWARP) {
      float mx = -INFINITY;
      for (int r = lane; r < PAGE; r += 32) mx = fmaxf(mx, sc[g * PAGE + r]);
      mx = warp_max(mx);
      const float m_old = m_s[g];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int r = lane; r < PAGE; r += 32) {
        const float s = sc[g * PAGE + r];
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        sc[g * PAGE + r] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float alpha = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
        a_s[g] = alpha;
        m_s[g] = m_new;
        l_s[g] = l_s[g] * alpha + sum;
      }
    }
    __syncthreads();
    // acc = acc*alpha + P V ; thread owns output dims tid, tid+THREADS, ...
#pragma unroll
    for (int i = 0; i < DIMS_PER_THREAD; ++i) {
      const int d = tid + i * THREADS;
      if (d < D) {
#pragma unroll
        for (int g = 0; g < G; ++g) acc[i][g] *= a_s[g];
        for (int r = 0; r < PAGE; ++r) {
          const float v = to_f32<T>(vt[r * D + d]);
#pragma unroll
          for (int g = 0; g < G; ++g) acc[i][g] = fmaf(sc[g * PAGE + r], v, acc[i][g]);
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < DIMS_PER_THREAD; ++i) {
    const int d = tid + i * THREADS;
    if (d >= D) continue;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int h = kvh * G + g;
      if (n_splits == 1) {
        const float l = l_s[g];
        out[((size_t)n * nH + h) * D + d] = from_f32<T>(l > 0.f ? acc[i][g] / l : 0.f);
      } else {
        part_o[(((size_t)n * nH + h) * n_splits + split) * D + d] = acc[i][g];
      }
    }
  }
  if (n_splits > 1 && tid < G) {
    size_t pi = ((size_t)n * nH + kvh * G + tid) * n_splits + split;
    part_ml[pi * 2] = m_s[tid];
    part_ml[pi * 2 + 1] = l_s[tid];
  }
}

// Combine the partials of one (row, head):  w_s = exp(m_s - max m);  o = sum w_s acc_s / sum w_s l_s.
template <typename T>
__global__ void attn_rows_reduce_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                        T* __restrict__ out, int n_splits) {
  const size_t rh = blockIdx.x;  // row * nH + head
  const float* ml = part_ml + rh * n_splits * 2;
  float mx = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, ml[s * 2]);
  float denom = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float m = ml[s * 2];
    if (m != -INFINITY) denom += expf(m - mx) * ml[s * 2 + 1];
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float num = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float m = ml[s * 2];
      if (m != -INFINITY) num += expf(m - mx) * part_o[(rh * n_splits + s) * D + d];
    }
    out[rh * D + d] = from_f32<T>(denom > 0.f ? num / denom : 0.f);
  }
}

template <typename T>
int launch(const void* q, const void* k_pages, const void* v_pages, const int* page_table, int max_pages,
           const int* tok_slot, const int* tok_pos, void* out, float* part_o, float* part_ml, int n_rows, int nKV,
           int n_splits, float scale, int window, cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (n_splits < 1 || nKV < 1 || nKV > 65535 || n_splits > 65535) return DRYFT_ERR_UNSUPPORTED;
  if (n_splits > 1 && (!part_o || !part_ml)) return DRYFT_ERR_UNSUPPORTED;
  const size_t smem = Smem<T>::bytes();
  if (smem > 227 * 1024) return DRYFT_ERR_UNSUPPORTED;
  // per instantiation and per device (the attribute belongs to the device's copy of the kernel); set outside any
  // stream capture by the first (eager) launch on that device
  static bool attr_set[64] = {false};
  if (smem > 48 * 1024) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DRYFT_ERR_UNSUPPORTED;
    if (!attr_set[dev]) {
      e = cudaFuncSetAttribute(attn_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      attr_set[dev] = true;
    }
  }
  dim3 grid(n_rows, nKV, n_splits);
  attn_rows_kernel<T><<<grid, THREADS, smem, st>>>((const T*)q, (const T*)k_pages, (const T*)v_pages, page_table,
                                                  max_pages, tok_slot, tok_pos, (T*)out, part_o, part_ml, nKV,
                                                  n_splits, scale, window);
  int rc = launch_status();
  if (rc || n_splits == 1) return rc;
  attn_rows_reduce_kernel<T><<<(unsigned)((size_t)n_rows * nKV * G), D < 128 ? 64 : 128, 0, st>>>(part_o, part_ml, (T*)out, n_splits);
  return launch_status();
}
}  // namespace

// The sizes this library was compiled for; the loader checks them against the model's.
DRYFT_API int dryft_attn_rows_head_dim() { return D; }
DRYFT_API int dryft_attn_rows_group() { return G; }
DRYFT_API int dryft_attn_rows_page() { return PAGE; }

DRYFT_API int dryft_attn_rows(int is_bf16, const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                              int max_pages, const int* tok_slot, const int* tok_pos, void* out, float* part_o,
                              float* part_ml, int n_rows, int nKV, int n_splits, float scale, int window, cudaStream_t st) {
  return is_bf16 ? launch<__nv_bfloat16>(q, k_pages, v_pages, page_table, max_pages, tok_slot, tok_pos, out, part_o, part_ml,
                                         n_rows, nKV, n_splits, scale, window, st)
                 : launch<float>(q, k_pages, v_pages, page_table, max_pages, tok_slot, tok_pos, out, part_o, part_ml,
                                 n_rows, nKV, n_splits, scale, window, st);
}

// ------------------------------------------------------------------------------------------
// The same attention for callers that cannot allocate device memory (see attn_rows_static.h).
// The split partials live in a file-scope device array instead of buffers handed in.  In host
// code the array's name is only a stand-in for the symbol, not a device address, so the address
// is asked of the runtime once per device, with that device current, and kept.
// ------------------------------------------------------------------------------------------
namespace {
static __device__ __align__(256) float g_static_scratch[DRYFT_ATTN_ROWS_STATIC_FLOATS];
constexpr int MAX_DEVICES = 64;
float* g_static_scratch_ptr[MAX_DEVICES] = {nullptr};
}  // namespace

DRYFT_API int dryft_attn_rows_static_scratch(int is_bf16, const void* q, const void* k_pages, const void* v_pages,
                                             const int* page_table, int max_pages, const int* tok_slot, const int* tok_pos,
                                             void* out, int n_rows, int nKV, int n_splits, float scale, int window,
                                             cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (n_splits < 1 || nKV < 1 || nKV > 65535 || n_splits > 65535) return DRYFT_ERR_UNSUPPORTED;  // the grid's limits
  // partial outputs [rows, heads, splits, D] and (max, sum) pairs [rows, heads, splits, 2].  The size check divides
  // instead of multiplying, so that no count, however large, can wrap around and pass.
  const unsigned long long heads = (unsigned long long)nKV * G;                      // < 2^20
  const unsigned long long per_row = heads * (unsigned long long)n_splits * (D + 2);  // < 2^45
  if (n_splits > 1 && (unsigned long long)n_rows > (unsigned long long)DRYFT_ATTN_ROWS_STATIC_FLOATS / per_row)
    return DRYFT_ERR_SCRATCH_TOO_SMALL;
  const unsigned long long need_o = (unsigned long long)n_rows * heads * n_splits * D;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return DRYFT_ERR_UNSUPPORTED;
  if (g_static_scratch_ptr[dev] == nullptr) {  // set-up, once per device: the first call on a device
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    g_static_scratch_ptr[dev] = ptr;
  }
  float* part_o = g_static_scratch_ptr[dev];
  float* part_ml = part_o + need_o;
  // Nothing in the scratch has to start at zero: every split writes its partial of every
  // (row, head) before the combining kernel reads any of them.
  return is_bf16 ? launch<__nv_bfloat16>(q, k_pages, v_pages, page_table, max_pages, tok_slot, tok_pos, out, part_o, part_ml,
                                         n_rows, nKV, n_splits, scale, window, st)
                 : launch<float>(q, k_pages, v_pages, page_table, max_pages, tok_slot, tok_pos, out, part_o, part_ml,
                                 n_rows, nKV, n_splits, scale, window, st);
}

DRYFT_API long long dryft_attn_rows_static_scratch_floats() { return (long long)DRYFT_ATTN_ROWS_STATIC_FLOATS; }
