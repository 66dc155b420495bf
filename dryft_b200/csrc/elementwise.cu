// Step metadata, embedding gather, RMSNorm (plain, fused with the residual add, gathered rows)
// and SiLU*mul.  None of these depends on a model size at compile time: widths are runtime
// arguments and need not be powers of two; vector width falls back to scalar when a row is not a
// multiple of the vector.
//
// Reference counterparts (hari495/dryft): F.embedding at engine/dryft_qwen3/model.py:132,226;
// kernels/rmsnorm.py:21-39 (add + RMSNorm, rounding points); kernels/silu_mul.py:23-32.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// Step metadata: token n of the packed batch -> (slot, position).
//   cu_q[b]..cu_q[b+1]-1 are the tokens of sequence b; seq_slot[b] < 0 marks a padding sequence.
//   position = seq_len[slot] + offset within the sequence's tokens of this step.
// Tokens at or beyond cu_q[B] are padding: slot -1.
// ------------------------------------------------------------------------------------------
__global__ void step_meta_kernel(const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
                                 const int* __restrict__ seq_len, int n_tokens, int n_seqs,
                                 int* __restrict__ tok_slot, int* __restrict__ tok_pos) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= n_tokens) return;
  int lo = 0, hi = n_seqs;  // find b with cu_q[b] <= n < cu_q[b+1]
  if (n >= cu_q[n_seqs]) {
    tok_slot[n] = -1;
    tok_pos[n] = 0;
    return;
  }
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (cu_q[mid] <= n) lo = mid; else hi = mid;
  }
  int slot = seq_slot[lo];
  tok_slot[n] = slot;
  tok_pos[n] = slot < 0 ? 0 : seq_len[slot] + (n - cu_q[lo]);
}

// After a step: seq_len[slot] += tokens the sequence appended.
__global__ void step_advance_kernel(const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
                                    int* __restrict__ seq_len, int n_seqs) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_seqs) return;
  int slot = seq_slot[b];
  if (slot >= 0) seq_len[slot] += cu_q[b + 1] - cu_q[b];
}

DRYFT_API int dryft_step_meta(const int* cu_q, const int* seq_slot, const int* seq_len, int n_tokens, int n_seqs,
                              int* tok_slot, int* tok_pos, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  step_meta_kernel<<<(n_tokens + 255) / 256, 256, 0, st>>>(cu_q, seq_slot, seq_len, n_tokens, n_seqs, tok_slot, tok_pos);
  return launch_status();
}
DRYFT_API int dryft_step_advance(const int* cu_q, const int* seq_slot, int* seq_len, int n_seqs, cudaStream_t st) {
  if (n_seqs <= 0) return 0;
  step_advance_kernel<<<(n_seqs + 127) / 128, 128, 0, st>>>(cu_q, seq_slot, seq_len, n_seqs);
  return launch_status();
}

// Decode input from the per-sequence state: tokens[b] = last_token[slot[b]] (0 for padding).
__global__ void tokens_from_state_kernel(const int* __restrict__ seq_slot, const int* __restrict__ last_token,
                                         int* __restrict__ tokens, int n_seqs) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_seqs) return;
  int slot = seq_slot[b];
  tokens[b] = slot < 0 ? 0 : last_token[slot];
}
DRYFT_API int dryft_tokens_from_state(const int* seq_slot, const int* last_token, int* tokens, int n_seqs, cudaStream_t st) {
  if (n_seqs <= 0) return 0;
  tokens_from_state_kernel<<<(n_seqs + 127) / 128, 128, 0, st>>>(seq_slot, last_token, tokens, n_seqs);
  return launch_status();
}

// ------------------------------------------------------------------------------------------
// Embedding gather: out[n, :] = table[tokens[n], :].  A token id outside [0, vocab) yields a
// zero row and raises *err (the host validates ids first; this is the second fence).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table, T* __restrict__ out,
                             int hidden, int vocab, int* __restrict__ err) {
  const int n = blockIdx.x;
  const int tok = tokens[n];
  T* o = out + (size_t)n * hidden;
  if (tok < 0 || tok >= vocab) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(0.f);
    if (threadIdx.x == 0 && err) atomicExch(err, 1);
    return;
  }
  const T* src = table + (size_t)tok * hidden;
  constexpr int V = 16 / sizeof(T);
  if (hidden % V == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* o4 = reinterpret_cast<uint4*>(o);
    for (int i = threadIdx.x; i < hidden / V; i += blockDim.x) o4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = src[i];
  }
}

template <typename T>
static int embed_launch(const int* tokens, const void* table, void* out, int n, int hidden, int vocab, int* err, cudaStream_t st) {
  if (n <= 0) return 0;
  embed_kernel<T><<<n, 128, 0, st>>>(tokens, (const T*)table, (T*)out, hidden, vocab, err);
  return launch_status();
}
DRYFT_API int dryft_embed(int is_bf16, const int* tokens, const void* table, void* out, int n, int hidden, int vocab,
                          int* err, cudaStream_t st) {
  return is_bf16 ? embed_launch<__nv_bfloat16>(tokens, table, out, n, hidden, vocab, err, st)
                 : embed_launch<float>(tokens, table, out, n, hidden, vocab, err, st);
}

// ------------------------------------------------------------------------------------------
// RMSNorm family, one block per output row r:
//   src  = rows ? rows[r] : r                         (gather, for the final norm at wanted places)
//   s    = x[src] (+ delta[src] if delta)             summed in 32-bit, rounded to T   (rmsnorm.py:34)
//   x_out[src] = s                                    (if x_out; the new residual stream)
//   h[r] = T( w * T( s * rsqrt(mean(s^2) + eps) ) )   weight applied after the cast   (model.py:28-32)
// The summed row lives in shared memory (hidden floats), so x and delta are read once.
// ------------------------------------------------------------------------------------------
// 16-byte vector of T <-> floats
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };
template <typename T> __device__ __forceinline__ void load_vec(const T* p, float* v) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec16<T>::N; ++i) v[i] = to_f32<T>(e[i]);
}
template <typename T> __device__ __forceinline__ void store_vec(T* p, const float* v) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec16<T>::N; ++i) e[i] = from_f32<T>(v[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

template <typename T>
__global__ void rmsnorm_kernel(const T* x, const T* __restrict__ delta, const float* __restrict__ w,
                               const int* __restrict__ rows, T* x_out, T* __restrict__ h, int hidden, float eps, int aligned) {
  // x and x_out may be the same buffer (in-place residual update): no __restrict__ on them
  extern __shared__ __align__(16) float row[];  // hidden floats + 33 scratch
  float* scratch = row + ((hidden + 3) & ~3);
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const T* xr = x + (size_t)src * hidden;
  const T* dr = delta ? delta + (size_t)src * hidden : nullptr;
  T* xo = x_out ? x_out + (size_t)src * hidden : nullptr;
  T* hr = h + (size_t)r * hidden;
  constexpr int V = Vec16<T>::N;
  const bool vec = aligned && hidden % V == 0;  // every row then starts on a 16-byte boundary
  float ss = 0.f;
  if (vec) {
    for (int i = threadIdx.x * V; i < hidden; i += blockDim.x * V) {
      float v[V], d[V];
      load_vec<T>(xr + i, v);
      if (dr) {
        load_vec<T>(dr + i, d);
#pragma unroll
        for (int e = 0; e < V; ++e) v[e] = rnd<T>(v[e] + d[e]);
      }
#pragma unroll
      for (int e = 0; e < V; ++e) { row[i + e] = v[e]; ss += v[e] * v[e]; }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = to_f32<T>(xr[i]);
      if (dr) v = rnd<T>(v + to_f32<T>(dr[i]));
      row[i] = v;
      ss += v * v;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  if (vec) {
    for (int i = threadIdx.x * V; i < hidden; i += blockDim.x * V) {
      float v[V], o[V];
#pragma unroll
      for (int e = 0; e < V; ++e) { v[e] = row[i + e]; o[e] = w[i + e] * rnd<T>(v[e] * inv); }
      if (xo) store_vec<T>(xo + i, v);
      store_vec<T>(hr + i, o);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = row[i];
      if (xo) xo[i] = from_f32<T>(v);
      hr[i] = from_f32<T>(w[i] * rnd<T>(v * inv));
    }
  }
}


// Many rows at once (a prompt): small blocks, so that every row of the step is in flight together, and
// the summed row stays in registers (up to RMS_REG_VECS 16-byte vectors a thread) instead of shared memory.
constexpr int RMS_REG_VECS = 4;
template <typename T>
__global__ void rmsnorm_rows_kernel(const T* x, const T* __restrict__ delta, const float* __restrict__ w,
                                    const int* __restrict__ rows, T* x_out, T* __restrict__ h, int hidden, float eps) {
  __shared__ float scratch[33];
  constexpr int V = Vec16<T>::N;
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const T* xr = x + (size_t)src * hidden;
  const T* dr = delta ? delta + (size_t)src * hidden : nullptr;
  T* xo = x_out ? x_out + (size_t)src * hidden : nullptr;
  T* hr = h + (size_t)r * hidden;
  float v[RMS_REG_VECS][V];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < RMS_REG_VECS; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * V;
    if (i < hidden) {
      load_vec<T>(xr + i, v[k]);
      if (dr) {
        float d[V];
        load_vec<T>(dr + i, d);
#pragma unroll
        for (int e = 0; e < V; ++e) v[k][e] = rnd<T>(v[k][e] + d[e]);
      }
#pragma unroll
      for (int e = 0; e < V; ++e) ss += v[k][e] * v[k][e];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int k = 0; k < RMS_REG_VECS; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * V;
    if (i < hidden) {
      float o[V], wv[V];
#pragma unroll
      for (int e = 0; e < V; e += 4)   // the weight in 16-byte pieces (hidden % V == 0 and allocations are aligned)
        *reinterpret_cast<float4*>(wv + e) = __ldg(reinterpret_cast<const float4*>(w + i + e));
#pragma unroll
      for (int e = 0; e < V; ++e) o[e] = wv[e] * rnd<T>(v[k][e] * inv);
      if (xo) store_vec<T>(xo + i, v[k]);
      store_vec<T>(hr + i, o);
    }
  }
}

template <typename T>
static int rmsnorm_launch(const void* x, const void* delta, const float* w, const int* rows, void* x_out, void* h,
                          int n_rows, int hidden, float eps, cudaStream_t st) {
  if (n_rows <= 0) return 0;
  constexpr int V = Vec16<T>::N;
  // 16-byte accesses need every base address on a 16-byte boundary (and hidden % V == 0 for the rows)
  const int aligned = !(((uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)x_out | (uintptr_t)h) & 15);
  if (aligned && n_rows >= 256 && hidden % V == 0 && hidden / V <= RMS_REG_VECS * 1024) {
    const int vecs = hidden / V;
    int threads = ((vecs + RMS_REG_VECS - 1) / RMS_REG_VECS + 31) & ~31;
    if (threads < 64) threads = 64;
    rmsnorm_rows_kernel<T><<<n_rows, threads, 0, st>>>((const T*)x, (const T*)delta, w, rows, (T*)x_out, (T*)h, hidden, eps);
    return launch_status();
  }
  size_t smem = (size_t)(((hidden + 3) & ~3) + 33) * sizeof(float);
  if (smem > 200 * 1024) return DRYFT_ERR_UNSUPPORTED;
  static size_t attr_bytes = 48 * 1024;  // per instantiation; raised by an eager launch before any capture
  if (smem > attr_bytes) {
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_bytes = smem;
  }
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  rmsnorm_kernel<T><<<n_rows, threads, smem, st>>>((const T*)x, (const T*)delta, w, rows, (T*)x_out, (T*)h, hidden, eps, aligned);
  return launch_status();
}
DRYFT_API int dryft_rmsnorm(int is_bf16, const void* x, const void* delta, const float* w, const int* rows, void* x_out,
                            void* h, int n_rows, int hidden, float eps, cudaStream_t st) {
  return is_bf16 ? rmsnorm_launch<__nv_bfloat16>(x, delta, w, rows, x_out, h, n_rows, hidden, eps, st)
                 : rmsnorm_launch<float>(x, delta, w, rows, x_out, h, n_rows, hidden, eps, st);
}

// Plain residual add (the last layer's feed-forward output when no norm follows): x = T(x + d).
template <typename T>
__global__ void residual_add_kernel(T* __restrict__ x, const T* __restrict__ d, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = from_f32<T>(to_f32<T>(x[i]) + to_f32<T>(d[i]));
}
DRYFT_API int dryft_residual_add(int is_bf16, void* x, const void* d, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  unsigned blocks = (unsigned)((n + 255) / 256);
  if (is_bf16) residual_add_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)d, (size_t)n);
  else residual_add_kernel<float><<<blocks, 256, 0, st>>>((float*)x, (const float*)d, (size_t)n);
  return launch_status();
}

// ------------------------------------------------------------------------------------------
// SiLU*mul over the fused gate|up product [rows, 2*inter] (gate columns first):
//   y = T( T(g / (1 + exp(-g))) * u )            (silu_mul.py:29-32; model.py:44-46)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ y, int inter, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  size_t r = i / inter;
  int c = (int)(i - r * inter);
  const T* base = gu + r * (size_t)(2 * inter);
  float g = to_f32<T>(base[c]);
  float u = to_f32<T>(base[inter + c]);
  float s = rnd<T>(g / (1.f + expf(-g)));
  y[i] = from_f32<T>(s * u);
}
// g / (1 + exp(-g)): exact division and exponential in the 32-bit path; where the result is rounded to
// bfloat16 right away, the fast exponential and division (a few ulp of 32-bit) are far inside that rounding
template <typename T> __device__ __forceinline__ float silu_f32(float g) { return g / (1.f + expf(-g)); }
template <> __device__ __forceinline__ float silu_f32<__nv_bfloat16>(float g) { return __fdividef(g, 1.f + __expf(-g)); }
// 16 bytes of gate and of up per thread (inter a multiple of the vector width)
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ y, int inter, size_t total_vecs) {
  constexpr int V = Vec16<T>::N;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_vecs) return;
  const int vpr = inter / V;
  size_t r = i / vpr;
  int c = (int)(i - r * vpr) * V;
  const T* base = gu + r * (size_t)(2 * inter);
  float g[V], u[V], o[V];
  load_vec<T>(base + c, g);
  load_vec<T>(base + inter + c, u);
#pragma unroll
  for (int e = 0; e < V; ++e) o[e] = rnd<T>(silu_f32<T>(g[e])) * u[e];
  store_vec<T>(y + r * (size_t)inter + c, o);
}
template <typename T>
static int silu_launch(const void* gu, void* y, int rows, int inter, cudaStream_t st) {
  constexpr int V = Vec16<T>::N;
  if (inter % V == 0 && !(((uintptr_t)gu | (uintptr_t)y) & 15)) {   // 16-byte accesses
    size_t total = (size_t)rows * (inter / V);
    silu_mul_vec_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const T*)gu, (T*)y, inter, total);
  } else {
    size_t total = (size_t)rows * inter;
    silu_mul_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const T*)gu, (T*)y, inter, total);
  }
  return launch_status();
}
DRYFT_API int dryft_silu_mul(int is_bf16, const void* gu, void* y, int rows, int inter, cudaStream_t st) {
  if ((size_t)rows * inter == 0) return 0;
  return is_bf16 ? silu_launch<__nv_bfloat16>(gu, y, rows, inter, st) : silu_launch<float>(gu, y, rows, inter, st);
}
