// Fused per-head q/k RMSNorm + rotate-half RoPE + write of K and V into the paged cache.
//
// One warp per (token, head).  Heads [0, nH) are query heads (norm, rotate, write to q_out);
// heads [nH, nH+nKV) are key heads (norm, rotate, write into the cache page of the token's
// position); heads [nH+nKV, nH+2nKV) are value heads (copied into the cache unchanged).
// Prefill and decode are the same launch: every token carries its own (slot, position).
//
// Formulas (hari495/dryft, engine/dryft_qwen3/kernels/rope_qknorm.py:38-47,73-99 and
// engine/dryft_qwen3/model.py:28-41,49-57):
//   n   = T( T(x * rsqrt(mean(x^2) + eps)) * w )
//   ang = float(pos) * inv_freq[j]                 32-bit angle, j = 0 .. R/2-1
//   c,s = T(cos(ang)), T(sin(ang))                 tables are cast to the activation type
//   o[j]       = T( T(n[j]*c)       - T(n[j+R/2]*s) )
//   o[j+R/2]   = T( T(n[j+R/2]*c)   + T(n[j]*s) )
// R (rotary_dim) may be smaller than the head size: the remaining dims pass through after the
// norm.  R = 0 disables the rotation; has_norm = 0 disables the norm.
#include "common.cuh"

template <typename T>
__global__ void qk_norm_rope_store_kernel(
    const T* __restrict__ qkv, int qkv_stride,                 // [N, qkv_stride]; q | k | v column blocks
    const float* __restrict__ wq, const float* __restrict__ wk,  // [D] each (ignored if !has_norm)
    const float* __restrict__ inv_freq,                         // [R/2]
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    T* __restrict__ q_out,                                      // [N, nH, D]
    T* __restrict__ k_pages, T* __restrict__ v_pages,           // [pages, nKV, page_size, D]
    const int* __restrict__ page_table, int max_pages,
    int n_tokens, int nH, int nKV, int D, int R, int page_size, float eps, int has_norm, int write_kv) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int heads_total = nH + (write_kv ? 2 * nKV : 0);
  const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (item >= (long long)n_tokens * heads_total) return;
  const int n = (int)(item / heads_total);
  const int head = (int)(item % heads_total);
  const int slot = tok_slot[n];
  const int pos = tok_pos[n];
  const T* src = qkv + (size_t)n * qkv_stride + (size_t)head * D;  // q heads, then k heads, then v heads

  T* dst;
  if (head < nH) {
    dst = q_out + ((size_t)n * nH + head) * D;
    if (slot < 0) {  // padding token: a defined (zero) query
      for (int i = lane; i < D; i += 32) dst[i] = from_f32<T>(0.f);
      return;
    }
  } else {
    if (slot < 0) return;  // padding token: nothing is cached
    const int kvh = (head - nH) % nKV;
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    const size_t off = (((size_t)page * nKV + kvh) * page_size + (pos % page_size)) * D;
    if (head >= nH + nKV) {  // value head: plain copy
      T* vd = v_pages + off;
      for (int i = lane; i < D; i += 32) vd[i] = src[i];
      return;
    }
    dst = k_pages + off;
  }

  float inv = 1.f;
  const float* w = head < nH ? wq : wk;
  if (has_norm) {
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
      float v = to_f32<T>(src[i]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)D + eps);
  }
  const int half = R >> 1;
  for (int j = lane; j < half; j += 32) {
    float a = to_f32<T>(src[j]);
    float b = to_f32<T>(src[j + half]);
    if (has_norm) {
      a = rnd<T>(rnd<T>(a * inv) * w[j]);
      b = rnd<T>(rnd<T>(b * inv) * w[j + half]);
    }
    float ang = (float)pos * inv_freq[j];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    cs = rnd<T>(cs);
    sn = rnd<T>(sn);
    // separate roundings of the two products, then of the sum (no fused multiply-add across them)
    float o1 = __fadd_rn(rnd<T>(__fmul_rn(a, cs)), -rnd<T>(__fmul_rn(b, sn)));
    float o2 = __fadd_rn(rnd<T>(__fmul_rn(b, cs)), rnd<T>(__fmul_rn(a, sn)));
    dst[j] = from_f32<T>(o1);
    dst[j + half] = from_f32<T>(o2);
  }
  for (int i = R + lane; i < D; i += 32) {  // dims beyond the rotary part
    float a = to_f32<T>(src[i]);
    if (has_norm) a = rnd<T>(rnd<T>(a * inv) * w[i]);
    dst[i] = from_f32<T>(a);
  }
}

template <typename T>
static int launch(const void* qkv, int qkv_stride, const float* wq, const float* wk, const float* inv_freq,
                  const int* tok_slot, const int* tok_pos, void* q_out, void* k_pages, void* v_pages,
                  const int* page_table, int max_pages, int n_tokens, int nH, int nKV, int D, int R, int page_size,
                  float eps, int has_norm, int write_kv, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (D <= 0 || (R & 1) || R > D || R < 0) return DRYFT_ERR_UNSUPPORTED;
  const int heads_total = nH + (write_kv ? 2 * nKV : 0);
  const long long items = (long long)n_tokens * heads_total;
  const int warps = 8;
  const long long blocks = (items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return DRYFT_ERR_UNSUPPORTED;
  qk_norm_rope_store_kernel<T><<<(unsigned)blocks, warps * 32, 0, st>>>(
      (const T*)qkv, qkv_stride, wq, wk, inv_freq, tok_slot, tok_pos, (T*)q_out, (T*)k_pages, (T*)v_pages, page_table,
      max_pages, n_tokens, nH, nKV, D, R, page_size, eps, has_norm, write_kv);
  return launch_status();
}

DRYFT_API int dryft_qk_norm_rope_store(int is_bf16, const void* qkv, int qkv_stride, const float* wq, const float* wk,
                                       const float* inv_freq, const int* tok_slot, const int* tok_pos, void* q_out,
                                       void* k_pages, void* v_pages, const int* page_table, int max_pages, int n_tokens,
                                       int nH, int nKV, int D, int R, int page_size, float eps, int has_norm,
                                       int write_kv, cudaStream_t st) {
  return is_bf16 ? launch<__nv_bfloat16>(qkv, qkv_stride, wq, wk, inv_freq, tok_slot, tok_pos, q_out, k_pages, v_pages,
                                         page_table, max_pages, n_tokens, nH, nKV, D, R, page_size, eps, has_norm, write_kv, st)
                 : launch<float>(qkv, qkv_stride, wq, wk, inv_freq, tok_slot, tok_pos, q_out, k_pages, v_pages,
                                 page_table, max_pages, n_tokens, nH, nKV, D, R, page_size, eps, has_norm, write_kv, st);
}
