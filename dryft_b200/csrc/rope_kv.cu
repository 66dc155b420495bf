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
//
// c and s depend on the token only, not on the layer: a step with many tokens evaluates them once
// (rope_table_kernel: [token][cos | sin][R/2], already rounded to T) and every layer's launch reads
// the table; without a table each warp evaluates its own.
#include "common.cuh"
#include <type_traits>

// two consecutive elements of T <-> two floats
template <typename T> __device__ __forceinline__ void load2(const T* p, float& a, float& b);
template <> __device__ __forceinline__ void load2<float>(const float* p, float& a, float& b) {
  const float2 v = *reinterpret_cast<const float2*>(p);
  a = v.x; b = v.y;
}
template <> __device__ __forceinline__ void load2<__nv_bfloat16>(const __nv_bfloat16* p, float& a, float& b) {
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p);
  a = __bfloat162float(v.x); b = __bfloat162float(v.y);
}
template <typename T> __device__ __forceinline__ void store2(T* p, float a, float b);
template <> __device__ __forceinline__ void store2<float>(float* p, float a, float b) {
  *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
template <> __device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// The rows of a token's page behind its own row, for one kv head, set to zero: `lanes` lanes (this one is
// `lane_in`) share the work.  Done by the value head of a sequence's last token of a step when the step's
// attention reads whole pages (tensor-core tiles): a page keeps what its last holder left there, the masked
// keys get probability zero, and 0 * v must stay 0 whatever v was (the reference zeroes its whole dense
// cache once instead, engine/dryft_qwen3/cache.py:43-47).
template <typename T>
__device__ __forceinline__ void zero_rows_behind(T* next_row, int n_rows, int D, int lane_in, int lanes) {
  const long long n = (long long)n_rows * D;
  if (((uintptr_t)next_row & 15) == 0 && (D * sizeof(T)) % 16 == 0) {
    uint4* p = reinterpret_cast<uint4*>(next_row);
    const long long n16 = n * (long long)sizeof(T) / 16;
    for (long long i = lane_in; i < n16; i += lanes) p[i] = make_uint4(0, 0, 0, 0);
  } else {
    for (long long i = lane_in; i < n; i += lanes) next_row[i] = from_f32<T>(0.f);
  }
}
// whether packed token n is the last one its sequence brings in this step (tokens of a sequence are consecutive)
__device__ __forceinline__ bool last_of_sequence(const int* __restrict__ tok_slot, int n, int n_tokens, int slot) {
  return n + 1 >= n_tokens || tok_slot[n + 1] != slot;
}

// A lane holds rotary pairs (j, j + R/2), two neighbouring j at a time; the head is read once,
// normalised, rotated and written.
constexpr int ROPE_WARPS = 4;
constexpr int MAX_PAIRS2 = 4;  // a lane holds up to 4 x 2 pairs: rotary dims up to 512

template <typename T>
__global__ void __launch_bounds__(ROPE_WARPS * 32) qk_norm_rope_store_kernel(
    const T* __restrict__ qkv, int qkv_stride,                 // [N, qkv_stride]; q | k | v column blocks
    const float* __restrict__ wq, const float* __restrict__ wk,  // [D] each (ignored if !has_norm)
    const float* __restrict__ inv_freq,                         // [R/2]
    const T* __restrict__ cs_table,                             // [N][2][R/2] cos | sin of each token, or null
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    T* __restrict__ q_out,                                      // [N, nH, D]
    T* __restrict__ k_pages, T* __restrict__ v_pages,           // [pages, nKV, page_size, D]
    const int* __restrict__ page_table, int max_pages,
    int n_tokens, int nH, int nKV, int D, int R, int page_size, float eps, int has_norm, int write_kv, int zero_tail) {
  // a warp per (token, head): plenty of warps in flight hide the latency of the few loads each one has;
  // grid (tokens, groups of ROPE_WARPS heads)
  const int lane = threadIdx.x & 31;
  const int heads_total = nH + (write_kv ? 2 * nKV : 0);
  const int n = blockIdx.x;
  const int head0 = blockIdx.y * ROPE_WARPS + (threadIdx.x >> 5);
  if (head0 >= heads_total) return;
  const int slot = tok_slot[n];
  const int pos = tok_pos[n];
  const int half = R >> 1;
  size_t page_off = 0;
  if (slot >= 0 && write_kv)
    page_off = ((size_t)page_table[(size_t)slot * max_pages + pos / page_size] * nKV * page_size + (pos % page_size)) * D;

  // the token's angles: cos/sin of pos * inv_freq[j] for this lane's pairs
  float cs[MAX_PAIRS2][2], sn[MAX_PAIRS2][2];
#pragma unroll
  for (int i = 0; i < MAX_PAIRS2; ++i) {
    if (cs_table != nullptr && (half & 1) == 0) {
      const int j = 2 * lane + 64 * i;
      cs[i][0] = cs[i][1] = 1.f;
      sn[i][0] = sn[i][1] = 0.f;
      if (j < half && head0 < nH + nKV && slot >= 0) {
        const T* row = cs_table + (size_t)n * R;
        load2<T>(row + j, cs[i][0], cs[i][1]);
        load2<T>(row + half + j, sn[i][0], sn[i][1]);
      }
      continue;
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int j = 2 * lane + 64 * i + e;
      cs[i][e] = 1.f;
      sn[i][e] = 0.f;
      if (j < half && head0 < nH + nKV && slot >= 0) {  // value heads and padding tokens rotate nothing
        float s_, c_;
        sincosf((float)pos * inv_freq[j], &s_, &c_);
        cs[i][e] = rnd<T>(c_);
        sn[i][e] = rnd<T>(s_);
      }
    }
  }

  for (int head = head0; head == head0; ++head) {
    const T* src = qkv + (size_t)n * qkv_stride + (size_t)head * D;  // q heads, then k heads, then v heads
    T* dst;
    if (head < nH) {
      dst = q_out + ((size_t)n * nH + head) * D;
      if (slot < 0) {  // padding token: a defined (zero) query
        for (int i = lane; i < D; i += 32) dst[i] = from_f32<T>(0.f);
        continue;
      }
    } else {
      if (slot < 0) continue;  // padding token: nothing is cached
      const int kvh = (head - nH) % nKV;
      const size_t off = page_off + (size_t)kvh * page_size * D;
      if (head >= nH + nKV) {  // value head: plain copy
        T* vd = v_pages + off;
        if ((D & 1) == 0) {
          for (int i = 2 * lane; i < D; i += 64) { float a, b; load2<T>(src + i, a, b); store2<T>(vd + i, a, b); }
        } else {
          for (int i = lane; i < D; i += 32) vd[i] = src[i];
        }
        if (zero_tail && last_of_sequence(tok_slot, n, n_tokens, slot))
          zero_rows_behind<T>(vd + D, page_size - 1 - pos % page_size, D, lane, 32);
        continue;
      }
      dst = k_pages + off;
    }
    const float* w = head < nH ? wq : wk;
    if ((half & 1) == 0 && half <= 64 * MAX_PAIRS2) {
      // vector path: the lane's pairs live in registers; one read of the head
      float a[MAX_PAIRS2][2], b[MAX_PAIRS2][2];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < MAX_PAIRS2; ++i) {
        const int j = 2 * lane + 64 * i;
        a[i][0] = a[i][1] = b[i][0] = b[i][1] = 0.f;
        if (j < half) {
          load2<T>(src + j, a[i][0], a[i][1]);
          load2<T>(src + j + half, b[i][0], b[i][1]);
          ss += a[i][0] * a[i][0] + a[i][1] * a[i][1] + b[i][0] * b[i][0] + b[i][1] * b[i][1];
        }
      }
      float inv = 1.f;
      if (has_norm) {
        for (int i = R + lane; i < D; i += 32) {  // dims beyond the rotary part count too
          const float v = to_f32<T>(src[i]);
          ss += v * v;
        }
        ss = warp_sum(ss);
        inv = rsqrtf(ss / (float)D + eps);
      }
#pragma unroll
      for (int i = 0; i < MAX_PAIRS2; ++i) {
        const int j = 2 * lane + 64 * i;
        if (j < half) {
          float o1[2], o2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float x = a[i][e], y = b[i][e];
            if (has_norm) {
              x = rnd<T>(rnd<T>(x * inv) * w[j + e]);
              y = rnd<T>(rnd<T>(y * inv) * w[j + e + half]);
            }
            // separate roundings of the two products, then of the sum (no fused multiply-add across them)
            o1[e] = __fadd_rn(rnd<T>(__fmul_rn(x, cs[i][e])), -rnd<T>(__fmul_rn(y, sn[i][e])));
            o2[e] = __fadd_rn(rnd<T>(__fmul_rn(y, cs[i][e])), rnd<T>(__fmul_rn(x, sn[i][e])));
          }
          store2<T>(dst + j, o1[0], o1[1]);
          store2<T>(dst + j + half, o2[0], o2[1]);
        }
      }
      for (int i = R + lane; i < D; i += 32) {  // dims beyond the rotary part
        float x = to_f32<T>(src[i]);
        if (has_norm) x = rnd<T>(rnd<T>(x * inv) * w[i]);
        dst[i] = from_f32<T>(x);
      }
    } else {
      // general path: any even rotary size, element by element
      float inv = 1.f;
      if (has_norm) {
        float ss = 0.f;
        for (int i = lane; i < D; i += 32) {
          const float v = to_f32<T>(src[i]);
          ss += v * v;
        }
        ss = warp_sum(ss);
        inv = rsqrtf(ss / (float)D + eps);
      }
      for (int j = lane; j < half; j += 32) {
        float x = to_f32<T>(src[j]);
        float y = to_f32<T>(src[j + half]);
        if (has_norm) {
          x = rnd<T>(rnd<T>(x * inv) * w[j]);
          y = rnd<T>(rnd<T>(y * inv) * w[j + half]);
        }
        float s_, c_;
        sincosf((float)pos * inv_freq[j], &s_, &c_);
        c_ = rnd<T>(c_);
        s_ = rnd<T>(s_);
        dst[j] = from_f32<T>(__fadd_rn(rnd<T>(__fmul_rn(x, c_)), -rnd<T>(__fmul_rn(y, s_))));
        dst[j + half] = from_f32<T>(__fadd_rn(rnd<T>(__fmul_rn(y, c_)), rnd<T>(__fmul_rn(x, s_))));
      }
      for (int i = R + lane; i < D; i += 32) {
        float x = to_f32<T>(src[i]);
        if (has_norm) x = rnd<T>(rnd<T>(x * inv) * w[i]);
        dst[i] = from_f32<T>(x);
      }
    }
  }
}


// The common case (rotary size = head size, R/2 even and at most 64 * NP): a warp takes ROPE_HPW
// consecutive heads of one token and issues every load of all of them before the first use, so that a
// warp's life is one memory round trip, not one per head.  Grid (tokens, groups of heads).
constexpr int ROPE_HPW = 4;
template <typename T, int NP>
__global__ void __launch_bounds__(ROPE_WARPS * 32) qk_norm_rope_store_fast_kernel(
    const T* __restrict__ qkv, int qkv_stride, const float* __restrict__ wq, const float* __restrict__ wk,
    const float* __restrict__ inv_freq, const T* __restrict__ cs_table, const int* __restrict__ tok_slot,
    const int* __restrict__ tok_pos, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
    const int* __restrict__ page_table, int max_pages, int nH, int nKV, int D, int page_size, float eps, int has_norm,
    int write_kv, int zero_tail) {
  const int lane = threadIdx.x & 31;
  const int heads_total = nH + (write_kv ? 2 * nKV : 0);
  const int n = blockIdx.x;
  const int head_base = (blockIdx.y * ROPE_WARPS + (threadIdx.x >> 5)) * ROPE_HPW;
  if (head_base >= heads_total) return;
  const int half = D >> 1;
  const T* row = qkv + (size_t)n * qkv_stride;
  // every load that needs no other load first
  float a[ROPE_HPW][NP][2], b[ROPE_HPW][NP][2];
#pragma unroll
  for (int u = 0; u < ROPE_HPW; ++u) {
    const int head = min(head_base + u, heads_total - 1);   // the last warp may repeat a head; it is not stored twice
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const int j = 2 * lane + 64 * i;
      a[u][i][0] = a[u][i][1] = b[u][i][0] = b[u][i][1] = 0.f;
      if (j < half) {
        load2<T>(row + (size_t)head * D + j, a[u][i][0], a[u][i][1]);
        load2<T>(row + (size_t)head * D + j + half, b[u][i][0], b[u][i][1]);
      }
    }
  }
  const int slot = tok_slot[n];
  const int pos = tok_pos[n];
  float cs[NP][2], sn[NP][2], wa[2][NP][2], wb[2][NP][2];
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int j = 2 * lane + 64 * i;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      cs[i][e] = 1.f; sn[i][e] = 0.f;
      wa[0][i][e] = wa[1][i][e] = wb[0][i][e] = wb[1][i][e] = 1.f;
    }
    if (j < half) {
      if (cs_table != nullptr) {
        load2<T>(cs_table + (size_t)n * D + j, cs[i][0], cs[i][1]);
        load2<T>(cs_table + (size_t)n * D + half + j, sn[i][0], sn[i][1]);
      }
      if (has_norm) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          wa[0][i][e] = wq[j + e]; wb[0][i][e] = wq[j + e + half];
          wa[1][i][e] = wk[j + e]; wb[1][i][e] = wk[j + e + half];
        }
      }
    }
  }
  if (slot < 0) {
    // padding token: a defined (zero) query, nothing cached
#pragma unroll
    for (int u = 0; u < ROPE_HPW; ++u) {
      const int head = head_base + u;
      if (head < nH)
        for (int i = 2 * lane; i < D; i += 64) store2<T>(q_out + ((size_t)n * nH + head) * D + i, 0.f, 0.f);
    }
    return;
  }
  size_t page_off = 0;
  if (write_kv)
    page_off = ((size_t)page_table[(size_t)slot * max_pages + pos / page_size] * nKV * page_size + (pos % page_size)) * D;
  if (cs_table == nullptr) {
#pragma unroll
    for (int i = 0; i < NP; ++i)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = 2 * lane + 64 * i + e;
        if (j < half) {
          float s_, c_;
          sincosf((float)pos * inv_freq[j], &s_, &c_);
          cs[i][e] = rnd<T>(c_);
          sn[i][e] = rnd<T>(s_);
        }
      }
  }
  // sums of squares of all heads together (value heads do not use theirs)
  float inv[ROPE_HPW];
#pragma unroll
  for (int u = 0; u < ROPE_HPW; ++u) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NP; ++i)
      ss += a[u][i][0] * a[u][i][0] + a[u][i][1] * a[u][i][1] + b[u][i][0] * b[u][i][0] + b[u][i][1] * b[u][i][1];
    inv[u] = ss;
  }
  if (has_norm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int u = 0; u < ROPE_HPW; ++u) inv[u] += __shfl_xor_sync(0xffffffffu, inv[u], o);
#pragma unroll
    for (int u = 0; u < ROPE_HPW; ++u) inv[u] = rsqrtf(inv[u] / (float)D + eps);
  }
#pragma unroll
  for (int u = 0; u < ROPE_HPW; ++u) {
    const int head = head_base + u;
    if (head >= heads_total) break;
    T* dst;
    const bool is_q = head < nH;
    if (is_q) {
      dst = q_out + ((size_t)n * nH + head) * D;
    } else {
      const int kvh = (head - nH) % nKV;
      const size_t off = page_off + (size_t)kvh * page_size * D;
      if (head >= nH + nKV) {  // value head: plain copy
#pragma unroll
        for (int i = 0; i < NP; ++i) {
          const int j = 2 * lane + 64 * i;
          if (j < half) {
            store2<T>(v_pages + off + j, a[u][i][0], a[u][i][1]);
            store2<T>(v_pages + off + j + half, b[u][i][0], b[u][i][1]);
          }
        }
        if (zero_tail && last_of_sequence(tok_slot, n, (int)gridDim.x, slot))
          zero_rows_behind<T>(v_pages + off + D, page_size - 1 - pos % page_size, D, lane, 32);
        continue;
      }
      dst = k_pages + off;
    }
#pragma unroll
    for (int i = 0; i < NP; ++i) {
      const int j = 2 * lane + 64 * i;
      if (j < half) {
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
          // the same roundings on pairs: x * inv in 32-bit rounded to a bfloat16 pair; every bfloat16
          // product and sum below is the exact result rounded once (the _rn forms are never fused)
          const __nv_bfloat162 cs2 = __floats2bfloat162_rn(cs[i][0], cs[i][1]), sn2 = __floats2bfloat162_rn(sn[i][0], sn[i][1]);
          __nv_bfloat162 x2, y2;
          if (has_norm) {
            const __nv_bfloat162 wa2 = is_q ? __floats2bfloat162_rn(wa[0][i][0], wa[0][i][1]) : __floats2bfloat162_rn(wa[1][i][0], wa[1][i][1]);
            const __nv_bfloat162 wb2 = is_q ? __floats2bfloat162_rn(wb[0][i][0], wb[0][i][1]) : __floats2bfloat162_rn(wb[1][i][0], wb[1][i][1]);
            x2 = __hmul2_rn(__floats2bfloat162_rn(a[u][i][0] * inv[u], a[u][i][1] * inv[u]), wa2);
            y2 = __hmul2_rn(__floats2bfloat162_rn(b[u][i][0] * inv[u], b[u][i][1] * inv[u]), wb2);
          } else {
            x2 = __floats2bfloat162_rn(a[u][i][0], a[u][i][1]);
            y2 = __floats2bfloat162_rn(b[u][i][0], b[u][i][1]);
          }
          *reinterpret_cast<__nv_bfloat162*>(dst + j) = __hsub2_rn(__hmul2_rn(x2, cs2), __hmul2_rn(y2, sn2));
          *reinterpret_cast<__nv_bfloat162*>(dst + j + half) = __hadd2_rn(__hmul2_rn(y2, cs2), __hmul2_rn(x2, sn2));
        } else {
          float o1[2], o2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float x = a[u][i][e], y = b[u][i][e];
            if (has_norm) {
              x = rnd<T>(rnd<T>(x * inv[u]) * (is_q ? wa[0][i][e] : wa[1][i][e]));
              y = rnd<T>(rnd<T>(y * inv[u]) * (is_q ? wb[0][i][e] : wb[1][i][e]));
            }
            // separate roundings of the two products, then of the sum (no fused multiply-add across them)
            o1[e] = __fadd_rn(rnd<T>(__fmul_rn(x, cs[i][e])), -rnd<T>(__fmul_rn(y, sn[i][e])));
            o2[e] = __fadd_rn(rnd<T>(__fmul_rn(y, cs[i][e])), rnd<T>(__fmul_rn(x, sn[i][e])));
          }
          store2<T>(dst + j, o1[0], o1[1]);
          store2<T>(dst + j + half, o2[0], o2[1]);
        }
      }
    }
  }
}

// bfloat16 with a cos / sin table, head sizes 16 * LPH (LPH = 1, 2, 4, 8 or 16 lanes a head): 16-byte loads
// and stores throughout.  A lane holds 8 elements of the first half of a head and the 8 they pair with in
// the second half; 32 / LPH heads go side by side in a warp, ROPE_VEC_PASSES such groups per warp, all
// loads issued before the first use.  Same formulas and roundings as the kernel above.
constexpr int ROPE_VEC_PASSES = 3;
__device__ __forceinline__ __nv_bfloat162 pair_of(const uint4& v, int e) {   // e is a constant after unrolling
  const unsigned u = e == 0 ? v.x : e == 1 ? v.y : e == 2 ? v.z : v.w;
  return *reinterpret_cast<const __nv_bfloat162*>(&u);
}
__device__ __forceinline__ unsigned bits_of(__nv_bfloat162 v) { return *reinterpret_cast<unsigned*>(&v); }
template <int LPH>
__global__ void __launch_bounds__(ROPE_WARPS * 32) qk_norm_rope_store_vec_kernel(
    const __nv_bfloat16* __restrict__ qkv, int qkv_stride, const float* __restrict__ wq, const float* __restrict__ wk,
    const __nv_bfloat16* __restrict__ cs_table, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
    const int* __restrict__ page_table, int max_pages, int nH, int nKV, int page_size, float eps, int has_norm, int write_kv,
    int zero_tail) {
  typedef __nv_bfloat16 bf16;
  typedef __nv_bfloat162 bf162;
  constexpr int D = 16 * LPH, half = D / 2, HPP = 32 / LPH;
  const int lane = threadIdx.x & 31;
  const int g = lane / LPH, c = lane % LPH;
  const int heads_total = nH + (write_kv ? 2 * nKV : 0);
  const int n = blockIdx.x;
  const int head0 = (blockIdx.y * ROPE_WARPS + (threadIdx.x >> 5)) * (HPP * ROPE_VEC_PASSES);
  if (head0 >= heads_total) return;
  const bf16* row = qkv + (size_t)n * qkv_stride;
  uint4 a[ROPE_VEC_PASSES], b[ROPE_VEC_PASSES];
#pragma unroll
  for (int u = 0; u < ROPE_VEC_PASSES; ++u) {
    const int head = min(head0 + u * HPP + g, heads_total - 1);   // lanes past the last head repeat it and store nothing
    a[u] = *reinterpret_cast<const uint4*>(row + (size_t)head * D + 8 * c);
    b[u] = *reinterpret_cast<const uint4*>(row + (size_t)head * D + half + 8 * c);
  }
  const int slot = tok_slot[n];
  const int pos = tok_pos[n];
  const uint4 cs4 = *reinterpret_cast<const uint4*>(cs_table + (size_t)n * D + 8 * c);
  const uint4 sn4 = *reinterpret_cast<const uint4*>(cs_table + (size_t)n * D + half + 8 * c);
  unsigned wqa[4] = {0, 0, 0, 0}, wqb[4] = {0, 0, 0, 0}, wka[4] = {0, 0, 0, 0}, wkb[4] = {0, 0, 0, 0};   // bfloat16 pairs
  if (has_norm) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 qa = *reinterpret_cast<const float2*>(wq + 8 * c + 2 * e), qb = *reinterpret_cast<const float2*>(wq + half + 8 * c + 2 * e);
      const float2 ka = *reinterpret_cast<const float2*>(wk + 8 * c + 2 * e), kb = *reinterpret_cast<const float2*>(wk + half + 8 * c + 2 * e);
      wqa[e] = bits_of(__floats2bfloat162_rn(qa.x, qa.y)); wqb[e] = bits_of(__floats2bfloat162_rn(qb.x, qb.y));
      wka[e] = bits_of(__floats2bfloat162_rn(ka.x, ka.y)); wkb[e] = bits_of(__floats2bfloat162_rn(kb.x, kb.y));
    }
  }
  if (slot < 0) {
    // padding token: a defined (zero) query, nothing cached
#pragma unroll
    for (int u = 0; u < ROPE_VEC_PASSES; ++u) {
      const int head = head0 + u * HPP + g;
      if (head < nH) {
        *reinterpret_cast<uint4*>(q_out + ((size_t)n * nH + head) * D + 8 * c) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(q_out + ((size_t)n * nH + head) * D + half + 8 * c) = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }
  size_t page_off = 0;
  if (write_kv)
    page_off = ((size_t)page_table[(size_t)slot * max_pages + pos / page_size] * nKV * page_size + (pos % page_size)) * D;
  float inv[ROPE_VEC_PASSES];
#pragma unroll
  for (int u = 0; u < ROPE_VEC_PASSES; ++u) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(pair_of(a[u], e)), y = __bfloat1622float2(pair_of(b[u], e));
      ss += x.x * x.x + x.y * x.y + y.x * y.x + y.y * y.y;
    }
    inv[u] = ss;
  }
  if (has_norm) {
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1)
#pragma unroll
      for (int u = 0; u < ROPE_VEC_PASSES; ++u) inv[u] += __shfl_xor_sync(0xffffffffu, inv[u], o);
#pragma unroll
    for (int u = 0; u < ROPE_VEC_PASSES; ++u) inv[u] = rsqrtf(inv[u] / (float)D + eps);
  }
#pragma unroll
  for (int u = 0; u < ROPE_VEC_PASSES; ++u) {
    const int head = head0 + u * HPP + g;
    if (head >= heads_total) continue;
    bf16* dst;
    const bool is_q = head < nH;
    if (is_q) {
      dst = q_out + ((size_t)n * nH + head) * D;
    } else {
      const int kvh = (head - nH) % nKV;
      const size_t off = page_off + (size_t)kvh * page_size * D;
      if (head >= nH + nKV) {  // value head: plain copy
        *reinterpret_cast<uint4*>(v_pages + off + 8 * c) = a[u];
        *reinterpret_cast<uint4*>(v_pages + off + half + 8 * c) = b[u];
        if (zero_tail && last_of_sequence(tok_slot, n, (int)gridDim.x, slot))
          zero_rows_behind<bf16>(v_pages + off + D, page_size - 1 - pos % page_size, D, c, LPH);
        continue;
      }
      dst = k_pages + off;
    }
    unsigned o1[4], o2[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // x * inv in 32-bit rounded to a bfloat16 pair; every bfloat16 product and sum below is the exact
      // result rounded once (the _rn forms are never fused)
      bf162 x2 = pair_of(a[u], e), y2 = pair_of(b[u], e);
      const bf162 cs2 = pair_of(cs4, e), sn2 = pair_of(sn4, e);
      if (has_norm) {
        const float2 xf = __bfloat1622float2(x2), yf = __bfloat1622float2(y2);
        const unsigned wa = is_q ? wqa[e] : wka[e], wb = is_q ? wqb[e] : wkb[e];
        x2 = __hmul2_rn(__floats2bfloat162_rn(xf.x * inv[u], xf.y * inv[u]), *reinterpret_cast<const bf162*>(&wa));
        y2 = __hmul2_rn(__floats2bfloat162_rn(yf.x * inv[u], yf.y * inv[u]), *reinterpret_cast<const bf162*>(&wb));
      }
      o1[e] = bits_of(__hsub2_rn(__hmul2_rn(x2, cs2), __hmul2_rn(y2, sn2)));
      o2[e] = bits_of(__hadd2_rn(__hmul2_rn(y2, cs2), __hmul2_rn(x2, sn2)));
    }
    *reinterpret_cast<uint4*>(dst + 8 * c) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *reinterpret_cast<uint4*>(dst + half + 8 * c) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
  }
}

template <int LPH>
static int launch_vec(const void* qkv, int qkv_stride, const float* wq, const float* wk, const void* cs_table, const int* tok_slot,
                      const int* tok_pos, void* q_out, void* k_pages, void* v_pages, const int* page_table, int max_pages,
                      int n_tokens, int nH, int nKV, int page_size, float eps, int has_norm, int write_kv, int zero_tail, cudaStream_t st) {
  typedef __nv_bfloat16 bf16;
  const int heads_total = nH + (write_kv ? 2 * nKV : 0);
  const int per_block = ROPE_WARPS * (32 / LPH) * ROPE_VEC_PASSES;
  const dim3 grid((unsigned)n_tokens, (unsigned)((heads_total + per_block - 1) / per_block));
  if (grid.y > 65535) return DRYFT_ERR_UNSUPPORTED;
  qk_norm_rope_store_vec_kernel<LPH><<<grid, ROPE_WARPS * 32, 0, st>>>(
      (const bf16*)qkv, qkv_stride, wq, wk, (const bf16*)cs_table, tok_slot, tok_pos, (bf16*)q_out, (bf16*)k_pages, (bf16*)v_pages,
      page_table, max_pages, nH, nKV, page_size, eps, has_norm, write_kv, zero_tail);
  return launch_status();
}

// cos / sin of every token's angles, rounded to T: table [n_tokens][2][half]
template <typename T>
__global__ void rope_table_kernel(const int* __restrict__ tok_pos, const float* __restrict__ inv_freq, T* __restrict__ table,
                                  int n_tokens, int half) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_tokens * half) return;
  const int n = (int)(i / half), j = (int)(i - (long long)n * half);
  float s_, c_;
  sincosf((float)tok_pos[n] * inv_freq[j], &s_, &c_);
  table[(size_t)n * 2 * half + j] = from_f32<T>(c_);
  table[(size_t)n * 2 * half + half + j] = from_f32<T>(s_);
}

DRYFT_API int dryft_rope_table(int is_bf16, const int* tok_pos, const float* inv_freq, void* table, int n_tokens, int R,
                               cudaStream_t st) {
  if (n_tokens <= 0 || R <= 0) return 0;
  if (R & 1) return DRYFT_ERR_UNSUPPORTED;
  const int half = R / 2;
  const long long items = (long long)n_tokens * half;
  const unsigned blocks = (unsigned)((items + 255) / 256);
  if (is_bf16) rope_table_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(tok_pos, inv_freq, (__nv_bfloat16*)table, n_tokens, half);
  else rope_table_kernel<float><<<blocks, 256, 0, st>>>(tok_pos, inv_freq, (float*)table, n_tokens, half);
  return launch_status();
}

template <typename T>
static int launch(const void* qkv, int qkv_stride, const float* wq, const float* wk, const float* inv_freq, const void* cs_table,
                  const int* tok_slot, const int* tok_pos, void* q_out, void* k_pages, void* v_pages,
                  const int* page_table, int max_pages, int n_tokens, int nH, int nKV, int D, int R, int page_size,
                  float eps, int has_norm, int write_kv, int zero_tail, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (D <= 0 || (R & 1) || R > D || R < 0) return DRYFT_ERR_UNSUPPORTED;
  const int heads_total = nH + (write_kv ? 2 * nKV : 0);
  if (std::is_same<T, __nv_bfloat16>::value && cs_table != nullptr && R == D && (D == 16 || D == 32 || D == 64 || D == 128 || D == 256) &&
      qkv_stride % 8 == 0 &&
      !(((uintptr_t)qkv | (uintptr_t)cs_table | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) &&
      !(((uintptr_t)wq | (uintptr_t)wk) & 7)) {
#define DRYFT_ROPE_VEC(L) launch_vec<L>(qkv, qkv_stride, wq, wk, cs_table, tok_slot, tok_pos, q_out, k_pages, v_pages, page_table, \
                                        max_pages, n_tokens, nH, nKV, page_size, eps, has_norm, write_kv, zero_tail, st)
    return D == 16 ? DRYFT_ROPE_VEC(1) : D == 32 ? DRYFT_ROPE_VEC(2) : D == 64 ? DRYFT_ROPE_VEC(4) : D == 128 ? DRYFT_ROPE_VEC(8) : DRYFT_ROPE_VEC(16);
#undef DRYFT_ROPE_VEC
  }
  if (R == D && (D & 3) == 0 && D <= 256) {
    const int per_block = ROPE_WARPS * ROPE_HPW;
    const dim3 grid((unsigned)n_tokens, (unsigned)((heads_total + per_block - 1) / per_block));
    if (grid.y > 65535) return DRYFT_ERR_UNSUPPORTED;
    if (D <= 128)
      qk_norm_rope_store_fast_kernel<T, 1><<<grid, ROPE_WARPS * 32, 0, st>>>(
          (const T*)qkv, qkv_stride, wq, wk, inv_freq, (const T*)cs_table, tok_slot, tok_pos, (T*)q_out, (T*)k_pages,
          (T*)v_pages, page_table, max_pages, nH, nKV, D, page_size, eps, has_norm, write_kv, zero_tail);
    else
      qk_norm_rope_store_fast_kernel<T, 2><<<grid, ROPE_WARPS * 32, 0, st>>>(
          (const T*)qkv, qkv_stride, wq, wk, inv_freq, (const T*)cs_table, tok_slot, tok_pos, (T*)q_out, (T*)k_pages,
          (T*)v_pages, page_table, max_pages, nH, nKV, D, page_size, eps, has_norm, write_kv, zero_tail);
    return launch_status();
  }
  const int head_groups = (heads_total + ROPE_WARPS - 1) / ROPE_WARPS;
  if (head_groups > 65535) return DRYFT_ERR_UNSUPPORTED;
  qk_norm_rope_store_kernel<T><<<dim3((unsigned)n_tokens, (unsigned)head_groups), ROPE_WARPS * 32, 0, st>>>(
      (const T*)qkv, qkv_stride, wq, wk, inv_freq, (const T*)cs_table, tok_slot, tok_pos, (T*)q_out, (T*)k_pages, (T*)v_pages, page_table,
      max_pages, n_tokens, nH, nKV, D, R, page_size, eps, has_norm, write_kv, zero_tail);
  return launch_status();
}

DRYFT_API int dryft_qk_norm_rope_store(int is_bf16, const void* qkv, int qkv_stride, const float* wq, const float* wk,
                                       const float* inv_freq, const void* cs_table, const int* tok_slot, const int* tok_pos, void* q_out,
                                       void* k_pages, void* v_pages, const int* page_table, int max_pages, int n_tokens,
                                       int nH, int nKV, int D, int R, int page_size, float eps, int has_norm,
                                       int write_kv, int zero_tail, cudaStream_t st) {
  return is_bf16 ? launch<__nv_bfloat16>(qkv, qkv_stride, wq, wk, inv_freq, cs_table, tok_slot, tok_pos, q_out, k_pages, v_pages,
                                         page_table, max_pages, n_tokens, nH, nKV, D, R, page_size, eps, has_norm, write_kv, zero_tail && write_kv, st)
                 : launch<float>(qkv, qkv_stride, wq, wk, inv_freq, cs_table, tok_slot, tok_pos, q_out, k_pages, v_pages,
                                 page_table, max_pages, n_tokens, nH, nKV, D, R, page_size, eps, has_norm, write_kv, zero_tail && write_kv, st);
}
