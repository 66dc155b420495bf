// Token choice over 32-bit logits, one block per row: greedy (first index of the maximum) and
// temperature / top-k sampling with a counter-based uniform.
//
// hari495/dryft chooses tokens with argmax only (engine/dryft_qwen3/model.py:187,262; ties go to
// the first index, AGENTS.md:174-175).  Sampling is this library's own definition:
//   keep the top_k largest logits (ties to the lower index; top_k <= 0 or >= vocab keeps all);
//   z_i = logit_i / temperature;  e_i = exp(z_i - max z);  total = sum of kept e_i;
//   u = uniform(seed, sequence, step) in [0,1);  choose the first kept index, in index order,
//   whose running sum of e exceeds u * total.
// The uniform is a 64-bit integer mix of (seed, sequence index, step), so a sequence's draws do not
// depend on its slot or on what else is in the batch.
//
// Both kernels can also record the choice as the sequence's last token (per-sequence state), which
// is what a captured decode step reads as its next input.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ float uniform24(unsigned long long seed, unsigned long long seq, unsigned long long step) {
  unsigned long long z = seed * 0x9E3779B97F4A7C15ULL + seq * 0xBF58476D1CE4E5B9ULL + step * 0x94D049BB133111EBULL +
                         0x2545F4914F6CDD1DULL;
  z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ULL;
  z ^= z >> 27; z *= 0x94D049BB133111EBULL;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// order-preserving map float -> uint32 (larger float, larger key)
__device__ __forceinline__ unsigned key_of(float f) {
  unsigned u = __float_as_uint(f + 0.0f);  // -0 and +0 are one value
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(THREADS) argmax_rows_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                                                              int* __restrict__ out, const int* __restrict__ row_slot,
                                                              int* __restrict__ last_token) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  const int r = blockIdx.x;
  const float* lg = logits + (size_t)r * row_stride;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  auto take = [&](float v, int i) {
    if (v > best || (v == best && i < idx) || idx == 0x7fffffff) { best = v; idx = i; }
  };
  // 16-byte loads, four of them in flight per thread, where the row allows; a thread sees its indices in rising order
  int done = 0;
  if ((reinterpret_cast<uintptr_t>(lg) & 15) == 0) {
    const float4* lg4 = reinterpret_cast<const float4*>(lg);
    const int n4 = vocab / 4;
    int i = threadIdx.x;
    for (; i + 3 * THREADS < n4; i += 4 * THREADS) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = lg4[i + u * THREADS];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int b = 4 * (i + u * THREADS);
        take(v[u].x, b); take(v[u].y, b + 1); take(v[u].z, b + 2); take(v[u].w, b + 3);
      }
    }
    for (; i < n4; i += THREADS) {
      const float4 v = lg4[i];
      take(v.x, 4 * i); take(v.y, 4 * i + 1); take(v.z, 4 * i + 2); take(v.w, 4 * i + 3);
    }
    done = n4 * 4;
  }
  for (int i = done + threadIdx.x; i < vocab; i += THREADS) take(lg[i], i);
  // (value desc, index asc) reduction
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
  __syncthreads();
  if (warp == 0) {
    best = bv[lane];
    idx = bi[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
    }
    if (lane == 0) {
      out[r] = idx;
      if (row_slot && last_token && row_slot[r] >= 0) last_token[row_slot[r]] = idx;
    }
  }
}

// Exclusive block scan of one value per thread (THREADS threads); returns the exclusive prefix and
// writes the block total to *total.  scratch: 33 floats.
__device__ __forceinline__ float block_excl_scan(float v, float* scratch, float* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    float w = scratch[lane];
    float winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    scratch[lane] = winc - w;  // exclusive prefix of the warp sums
    if (lane == 31) scratch[32] = winc;
  }
  __syncthreads();
  *total = scratch[32];
  return scratch[warp] + inc - v;
}
__device__ __forceinline__ int block_excl_scan_int(int v, int* scratch, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = scratch[lane];
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    scratch[lane] = winc - w;
    if (lane == 31) scratch[32] = winc;
  }
  __syncthreads();
  *total = scratch[32];
  return scratch[warp] + inc - v;
}

__global__ void __launch_bounds__(THREADS) sample_rows_kernel(
    const float* __restrict__ logits, int vocab, long long row_stride, float temperature, int top_k,
    unsigned long long seed, const int* __restrict__ row_seq, const int* __restrict__ row_step, int step_base,
    int* __restrict__ out, const int* __restrict__ row_slot, int* __restrict__ last_token) {
  __shared__ unsigned hist[256];
  __shared__ float fscratch[33];
  __shared__ int iscratch[33];
  __shared__ unsigned sh_prefix, sh_remaining;
  __shared__ int sh_choice;
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* lg = logits + (size_t)r * row_stride;

  // ---- threshold key of the top_k-th largest logit (radix select, 4 passes of 8 bits) ----
  unsigned thr_key = 0;       // keep keys > thr_key, and the first n_eq keys == thr_key
  int n_eq = 0x7fffffff;      // how many elements equal to the threshold are kept
  const bool use_topk = top_k > 0 && top_k < vocab;
  if (use_topk) {
    if (tid == 0) { sh_prefix = 0; sh_remaining = (unsigned)top_k; }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int i = tid; i < 256; i += THREADS) hist[i] = 0;
      __syncthreads();
      const unsigned prefix = sh_prefix;
      const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < vocab; i += THREADS) {
        const unsigned k = key_of(lg[i]);
        if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned rem = sh_remaining;
        int b = 255;
        for (; b > 0; --b) {  // walk from the largest digit down
          if (hist[b] >= rem) break;
          rem -= hist[b];
        }
        sh_prefix = prefix | ((unsigned)b << shift);
        sh_remaining = rem;  // rank of the wanted element inside bucket b
      }
      __syncthreads();
    }
    thr_key = sh_prefix;
    n_eq = (int)sh_remaining;
  }

  // ---- each thread owns a contiguous chunk of the vocabulary (index order matters) ----
  const int chunk = (vocab + THREADS - 1) / THREADS;
  const int lo = min(tid * chunk, vocab), hi = min(lo + chunk, vocab);

  // elements equal to the threshold before this thread's chunk
  int eq_before = 0;
  if (use_topk) {
    int eq_local = 0;
    for (int i = lo; i < hi; ++i) eq_local += key_of(lg[i]) == thr_key;
    int eq_total;
    eq_before = block_excl_scan_int(eq_local, iscratch, &eq_total);
  }

  // maximum of the logits (the kept set always contains it)
  float mx = -INFINITY;
  for (int i = lo; i < hi; ++i) mx = fmaxf(mx, lg[i]);
  mx = warp_max(mx);
  __syncthreads();
  if ((tid & 31) == 0) fscratch[tid >> 5] = mx;
  __syncthreads();
  if (tid < 32) {
    float t = fscratch[tid];
    t = warp_max(t);
    if (tid == 0) fscratch[32] = t;
  }
  __syncthreads();
  const float zmax = fscratch[32] / temperature;
  __syncthreads();

  // kept weights of this chunk
  float local = 0.f;
  {
    int eq_seen = eq_before;
    for (int i = lo; i < hi; ++i) {
      const float v = lg[i];
      bool keep = true;
      if (use_topk) {
        const unsigned k = key_of(v);
        keep = k > thr_key || (k == thr_key && eq_seen++ < n_eq);
      }
      if (keep) local += expf(v / temperature - zmax);
    }
  }
  float total;
  const float before = block_excl_scan(local, fscratch, &total);
  const int seq = row_seq ? row_seq[r] : r;
  const int step = step_base + (row_step ? row_step[r] : 0);
  const float target = uniform24(seed, (unsigned long long)seq, (unsigned long long)step) * total;

  // the first chunk, in index order, whose inclusive running sum passes the target holds the choice
  if (tid == 0) sh_choice = THREADS;
  __syncthreads();
  if (local > 0.f && before + local > target) atomicMin(&sh_choice, tid);
  __syncthreads();
  const int owner = sh_choice;
  __syncthreads();
  if (tid == 0) sh_choice = -1;
  __syncthreads();
  if (owner == tid) {
    float run = before;
    int eq_seen = eq_before;
    int pick = -1, last_kept = -1;
    for (int i = lo; i < hi; ++i) {
      const float v = lg[i];
      bool keep = true;
      if (use_topk) {
        const unsigned k = key_of(v);
        keep = k > thr_key || (k == thr_key && eq_seen++ < n_eq);
      }
      if (!keep) continue;
      last_kept = i;
      run += expf(v / temperature - zmax);
      if (run > target) { pick = i; break; }
    }
    sh_choice = pick >= 0 ? pick : last_kept;
  } else if (owner == THREADS) {
    // rounding left the target at or beyond the total: take the last kept index
    int last_kept = -1;
    int eq_seen = eq_before;
    for (int i = lo; i < hi; ++i) {
      bool keep = true;
      if (use_topk) {
        const unsigned k = key_of(lg[i]);
        keep = k > thr_key || (k == thr_key && eq_seen++ < n_eq);
      }
      if (keep) last_kept = i;
    }
    if (last_kept >= 0) atomicMax(&sh_choice, last_kept);
  }
  __syncthreads();
  if (tid == 0) {
    const int c = sh_choice < 0 ? 0 : sh_choice;
    out[r] = c;
    if (row_slot && last_token && row_slot[r] >= 0) last_token[row_slot[r]] = c;
  }
}
}  // namespace

DRYFT_API int dryft_argmax_rows(const float* logits, int n_rows, int vocab, long long row_stride, int* out,
                                const int* row_slot, int* last_token, cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (vocab <= 0) return DRYFT_ERR_UNSUPPORTED;
  argmax_rows_kernel<<<n_rows, THREADS, 0, st>>>(logits, vocab, row_stride, out, row_slot, last_token);
  return launch_status();
}

DRYFT_API int dryft_sample_rows(const float* logits, int n_rows, int vocab, long long row_stride, float temperature,
                                int top_k, unsigned long long seed, const int* row_seq, const int* row_step, int step_base, int* out,
                                const int* row_slot, int* last_token, cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (vocab <= 0 || !(temperature > 0.f)) return DRYFT_ERR_UNSUPPORTED;
  sample_rows_kernel<<<n_rows, THREADS, 0, st>>>(logits, vocab, row_stride, temperature, top_k, seed, row_seq, row_step,
                                                 step_base, out, row_slot, last_token);
  return launch_status();
}
