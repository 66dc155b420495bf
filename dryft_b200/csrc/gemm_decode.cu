// Decode matrix product for one K, fixed at compile time (-DDRYFT_K, a multiple of 256): the same
// operation, fusions and launch overlap as csrc/gemm_small_m.cu, but with every loop over k unrolled
// and every offset an immediate, so that an instruction moves as many bytes as it can.  It is what a
// model's decode step uses when its widths allow; gemm_small_m.cu remains the general form.
//
//   C[M,N] = A[M,K] * W[N,K]^T,  M <= 8 or <= 16,  bfloat16 operands, 32-bit accumulation,
//   every weight byte read from HBM exactly once (hari495/dryft: cuBLAS via F.linear,
//   engine/dryft_qwen3/model.py:237,258,260,261).
//   norm prologue (kernels/rmsnorm.py:21-39), residual epilogue with sums of squares for the next
//   norm (rmsnorm.py:34), SiLU*mul epilogue (kernels/silu_mul.py:29-32; weights.py:98-100).
//
// A group of 8 warps takes 16 rows of W at a time; groups are persistent, two per SM -- two blocks of one
// group, or, with the norm on the way in, one block of two groups that share the staged activations --
// each walking over every grid-th tile.  The warps of a group split K into 8 equal ranges.  A thread keeps a ring of up to ten 32-wide k steps of its two weight rows in
// registers -- 16-byte loads that bypass L1, all in flight together -- and feeds them to
// mma.sync.m16n8k16 with W as the 16 x 16 operand and 8 batch rows as the 16 x 8 operand (the k index
// permuted identically in both operands, so that a thread's fragment is one contiguous 16-byte piece);
// the registers of a step just multiplied take the step a ring's length further on, of this tile or of
// the block's next one, so a warp's requests never drain.  With the norm prologue the normalised
// activations are made once per block and stay in shared memory (the M rows there are and one row of
// zeros for the rest of the operand); otherwise they are read through L2, a few steps ahead.  The 8
// partial sums are added in warp order through shared memory: a row's result depends neither on the
// other rows nor on M (the split of K is chosen by the sizes of the product and by whether M is up to 8 or
// up to 16, never by M itself).
//
// The norm can also be split between two launches, which takes it off the consumer's critical path: a
// residual product that knows the next norm's weight w leaves, beside the new stream x, the weighted
// activations xw = T(x * w); the next product then multiplies xw as plain activations (no prologue at
// all) and scales its sums by inv[m] = rsqrt(mean(x[m]^2) + eps) in the epilogue, in 32-bit:
// inv * sum_k T(x*w) W in place of sum_k T(T(x*inv)*w) W -- one rounding of the activations fewer than the
// reference makes (model.py:28-32), the statistics still in 32-bit.
//
// The kernel may be launched as a programmatic dependent of the launch before it: it requests its
// first weights, which depend on nothing, and only then waits for the earlier grid.
// No block waits on another block of its grid; there is no spin in this file.
#include "common.cuh"

#if !defined(DRYFT_K)
#error "compile with -DDRYFT_K=<inner size, a multiple of 256>"
#endif

namespace {
typedef __nv_bfloat16 bf16;
constexpr int K = DRYFT_K;
static_assert(K % 256 == 0, "this kernel takes inner sizes that are multiples of 256");
constexpr int ROWS = 16;
// The warps of a group (8, or 16) split K evenly: SPW 32-wide k steps a warp.
// A thread keeps CHUNK steps of its two weight rows in registers, as a ring: the registers of the step just
// multiplied take the step CHUNK further on, of this tile or of the block's next one, so that a warp's
// requests never drain.  The ring's slot of a step is (step mod CHUNK) in every tile, so a tile is walked in
// SPWP steps, a multiple of CHUNK; the steps from SPW on are empty.  CHUNK is the ring of 6 to 10 steps that
// keeps most steps in flight after those empty ones.
__host__ __device__ constexpr int pick_chunk(int SPW, int most) {
  if (SPW <= most) return SPW;
  int best = most, best_score = 0;
  for (int c = 6; c <= most; ++c) {
    const int score = SPW * c * 64 / ((SPW + c - 1) / c * c);
    if (score > best_score) { best = c; best_score = score; }   // ties: the shorter ring
  }
  return best;
}
// plain activations come from L2 a few steps ahead, in a ring of registers of their own whose length divides
// the weights' ring; 16 rows of them take twice the registers, so the weights' ring is at most 8 steps there
__host__ __device__ constexpr int pick_ahead(int chunk, int most) {
  int d = 1;
  for (int c = 1; c <= most; ++c)
    if (chunk % c == 0) d = c;
  return d;
}
constexpr int SS_STRIDE = 64;
constexpr int KA = K + ((64 - (K * 2) % 128 + 128) % 128) / 2;  // resident row stride: bytes = 64 mod 128

// Shared memory and L1 are one 256 KB array per SM, cut at one of a few places, and the weights on their way
// into registers are held in L1: an SM streams at full rate only while the L1 that the cut leaves is about as
// large as the bytes its blocks keep in flight (two blocks: 160 KB).  Measured on the gate|up product of a
// 5,120-wide model (524 MB): 80 us with 10 KB of shared memory a block, 162 us with 101 KB (two blocks: the
// 228 KB cut), 83 us with 126 KB (one block an SM, the 132 KB cut).  So every instantiation asks for the
// 100 KB cut (also so that neighbouring launches, which overlap, agree on it: a batch-8 step of a 2,560-wide
// model takes 2.12 ms this way, 2.26 ms when each launch is left to the driver's choice), stages only the rows
// there are, once per SM, and runs one group an SM where two would not fit under that cut.
constexpr int CARVEOUT_PCT = 43;
constexpr size_t CARVEOUT_BYTES = 100 * 1024;
constexpr size_t SMEM_MOST = 164 * 1024;   // one block under the 164 KB cut: L1 still holds one block's requests

enum Mode { STORE_BF16 = 0, STORE_F32 = 1, RESIDUAL = 2, SILU = 3 };
// what happens to the activations: nothing; RMSNorm in the prologue (rows normalised into shared memory);
// or they come weighted already (T(x * w)) and the sums are scaled by inv[m] in the epilogue
enum Pro { PLAIN = 0, NORMED = 1, SCALED = 2 };

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bfr(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// bytes of the partial sums, which also hold the norm's weight while the activations are normalised
template <int MB, int PRO, int GROUPS, int GW> __host__ __device__ constexpr size_t head_bytes() {
  const size_t red = (size_t)GROUPS * GW * ROWS * (8 * MB + 1) * 4, nw = PRO == NORMED ? (size_t)K * 2 : 0;
  return ((red > nw ? red : nw) + 15) / 16 * 16;
}

// GROUPS = 2: two groups of 8 warps in one block, each walking tiles of its own as a block of its own would
// (its own partial sums, its own named barrier), but sharing one copy of the staged activations, which all
// 16 warps make together.
// GW = 16: the 16 warps of the block split K of ONE tile 16 ways, for inner sizes that still leave a warp 8 steps
// or more and products with tiles for every SM twice over: one staged copy, one tile's epilogue at a time, and
// half as long a wait for the slowest block at the end.
template <int MB, int MODE, int PRO, int GROUPS, int GW>
__global__ void __launch_bounds__(GW * 32 * GROUPS, GW * GROUPS == 8 ? 2 : 1) gemm_decode_kernel(
    const bf16* __restrict__ A, int lda, const bf16* __restrict__ W, void* C, int ldc, int M, int N,
    const float* __restrict__ norm_w, const float* __restrict__ ss_in, int ss_parts, float eps, float* __restrict__ ss_out,
    const float* __restrict__ next_w, bf16* __restrict__ xw_out, int rs) {
  constexpr bool NORM = PRO == NORMED;
  constexpr int MP = 8 * MB;
  constexpr int WARPS = GW, THREADS = GW * 32, SPW = K / 32 / GW;   // of a group; SPW: 32-wide k steps a warp
  constexpr int RED = WARPS * ROWS * (MP + 1);
  constexpr int CHUNK = pick_chunk(SPW, MB == 2 && PRO == PLAIN ? 8 : 10);
  constexpr int SPWP = (SPW + CHUNK - 1) / CHUNK * CHUNK;
  extern __shared__ __align__(16) unsigned char smem[];
  // [WARPS][ROWS][MP + 1] partial sums (the norm's weight lies in the same bytes until the first tile is
  // reduced), 64 floats of inv, then the resident activations: the rs = min(M, MP) rows there are, and one
  // row of zeros behind them that stands for every row from M on
  constexpr int CT = THREADS * GROUPS;                         // threads of the block
  const int ctid = threadIdx.x, group = GROUPS == 1 ? 0 : ctid / THREADS;
  const int tid = ctid - group * THREADS, warp = tid >> 5, lane = tid & 31;   // within the group
  float* red = reinterpret_cast<float*>(smem) + group * RED;
  float* inv_s = reinterpret_cast<float*>(smem + head_bytes<MB, PRO, GROUPS, GW>());
  bf16* a_res = reinterpret_cast<bf16*>(inv_s + SS_STRIDE);
  auto group_sync = [&]() {
    if (GROUPS == 1) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "n"(GW * 32) : "memory");
  };

  const int g = lane >> 2, t = lane & 3;
  constexpr int TILE_N = MODE == SILU ? 8 : ROWS;
  const int n_tiles = (N + TILE_N - 1) / TILE_N;
  const int k_warp = warp * SPW * 32 + t * 8;   // this thread's first k
  pdl_launch_dependents();

  uint4 wa[CHUNK], wb[CHUNK];
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // this thread's two weight rows of a tile (tile rows g and g+8; SILU: gate row and matching up row)
  auto rows_of = [&](int tile, const bf16*& w0, const bf16*& w1) {
    const int n0 = tile * TILE_N;
    int r0, r1;
    bool ok0, ok1;
    if (MODE == SILU) { r0 = n0 + g; r1 = N + n0 + g; ok0 = ok1 = n0 + g < N; }
    else { r0 = n0 + g; r1 = n0 + g + 8; ok0 = r0 < N; ok1 = r1 < N; }
    w0 = ok0 ? W + (size_t)r0 * K + k_warp : nullptr;
    w1 = ok1 ? W + (size_t)r1 * K + k_warp : nullptr;
  };
  int tile = blockIdx.x * GROUPS + group;
  const bf16 *w0 = nullptr, *w1 = nullptr;
  if (tile < n_tiles) {
    rows_of(tile, w0, w1);
#pragma unroll
    for (int u = 0; u < CHUNK; ++u) {   // the first tile's first steps: weights depend on no earlier launch
      wa[u] = w0 ? ld_stream(w0 + u * 32) : zero;
      wb[u] = w1 ? ld_stream(w1 + u * 32) : zero;
    }
  }

  bf16* nw_s = reinterpret_cast<bf16*>(smem);   // the norm's weight as bfloat16 (its values are bfloat16 values held in 32-bit)
  if (NORM) {
    // the norm's weight depends on no earlier launch either: into shared memory before the wait
    for (int i = ctid; i < K / 4; i += CT) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(norm_w) + i);
      reinterpret_cast<__nv_bfloat162*>(nw_s)[2 * i] = __floats2bfloat162_rn(v.x, v.y);
      reinterpret_cast<__nv_bfloat162*>(nw_s)[2 * i + 1] = __floats2bfloat162_rn(v.z, v.w);
    }
  }

  pdl_wait();  // from here on, what earlier launches wrote (activations, sums of squares) is visible

  // SCALED: the rows' sums of squares are requested now and added after the first tile's products, so
  // that nothing waits for them: warp w owns rows w, w + 8, ...; a lane holds up to SSL blocks per row
  constexpr int SSL = 8;
  float ssv[MB][SSL];
  if (PRO == SCALED) {
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < SSL; ++i) {
        const int m = warp + 8 * mb, part = lane + 32 * i;
        ssv[mb][i] = (m < M && part < ss_parts) ? ld_prev(ss_in + (size_t)part * SS_STRIDE + m) : 0.f;
      }
  }
  bool inv_done = false;

  if (PRO == SCALED) {
    // the weighted activations go to shared memory once per block (one trip through L2, no arithmetic):
    // every tile of the block reads them from there
    constexpr int CHUNKS = K / 8;
    constexpr int BATCH = 5;    // pieces a thread requests together (registers also hold the first weights)
    const int items = rs * CHUNKS;
    if (rs < MP)
      for (int c = tid; c < CHUNKS; c += THREADS) *reinterpret_cast<uint4*>(a_res + (size_t)rs * KA + c * 8) = zero;
#pragma unroll 1
    for (int first = tid; first < items; first += BATCH * THREADS) {
      uint4 raw[BATCH];
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int i = first + u * THREADS;
        const int m = i / CHUNKS, c = i - m * CHUNKS;
        raw[u] = i < items ? ld_prev(reinterpret_cast<const uint4*>(A + (size_t)m * lda + c * 8)) : zero;
      }
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int i = first + u * THREADS;
        if (i >= items) break;
        const int m = i / CHUNKS, c = i - m * CHUNKS;
        *reinterpret_cast<uint4*>(a_res + (size_t)m * KA + c * 8) = raw[u];
      }
    }
    __syncthreads();
  }

  if (NORM) {
    // inv[m] = rsqrt(mean(x[m]^2) + eps): warp m adds the blocks of sums of squares in a fixed order;
    // then the normalised rows a[m,k] = T(T(x[m,k] * inv[m]) * w[k]) go to shared memory once per block.
    // The activations are requested together with the sums of squares, a batch of loads per thread
    // at once, so that the whole prologue is one or two trips to memory.
    constexpr int CHUNKS = K / 8;                 // 16-byte pieces of a row
    constexpr int BATCH = 5;                      // pieces a thread requests together (registers also hold the first weights)
    const int items = rs * CHUNKS;
    uint4 raw[BATCH];
    auto fetch = [&](int first) {
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int i = first + u * CT;
        const int m = i / CHUNKS, c = i - m * CHUNKS;
        raw[u] = i < items ? ld_prev(reinterpret_cast<const uint4*>(A + (size_t)m * lda + c * 8)) : zero;
      }
    };
    fetch(ctid);
    if (rs < MP)
      for (int c = ctid; c < CHUNKS; c += CT) *reinterpret_cast<uint4*>(a_res + (size_t)rs * KA + c * 8) = zero;
    for (int m = ctid >> 5; m < MP; m += WARPS * GROUPS) {
      float s = 0.f;
      if (m < M)
        for (int p = lane; p < ss_parts; p += 32) s += ld_prev(ss_in + (size_t)p * SS_STRIDE + m);
      s = warp_sum(s);
      if (lane == 0) inv_s[m] = rsqrtf(s / (float)K + eps);
    }
    __syncthreads();   // inv_s and the norm's weight are in shared memory
#pragma unroll 1
    for (int first = ctid; first < items; first += BATCH * CT) {
      if (first != ctid) fetch(first);
#pragma unroll
      for (int u = 0; u < BATCH; ++u) {
        const int i = first + u * CT;
        if (i >= items) break;
        const int m = i / CHUNKS, c = i - m * CHUNKS;
        uint4 out = zero;
        {
          // two elements at a time: x * inv in 32-bit, rounded to a bfloat16 pair, times the weight pair
          // (a bfloat16 product rounded once: the same value as the 32-bit product rounded)
          const uint4 wraw = *reinterpret_cast<const uint4*>(nw_s + c * 8);
          const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wraw);
          const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
          const float inv = inv_s[m];
          __align__(16) __nv_bfloat162 o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(e[j]);
            o[j] = __hmul2(__floats2bfloat162_rn(f.x * inv, f.y * inv), wp[j]);
          }
          out = *reinterpret_cast<const uint4*>(o);
        }
        *reinterpret_cast<uint4*>(a_res + (size_t)m * KA + c * 8) = out;
      }
    }
    __syncthreads();
  }
  // this thread's activation fragments: batch row mb*8 + g, k as for the weights
  constexpr bool STAGED = PRO != PLAIN;   // the block's activations are in shared memory
  const bf16* a_frag = A + (size_t)g * lda + k_warp;
  const size_t a_mb = (size_t)8 * lda;
  const bf16* a_row[MB];   // STAGED: where batch row mb * 8 + g lies (the row of zeros from rs on)
#pragma unroll
  for (int mb = 0; mb < MB; ++mb) a_row[mb] = a_res + (size_t)(mb * 8 + g < rs ? mb * 8 + g : rs) * KA + k_warp;
  // plain activations come from L2 AD steps ahead, in a ring of registers of their own
  constexpr int AD = STAGED ? 1 : pick_ahead(CHUNK, MB == 1 ? 5 : 4);
  uint4 ar[MB][AD];
  auto plain_a = [&](int mb, int step) {
    return mb * 8 + g < M ? ld_prev(reinterpret_cast<const uint4*>(a_frag + mb * a_mb + step * 32)) : zero;
  };
  if (!STAGED && tile < n_tiles) {
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int u = 0; u < AD; ++u) ar[mb][u] = plain_a(mb, u);
  }
  for (; tile < n_tiles; tile += gridDim.x * GROUPS) {
    float acc[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mb][i] = 0.f;
    const int next = tile + gridDim.x * GROUPS;
    const bool has_next = next < n_tiles;
    const bf16 *nw0 = nullptr, *nw1 = nullptr;
    if (has_next) rows_of(next, nw0, nw1);

#pragma unroll
    for (int s = 0; s < SPWP; ++s) {
      const int u = s % CHUNK;
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        if (s < SPW) {
          const uint4 a = STAGED ? *reinterpret_cast<const uint4*>(a_row[mb] + s * 32) : ar[mb][s % AD];
          mma16816(acc[mb], wa[u].x, wb[u].x, wa[u].y, wb[u].y, a.x, a.y);
          mma16816(acc[mb], wa[u].z, wb[u].z, wa[u].w, wb[u].w, a.z, a.w);
        }
        if (!STAGED) {   // the slot takes the step AD further on; the activations are the same for every tile
          const int ta = s + AD < SPWP ? s + AD : s + AD - SPWP;
          if (ta < SPW && (s + AD < SPWP || has_next)) ar[mb][s % AD] = plain_a(mb, ta);
        }
      }
      // these registers take the step CHUNK further on: of this tile, or of the block's next one, whose
      // first weights thus fly while this tile is reduced and written
      if (s + CHUNK < SPWP) {
        if (s + CHUNK < SPW) {
          wa[u] = w0 ? ld_stream(w0 + (s + CHUNK) * 32) : zero;
          wb[u] = w1 ? ld_stream(w1 + (s + CHUNK) * 32) : zero;
        }
      } else if (has_next && s + CHUNK - SPWP < SPW) {
        wa[u] = nw0 ? ld_stream(nw0 + (s + CHUNK - SPWP) * 32) : zero;
        wb[u] = nw1 ? ld_stream(nw1 + (s + CHUNK - SPWP) * 32) : zero;
      }
    }
    w0 = nw0;
    w1 = nw1;

    if (PRO == SCALED && !inv_done) {
      inv_done = true;
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        float sm = 0.f;
#pragma unroll
        for (int i = 0; i < SSL; ++i) sm += ssv[mb][i];
        for (int part = lane + 32 * SSL; part < ss_parts; part += 32)   // more blocks than the registers hold
          if (warp + 8 * mb < M) sm += ld_prev(ss_in + (size_t)part * SS_STRIDE + warp + 8 * mb);
        sm = warp_sum(sm);
        if (lane == 0) inv_s[warp + 8 * mb] = rsqrtf(sm / (float)K + eps);   // visible after the barrier below
      }
    }
    // partial sums -> shared memory, once the tile before this one has been read from there
    group_sync();
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      red[(warp * ROWS + g) * (MP + 1) + mb * 8 + 2 * t] = acc[mb][0];
      red[(warp * ROWS + g) * (MP + 1) + mb * 8 + 2 * t + 1] = acc[mb][1];
      red[(warp * ROWS + g + 8) * (MP + 1) + mb * 8 + 2 * t] = acc[mb][2];
      red[(warp * ROWS + g + 8) * (MP + 1) + mb * 8 + 2 * t + 1] = acc[mb][3];
    }
    group_sync();
    auto total = [&](int row, int m) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) s += red[(w * ROWS + row) * (MP + 1) + m];
      return PRO == SCALED ? s * inv_s[m] : s;
    };
    const int n0 = tile * TILE_N;
    if (MODE == SILU) {
      bf16* out = reinterpret_cast<bf16*>(C);
      if (tid < 8 * MP) {
        const int j = tid & 7, m = tid >> 3;
        if (m < M && n0 + j < N) {
          const float gt = bfr(total(j, m)), up = bfr(total(j + 8, m));
          const float s = bfr(gt / (1.f + expf(-gt)));
          out[(size_t)m * ldc + n0 + j] = __float2bfloat16_rn(s * up);
        }
      }
    } else if (MODE == RESIDUAL) {
      bf16* x = reinterpret_cast<bf16*>(C);
      // thread -> (row = tid % 16, m = tid / 16): a half-warp covers the 16 columns of one batch row
      if (tid < ROWS * MP) {
        const int row = tid & 15, m = tid >> 4;
        const int n = n0 + row;
        float sq = 0.f;
        if (m < M && n < N) {
          const float v = bfr(ld_prev_bf16(x + (size_t)m * ldc + n) + bfr(total(row, m)));
          x[(size_t)m * ldc + n] = __float2bfloat16_rn(v);
          if (xw_out) xw_out[(size_t)m * ldc + n] = __float2bfloat16_rn(v * next_w[n]);   // for the next norm
          sq = v * v;
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (ss_out && row == 0 && m < M) ss_out[(size_t)tile * SS_STRIDE + m] = sq;
      }
    } else {
      if (tid < ROWS * MP) {
        const int row = tid & 15, m = tid >> 4;
        const int n = n0 + row;
        if (m < M && n < N) {
          const float s = total(row, m);
          if (MODE == STORE_F32) reinterpret_cast<float*>(C)[(size_t)m * ldc + n] = s;
          else reinterpret_cast<bf16*>(C)[(size_t)m * ldc + n] = __float2bfloat16_rn(s);
        }
      }
    }
  }
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    sms = n > 0 ? n : 148;
  }
  return sms;
}
template <int MB, int PRO, int GROUPS, int GW> size_t smem_of(int staged) {
  return head_bytes<MB, PRO, GROUPS, GW>() + SS_STRIDE * 4 + (size_t)staged * KA * 2;
}
template <int MB, int MODE, int PRO, int GROUPS, int GW>
int launch4(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, const float* norm_w,
            const float* ss_in, int ss_parts, float eps, float* ss_out, const float* next_w, void* xw_out, int pdl,
            int rs, int staged, int blocks_per_sm, cudaStream_t st) {
  constexpr int MP = 8 * MB;
  const size_t smem = smem_of<MB, PRO, GROUPS, GW>(staged);
  const size_t smem_max = smem_of<MB, PRO, GROUPS, GW>(PRO == PLAIN ? 0 : MP);
  if (smem + 1024 > SMEM_MOST) return DRYFT_ERR_UNSUPPORTED;
  static bool attr_done = false;  // per instantiation; set by an eager launch before any capture
  if (!attr_done) {
    const size_t most = smem_max + 1024 > SMEM_MOST ? SMEM_MOST - 1024 : smem_max;
    cudaError_t e = cudaFuncSetAttribute(gemm_decode_kernel<MB, MODE, PRO, GROUPS, GW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_decode_kernel<MB, MODE, PRO, GROUPS, GW>, cudaFuncAttributePreferredSharedMemoryCarveout, CARVEOUT_PCT);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  // Persistent blocks, each (group) taking every grid-th tile.  What an SM can pull from memory is
  // bounded by the requests its blocks keep in flight, so the tiles are spread over all SMs as evenly as
  // they go: with the usual placement (block b beside block b + SMs) the SMs' totals differ by one tile.
  const int max_blocks = sm_count();
  const int n_tiles = MODE == SILU ? (N + 7) / 8 : (N + ROWS - 1) / ROWS;
  const int want = (n_tiles + GROUPS - 1) / GROUPS;
  const unsigned blocks = (unsigned)(want < blocks_per_sm * max_blocks ? want : blocks_per_sm * max_blocks);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(GW * 32 * GROUPS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_decode_kernel<MB, MODE, PRO, GROUPS, GW>, (const bf16*)A, lda, (const bf16*)W, C, ldc,
                                     M, N, norm_w, ss_in, ss_parts, eps, ss_out, next_w, (bf16*)xw_out, rs);
  if (e != cudaSuccess) return (int)e;
  return launch_status();
}
// With the norm on the way in: one block an SM of two groups that share the staged rows (half the bytes to
// stage per SM, by twice the threads: the batch-8 step of a 2,560-wide model takes 1.95 ms this way, 2.05 ms
// with two blocks of one group; the 4,096-wide one 3.05 against 3.35 ms, where two blocks' rows do not fit
// the cut and an SM held one); one group where even that does not fit.  Else two blocks an SM where both fit
// under the cut, else one.
template <int MB, int MODE, int PRO>
int launch3(const void* A, int lda, const void* W, void* C, int ldc, int M, int N, const float* norm_w,
            const float* ss_in, int ss_parts, float eps, float* ss_out, const float* next_w, void* xw_out, int pdl,
            cudaStream_t st) {
  constexpr int MP = 8 * MB;
  const int rs = M < MP ? M : MP;                                  // activation rows there are
  const int staged = PRO == PLAIN ? 0 : (rs < MP ? rs + 1 : MP);   // and the row of zeros behind them
#define DRYFT_GO(GROUPS, GW, PER_SM) \
  launch4<MB, MODE, PRO, GROUPS, GW>(A, lda, W, C, ldc, M, N, norm_w, ss_in, ss_parts, eps, ss_out, next_w, xw_out, pdl, rs, staged, PER_SM, st)
  constexpr int WIDE = (K % 512 == 0 && K / 512 >= 8 && PRO != SCALED) ? 16 : 8;   // 16 warps on one tile where a warp keeps 8 steps
  const int n_tiles = MODE == SILU ? (N + 7) / 8 : (N + ROWS - 1) / ROWS;
  // (decided by what 8 / 16 rows would need, not by M: the split of K, and with it the order of the sums,
  // is then the same for every M up to 8, and for every M from 9 to 16)
  if (WIDE == 16 && n_tiles >= 2 * sm_count() && smem_of<MB, PRO, 1, WIDE>(PRO == PLAIN ? 0 : MP) + 1024 <= CARVEOUT_BYTES)
    return DRYFT_GO(1, WIDE, 1);
  if (PRO != NORMED && 2 * (smem_of<MB, PRO, 1, 8>(staged) + 1024) <= CARVEOUT_BYTES) return DRYFT_GO(1, 8, 2);
  if (PRO == NORMED && smem_of<MB, PRO, 2, 8>(staged) + 1024 <= CARVEOUT_BYTES) return DRYFT_GO((PRO == NORMED ? 2 : 1), 8, 1);
  return DRYFT_GO(1, 8, 1);
#undef DRYFT_GO
}
struct Args {
  const void* A; int lda; const void* W; void* C; int ldc; int M; int N;
  const float* norm_w; const float* ss_in; int ss_parts; float eps; float* ss_out; const float* next_w; void* xw_out;
  int pdl; cudaStream_t st;
};
template <int MB, int MODE, int PRO>
int launch_a(const Args& a) {
  return launch3<MB, MODE, PRO>(a.A, a.lda, a.W, a.C, a.ldc, a.M, a.N, a.norm_w, a.ss_in, a.ss_parts, a.eps, a.ss_out, a.next_w,
                                a.xw_out, a.pdl, a.st);
}
template <int MB, int MODE>
int launch2(int pro, const Args& a) {
  return pro == NORMED ? launch_a<MB, MODE, NORMED>(a) : pro == SCALED ? launch_a<MB, MODE, SCALED>(a) : launch_a<MB, MODE, PLAIN>(a);
}
template <int MB>
int launch1(int mode, int pro, const Args& a) {
  switch (mode) {
    case STORE_BF16: return launch2<MB, STORE_BF16>(pro, a);
    case STORE_F32: return launch2<MB, STORE_F32>(pro, a);
    case RESIDUAL: return launch2<MB, RESIDUAL>(pro, a);
    case SILU: return launch2<MB, SILU>(pro, a);
  }
  return DRYFT_ERR_UNSUPPORTED;
}
}  // namespace

DRYFT_API int dryft_gemm_decode_k() { return K; }

// Same contract as dryft_gemm_small_m (csrc/gemm_small_m.cu) for this library's K.  A residual product
// of N outputs leaves ceil(N/16) blocks of sums of squares in ss_out and, given the next norm's weight
// next_w [N] and xw_out [M, ldc], the weighted activations T(x * next_w) for the product after it.
// scaled != 0: A holds such weighted activations; the sums are scaled by rsqrt(mean(x^2) + eps) from
// ss_in (norm_w is not read).
DRYFT_API int dryft_gemm_decode(const void* A, int lda, const void* W, void* C, int ldc, int mode, int M, int N,
                                const float* norm_w, const float* ss_in, int ss_parts, float eps, float* ss_out, int pdl,
                                int scaled, const float* next_w, void* xw_out, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if ((lda & 7) || M > 16) return DRYFT_ERR_UNSUPPORTED;
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return DRYFT_ERR_UNSUPPORTED;
  const int pro = scaled ? SCALED : (norm_w != nullptr ? NORMED : PLAIN);
  if (pro != PLAIN && (!ss_in || ss_parts <= 0)) return DRYFT_ERR_UNSUPPORTED;
  if (pro == NORMED && ((uintptr_t)norm_w & 15)) return DRYFT_ERR_UNSUPPORTED;
  if ((xw_out != nullptr) != (next_w != nullptr) || (xw_out && mode != RESIDUAL)) return DRYFT_ERR_UNSUPPORTED;
  Args a = {A, lda, W, C, ldc, M, N, norm_w, ss_in, ss_parts, eps, ss_out, next_w, xw_out, pdl, st};
  return M <= 8 ? launch1<1>(mode, pro, a) : launch1<2>(mode, pro, a);
}
