// Shared helpers of the dryft_b200 kernels (sm_100a).
//
// Every kernel is a template over the activation type T (float or __nv_bfloat16).  All
// arithmetic is done in 32-bit; `rnd<T>` marks the places where the bfloat16 path rounds an
// intermediate (the rounding points hari495/dryft documents at engine/dryft_qwen3/model.py:4-13)
// and is the identity in the 32-bit path.
//
// Launchers are `extern "C"`, take raw device pointers and a stream, launch, and return the
// cudaError_t of the launch as an int (0 = ok).  They allocate nothing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DRYFT_API extern "C" __attribute__((visibility("default")))

// error codes of the launchers beyond cudaError_t (negative so they cannot collide)
#define DRYFT_ERR_UNSUPPORTED (-2)

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Round a 32-bit intermediate to T and back: a rounding point of the bfloat16 path.
template <typename T> __device__ __forceinline__ float rnd(float v) { return to_f32<T>(from_f32<T>(v)); }

// Data that the launch before this one wrote (activations, sums of squares, the residual stream) is read
// through L2 only in kernels that may run as programmatic dependents.  Such a grid is resident while its
// predecessor still runs, so that data is not read-only for the grid's lifetime: the non-coherent path
// (ld.global.nc, which the compiler also picks by itself for const __restrict__ pointers) may return lines
// that an earlier grid left in this SM's L1.  Weights never change and keep the cached paths.
template <typename T> __device__ __forceinline__ T ld_prev(const T* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_prev_bf16(const __nv_bfloat16* p) {
  return __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(p))));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `scratch` holds >= 33 floats of shared memory.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

static inline int launch_status() { return (int)cudaGetLastError(); }
