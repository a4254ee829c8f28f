// Shared helpers for the engine's CUDA kernels (sm_100a).
//
// Every launcher is a plain C function: raw device pointers, sizes, a stream; it
// returns the cudaError_t of the launch as an int (0 = ok).  Activations and
// cache pages are either float (dtype code 0) or __nv_bfloat16 (code 1); all
// arithmetic inside a kernel is float.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define BF_DTYPE_F32 0
#define BF_DTYPE_BF16 1

// Bits of the device error word that kernels set instead of faulting.
#define BF_ERR_TOKEN_ID 1      // token id outside the vocabulary
#define BF_ERR_SLOT 2          // cache slot outside the pool
#define BF_ERR_PAGE 4          // page id outside the pool
#define BF_ERR_WAIT 8          // a bounded wait gave up

#define BF_EXPORT extern "C" __attribute__((visibility("default")))

__device__ __forceinline__ float bf_ld(const float* p) { return *p; }
__device__ __forceinline__ float bf_ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void bf_st(float* p, float v) { *p = v; }
__device__ __forceinline__ void bf_st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

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

// Sum over a whole block; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  float r = scratch[32];
  __syncthreads();
  return r;
}

static inline int bf_launch_status() { return (int)cudaGetLastError(); }
