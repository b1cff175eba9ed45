// Shared device helpers for the sm_100a kernels of this engine.
//
// Conventions used by every kernel file:
//   * activations and weights come as T = float (the true 32-bit path) or __nv_bfloat16 (the
//     serving path); statistics, softmax state, angles and the residual stream are float in both;
//   * every exported function is `extern "C" int q25_<name>_<f32|bf16>(..., void* stream)` and
//     returns the cudaError_t of its launch (0 = success), so Python can call it through ctypes
//     with raw device pointers and the stream it is recording or capturing on;
//   * no kernel waits on another kernel or on a flag: everything is stream-ordered.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

#define Q25_EXPORT extern "C" __attribute__((visibility("default")))

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a thread block in a fixed order (lanes by butterfly, then warps in index order),
// so the result for a row never depends on what else is in the batch.  `scratch` holds 32
// floats.  Every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}

static inline int launch_status() { return (int)cudaGetLastError(); }
