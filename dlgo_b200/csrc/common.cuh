// Shared helpers of the hand-written sm_100a kernels.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and the
// stream to launch on, allocates nothing, and returns a status: 0, a positive
// cudaError_t from the launch, or a negative DLGO_ERR_* when it refuses the sizes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DLGO_OK 0
#define DLGO_ERR_SIZE (-1)      // a size the kernel does not take (never a wrong result)
#define DLGO_ERR_ALIGN (-2)     // a pointer or stride that breaks an alignment rule
#define DLGO_ERR_DTYPE (-3)     // unknown element type code
#define DLGO_ERR_DRIVER (-4)    // a driver entry point could not be found
#define DLGO_ERR_DEVICE (-5)    // the kernel gave up a bounded wait and set its error word

// element type codes shared with the Python side
#define DLGO_F32 0
#define DLGO_BF16 1

#define DLGO_EXPORT extern "C" __attribute__((visibility("default")))

namespace dlgo {

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
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

// Sum over a block of up to 1024 threads in a fixed order (warp trees, then the
// warp partials in warp order), so a row's result does not depend on what else
// is in the launch.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nwarps; ++w) t += scratch[w];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = scratch[0];
  for (int w = 1; w < nwarps; ++w) t = fmaxf(t, scratch[w]);
  return t;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DLGO_OK : (int)e;
}

}  // namespace dlgo
