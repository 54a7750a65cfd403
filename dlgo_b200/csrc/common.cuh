// Shared helpers of the hand-written sm_100a kernels.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and the
// stream to launch on, allocates nothing, and returns a status: 0, a positive
// cudaError_t from the launch, or a negative DLGO_ERR_* when it refuses the sizes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

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

// Programmatic dependent launch: a kernel may be scheduled while its predecessor on the stream is
// still draining, so that launch latency and prologues overlap the predecessor's tail.  Every kernel
// of this package calls pdl_launch_dependents() at its start and pdl_wait() before it reads or writes
// anything a predecessor may have touched; pdl_wait() returns once all predecessors have completed
// and their writes are visible.  Both are no-ops for a kernel launched without the attribute.
// Before the wait a kernel may read only what no kernel of the same step writes: weights, tables,
// and the step's own inputs (token positions, slots, page tables), which are in place before the
// step's first kernel starts.  That first kernel (the embedding) is launched WITHOUT the attribute
// (launch_kernel_first), so it starts only after everything before it on the stream has completed;
// every later kernel of the chain starts after it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("DLGO_PDL");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// For the first kernel of a step: an ordinary launch, ordered after all earlier work of the stream.
template <typename... KArgs, typename... Args>
inline void launch_kernel_first(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = nullptr;
  cfg.numAttrs = 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with a thread-block cluster of `cluster` blocks (grid must be a multiple of it).
template <typename... KArgs, typename... Args>
inline void launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Diagnostic build (-DDLGO_TIMING): kernels stamp the global timer at named points, per block, and
// the library exports dlgo_times() to fetch the stamps (8 per block, the first 1024 blocks).
#ifdef DLGO_TIMING
__device__ unsigned long long g_times[1024 * 8];
#define TSTAMP(k)                                                                              \
  do {                                                                                         \
    const int c_ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;             \
    if (c_ < 1024) {                                                                           \
      unsigned long long t_;                                                                   \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                   \
      g_times[c_ * 8 + (k)] = t_;                                                              \
    }                                                                                          \
  } while (0)
#define DLGO_TIMES_EXPORT                                                                      \
  extern "C" __attribute__((visibility("default"))) int dlgo_times(unsigned long long* out) {  \
    return cudaMemcpyFromSymbol(out, dlgo::g_times, sizeof(unsigned long long) * 1024 * 8) == cudaSuccess ? 0 : -1; \
  }
#else
#define TSTAMP(k) do {} while (0)
#define DLGO_TIMES_EXPORT
#endif

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DLGO_OK : (int)e;
}

}  // namespace dlgo
