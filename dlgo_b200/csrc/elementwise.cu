// Embedding gather, RMSNorm and SwiGLU.
//
// Formulas (reference, computerex/dlgo):
//   embedding  x = E[token, :]                                models/llm/forward.go:132
//   RMSNorm    ss = sum x^2 (fp32); s = 1/sqrt(ss/n + eps) with the square root and
//              the reciprocal in double, cast to fp32; out = x*s*w   ops/norm.go:10-32
//   SwiGLU     out = g / (1 + exp(-g)) * u                    ops/activation.go:8-38
// The residual stream is fp32 in both precisions; T is the element type of the
// activations handed to the next contraction (float or bfloat16).
#include "common.cuh"

namespace dlgo {

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             float* __restrict__ out, int d, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  const bool ok = tok >= 0 && tok < vocab;
  const TW* row = table + (size_t)(ok ? tok : 0) * d;
  float* o = out + (size_t)t * d;
  if (sizeof(TW) == 2 && (d & 7) == 0 && ((uintptr_t)table & 15) == 0) {
    // 16 bytes of the row per thread and trip: the whole row is in flight at once
    for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
      uint4 u = ok ? __ldg(reinterpret_cast<const uint4*>(row + i)) : make_uint4(0u, 0u, 0u, 0u);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
      const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
      const float2 c = __bfloat1622float2(h[2]), e = __bfloat1622float2(h[3]);
      *reinterpret_cast<float4*>(o + i) = make_float4(a.x, a.y, b.x, b.y);
      *reinterpret_cast<float4*>(o + i + 4) = make_float4(c.x, c.y, e.x, e.y);
    }
    return;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = ok ? to_float(row[i]) : 0.f;
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row.  `rows` (optional) picks the input row of each
// output row, so the final norm runs on the wanted positions only.
// 1 / sqrt(mean + eps): as the reference computes it (square root and reciprocal in double, ops/norm.go:21)
// for the float32 path; for bfloat16 activations, whose 8 bits of mantissa hide the last ulps, in
// fp32 (a double-precision square root and division cost microseconds on this GPU).
template <typename TO> __device__ __forceinline__ float norm_scale(float mean_eps);
template <> __device__ __forceinline__ float norm_scale<float>(float mean_eps) {
  return (float)(1.0 / sqrt((double)mean_eps));
}
template <> __device__ __forceinline__ float norm_scale<__nv_bfloat16>(float mean_eps) {
  return 1.0f / sqrtf(mean_eps);
}

template <typename TO> __device__ __forceinline__ void store4(TO* o, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* o, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* o, float a, float b, float c, float d) {
  __nv_bfloat162 h[2] = {__floats2bfloat162_rn(a, b), __floats2bfloat162_rn(c, d)};
  *reinterpret_cast<uint2*>(o) = *reinterpret_cast<uint2*>(h);
}

template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               TO* __restrict__ out, const int* __restrict__ rows, int d, float eps) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  __shared__ float scale_s;
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * d;   // (`rows` is an input of the step, not a result)
  TO* o = out + (size_t)r * d;
  constexpr int KEEP = 4;   // float4s of the row a thread keeps in registers between the two passes
  if ((d & 3) == 0 && d <= (int)blockDim.x * 4 * KEEP) {
    // the weight is nobody's output: it is fetched before the wait for the predecessor
    float4 ww[KEEP];
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      const int i = (threadIdx.x + j * blockDim.x) * 4;
      ww[j] = i < d ? __ldg(reinterpret_cast<const float4*>(w + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    // the row is read once, 16 bytes at a time, and stays in registers for the second pass
    float4 v[KEEP];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      const int i = (threadIdx.x + j * blockDim.x) * 4;
      v[j] = i < d ? *reinterpret_cast<const float4*>(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      ss = fmaf(v[j].x, v[j].x, ss);
      ss = fmaf(v[j].y, v[j].y, ss);
      ss = fmaf(v[j].z, v[j].z, ss);
      ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = block_sum(ss, scratch);
    if (threadIdx.x == 0) scale_s = norm_scale<TO>(ss / (float)d + eps);
    __syncthreads();
    const float s = scale_s;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      const int i = (threadIdx.x + j * blockDim.x) * 4;
      if (i < d)
        store4<TO>(o + i, v[j].x * s * ww[j].x, v[j].y * s * ww[j].y, v[j].z * s * ww[j].z, v[j].w * s * ww[j].w);
    }
    return;
  }
  pdl_wait();
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = xr[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) scale_s = norm_scale<TO>(ss / (float)d + eps);
  __syncthreads();
  const float s = scale_s;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_float<TO>(xr[i] * s * w[i]);
}

// ------------------------------------------- residual += sum of partials, then RMSNorm
// Many rows (prompts): one WARP per row, the row in registers (KV float4 per lane), no block-wide
// barrier; a block of eight warps takes eight rows.  d <= 32 * 4 * KV and d % 4 == 0.
template <typename TO, int KV>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                           TO* __restrict__ out, const int* __restrict__ rows, int R,
                                                           int d, float eps) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int src = (r < R && rows) ? rows[r] : r;
  pdl_wait();
  if (r >= R) return;
  const float* xr = x + (size_t)src * d;
  float4 v[KV];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < KV; ++j) {
    const int i = (lane + 32 * j) * 4;
    v[j] = i < d ? *reinterpret_cast<const float4*>(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int j = 0; j < KV; ++j) ss += (v[j].x * v[j].x + v[j].y * v[j].y) + (v[j].z * v[j].z + v[j].w * v[j].w);
  ss = warp_sum(ss);
  const float s = norm_scale<TO>(ss / (float)d + eps);
  TO* o = out + (size_t)r * d;
#pragma unroll
  for (int j = 0; j < KV; ++j) {
    const int i = (lane + 32 * j) * 4;
    if (i < d) {
      const float4 ww = *reinterpret_cast<const float4*>(w + i);
      store4<TO>(o + i, v[j].x * s * ww.x, v[j].y * s * ww.y, v[j].z * s * ww.z, v[j].w * s * ww.w);
    }
  }
}

// The contraction before a residual add may leave its K-slices unsummed ([S][T][d] fp32).  This
// kernel adds them to the residual in slice order (models/llm/forward.go:163,169), writes the
// residual back, and normalises the new row in the same pass (ops/norm.go:10-32).  With
// `w == nullptr` it only settles the sum.  One block per row; `rows` picks the rows to do.
template <typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ parts, int S, size_t part_stride,
                                   const float* __restrict__ w, TO* __restrict__ out, const int* __restrict__ rows,
                                   int d, float eps) {
  pdl_launch_dependents();
  extern __shared__ float row_s[];   // the new row, kept for the second pass
  __shared__ float scratch[32];
  __shared__ float scale_s;
  const int r = blockIdx.x;
  const bool vec = (d & 3) == 0 && (part_stride & 3) == 0;
  // the norm's weight does not depend on earlier kernels: this thread's first piece of it is
  // fetched before waiting for them
  float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (vec && w != nullptr && threadIdx.x * 4 < d) w0 = *reinterpret_cast<const float4*>(w + threadIdx.x * 4);
  const int src = rows ? rows[r] : r;   // (the row list is the step's own input, like the weights)
  pdl_wait();
  float* xr = x + (size_t)src * d;
  const float* pr = parts + (size_t)src * d;
  float ss = 0.f;
  float4 first = make_float4(0.f, 0.f, 0.f, 0.f);
  if (vec) {
    // 16-byte accesses; sixteen slices' loads and the residual's are in flight before the first add,
    // so a row costs one round trip to memory per sixteen slices
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + i);
      for (int s0 = 0; s0 < S; s0 += 16) {
        float4 t[16];
#pragma unroll
        for (int j = 0; j < 16; ++j)
          t[j] = (s0 + j < S) ? __ldcg(reinterpret_cast<const float4*>(pr + (size_t)(s0 + j) * part_stride + i))
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (s0 + j < S) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
        }
      }
      *reinterpret_cast<float4*>(xr + i) = v;
      if (i == threadIdx.x * 4) first = v; else *reinterpret_cast<float4*>(row_s + i) = v;
      ss = fmaf(v.x, v.x, ss);
      ss = fmaf(v.y, v.y, ss);
      ss = fmaf(v.z, v.z, ss);
      ss = fmaf(v.w, v.w, ss);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float v = xr[i];
      for (int s = 0; s < S; ++s) v += pr[(size_t)s * part_stride + i];
      xr[i] = v;
      row_s[i] = v;
      ss = fmaf(v, v, ss);
    }
  }
  if (w == nullptr) return;
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) scale_s = norm_scale<TO>(ss / (float)d + eps);
  __syncthreads();
  const float sc = scale_s;
  TO* o = out + (size_t)r * d;
  if (vec) {
    // the thread's first piece never left its registers; the rest (rows wider than four times the
    // block) comes back from shared memory
    if (threadIdx.x * 4 < d) {
      store4<TO>(o + threadIdx.x * 4, first.x * sc * w0.x, first.y * sc * w0.y, first.z * sc * w0.z,
                 first.w * sc * w0.w);
    }
    for (int i = (threadIdx.x + blockDim.x) * 4; i < d; i += blockDim.x * 4) {
      const float4 ww = *reinterpret_cast<const float4*>(w + i);
      store4<TO>(o + i, row_s[i] * sc * ww.x, row_s[i + 1] * sc * ww.y, row_s[i + 2] * sc * ww.z,
                 row_s[i + 3] * sc * ww.w);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_float<TO>(row_s[i] * sc * w[i]);
  }
}

// The same with a row spread over the CTAs of a thread-block cluster (few rows, wide rows: decode
// steps).  A row's K-slices are S * d * 4 bytes that one SM pulls out of L2 no faster than ~100 GB/s;
// NC CTAs pull NC times as fast.  Every CTA settles and keeps its stretch of the row in registers,
// sends its sum of squares to all CTAs of the cluster (distributed shared memory), and after one
// cluster barrier each adds the NC sums in rank order (the same order everywhere) and writes its
// stretch of the normalised row.  blockDim.x * 4 >= chunk (the columns per CTA, a multiple of 4).
template <typename TO>
__global__ void add_rmsnorm_cluster_kernel(float* __restrict__ x, const float* __restrict__ parts, int S,
                                           size_t part_stride, const float* __restrict__ w, TO* __restrict__ out,
                                           const int* __restrict__ rows, int d, float eps, int chunk) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  __shared__ float ss_all[8];
  const int r = blockIdx.y;
  unsigned rank, nc;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(nc));
  const int i = (int)rank * chunk + threadIdx.x * 4;
  const bool live = threadIdx.x * 4 < chunk && i < d;
  float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live && w != nullptr) w0 = *reinterpret_cast<const float4*>(w + i);
  const int src = rows ? rows[r] : r;
  pdl_wait();
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    float* xr = x + (size_t)src * d;
    const float* pr = parts + (size_t)src * d;
    v = *reinterpret_cast<const float4*>(xr + i);
    for (int s0 = 0; s0 < S; s0 += 16) {
      float4 t[16];
#pragma unroll
      for (int j = 0; j < 16; ++j)
        t[j] = (s0 + j < S) ? __ldcg(reinterpret_cast<const float4*>(pr + (size_t)(s0 + j) * part_stride + i))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (s0 + j < S) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
      }
    }
    *reinterpret_cast<float4*>(xr + i) = v;
  }
  if (w == nullptr) return;     // (uniform over the cluster: nobody reaches the barrier)
  float ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
  ss = block_sum(ss, scratch);
  if (threadIdx.x < nc) {
    unsigned local = (unsigned)__cvta_generic_to_shared(&ss_all[rank]), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"((unsigned)threadIdx.x));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(ss) : "memory");
  }
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  float total = 0.f;
  for (unsigned k = 0; k < nc; ++k) total += ss_all[k];
  const float sc = norm_scale<TO>(total / (float)d + eps);
  if (live) store4<TO>(out + (size_t)r * d + i, v.x * sc * w0.x, v.y * sc * w0.y, v.z * sc * w0.z, v.w * sc * w0.w);
}

// ------------------------------------------------------------------- SwiGLU
// in: [T, 2F] with the gate in columns [0, F) and the up projection in [F, 2F).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ in, T* __restrict__ out, int F, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  size_t t = i / F;
  int c = (int)(i - t * F);
  float g = to_float(in[t * 2 * F + c]);
  float u = to_float(in[t * 2 * F + F + c]);
  float h = g / (1.0f + expf(-g)) * u;
  out[i] = from_float<T>(h);
}

}  // namespace dlgo

using namespace dlgo;

// tokens[T] int32, table[vocab, d] (f32 or bf16), out[T, d] f32
DLGO_EXPORT int dlgo_embed(const int* tokens, const void* table, int table_dtype, float* out, int T, int d,
                           int vocab, cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (d <= 0 || vocab <= 0) return DLGO_ERR_SIZE;
  const int threads = d >= 1024 ? 256 : 128;
  if (table_dtype == DLGO_F32)
    launch_kernel_first(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, tokens, (const float*)table, out, d, vocab);
  else if (table_dtype == DLGO_BF16)
    launch_kernel_first(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, tokens, (const __nv_bfloat16*)table, out, d, vocab);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

// x[*, d] f32, w[d] f32, out[R, d] (f32 or bf16); rows[R] int32 or null (then row r of x)
DLGO_EXPORT int dlgo_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int* rows, int R,
                             int d, float eps, cudaStream_t stream) {
  if (R <= 0) return DLGO_OK;
  if (d <= 0) return DLGO_ERR_SIZE;
  if (out_dtype != DLGO_F32 && out_dtype != DLGO_BF16) return DLGO_ERR_DTYPE;
  if (R >= 256 && (d & 3) == 0 && d <= 32 * 4 * 32) {
    // many rows: a warp per row
    const dim3 grid((R + 7) / 8);
#define DLGO_ROWS(KV)                                                                                             \
  do {                                                                                                            \
    if (out_dtype == DLGO_F32)                                                                                    \
      launch_kernel(rmsnorm_rows_kernel<float, KV>, grid, dim3(256), 0, stream, x, w, (float*)out, rows, R, d, eps); \
    else                                                                                                          \
      launch_kernel(rmsnorm_rows_kernel<__nv_bfloat16, KV>, grid, dim3(256), 0, stream, x, w, (__nv_bfloat16*)out,  \
                    rows, R, d, eps);                                                                             \
  } while (0)
    if (d <= 32 * 4 * 4) DLGO_ROWS(4);
    else if (d <= 32 * 4 * 8) DLGO_ROWS(8);
    else if (d <= 32 * 4 * 16) DLGO_ROWS(16);
    else DLGO_ROWS(32);
#undef DLGO_ROWS
    return launch_status();
  }
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  if (out_dtype == DLGO_F32)
    launch_kernel(rmsnorm_kernel<float>, dim3(R), dim3(threads), 0, stream, x, w, (float*)out, rows, d, eps);
  else if (out_dtype == DLGO_BF16)
    launch_kernel(rmsnorm_kernel<__nv_bfloat16>, dim3(R), dim3(threads), 0, stream, x, w, (__nv_bfloat16*)out, rows, d, eps);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

// in[T, 2F], out[T, F], same element type
DLGO_EXPORT int dlgo_swiglu(const void* in, void* out, int dtype, int T, int F, cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (F <= 0) return DLGO_ERR_SIZE;
  const size_t total = (size_t)T * F;
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  if (dtype == DLGO_F32)
    launch_kernel(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)in, (float*)out, F, total);
  else if (dtype == DLGO_BF16)
    launch_kernel(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, F,
                                                                 total);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

// x[*, d] f32 (updated in place), parts[S][*, d] f32 (slice stride part_stride floats), w[d] f32 or null,
// out[R, d] (f32 or bf16, unused when w is null); rows[R] int32 or null
DLGO_EXPORT int dlgo_add_rmsnorm(float* x, const float* parts, int S, long long part_stride, const float* w,
                                 void* out, int out_dtype, const int* rows, int R, int d, float eps,
                                 cudaStream_t stream) {
  if (R <= 0) return DLGO_OK;
  if (d <= 0 || S < 0 || (size_t)d * sizeof(float) > 200 * 1024) return DLGO_ERR_SIZE;
  if (out_dtype != DLGO_F32 && out_dtype != DLGO_BF16) return DLGO_ERR_DTYPE;
  static const int cluster_on = [] { const char* e = getenv("DLGO_NORM_CLUSTER"); return e ? atoi(e) : 8; }();
  if (cluster_on > 1 && R <= 256 && d >= 1024 && (d & 3) == 0 && (part_stride & 3) == 0 && S > 0) {
    // few wide rows: a cluster of CTAs per row (at least 128 columns each)
    int nc = cluster_on > 8 ? 8 : cluster_on;
    while (nc > 1 && d / nc < 128) nc >>= 1;
    const int chunk = (((d + nc - 1) / nc) + 3) / 4 * 4;
    const int threads = ((chunk / 4) + 31) / 32 * 32;
    if (nc > 1 && threads <= 1024) {
      if (out_dtype == DLGO_F32)
        launch_kernel_cluster(add_rmsnorm_cluster_kernel<float>, dim3(nc, R), dim3(threads), 0, stream, dim3(nc, 1, 1),
                              x, parts, S, (size_t)part_stride, w, (float*)out, rows, d, eps, chunk);
      else
        launch_kernel_cluster(add_rmsnorm_cluster_kernel<__nv_bfloat16>, dim3(nc, R), dim3(threads), 0, stream,
                              dim3(nc, 1, 1), x, parts, S, (size_t)part_stride, w, (__nv_bfloat16*)out, rows, d, eps,
                              chunk);
      return launch_status();
    }
  }
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  const size_t smem = (size_t)d * sizeof(float);
  if (out_dtype == DLGO_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(add_rmsnorm_kernel<float>, dim3(R), dim3(threads), smem, stream, x, parts, S, (size_t)part_stride, w,
                  (float*)out, rows, d, eps);
  } else if (out_dtype == DLGO_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(add_rmsnorm_kernel<__nv_bfloat16>, dim3(R), dim3(threads), smem, stream, x, parts, S,
                  (size_t)part_stride, w, (__nv_bfloat16*)out, rows, d, eps);
  } else {
    return DLGO_ERR_DTYPE;
  }
  return launch_status();
}
