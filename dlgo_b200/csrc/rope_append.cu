// Rotary position encoding of the query and key heads and the append of this
// step's keys and values to the paged cache, in one pass over the fused
// projection output.
//
// Reference: rotation of every Q and K head at the token's absolute position
// from precomputed cos/sin tables (models/llm/forward.go:246-252,
// models/llm/workers.go:182-215; pairings ops/rope.go:21-31), then
// `Store(pos, k, v)` (models/llm/forward.go:257, memory/kvcache.go:30-36).
// Only the first `rot` dims of a head are rotated, the rest pass through
// (workers.go:151-159).  The rotation is computed in fp32.
//
// qkv[T, ld]: q heads, then k heads, then v heads, `hd` elements each (or, with
// `parts`, the unsummed fp32 K-slices [S][T][ld] of the projection, which are
// added here; qkv then only receives the rotated q).  q is rotated in place; k (rotated) and v go to the page of their position:
// pages[page_table[slot][pos / PS]][kv_head][pos % PS][:].
#include "common.cuh"

namespace dlgo {

// Set when a token's position had no page in the table (-1): the append is skipped, never written
// through a negative page number, and the host reads the word (dlgo_rope_append_error).
__device__ int g_rope_append_error = 0;

template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, const int* __restrict__ token_pos,
                                   const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                   const int* __restrict__ page_table, int max_pages, T* __restrict__ kpages,
                                   T* __restrict__ vpages, int Hq, int Hkv, int hd, int rot, int page_size,
                                   int interleaved, int write_cache, const float* __restrict__ parts, int S,
                                   size_t part_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = hd / 2, rhalf = rot / 2;
  const int items = (Hq + 2 * Hkv) * half;
  const int pos = token_pos[t];
  T* row = qkv + (size_t)t * ld;
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (write_cache) {
    const int slot = seq_slot[token_seq[t]];
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    if (page < 0) {
      write_cache = 0;
      if (threadIdx.x == 0) atomicExch(&g_rope_append_error, 1);
    }
    const size_t base = ((size_t)max(page, 0) * Hkv) * page_size * hd + (size_t)(pos % page_size) * hd;
    kdst = kpages + base;
    vdst = vpages + base;
  }
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    const int head = it / half, i = it - head * half;
    T* h = row + (size_t)head * hd;
    int i0, i1;
    bool rotate = i < rhalf;
    if (rotate) {
      if (interleaved) { i0 = 2 * i; i1 = 2 * i + 1; }
      else { i0 = i; i1 = i + rhalf; }
    } else {
      i0 = rot + 2 * (i - rhalf);
      i1 = i0 + 1;
    }
    float x0, x1;
    if (parts != nullptr) {
      // the projection left its K-slices unsummed ([S][T][ld] fp32): add them in order here
      const float* pp = parts + (size_t)t * ld + (size_t)head * hd;
      x0 = 0.f;
      x1 = 0.f;
      for (int sp = 0; sp < S; ++sp) {
        x0 += pp[(size_t)sp * part_stride + i0];
        x1 += pp[(size_t)sp * part_stride + i1];
      }
    } else {
      x0 = to_float(h[i0]);
      x1 = to_float(h[i1]);
    }
    if (head < Hq + Hkv && rotate) {
      const float c = cos_t[(size_t)pos * rhalf + i], s = sin_t[(size_t)pos * rhalf + i];
      const float y0 = x0 * c - x1 * s;
      const float y1 = x0 * s + x1 * c;
      x0 = y0;
      x1 = y1;
    }
    if (head < Hq) {
      h[i0] = from_float<T>(x0);
      h[i1] = from_float<T>(x1);
    } else if (write_cache) {
      const bool is_k = head < Hq + Hkv;
      const int kvh = is_k ? head - Hq : head - Hq - Hkv;
      T* dst = (is_k ? kdst : vdst) + (size_t)kvh * page_size * hd;
      dst[i0] = from_float<T>(x0);
      dst[i1] = from_float<T>(x1);
    }
  }
}

// The same for the common layout (pairs (i, i + hd/2), the whole head rotated, no K-slices to add):
// a thread takes 16 bytes from the low half of a head and the 16 bytes they pair with in the high
// half, so prompts move through this kernel at memory speed.
template <typename T> struct RVec;
template <> struct RVec<float> { static constexpr int N = 4; };
template <> struct RVec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ void rv_load(const T* p, float* o);
template <> __device__ __forceinline__ void rv_load<float>(const float* p, float* o) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <> __device__ __forceinline__ void rv_load<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}
template <typename T>
__device__ __forceinline__ void rv_store(T* p, const float* o);
template <> __device__ __forceinline__ void rv_store<float>(float* p, const float* o) {
  *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
}
template <> __device__ __forceinline__ void rv_store<__nv_bfloat16>(__nv_bfloat16* p, const float* o) {
  __nv_bfloat162 h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(h);
}

template <typename T>
__global__ void rope_append_vec_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, const int* __restrict__ token_pos,
                                       const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                       const int* __restrict__ page_table, int max_pages, T* __restrict__ kpages,
                                       T* __restrict__ vpages, int Hq, int Hkv, int hd, int page_size,
                                       int write_cache) {
  pdl_launch_dependents();
  constexpr int N = RVec<T>::N;
  const int t = blockIdx.x;
  const int rhalf = hd / 2, per_head = rhalf / N;
  const int items = (Hq + 2 * Hkv) * per_head;
  // the step's own inputs: read before waiting for the projection
  const int pos = token_pos[t];
  T* row = qkv + (size_t)t * ld;
  size_t base = 0;
  if (write_cache) {
    const int slot = seq_slot[token_seq[t]];
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    if (page < 0) {
      write_cache = 0;
      if (threadIdx.x == 0) atomicExch(&g_rope_append_error, 1);
    }
    base = ((size_t)max(page, 0) * Hkv) * page_size * hd + (size_t)(pos % page_size) * hd;
  }
  pdl_wait();
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    const int head = it / per_head, i = (it - head * per_head) * N;
    T* h = row + (size_t)head * hd;
    float lo[N], hi[N];
    rv_load<T>(h + i, lo);
    rv_load<T>(h + i + rhalf, hi);
    if (head < Hq + Hkv) {
      float c[N], sn[N];
#pragma unroll
      for (int e = 0; e < N; e += 4) {
        const float4 cc = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * rhalf + i + e);
        const float4 ss = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * rhalf + i + e);
        c[e] = cc.x; c[e + 1] = cc.y; c[e + 2] = cc.z; c[e + 3] = cc.w;
        sn[e] = ss.x; sn[e + 1] = ss.y; sn[e + 2] = ss.z; sn[e + 3] = ss.w;
      }
#pragma unroll
      for (int e = 0; e < N; ++e) {
        const float x0 = lo[e], x1 = hi[e];
        lo[e] = x0 * c[e] - x1 * sn[e];
        hi[e] = x0 * sn[e] + x1 * c[e];
      }
    }
    if (head < Hq) {
      rv_store<T>(h + i, lo);
      rv_store<T>(h + i + rhalf, hi);
    } else if (write_cache) {
      const bool is_k = head < Hq + Hkv;
      const int kvh = is_k ? head - Hq : head - Hq - Hkv;
      T* dst = (is_k ? kpages : vpages) + base + (size_t)kvh * page_size * hd;
      rv_store<T>(dst + i, lo);
      rv_store<T>(dst + i + rhalf, hi);
    }
  }
}

// The same when the projection left its K-slices unsummed (decode steps): one warp per (token, head),
// so that a step's few tokens still spread over many SMs.  Everything that does not depend on the
// projection (position, page, cos / sin) is fetched before the kernel waits for it; after the wait
// a lane has eight slices' loads of a pair in flight at once.
// SUM: `parts` is one fp32 sum that the projection's K-slices added themselves into (S = 1); it is read
// once, here, and left zero for the next step's projection.
constexpr int RP_WARPS = 4;
template <typename T, bool SUM>
__global__ void __launch_bounds__(RP_WARPS * 32)
rope_append_parts_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ cos_t,
                         const float* __restrict__ sin_t, const int* __restrict__ token_pos,
                         const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                         const int* __restrict__ page_table, int max_pages, T* __restrict__ kpages,
                         T* __restrict__ vpages, int Hq, int Hkv, int hd, int rot, int page_size,
                         int interleaved, int write_cache, const float* __restrict__ parts, int S,
                         size_t part_stride) {
  pdl_launch_dependents();
  const int t = blockIdx.y;
  const int head = blockIdx.x * RP_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int half = hd / 2, rhalf = rot / 2;
  const bool active = head < Hq + 2 * Hkv;
  const int pos = token_pos[t];
  T* dst = nullptr;                       // where the head goes: q in place, k and v to their page
  if (active) {
    if (head < Hq) {
      dst = qkv + (size_t)t * ld + (size_t)head * hd;
    } else if (write_cache) {
      const int slot = seq_slot[token_seq[t]];
      const int page = page_table[(size_t)slot * max_pages + pos / page_size];
      const bool is_k = head < Hq + Hkv;
      const int kvh = is_k ? head - Hq : head - Hq - Hkv;
      if (page >= 0)
        dst = (is_k ? kpages : vpages) + (((size_t)page * Hkv + kvh) * page_size + (size_t)(pos % page_size)) * hd;
      else if (lane == 0)
        atomicExch(&g_rope_append_error, 1);
    }
  }
  const bool rotates = active && head < Hq + Hkv;
  // first pair of this lane: its angle is ready before the wait
  float c0 = 1.f, s0 = 0.f;
  if (rotates && lane < rhalf) {
    c0 = cos_t[(size_t)pos * rhalf + lane];
    s0 = sin_t[(size_t)pos * rhalf + lane];
  }
  pdl_wait();
  if (!active || (dst == nullptr && !SUM)) return;
  const float* pp = parts + (size_t)t * ld + (size_t)head * hd;
  for (int i = lane; i < half; i += 32) {
    int i0, i1;
    const bool rotate = i < rhalf;
    if (rotate) {
      if (interleaved) { i0 = 2 * i; i1 = 2 * i + 1; }
      else { i0 = i; i1 = i + rhalf; }
    } else {
      i0 = rot + 2 * (i - rhalf);
      i1 = i0 + 1;
    }
    float x0 = 0.f, x1 = 0.f;
    if constexpr (SUM) {
      float* sum = const_cast<float*>(pp);
      x0 = __ldcg(sum + i0);
      x1 = __ldcg(sum + i1);
      sum[i0] = 0.f;
      sum[i1] = 0.f;
      if (dst == nullptr) continue;
    }
    for (int sb = 0; !SUM && sb < S; sb += 8) {
      float a[8], b[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] = (sb + j < S) ? __ldcg(pp + (size_t)(sb + j) * part_stride + i0) : 0.f;
        b[j] = (sb + j < S) ? __ldcg(pp + (size_t)(sb + j) * part_stride + i1) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (sb + j < S) { x0 += a[j]; x1 += b[j]; }
      }
    }
    if (rotates && rotate) {
      float c = c0, sn = s0;
      if (i != lane) {
        c = cos_t[(size_t)pos * rhalf + i];
        sn = sin_t[(size_t)pos * rhalf + i];
      }
      const float y0 = x0 * c - x1 * sn;
      const float y1 = x0 * sn + x1 * c;
      x0 = y0;
      x1 = y1;
    }
    dst[i0] = from_float<T>(x0);
    dst[i1] = from_float<T>(x1);
  }
}

}  // namespace dlgo

using namespace dlgo;

DLGO_EXPORT int dlgo_rope_append(void* qkv, int dtype, int T, int ld, const float* cos_t, const float* sin_t,
                                 const int* token_pos, const int* token_seq, const int* seq_slot,
                                 const int* page_table, int max_pages, void* kpages, void* vpages, int Hq, int Hkv,
                                 int hd, int rot, int page_size, int interleaved, int write_cache,
                                 const float* parts, int S, long long part_stride, int clear_parts,
                                 cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (hd <= 0 || hd % 2 || rot < 0 || rot > hd || rot % 2 || Hq <= 0 || Hkv <= 0 || page_size <= 0 ||
      ld < (Hq + 2 * Hkv) * hd)
    return DLGO_ERR_SIZE;
  const int vec = dtype == DLGO_BF16 ? 8 : 4;
  if (parts == nullptr && !interleaved && rot == hd && (hd / 2) % vec == 0 && ld % vec == 0 &&
      ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)kpages & 15) == 0 && ((uintptr_t)vpages & 15) == 0) {
    const int vitems = (Hq + 2 * Hkv) * (hd / 2 / vec);
    const int vthreads = vitems >= 256 ? 256 : (vitems >= 128 ? 128 : 64);
    if (dtype == DLGO_F32)
      launch_kernel(rope_append_vec_kernel<float>, dim3(T), dim3(vthreads), 0, stream, (float*)qkv, ld, cos_t, sin_t,
                    token_pos, token_seq, seq_slot, page_table, max_pages, (float*)kpages, (float*)vpages, Hq, Hkv, hd,
                    page_size, write_cache);
    else if (dtype == DLGO_BF16)
      launch_kernel(rope_append_vec_kernel<__nv_bfloat16>, dim3(T), dim3(vthreads), 0, stream, (__nv_bfloat16*)qkv, ld,
                    cos_t, sin_t, token_pos, token_seq, seq_slot, page_table, max_pages, (__nv_bfloat16*)kpages,
                    (__nv_bfloat16*)vpages, Hq, Hkv, hd, page_size, write_cache);
    else
      return DLGO_ERR_DTYPE;
    return launch_status();
  }
  if (clear_parts && (parts == nullptr || S != 1 || T > 65535)) return DLGO_ERR_SIZE;
  if (parts != nullptr && T <= 65535) {
    const dim3 grid((Hq + 2 * Hkv + RP_WARPS - 1) / RP_WARPS, T);
#define DLGO_ROPE_PARTS(TT, SUM)                                                                                  \
  launch_kernel(rope_append_parts_kernel<TT, SUM>, grid, dim3(RP_WARPS * 32), 0, stream, (TT*)qkv, ld, cos_t, sin_t, \
                token_pos, token_seq, seq_slot, page_table, max_pages, (TT*)kpages, (TT*)vpages, Hq, Hkv, hd, rot, \
                page_size, interleaved, write_cache, parts, S, (size_t)part_stride)
    if (dtype == DLGO_F32) {
      if (clear_parts) DLGO_ROPE_PARTS(float, true); else DLGO_ROPE_PARTS(float, false);
    } else if (dtype == DLGO_BF16) {
      if (clear_parts) DLGO_ROPE_PARTS(__nv_bfloat16, true); else DLGO_ROPE_PARTS(__nv_bfloat16, false);
    } else {
      return DLGO_ERR_DTYPE;
    }
#undef DLGO_ROPE_PARTS
    return launch_status();
  }
  const int items = (Hq + 2 * Hkv) * (hd / 2);
  const int threads = items >= 1024 ? 256 : 128;
  if (dtype == DLGO_F32)
    launch_kernel(rope_append_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)qkv, ld, cos_t, sin_t, token_pos, token_seq, seq_slot,
                                                         page_table, max_pages, (float*)kpages, (float*)vpages, Hq,
                                                         Hkv, hd, rot, page_size, interleaved, write_cache, parts, S,
                                                         (size_t)part_stride);
  else if (dtype == DLGO_BF16)
    launch_kernel(rope_append_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, 
        (__nv_bfloat16*)qkv, ld, cos_t, sin_t, token_pos, token_seq, seq_slot, page_table, max_pages,
        (__nv_bfloat16*)kpages, (__nv_bfloat16*)vpages, Hq, Hkv, hd, rot, page_size, interleaved, write_cache, parts,
        S, (size_t)part_stride);
  else
    return DLGO_ERR_DTYPE;
  return launch_status();
}

// 1 if an append was skipped since the last call because its position had no page (clears the word).
DLGO_EXPORT int dlgo_rope_append_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_rope_append_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_rope_append_error, &zero, sizeof(int));
  return v;
}
