// Attention for decode steps: one new token per sequence against its cached keys and values.
//
// Same formulas as attention.cu (models/llm/forward.go:258-278): scores q.k * scale over the keys
// t <= pos (t > pos - window if windowed), softmax, weighted sum of the values, all in fp32.  Decode
// reads every cached key and value once and does a handful of flops per byte, so the kernel is
// shaped for memory latency, not arithmetic:
//   * a block takes one sequence, one kv head (up to 4 of its query heads) and a slice of the pages;
//   * a warp takes tiles of keys; LPK lanes share a key, each loading 16 bytes of it straight from
//     global memory (coalesced rows of the page), so nothing is staged in shared memory;
//   * scores of a tile are kept in registers, the running maximum is made uniform across the warp,
//     and the values of the same tile are then streamed with the probabilities as weights;
//   * lanes, then warps, merge their partial sums; with several slices the partial (max, sum,
//     output) go to scratch and attention_combine_kernel finishes.
#include <cooperative_groups.h>
#include <math.h>

#include "attention_combine.cuh"
#include "common.cuh"

namespace dlgo {

constexpr int DEC_THREADS = 128;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int DEC_GMAX = 4;   // query heads of a kv head per block
constexpr int DEC_ITER = 4;   // keys per lane group and tile

struct DecParams {
  const void* q;
  int ldq;
  const void* kpages;
  const void* vpages;
  const int* page_table;
  int max_pages;
  const int* seq_slot;   // [B]
  const int* token_pos;  // [B] position of the new token (its key is already in the cache)
  void* out;
  int ldo;
  float* part_acc;
  float* part_ml;
  int* counters;         // [B * Hkv * n_gchunks] zero before the first launch and left zero, or null
  int Hq, Hkv, page_size, n_splits, n_gchunks, window;
  int cluster;           // 1: the slices of a (sequence, kv head) form one thread-block cluster and combine
                         // through distributed shared memory; no scratch, no counters
  float scale;
};

template <typename T> struct Ld16;
template <> struct Ld16<float> {
  static constexpr int VEC = 4;
  __device__ static void load(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct Ld16<__nv_bfloat16> {
  static constexpr int VEC = 8;
  __device__ static void load(const __nv_bfloat16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      o[2 * i] = f.x;
      o[2 * i + 1] = f.y;
    }
  }
};

template <typename T> __device__ __forceinline__ void cvt16(const uint4& raw, float* o);
template <> __device__ __forceinline__ void cvt16<float>(const uint4& raw, float* o) {
  o[0] = __uint_as_float(raw.x); o[1] = __uint_as_float(raw.y); o[2] = __uint_as_float(raw.z); o[3] = __uint_as_float(raw.w);
}
template <> __device__ __forceinline__ void cvt16<__nv_bfloat16>(const uint4& raw, float* o) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}

// exp(x) for the softmax: exact expf in the float32 path; in the bfloat16 path one ex2.approx (the
// result is rounded to far fewer bits than it loses)
template <typename T> __device__ __forceinline__ float soft_exp(float x);
template <> __device__ __forceinline__ float soft_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ float soft_exp<__nv_bfloat16>(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}

// LPK lanes per key; head_dim = LPK * VEC.
template <typename T, int LPK>
__global__ void __launch_bounds__(DEC_THREADS, 4) attention_decode_kernel(DecParams p) {
  pdl_launch_dependents();
  if (threadIdx.x == 0) TSTAMP(0);
  constexpr int VEC = Ld16<T>::VEC;
  constexpr int HD = LPK * VEC;
  constexpr int KPW = 32 / LPK;            // keys a warp covers per iteration
  constexpr int TILE = KPW * DEC_ITER;     // keys per tile (divides the page size)
  __shared__ float sm_acc[DEC_WARPS][DEC_GMAX][HD];
  __shared__ float sm_ml[DEC_WARPS][DEC_GMAX][2];
  __shared__ int sm_last;
  __shared__ __align__(16) T sm_v[DEC_WARPS][TILE * HD];   // a warp's tile of values, copied in asynchronously
  __shared__ float cl_acc[DEC_GMAX][HD];   // this block's merged result, read by the cluster's first block
  __shared__ float cl_ml[DEC_GMAX][2];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPK;              // which 16 bytes of the key
  const int grp = lane / LPK;              // which key of the iteration
  const int b = blockIdx.x;
  const int kvh = blockIdx.y / p.n_gchunks, gc = blockIdx.y - kvh * p.n_gchunks;
  const int split = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int g0 = gc * DEC_GMAX;
  const int GC = min(DEC_GMAX, G - g0);
  const int PS = p.page_size;
  const int slot = p.seq_slot[b];
  const int pos = p.token_pos[b];
  const int t_end = pos + 1;
  const int t_begin = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int pg_first = t_begin / PS, pg_last = pos / PS;
  const int per = (pg_last - pg_first + 1 + p.n_splits - 1) / p.n_splits;
  const int pg_b = pg_first + split * per;
  const int pg_e = min(pg_last + 1, pg_b + per);

  const int tiles_per_page = PS / TILE;
  const int n_tiles = max(0, pg_e - pg_b) * tiles_per_page;
  // Before waiting for the kernels that make q (and the newest key): the step's own inputs above
  // (slot, position, page ids: later loads of them hit L1) and a hint that pulls this block's keys
  // and values into L2, so that the loads after the wait are short round trips.  The cache lines of
  // the newest position may still be written; a prefetch of them is harmless (L2 is coherent).
  for (int tile = warp; tile < n_tiles; tile += DEC_WARPS) {
    const int pg = pg_b + tile / tiles_per_page;
    const int key0 = (tile % tiles_per_page) * TILE;
    if (pg * PS + key0 >= t_end) continue;
    const int page = p.page_table[(size_t)slot * p.max_pages + pg];
    const size_t base = (((size_t)page * p.Hkv + kvh) * PS + key0) * HD;
    const char* kp = (const char*)((const T*)p.kpages + base);
    const char* vp = (const char*)((const T*)p.vpages + base);
    constexpr int LINES = TILE * HD * (int)sizeof(T) / 128;
    if (n_tiles <= 4 * DEC_WARPS) {   // short slices only: hinting a long slice all at once slows it down
      for (int ln = lane; ln < LINES; ln += 32) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(kp + (size_t)ln * 128));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(vp + (size_t)ln * 128));
      }
    }
  }
  if (threadIdx.x == 0) TSTAMP(1);
  pdl_wait();
  if (threadIdx.x == 0) TSTAMP(2);

  float q[DEC_GMAX][VEC], acc[DEC_GMAX][VEC], m[DEC_GMAX], l[DEC_GMAX];
  {
    const T* qrow = (const T*)p.q + (size_t)b * p.ldq + (size_t)(kvh * G + g0) * HD + sub * VEC;
#pragma unroll
    for (int g = 0; g < DEC_GMAX; ++g) {
      if (g < GC) Ld16<T>::load(qrow + (size_t)g * HD, q[g]);
      else
#pragma unroll
        for (int e = 0; e < VEC; ++e) q[g][e] = 0.f;
    }
  }
#pragma unroll
  for (int g = 0; g < DEC_GMAX; ++g) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[g][e] = 0.f;
    m[g] = -INFINITY;
    l[g] = 0.f;
  }

  for (int tile = warp; tile < n_tiles; tile += DEC_WARPS) {
    const int pg = pg_b + tile / tiles_per_page;
    const int key0 = (tile % tiles_per_page) * TILE;
    if (pg * PS + key0 >= t_end) continue;                       // wholly beyond the sequence (warp-uniform)
    const int page = p.page_table[(size_t)slot * p.max_pages + pg];
    const size_t base = ((size_t)page * p.Hkv + kvh) * PS * HD;
    const T* kp = (const T*)p.kpages + base;
    const T* vp = (const T*)p.vpages + base;
    float s[DEC_GMAX][DEC_ITER];
    bool live[DEC_ITER];
    float tmax[DEC_GMAX];
    // All of the tile's keys AND values are requested before any arithmetic: one memory round trip.
    // The keys come into registers; the values, needed later, are copied asynchronously into this
    // lane's own 16 bytes of shared memory (no registers held meanwhile, nothing shared between lanes).
    uint4 kraw[DEC_ITER];
#pragma unroll
    for (int it = 0; it < DEC_ITER; ++it) {
      const int key = key0 + it * KPW + grp;
      const int t = pg * PS + key;
      live[it] = t < t_end && t >= t_begin;
      kraw[it] = make_uint4(0u, 0u, 0u, 0u);
      if (live[it]) {
        kraw[it] = *reinterpret_cast<const uint4*>(kp + (size_t)key * HD + sub * VEC);
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&sm_v[warp][(it * KPW + grp) * HD + sub * VEC]);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(vp + (size_t)key * HD + sub * VEC)
                     : "memory");
      }
    }
#pragma unroll
    for (int g = 0; g < DEC_GMAX; ++g) tmax[g] = -INFINITY;
#pragma unroll
    for (int it = 0; it < DEC_ITER; ++it) {
      float kf[VEC];
      cvt16<T>(kraw[it], kf);
#pragma unroll
      for (int g = 0; g < DEC_GMAX; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < VEC; ++e) d = fmaf(q[g][e], kf[e], d);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        s[g][it] = live[it] ? d * p.scale : -INFINITY;
        tmax[g] = fmaxf(tmax[g], s[g][it]);
      }
    }
    // one running maximum per head for the whole warp, so partial sums of its lane groups add up
#pragma unroll
    for (int g = 0; g < DEC_GMAX; ++g) {
#pragma unroll
      for (int o = 16; o >= LPK; o >>= 1) tmax[g] = fmaxf(tmax[g], __shfl_xor_sync(0xffffffffu, tmax[g], o));
      const float m_new = fmaxf(m[g], tmax[g]);
      const float c = (m[g] == -INFINITY) ? 0.f : soft_exp<T>(m[g] - m_new);
      m[g] = m_new;
      l[g] *= c;
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[g][e] *= c;
#pragma unroll
      for (int it = 0; it < DEC_ITER; ++it) {
        const float pr = (s[g][it] == -INFINITY) ? 0.f : soft_exp<T>(s[g][it] - m_new);
        s[g][it] = pr;
        l[g] += pr;
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
#pragma unroll
    for (int it = 0; it < DEC_ITER; ++it) {
      float vf[VEC];
      // zeros where the key is not live (nothing was copied there; its probability is zero as well)
      const uint4 vraw = live[it] ? *reinterpret_cast<const uint4*>(&sm_v[warp][(it * KPW + grp) * HD + sub * VEC])
                                  : make_uint4(0u, 0u, 0u, 0u);
      cvt16<T>(vraw, vf);
#pragma unroll
      for (int g = 0; g < DEC_GMAX; ++g)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[g][e] = fmaf(s[g][it], vf[e], acc[g][e]);
    }
  }

  if (threadIdx.x == 0) TSTAMP(3);
  // lane groups of a warp share their maximum: sums add up.  l was counted once per lane of a
  // group, so only lanes with sub == 0 contribute it.
#pragma unroll
  for (int g = 0; g < DEC_GMAX; ++g) {
    float lg = (sub == 0) ? l[g] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lg += __shfl_xor_sync(0xffffffffu, lg, o);
    l[g] = lg;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float a = acc[g][e];
#pragma unroll
      for (int o = 16; o >= LPK; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      acc[g][e] = a;
    }
    if (grp == 0) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) sm_acc[warp][g][sub * VEC + e] = acc[g][e];
      if (sub == 0) {
        sm_ml[warp][g][0] = m[g];
        sm_ml[warp][g][1] = l[g];
      }
    }
  }
  __syncthreads();
  // merge the warps: thread -> (head g, dim d)
  for (int idx = threadIdx.x; idx < GC * HD; idx += DEC_THREADS) {
    const int g = idx / HD, d = idx - g * HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, sm_ml[w][g][0]);
    float a = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float mw = sm_ml[w][g][0];
      if (mw != -INFINITY) {
        const float c = expf(mw - mm);
        a = fmaf(c, sm_acc[w][g][d], a);
        ll = fmaf(c, sm_ml[w][g][1], ll);
      }
    }
    const int head = kvh * G + g0 + g;
    if (p.n_splits == 1) {
      ((T*)p.out)[(size_t)b * p.ldo + (size_t)head * HD + d] = from_float<T>(a / ll);
    } else if (p.cluster) {
      cl_acc[g][d] = a;
      if (d == 0) {
        cl_ml[g][0] = mm;
        cl_ml[g][1] = ll;
      }
    } else {
      const size_t o = ((size_t)b * p.Hq + head) * p.n_splits + split;
      p.part_acc[o * HD + d] = a;
      if (d == 0) {
        p.part_ml[o * 2] = mm;
        p.part_ml[o * 2 + 1] = ll;
      }
    }
  }
  if (p.n_splits > 1 && p.cluster) {
    // The slices of this (sequence, kv head, head chunk) are the blocks of one cluster: each leaves
    // its merged (max, sum, output) in its own shared memory, the first block reads them all through
    // distributed shared memory and writes the result.  No global round trip, fence or ticket.
    namespace cg = cooperative_groups;
    cg::cluster_group cl = cg::this_cluster();
    if (threadIdx.x == 0) TSTAMP(4);
    cl.sync();
    if (threadIdx.x == 0) TSTAMP(5);
    if (cl.block_rank() == 0) {
      const int NS = p.n_splits;
      for (int idx = threadIdx.x; idx < GC * HD; idx += DEC_THREADS) {
        const int g = idx / HD, d = idx - g * HD;
        float ms[8], ls[8], as[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (r < NS) {
            const float* rml = cl.map_shared_rank(&cl_ml[0][0], r);
            const float* racc = cl.map_shared_rank(&cl_acc[0][0], r);
            ms[r] = rml[g * 2];
            ls[r] = rml[g * 2 + 1];
            as[r] = racc[g * HD + d];
          } else {
            ms[r] = -INFINITY;
            ls[r] = 0.f;
            as[r] = 0.f;
          }
        }
        float mm = -INFINITY;
#pragma unroll
        for (int r = 0; r < 8; ++r) mm = fmaxf(mm, ms[r]);
        float a = 0.f, ll = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const float c = (ms[r] == -INFINITY) ? 0.f : expf(ms[r] - mm);
          a = fmaf(c, as[r], a);
          ll = fmaf(c, ls[r], ll);
        }
        ((T*)p.out)[(size_t)b * p.ldo + (size_t)(kvh * G + g0 + g) * HD + d] = from_float<T>(a / ll);
      }
    }
    if (threadIdx.x == 0) TSTAMP(6);
    cl.sync();   // nobody leaves while its shared memory may still be read
    if (threadIdx.x == 0) TSTAMP(7);
    return;
  }
  if (p.n_splits == 1 || p.counters == nullptr) return;
  // the block that finishes last among the slices of this (sequence, kv head, head chunk) combines them
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* c = p.counters + (size_t)b * gridDim.y + blockIdx.y;
    const int ticket = atomicAdd(c, 1);
    sm_last = ticket == p.n_splits - 1;
    if (sm_last) *c = 0;
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  // Weights of the slices first (one round trip for all of them, through shared memory), then the
  // weighted sum with several slices' loads in flight: no load waits on a branch.
  float* w_s = &sm_acc[0][0][0];                 // [GC][n_splits] weights, then [GC] 1 / denominators
  const int NS = p.n_splits;
  const bool fits = GC * (NS + 1) <= DEC_WARPS * DEC_GMAX * HD;
  float* l_sm = w_s + GC * (NS + 1);             // [GC][n_splits] the slices' sums
  const bool fits2 = GC * (2 * NS + 1) <= DEC_WARPS * DEC_GMAX * HD;
  if (fits && fits2) {
    for (int idx = threadIdx.x; idx < GC * NS; idx += DEC_THREADS) {
      const int g = idx / NS, sp = idx - g * NS;
      const size_t o = ((size_t)b * p.Hq + kvh * G + g0 + g) * NS + sp;
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(&p.part_ml[o * 2]));
      w_s[idx] = ml.x;                           // the slice's maximum for now
      l_sm[idx] = ml.y;
    }
    __syncthreads();
    if (threadIdx.x < GC) {
      const int g = threadIdx.x;
      float mm = -INFINITY;
      for (int sp = 0; sp < NS; ++sp) mm = fmaxf(mm, w_s[g * NS + sp]);
      float ll = 0.f;
      for (int sp = 0; sp < NS; ++sp) {
        const float ms = w_s[g * NS + sp];
        const float c = (ms == -INFINITY) ? 0.f : expf(ms - mm);
        w_s[g * NS + sp] = c;
        ll = fmaf(c, l_sm[g * NS + sp], ll);
      }
      w_s[GC * NS + g] = 1.0f / ll;
    }
    __syncthreads();
  }
  for (int idx = threadIdx.x; idx < GC * HD; idx += DEC_THREADS) {
    const int g = idx / HD, d = idx - g * HD;
    const int head = kvh * G + g0 + g;
    const size_t o = ((size_t)b * p.Hq + head) * NS;
    float a = 0.f, inv;
    if (fits && fits2) {
      int sp = 0;
      for (; sp + 4 <= NS; sp += 4) {
        const float x0 = __ldcg(&p.part_acc[(o + sp) * HD + d]), x1 = __ldcg(&p.part_acc[(o + sp + 1) * HD + d]);
        const float x2 = __ldcg(&p.part_acc[(o + sp + 2) * HD + d]), x3 = __ldcg(&p.part_acc[(o + sp + 3) * HD + d]);
        a = fmaf(w_s[g * NS + sp], x0, a);
        a = fmaf(w_s[g * NS + sp + 1], x1, a);
        a = fmaf(w_s[g * NS + sp + 2], x2, a);
        a = fmaf(w_s[g * NS + sp + 3], x3, a);
      }
      for (; sp < NS; ++sp) a = fmaf(w_s[g * NS + sp], __ldcg(&p.part_acc[(o + sp) * HD + d]), a);
      inv = w_s[GC * NS + g];
    } else {
      float mm = -INFINITY, ll = 0.f;
      for (int sp = 0; sp < NS; ++sp) mm = fmaxf(mm, __ldcg(&p.part_ml[(o + sp) * 2]));
      for (int sp = 0; sp < NS; ++sp) {
        const float ms = __ldcg(&p.part_ml[(o + sp) * 2]);
        const float c = (ms == -INFINITY) ? 0.f : expf(ms - mm);
        a = fmaf(c, __ldcg(&p.part_acc[(o + sp) * HD + d]), a);
        ll = fmaf(c, __ldcg(&p.part_ml[(o + sp) * 2 + 1]), ll);
      }
      inv = 1.0f / ll;
    }
    ((T*)p.out)[(size_t)b * p.ldo + (size_t)head * HD + d] = from_float<T>(a * inv);
  }
}

template <typename T, int LPK>
int launch_decode(const DecParams& p, int B, cudaStream_t stream) {
  constexpr int HD = LPK * Ld16<T>::VEC;
  dim3 grid(B, p.Hkv * p.n_gchunks, p.n_splits);
  if (p.cluster && p.n_splits > 1) {
    launch_kernel_cluster(attention_decode_kernel<T, LPK>, grid, dim3(DEC_THREADS), 0, stream, dim3(1, 1, p.n_splits), p);
    return launch_status();
  }
  launch_kernel(attention_decode_kernel<T, LPK>, dim3(grid), dim3(DEC_THREADS), 0, stream, p);
  int st = launch_status();
  if (st != DLGO_OK || p.n_splits == 1 || p.counters != nullptr) return st;
  dim3 cgrid(B, p.Hq);
  const int threads = HD >= 128 ? 128 : (HD >= 64 ? 64 : 32);
  launch_kernel(attention_combine_kernel<T>, dim3(cgrid), dim3(threads), 0, stream, p.part_acc, p.part_ml, (T*)p.out, p.ldo, p.Hq, HD,
                                                             p.n_splits);
  return launch_status();
}

template <typename T>
int dispatch_decode(const DecParams& p, int B, int hd, cudaStream_t stream) {
  switch (hd / Ld16<T>::VEC) {
    case 2: return launch_decode<T, 2>(p, B, stream);
    case 4: return launch_decode<T, 4>(p, B, stream);
    case 8: return launch_decode<T, 8>(p, B, stream);
    case 16: return launch_decode<T, 16>(p, B, stream);
    case 32: return launch_decode<T, 32>(p, B, stream);
    default: return DLGO_ERR_SIZE;
  }
}

}  // namespace dlgo

using namespace dlgo;

namespace {
int decode_common(DecParams& p, int dtype, int B, int hd, cudaStream_t stream) {
  if (dtype == DLGO_F32) return dispatch_decode<float>(p, B, hd, stream);
  return dispatch_decode<__nv_bfloat16>(p, B, hd, stream);
}
}  // namespace

// 1 if the kernel takes this head size for this element type (16 bytes per lane, 2..32 lanes per key)
DLGO_EXPORT int dlgo_attention_decode_takes(int dtype, int hd, int page_size) {
  const int vec = dtype == DLGO_BF16 ? 8 : 4;
  if (hd % vec) return 0;
  const int lpk = hd / vec;
  if (!(lpk == 2 || lpk == 4 || lpk == 8 || lpk == 16 || lpk == 32)) return 0;
  const int tile = (32 / lpk) * DEC_ITER;
  return page_size % tile == 0;
}

// q[B, .] (row stride ldq, head h at column h*hd), one token per sequence at position token_pos[b];
// scratch: B * Hq * n_splits * (hd + 2) floats when n_splits > 1.  counters: B * Hkv * ceil(G / 4) ints,
// zero before the first call (the kernel leaves them zero): the last slice to finish then combines the
// partial results itself; with counters == null a second kernel does.  With scratch == null and
// 2 <= n_splits <= 8 the slices form a thread-block cluster and combine through distributed shared memory.
DLGO_EXPORT int dlgo_attention_decode(const void* q, int dtype, int B, int ldq, const void* kpages,
                                      const void* vpages, const int* page_table, int max_pages,
                                      const int* seq_slot, const int* token_pos, void* out, int ldo, float* scratch,
                                      int* counters, int Hq, int Hkv, int hd, int page_size, int n_splits,
                                      int window, float scale, cudaStream_t stream) {
  if (B <= 0) return DLGO_OK;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || n_splits <= 0 || n_splits > 65535) return DLGO_ERR_SIZE;
  if (dtype != DLGO_F32 && dtype != DLGO_BF16) return DLGO_ERR_DTYPE;
  if (!dlgo_attention_decode_takes(dtype, hd, page_size)) return DLGO_ERR_SIZE;
  const int use_cluster = (n_splits > 1 && n_splits <= 8 && scratch == nullptr) ? 1 : 0;
  if (n_splits > 1 && scratch == nullptr && !use_cluster) return DLGO_ERR_SIZE;
  const int G = Hq / Hkv;
  DecParams p;
  p.cluster = use_cluster;
  p.q = q; p.ldq = ldq; p.kpages = kpages; p.vpages = vpages; p.page_table = page_table; p.max_pages = max_pages;
  p.seq_slot = seq_slot; p.token_pos = token_pos; p.out = out; p.ldo = ldo;
  p.part_acc = scratch;
  p.part_ml = scratch ? scratch + (size_t)B * Hq * n_splits * hd : nullptr;
  p.counters = counters;
  p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size; p.n_splits = n_splits;
  p.n_gchunks = (G + DEC_GMAX - 1) / DEC_GMAX;
  p.window = window; p.scale = scale;
  if ((long long)Hkv * p.n_gchunks > 65535) return DLGO_ERR_SIZE;
  return decode_common(p, dtype, B, hd, stream);
}

DLGO_TIMES_EXPORT
