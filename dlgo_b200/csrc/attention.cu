// Grouped-query attention over the paged cache, for prompts and for decode.
//
// Reference: for query head h, kv head g = h / (Hq / Hkv):
//   s_t = (q_h . k_{t,g}) * scale  for t in [0, pos]   (causal by the loop bound,
//   never a -inf fill), softmax (subtract max, exp, sum, times 1/sum), then
//   o_h = sum_t p_t * v_{t,g}                     models/llm/forward.go:258-278
// Prompts attend the same way, reading keys and values back from the cache
// (models/llm/forward_batch.go:188-207), so this one kernel serves both: a
// block takes a tile of consecutive tokens of ONE sequence, one kv head (a
// chunk of its query heads), and one slice of the sequence's pages, and runs an
// online softmax in fp32 over 64-key pages.  With more than one slice the
// partial (max, sum, unnormalised output) go to scratch and a second kernel
// combines them.  A window w > 0 keeps keys t > pos - w only.
//
// Storage type T (float or bfloat16) is what q, the pages and the output hold;
// scores, softmax and the weighted sum are fp32 with expf.
#include <math.h>

#include "common.cuh"
#include "attention_combine.cuh"

namespace dlgo {

constexpr int ATT_THREADS = 128;
constexpr int ATT_MAX_ACC = 32;  // accumulators per thread: rows * hd <= 128 * 32

struct AttnParams {
  const void* q;
  int ldq;
  const void* kpages;
  const void* vpages;
  const int* page_table;
  int max_pages;
  const int* tiles;  // [n_tiles][3]: sequence index in the batch, first packed token, token count
  const int* seq_slot;
  const int* token_pos;
  void* out;
  int ldo;
  float* part_acc;  // [T, Hq, n_splits, hd]
  float* part_ml;   // [T, Hq, n_splits, 2]
  int Hq, Hkv, hd, page_size, n_splits, gchunk, n_gchunks, rows_max, window;
  float scale;
};

template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* o) {
    float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float* o) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      o[2 * i] = f.x;
      o[2 * i + 1] = f.y;
    }
  }
};

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS) attention_kernel(AttnParams p) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int hd = p.hd, PS = p.page_size, kstride = hd + 1;
  const int G = p.Hq / p.Hkv;
  const int tile = blockIdx.x;
  const int kvh = blockIdx.y / p.n_gchunks, gc = blockIdx.y - kvh * p.n_gchunks;
  const int split = blockIdx.z;
  const int g0 = gc * p.gchunk;
  const int GC = min(p.gchunk, G - g0);
  const int seq = p.tiles[3 * tile], tok0 = p.tiles[3 * tile + 1], ntok = p.tiles[3 * tile + 2];
  const int R = ntok * GC;
  const int slot = p.seq_slot[seq];
  const int pos0 = p.token_pos[tok0];
  const int t_end = pos0 + ntok;  // one past the last key any row may see
  const int t_begin = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int pg_first = t_begin / PS, pg_last = (t_end - 1) / PS;
  const int per = (pg_last - pg_first + 1 + p.n_splits - 1) / p.n_splits;
  const int pg_b = pg_first + split * per;
  const int pg_e = min(pg_last + 1, pg_b + per);

  float* q_s = smem;                          // [rows_max][hd]
  float* k_s = q_s + p.rows_max * hd;         // [PS][hd + 1]
  float* v_s = k_s + PS * kstride;            // [PS][hd]
  float* p_s = v_s + PS * hd;                 // [rows_max][PS]
  float* m_s = p_s + p.rows_max * PS;         // [rows_max] running max
  float* l_s = m_s + p.rows_max;              // [rows_max] running sum
  float* c_s = l_s + p.rows_max;              // [rows_max] correction of this page

  const T* q = (const T*)p.q;
  for (int idx = tid; idx < R * hd; idx += ATT_THREADS) {
    const int r = idx / hd, d = idx - r * hd;
    const int tq = r / GC, g = r - tq * GC;
    q_s[idx] = to_float(q[(size_t)(tok0 + tq) * p.ldq + (size_t)(kvh * G + g0 + g) * hd + d]);
  }
  for (int r = tid; r < R; r += ATT_THREADS) {
    m_s[r] = -INFINITY;
    l_s[r] = 0.f;
  }
  float acc[ATT_MAX_ACC];
#pragma unroll
  for (int i = 0; i < ATT_MAX_ACC; ++i) acc[i] = 0.f;
  __syncthreads();

  constexpr int VN = Vec<T>::N;
  const int vec_per_row = hd / VN;
  for (int pg = pg_b; pg < pg_e; ++pg) {
    const int page = p.page_table[(size_t)slot * p.max_pages + pg];
    const size_t base = ((size_t)page * p.Hkv + kvh) * PS * hd;
    const T* kp = (const T*)p.kpages + base;
    const T* vp = (const T*)p.vpages + base;
    for (int idx = tid; idx < PS * vec_per_row; idx += ATT_THREADS) {
      const int key = idx / vec_per_row, dv = (idx - key * vec_per_row) * VN;
      const bool live = pg * PS + key < t_end;  // what lies beyond was never written
      float kf[VN], vf[VN];
      if (live) {
        Vec<T>::load(kp + (size_t)key * hd + dv, kf);
        Vec<T>::load(vp + (size_t)key * hd + dv, vf);
      } else {
#pragma unroll
        for (int j = 0; j < VN; ++j) kf[j] = vf[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < VN; ++j) {
        k_s[key * kstride + dv + j] = kf[j];
        v_s[key * hd + dv + j] = vf[j];
      }
    }
    __syncthreads();
    // scores
    for (int idx = tid; idx < R * PS; idx += ATT_THREADS) {
      const int r = idx / PS, key = idx - r * PS;
      const int t = pg * PS + key;
      const int pos_r = pos0 + r / GC;
      const bool valid = t <= pos_r && (p.window <= 0 || t > pos_r - p.window);
      float s = -INFINITY;
      if (valid) {
        const float* qr = q_s + r * hd;
        const float* kr = k_s + key * kstride;
        float dot = 0.f;
        for (int d = 0; d < hd; ++d) dot = fmaf(qr[d], kr[d], dot);
        s = dot * p.scale;
      }
      p_s[idx] = s;
    }
    __syncthreads();
    // online softmax: one warp per row
    for (int r = warp; r < R; r += ATT_THREADS / 32) {
      float mx = -INFINITY;
      for (int key = lane; key < PS; key += 32) mx = fmaxf(mx, p_s[r * PS + key]);
      mx = warp_max(mx);
      const float m_old = m_s[r];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int key = lane; key < PS; key += 32) {
        const float s = p_s[r * PS + key];
        const float e = (m_new == -INFINITY || s == -INFINITY) ? 0.f : expf(s - m_new);
        p_s[r * PS + key] = e;
        sum += e;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float c = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
        c_s[r] = c;
        l_s[r] = l_s[r] * c + sum;
        m_s[r] = m_new;
      }
    }
    __syncthreads();
    // weighted sum of the values
#pragma unroll
    for (int i = 0; i < ATT_MAX_ACC; ++i) {
      const int idx = tid + ATT_THREADS * i;
      if (idx < R * hd) {
        const int r = idx / hd, d = idx - r * hd;
        float a = acc[i] * c_s[r];
        const float* pr = p_s + r * PS;
        for (int key = 0; key < PS; ++key) a = fmaf(pr[key], v_s[key * hd + d], a);
        acc[i] = a;
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < ATT_MAX_ACC; ++i) {
    const int idx = tid + ATT_THREADS * i;
    if (idx < R * hd) {
      const int r = idx / hd, d = idx - r * hd;
      const int tq = r / GC, g = r - tq * GC;
      const int head = kvh * G + g0 + g;
      const size_t token = tok0 + tq;
      if (p.n_splits == 1) {
        ((T*)p.out)[token * p.ldo + (size_t)head * hd + d] = from_float<T>(acc[i] / l_s[r]);
      } else {
        const size_t o = (token * p.Hq + head) * p.n_splits + split;
        p.part_acc[o * hd + d] = acc[i];
        if (d == 0) {
          p.part_ml[o * 2] = m_s[r];
          p.part_ml[o * 2 + 1] = l_s[r];
        }
      }
    }
  }
}

template <typename T>
int launch_attention(const AttnParams& p, int n_tiles, int T_tokens, cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)p.rows_max * p.hd + (size_t)p.page_size * (p.hd + 1) +
                                       (size_t)p.page_size * p.hd + (size_t)p.rows_max * p.page_size +
                                       3 * (size_t)p.rows_max);
  if (smem > 227 * 1024) return DLGO_ERR_SIZE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(n_tiles, p.Hkv * p.n_gchunks, p.n_splits);
  launch_kernel(attention_kernel<T>, dim3(grid), dim3(ATT_THREADS), smem, stream, p);
  int st = launch_status();
  if (st != DLGO_OK || p.n_splits == 1) return st;
  dim3 cgrid(T_tokens, p.Hq);
  const int threads = p.hd >= 128 ? 128 : (p.hd >= 64 ? 64 : 32);
  launch_kernel(attention_combine_kernel<T>, dim3(cgrid), dim3(threads), 0, stream, p.part_acc, p.part_ml, (T*)p.out, p.ldo, p.Hq, p.hd,
                                                             p.n_splits);
  return launch_status();
}

}  // namespace dlgo

using namespace dlgo;

// Floats of scratch the call needs for `n_splits` > 1 (0 for one slice):
// part_acc [T, Hq, n_splits, hd] followed by part_ml [T, Hq, n_splits, 2].
DLGO_EXPORT long long dlgo_attention_scratch_floats(int T, int Hq, int hd, int n_splits) {
  if (n_splits <= 1) return 0;
  return (long long)T * Hq * n_splits * (hd + 2);
}

// q[T, .] with row stride ldq (head h at column h*hd); pages [n_pages, Hkv, page_size, hd];
// tiles[n_tiles][3]; rows_max = (largest token count of a tile) * gchunk;
// out[T, Hq*hd] with row stride ldo.  `scratch` as sized above.
DLGO_EXPORT int dlgo_attention(const void* q, int dtype, int T, int ldq, const void* kpages, const void* vpages,
                               const int* page_table, int max_pages, const int* tiles, int n_tiles,
                               int tile_tokens_max, const int* seq_slot, const int* token_pos, void* out, int ldo,
                               float* scratch, int Hq, int Hkv, int hd, int page_size, int n_splits, int gchunk,
                               int window, float scale, cudaStream_t stream) {
  if (T <= 0 || n_tiles <= 0) return DLGO_OK;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || hd <= 0 || page_size <= 0 || page_size % 32 || n_splits <= 0 ||
      gchunk <= 0 || tile_tokens_max <= 0)
    return DLGO_ERR_SIZE;
  if (hd % (dtype == DLGO_BF16 ? 8 : 4)) return DLGO_ERR_SIZE;
  const int G = Hq / Hkv;
  if (gchunk > G) gchunk = G;
  AttnParams p;
  p.q = q; p.ldq = ldq; p.kpages = kpages; p.vpages = vpages; p.page_table = page_table; p.max_pages = max_pages;
  p.tiles = tiles; p.seq_slot = seq_slot; p.token_pos = token_pos; p.out = out; p.ldo = ldo;
  p.part_acc = scratch;
  p.part_ml = scratch ? scratch + (size_t)T * Hq * n_splits * hd : nullptr;
  p.Hq = Hq; p.Hkv = Hkv; p.hd = hd; p.page_size = page_size; p.n_splits = n_splits; p.gchunk = gchunk;
  p.n_gchunks = (G + gchunk - 1) / gchunk;
  p.rows_max = tile_tokens_max * gchunk;
  p.window = window; p.scale = scale;
  if ((long long)p.rows_max * hd > (long long)ATT_THREADS * ATT_MAX_ACC) return DLGO_ERR_SIZE;
  if (n_splits > 1 && scratch == nullptr) return DLGO_ERR_SIZE;
  if ((long long)Hkv * p.n_gchunks > 65535 || n_splits > 65535) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32) return launch_attention<float>(p, n_tiles, T, stream);
  if (dtype == DLGO_BF16) return launch_attention<__nv_bfloat16>(p, n_tiles, T, stream);
  return DLGO_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------
// The entry point that allocates nothing (see attention_noalloc.h for who needs it and its rules).
#include "attention_noalloc.h"

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress, never a
// device address: a kernel must be given the looked-up pointer.
static __device__ __align__(256) float g_attention_scratch[DLGO_ATTENTION_NOALLOC_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch on the current device; looked up once per device.
int scratch_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return DLGO_ERR_SIZE;
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_attention_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return DLGO_ERR_DRIVER;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return DLGO_OK;
}
}  // namespace

DLGO_EXPORT long long dlgo_attention_noalloc_needs(int T, int Hq, int hd, int n_splits) {
  return dlgo_attention_scratch_floats(T, Hq, hd, n_splits);
}

DLGO_EXPORT int dlgo_attention_noalloc(const void* q, int dtype, int T, int ldq, const void* kpages,
                                       const void* vpages, const int* page_table, int max_pages, const int* tiles,
                                       int n_tiles, int tile_tokens_max, const int* seq_slot, const int* token_pos,
                                       void* out, int ldo, int Hq, int Hkv, int hd, int page_size, int n_splits,
                                       int gchunk, int window, float scale, cudaStream_t stream) {
  if (T <= 0 || n_tiles <= 0) return DLGO_OK;
  if (Hq <= 0 || hd <= 0 || n_splits <= 0) return DLGO_ERR_SIZE;
  const long long need = dlgo_attention_scratch_floats(T, Hq, hd, n_splits);
  if (need > (long long)DLGO_ATTENTION_NOALLOC_FLOATS) return DLGO_ERR_SIZE;  // beyond the stated maximum
  float* scratch = nullptr;
  if (need > 0) {
    const int st = scratch_address(&scratch);
    if (st != DLGO_OK) return st;
  }
  return dlgo_attention(q, dtype, T, ldq, kpages, vpages, page_table, max_pages, tiles, n_tiles, tile_tokens_max,
                        seq_slot, token_pos, out, ldo, scratch, Hq, Hkv, hd, page_size, n_splits, gchunk, window,
                        scale, stream);
}
