// Greedy and temperature sampling on the device: only token ids go to the host.
//
// Reference (ops/sampling.go, ops/ops.go):
//   greedy       first index of the maximum, strict '>'            ops/ops.go:272-285
//   temperature  logits * (1/T), softmax, then the first index whose running
//                sum of probabilities reaches a uniform draw r in [0, 1);
//                the last index if none does           ops/sampling.go:72-80,167-181
// Filters that set logits to -inf beforehand (top-k, top-p, min-p) are honoured:
// a -inf logit has probability 0.
//
// The reference draws r from one generator per request, seeded by the caller
// (models/llm/generate.go:92-95).  Here r = philox4x32-10(key = seed,
// counter = (draw index, request index)), so a request's draws do not depend on
// which other requests share its batch.
#include <math.h>

#include "common.cuh"

namespace dlgo {

__device__ __forceinline__ void philox_round(uint32_t& c0, uint32_t& c1, uint32_t& c2, uint32_t& c3, uint32_t k0,
                                             uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
  const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
  c0 = n0; c1 = n1; c2 = n2; c3 = n3;
}

// uniform in [0, 1) with 24 bits
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint32_t draw, uint32_t request) {
  uint32_t c0 = draw, c1 = request, c2 = 0u, c3 = 0u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    philox_round(c0, c1, c2, c3, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return (float)(c0 >> 8) * (1.0f / 16777216.0f);
}

constexpr int SAMPLE_THREADS = 1024;

// (value, index) of the first maximum among row[begin, end): larger value wins, ties go to the
// smaller index.  Called by every thread of the block; the result is valid in thread 0.
__device__ __forceinline__ void block_argmax(const float* __restrict__ row, int begin, int end, float& best,
                                             int& besti) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  best = -INFINITY;
  besti = 0x7fffffff;
  if ((((uintptr_t)(row + begin)) & 15) == 0 && end - begin >= 4 * (int)blockDim.x) {
    // 16-byte loads, two in flight per thread; a thread's indices still rise, so strict '>' keeps
    // the first maximum
    const int n4 = (end - begin) / 4;
    const float4* r4 = reinterpret_cast<const float4*>(row + begin);
    int k = threadIdx.x;
    for (; k + (int)blockDim.x < n4; k += 2 * blockDim.x) {
      const float4 a = r4[k], b = r4[k + blockDim.x];
      const float va[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int i = begin + 4 * (e < 4 ? k : k + (int)blockDim.x) + (e & 3);
        if (va[e] > best || besti == 0x7fffffff) { best = va[e]; besti = i; }
      }
    }
    for (; k < n4; k += blockDim.x) {
      const float4 a = r4[k];
      const float va[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = begin + 4 * k + e;
        if (va[e] > best || besti == 0x7fffffff) { best = va[e]; besti = i; }
      }
    }
    for (int i = begin + 4 * n4 + threadIdx.x; i < end; i += blockDim.x) {   // the ragged end (indices above all others)
      const float v = row[i];
      if (v > best || besti == 0x7fffffff) { best = v; besti = i; }
    }
  } else {
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
      const float v = row[i];
      // a strided scan visits indices in rising order, so strict '>' keeps the first maximum
      if (v > best || besti == 0x7fffffff) { best = v; besti = i; }
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { bv[warp] = best; bi[warp] = besti; }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    for (int w = 1; w < nw; ++w)
      if (bv[w] > best || (bv[w] == best && bi[w] < besti)) { best = bv[w]; besti = bi[w]; }
  }
}

// grid (rows, nblk): block (r, c) scans its chunk of the vocabulary.  With nblk == 1 it writes the
// answer; otherwise its (value, index) go to scratch for argmax_finish_kernel.
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int V, int* __restrict__ out, float* __restrict__ part_v,
              int* __restrict__ part_i) {
  pdl_launch_dependents();
  pdl_wait();
  const int nblk = gridDim.y;
  const int chunk = (V + nblk - 1) / nblk;
  const int begin = blockIdx.y * chunk, end = min(V, begin + chunk);
  float best;
  int besti;
  block_argmax(logits + (size_t)blockIdx.x * ld, begin, end, best, besti);
  if (threadIdx.x == 0) {
    if (nblk == 1) out[blockIdx.x] = besti == 0x7fffffff ? 0 : besti;
    else {
      part_v[blockIdx.x * nblk + blockIdx.y] = best;
      part_i[blockIdx.x * nblk + blockIdx.y] = besti;
    }
  }
}

__global__ void argmax_finish_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int nblk,
                                     int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  // one warp per row; chunks are in rising index order
  const int r = blockIdx.x;
  float best = -INFINITY;
  int besti = 0x7fffffff;
  for (int c = threadIdx.x; c < nblk; c += 32) {
    const float v = part_v[r * nblk + c];
    const int i = part_i[r * nblk + c];
    if (v > best || (v == best && i < besti)) { best = v; besti = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
  }
  if (threadIdx.x == 0) out[r] = besti == 0x7fffffff ? 0 : besti;
}

// One block per row.  Each WARP owns a contiguous chunk of the vocabulary and walks it 32 consecutive
// entries at a time (coalesced), so "first index whose running sum reaches the target" keeps its meaning:
// warps in order, groups of 32 in order, lanes in order.
__device__ __forceinline__ void sample_row(const float* __restrict__ row, int V, float inv_t, float u,
                                           int* __restrict__ out_r) {
  __shared__ float scratch[32];
  __shared__ float wsum[SAMPLE_THREADS / 32];
  __shared__ int chosen;
  __shared__ float rest_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int chunk = ((V + n_warps - 1) / n_warps + 31) / 32 * 32;   // whole groups of 32 per warp
  const int b = warp * chunk, e = min(V, b + chunk);
  float mx = -INFINITY;
  for (int i = b + lane; i < e; i += 32) mx = fmaxf(mx, row[i] * inv_t);
  mx = block_max(mx, scratch);
  float s = 0.f;
  for (int i = b + lane; i < e; i += 32) {
    const float v = row[i] * inv_t;
    s += (v == -INFINITY) ? 0.f : expf(v - mx);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) wsum[warp] = s;
  if (threadIdx.x == 0) chosen = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int i = 0; i < n_warps; ++i) total += wsum[i];
    const float target = u * total;
    float run = 0.f;
    int owner = -1;
    for (int i = 0; i < n_warps; ++i) {
      if (run + wsum[i] >= target && wsum[i] > 0.f) { owner = i; break; }
      run += wsum[i];
    }
    if (owner < 0) {
      // rounding left the target above the total: the last chunk with weight
      for (int i = n_warps - 1; i >= 0; --i)
        if (wsum[i] > 0.f) { owner = i; break; }
      rest_s = -1.f;  // sentinel: take the chunk's last weighted index
    } else {
      rest_s = target - run;
    }
    chosen = owner;
  }
  __syncthreads();
  if (warp == chosen) {
    const float rest = rest_s;
    float run = 0.f;
    int pick = -1, last = -1;
    for (int g = b; g < e && pick < 0; g += 32) {
      const int i = g + lane;
      float pr = 0.f;
      if (i < e) {
        const float v = row[i] * inv_t;
        pr = (v == -INFINITY) ? 0.f : expf(v - mx);
      }
      float incl = pr;                       // inclusive scan over the lanes, in lane order
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const unsigned weighted = __ballot_sync(0xffffffffu, pr > 0.f);
      if (weighted) last = g + 31 - __clz(weighted);
      const unsigned hit = __ballot_sync(0xffffffffu, rest >= 0.f && pr > 0.f && run + incl >= rest);
      if (hit) pick = g + __ffs(hit) - 1;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) *out_r = pick >= 0 ? pick : (last >= 0 ? last : b);
  }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ request, const int* __restrict__ draw, uint64_t seed,
              const unsigned long long* __restrict__ seed_dev, int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  if (seed_dev != nullptr) seed = *seed_dev;   // (a captured step takes its seed from memory)
  const int r = blockIdx.x;
  sample_row(logits + (size_t)r * ld, V, 1.0f / temperature[r],
             philox_uniform(seed, (uint32_t)draw[r], (uint32_t)request[r]), out + r);
}


// ---------------------------------------------------------------------------------------------
// The reference's filters in one kernel (ops/sampling.go:53-165): repetition penalty over the recent tokens (positive logits / penalty, negative * penalty, each
// token once), temperature, top-k (everything below the k-th largest value goes to -inf, ties at the
// cutoff stay), then among the survivors top-p (the shortest prefix of the descending order whose
// probabilities reach p) and min-p (drop below min_p times the largest probability).  One block per
// row writes the filtered, temperature-scaled logits to `work`; the draw itself is sample_kernel's.
constexpr int FILTER_THREADS = 1024;
constexpr int FILTER_CAP = 2048;     // survivors kept for top-p / min-p (k plus ties at the cutoff)
constexpr int FILTER_RECENT = 64;

__device__ __forceinline__ uint32_t order_key(float x) {     // monotone: a < b  <=>  key(a) < key(b)
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// The k-th largest of the order-preserving keys of vals[0, n) (1 <= k <= n), digit by digit from the top (11,
// 11 and 10 bits): a histogram of the digit over the keys that share the digits found so far, then the highest
// bin at which the count from the top reaches what is still wanted.  Three passes over the values.  Called by
// every thread of the block (any size that is a multiple of 32); `hist` holds 2048 ints of shared memory.
__device__ __forceinline__ uint32_t kth_largest_key(const float* vals, int n, int k, int* hist) {
  __shared__ unsigned int want_s, digit_s;
  const int tid = threadIdx.x, nthr = blockDim.x;
  uint32_t lo = 0u;                       // the digits found so far, in place
  if (tid == 0) want_s = (unsigned int)k;
  for (int level = 0; level < 3; ++level) {
    const int shift = level == 0 ? 21 : (level == 1 ? 10 : 0);
    const int nb = level < 2 ? 2048 : 1024;
    const uint32_t above = level == 0 ? 0u : ~((1u << (shift + (level < 2 ? 11 : 10))) - 1u);
    for (int i = tid; i < nb; i += nthr) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += nthr) {
      const uint32_t key = order_key(vals[i]);
      if ((key & above) == lo) atomicAdd(&hist[(key >> shift) & (uint32_t)(nb - 1)], 1);
    }
    __syncthreads();
    if (tid < 32) {
      // lane l owns bins [nb - (l + 1) * per, nb - l * per): lane 0 the highest
      const int per = nb / 32;
      const int top = nb - tid * per;
      unsigned int mine = 0;
      for (int j = 0; j < per; ++j) mine += (unsigned int)hist[top - 1 - j];
      unsigned int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (tid >= o) incl += t;
      }
      const unsigned int want = want_s;
      const unsigned int before = incl - mine;                     // keys in the lanes above this one
      const unsigned owners = __ballot_sync(0xffffffffu, incl >= want);
      const int owner = owners ? __ffs(owners) - 1 : 31;         // (k <= n: some lane reaches it)
      if (tid == owner) {
        unsigned int run = before;
        int bin = top - per;
        for (int j = 0; j < per; ++j) {
          run += (unsigned int)hist[top - 1 - j];
          if (run >= want) { bin = top - 1 - j; run -= (unsigned int)hist[bin]; break; }
        }
        digit_s = (unsigned int)bin;
        want_s = want - run;                                       // still wanted inside the bin
      }
    }
    __syncthreads();
    lo |= digit_s << shift;
    __syncthreads();
  }
  return lo;
}

// The row's recent tokens into shared memory: duplicates and ids outside the vocabulary become -1.
__device__ __forceinline__ void distinct_recent(const int* __restrict__ recent_row, int n_recent, int V, int* rec_s) {
  const int tid = threadIdx.x;
  int tok = -1;
  if (tid < FILTER_RECENT) {
    tok = (recent_row != nullptr && tid < n_recent) ? recent_row[tid] : -1;
    if (tok >= V) tok = -1;
    rec_s[tid] = tok;
  }
  __syncthreads();
  bool again = false;                    // (compared in shared memory: a chain of loads from memory costs 20 us)
  if (tid < FILTER_RECENT && tok >= 0)
    for (int j = 0; j < tid; ++j) again |= rec_s[j] == tok;
  __syncthreads();
  if (again) rec_s[tid] = -1;
  __syncthreads();
}

// Thread 0: how many of the n survivors, sorted by value (descending), top-p and min-p keep.
__device__ __forceinline__ int kept_of_sorted(const float* sv, int n, float top_p, float min_p) {
  const float mx = sv[0];
  float total = 0.f;
  for (int i = 0; i < n; ++i) total += expf(sv[i] - mx);
  int keep = n;
  if (top_p < 1.0f) {
    float cum = 0.f;
    for (int i = 0; i < n; ++i) {
      cum += expf(sv[i] - mx) / total;
      if (cum >= top_p) { keep = i + 1; break; }
    }
  }
  if (min_p > 0.f) {
    // prob_i < min_p * prob_max  <=>  exp(v_i - mx) < min_p
    int k2 = 0;
    while (k2 < keep && expf(sv[k2] - mx) >= min_p) ++k2;
    keep = k2 < 1 ? 1 : k2;
  }
  return keep;
}

// One row through the filters; FILTER_THREADS threads.
__device__ __forceinline__ void filter_row(const float* __restrict__ row, int V, float* __restrict__ out, float inv_t,
                                           int top_k, float top_p, float min_p, float penalty,
                                           const int* __restrict__ recent_row, int n_recent) {
  __shared__ int rec_s[FILTER_RECENT];
  __shared__ unsigned int count_s;
  __shared__ float sv[FILTER_CAP];
  __shared__ int si[FILTER_CAP];
  __shared__ float red[32];
  __shared__ float cut_s;
  const int tid = threadIdx.x;
  distinct_recent(recent_row, n_recent, V, rec_s);
  // pass 0: temperature -> work; then the penalty on the (few, distinct) recent tokens
  for (int i = tid; i < V; i += FILTER_THREADS) out[i] = row[i] * inv_t;
  __syncthreads();
  if (penalty > 1.0f && tid < FILTER_RECENT && rec_s[tid] >= 0) {
    const float v = row[rec_s[tid]];
    out[rec_s[tid]] = (v > 0.f ? v / penalty : v * penalty) * inv_t;
  }
  __syncthreads();
  if (top_k <= 0 || top_k >= V) {
    // No top-k: nothing bounds the survivors, so there is no list to sort.  Top-p by bisection on the
    // probability mass instead: the cutoff is the largest key whose tokens at or above it carry at
    // least p of the mass (the shortest prefix of the descending order that reaches p; tokens that tie
    // with the cutoff all stay).  Min-p is a threshold against the maximum.
    float mx = -INFINITY;
    for (int i = tid; i < V; i += FILTER_THREADS) mx = fmaxf(mx, out[i]);
    mx = block_max(mx, red);
    if (top_p < 1.0f) {
      float tot = 0.f;
      for (int i = tid; i < V; i += FILTER_THREADS) tot += expf(out[i] - mx);
      tot = block_sum(tot, red);
      const float target = top_p * tot;
      uint32_t cut = 0u;     // invariant: mass(key >= cut) >= target
      for (int bit = 31; bit >= 0; --bit) {
        const uint32_t mid = cut | (1u << bit);
        float m = 0.f;
        for (int i = tid; i < V; i += FILTER_THREADS) {
          const float v = out[i];
          if (order_key(v) >= mid) m += expf(v - mx);
        }
        m = block_sum(m, red);
        if (m >= target) cut = mid;     // (the same value in every thread)
      }
      for (int i = tid; i < V; i += FILTER_THREADS)
        if (order_key(out[i]) < cut) out[i] = -INFINITY;
    }
    if (min_p > 0.f) {
      const float thr = mx + logf(min_p);     // exp(v - mx) < min_p  <=>  v < mx + ln(min_p)
      for (int i = tid; i < V; i += FILTER_THREADS)
        if (out[i] < thr) out[i] = -INFINITY;
    }
    return;
  }
  // top-k: everything below the k-th largest value goes to -inf (the survivors' list is not in use yet: its
  // 2048 ints hold the histogram)
  const uint32_t lo = kth_largest_key(out, V, top_k, si);
  // survivors (key >= lo) into shared memory, the rest to -inf
  if (tid == 0) count_s = 0;
  __syncthreads();
  for (int i = tid; i < V; i += FILTER_THREADS) {
    const float v = out[i];
    if (order_key(v) >= lo) {
      const unsigned int at = atomicAdd(&count_s, 1u);
      if (at < FILTER_CAP) { sv[at] = v; si[at] = i; }
    } else {
      out[i] = -INFINITY;
    }
  }
  __syncthreads();
  const int n = (int)count_s;
  if (n > FILTER_CAP || (top_p >= 1.0f && min_p <= 0.f)) return;   // (more ties than fit: top-k alone stands)
  // sort the survivors by value, descending (bitonic over the next power of two, padded with -inf)
  int m = 1;
  while (m < n) m <<= 1;
  for (int i = n + tid; i < m; i += FILTER_THREADS) { sv[i] = -INFINITY; si[i] = -1; }
  __syncthreads();
  for (int k = 2; k <= m; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < m; i += FILTER_THREADS) {
        const int l = i ^ j;
        if (l > i) {
          const bool desc = (i & k) == 0;
          const float a = sv[i], b = sv[l];
          if (desc ? a < b : a > b) {
            sv[i] = b; sv[l] = a;
            const int t = si[i]; si[i] = si[l]; si[l] = t;
          }
        }
      }
      __syncthreads();
    }
  }
  // probabilities of the survivors and the cut: thread 0 walks the (short) sorted list
  if (tid == 0) {
    const int keep = kept_of_sorted(sv, n, top_p, min_p);
    cut_s = keep < n ? (float)keep : -1.f;
  }
  __syncthreads();
  // positions keep .. n-1 of the sorted list are dropped (ties between kept and dropped values are
  // resolved by position in the sorted order, as the reference's sort does)
  const int keep = cut_s < 0.f ? n : (int)cut_s;
  for (int i = keep + tid; i < n; i += FILTER_THREADS) out[si[i]] = -INFINITY;
}

__global__ void __launch_bounds__(FILTER_THREADS)
filter_kernel(const float* __restrict__ logits, int ld, int V, float* __restrict__ work, float inv_t, int top_k,
              float top_p, float min_p, float penalty, const int* __restrict__ recent, int n_recent) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  filter_row(logits + (size_t)r * ld, V, work + (size_t)r * V, inv_t, top_k, top_p, min_p, penalty,
             recent != nullptr ? recent + (size_t)r * n_recent : nullptr, n_recent);
}

// ---------------------------------------------------------------------------------------------
// Filters and draw for a small top-k (the reference's default sampler: top-k 40) without a pass of one block
// over the whole row: what top-k keeps is all that top-p, min-p and the draw ever look at.
//   1. candidates_kernel, grid (rows, chunks of FD_CHUNK entries): a block holds its chunk (temperature and
//      repetition penalty applied) in shared memory; every thread takes the maximum of its 16 entries, the
//      k-th largest of these 512 maxima is at most the chunk's k-th largest value, which is at most the row's;
//      every entry at or above it goes, value and index, to the row's candidate list (a few more than k per
//      chunk).  Every entry that the row's top-k keeps is among them.
//   2. filter_draw_kernel, a block per row: sorts the candidates by value; the k-th is the row's cutoff and
//      what lies at or above it survives (ties included); top-p and min-p as filter_row does; what is kept is
//      sorted by index, and the draw walks it in index order as sample_row does.
// More ties than a list holds (cand_n > cap, more than FD_MAX_CAND candidates or FILTER_CAP survivors in a
// row): that row's block runs filter_row and sample_row instead, through `work`.
constexpr int FD_CHUNK = 8192;
constexpr int FD_THREADS = 512;
constexpr int FD_PER_THREAD = FD_CHUNK / FD_THREADS;
constexpr int FD_MAX_CAND = 4096;

// a before b in "value descending, then index ascending"
__device__ __forceinline__ bool by_value_first(float va, int ia, float vb, int ib) {
  return va > vb || (va == vb && ia < ib);
}

__global__ void __launch_bounds__(FD_THREADS)
candidates_kernel(const float* __restrict__ logits, int ld, int V, float inv_t, int top_k, float penalty,
                  const int* __restrict__ recent, int n_recent, int cap, float* __restrict__ cand_v,
                  int* __restrict__ cand_i, int* __restrict__ cand_n) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float vals[FD_CHUNK];
  __shared__ int rec_s[FILTER_RECENT];
  __shared__ unsigned int count_s;
  const int r = blockIdx.x, c = blockIdx.y, C = gridDim.y, tid = threadIdx.x;
  const float* row = logits + (size_t)r * ld;
  const int b = c * FD_CHUNK, n = min(V, b + FD_CHUNK) - b;
  {
    float x[FD_PER_THREAD];                 // all of the thread's loads are on their way before the first is used
#pragma unroll
    for (int j = 0; j < FD_PER_THREAD; ++j) {
      const int i = tid + j * FD_THREADS;
      x[j] = i < n ? row[b + i] : -INFINITY;
    }
#pragma unroll
    for (int j = 0; j < FD_PER_THREAD; ++j) vals[tid + j * FD_THREADS] = x[j] * inv_t;
  }
  if (tid == 0) count_s = 0;
  distinct_recent(recent != nullptr ? recent + (size_t)r * n_recent : nullptr, n_recent, V, rec_s);
  if (penalty > 1.0f && tid < FILTER_RECENT && rec_s[tid] >= b && rec_s[tid] < b + n) {
    const float v = row[rec_s[tid]];
    vals[rec_s[tid] - b] = (v > 0.f ? v / penalty : v * penalty) * inv_t;
  }
  __syncthreads();
  uint32_t lo = 0u;
  if (n > top_k) {                          // (block-uniform; else everything is a candidate)
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < FD_PER_THREAD; ++j)
      if (tid + j * FD_THREADS < n) mx = fmaxf(mx, vals[tid + j * FD_THREADS]);
    // the k-th largest of the threads' maxima (top_k <= 256 < FD_THREADS, and more than top_k threads hold
    // entries; a thread without entries has key 0, which nothing real has), by bisection on the order key's
    // bits with a barrier that counts
    const uint32_t key = tid < n ? order_key(mx) : 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t mid = lo | (1u << bit);          // invariant: at least top_k keys are >= lo
      if (__syncthreads_count(key >= mid) >= top_k) lo = mid;
    }
  }
  const size_t base = ((size_t)r * C + c) * cap;
#pragma unroll
  for (int j = 0; j < FD_PER_THREAD; ++j) {
    const int i = tid + j * FD_THREADS;
    if (i < n) {
      const float v = vals[i];
      if (order_key(v) >= lo) {
        const unsigned int at = atomicAdd(&count_s, 1u);
        if (at < (unsigned int)cap) { cand_v[base + at] = v; cand_i[base + at] = b + i; }
      }
    }
  }
  __syncthreads();
  if (tid == 0) cand_n[r * C + c] = (int)count_s;
}

// Sorts (v, idx)[0, n) by value descending and index ascending, by ONE warp (all 32 lanes call it): up to 64
// entries by ranking every entry against all others (the usual case: some forty survivors), longer lists by a
// bitonic network over the next power of two, which must fit the arrays (padding is written behind n).
// `tv`, `ti`: room for 64 entries.
__device__ __forceinline__ void warp_sort_by_value(float* v, int* idx, int n, float* tv, int* ti) {
  const int lane = threadIdx.x & 31;
  if (n <= 64) {
    float mv[2];
    int mi[2], rank[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int i = lane + 32 * e;
      mv[e] = i < n ? v[i] : -INFINITY;
      mi[e] = i < n ? idx[i] : 0x7fffffff;
      rank[e] = 0;
    }
    for (int j = 0; j < n; ++j) {
      const float vj = v[j];
      const int ij = idx[j];
#pragma unroll
      for (int e = 0; e < 2; ++e) rank[e] += by_value_first(vj, ij, mv[e], mi[e]) ? 1 : 0;
    }
#pragma unroll
    for (int e = 0; e < 2; ++e)
      if (lane + 32 * e < n) { tv[rank[e]] = mv[e]; ti[rank[e]] = mi[e]; }      // (entries are distinct: so are ranks)
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 2; ++e)
      if (lane + 32 * e < n) { v[lane + 32 * e] = tv[lane + 32 * e]; idx[lane + 32 * e] = ti[lane + 32 * e]; }
    __syncwarp();
    return;
  }
  int m = 1;
  while (m < n) m <<= 1;
  for (int i = n + lane; i < m; i += 32) { v[i] = -INFINITY; idx[i] = 0x7fffffff; }
  __syncwarp();
  for (int k = 2; k <= m; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = lane; i < m; i += 32) {
        const int l = i ^ j;
        if (l > i) {
          const bool desc = (i & k) == 0;
          const float a = v[i], b = v[l];
          const int ia = idx[i], ib = idx[l];
          if (desc ? by_value_first(b, ib, a, ia) : by_value_first(a, ia, b, ib)) {
            v[i] = b; v[l] = a;
            idx[i] = ib; idx[l] = ia;
          }
        }
      }
      __syncwarp();
    }
  }
}

__global__ void __launch_bounds__(FILTER_THREADS)
filter_draw_kernel(const float* __restrict__ logits, int ld, int V, float* __restrict__ work, float inv_t, int top_k,
                   float top_p, float min_p, float penalty, const int* __restrict__ recent, int n_recent, int C,
                   int cap, const float* __restrict__ cand_v, const int* __restrict__ cand_i,
                   const int* __restrict__ cand_n, const int* __restrict__ request, const int* __restrict__ draw,
                   uint64_t seed, const unsigned long long* __restrict__ seed_dev, int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  if (seed_dev != nullptr) seed = *seed_dev;
  extern __shared__ __align__(16) uint8_t fd_smem[];
  float* cv = reinterpret_cast<float*>(fd_smem);            // [FD_MAX_CAND] the row's candidates
  int* ci = reinterpret_cast<int*>(cv + FD_MAX_CAND);        // [FD_MAX_CAND]
  float* sv = reinterpret_cast<float*>(ci + FD_MAX_CAND);    // [FILTER_CAP] survivors of top-k
  int* si = reinterpret_cast<int*>(sv + FILTER_CAP);         // [FILTER_CAP]
  float* ev = reinterpret_cast<float*>(si + FILTER_CAP);     // [FILTER_CAP] their exponentials
  __shared__ int first_s[65];
  __shared__ int slow_s, n_s;
  __shared__ float tv[64];
  __shared__ int ti[64];
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
  const float u = philox_uniform(seed, (uint32_t)draw[r], (uint32_t)request[r]);
  if (tid < 32) {
    // the chunks' counts (at most 64: two per lane), their running sum, and whether any list overflowed
    const int n0 = tid < C ? cand_n[r * C + tid] : 0, n1 = tid + 32 < C ? cand_n[r * C + tid + 32] : 0;
    const unsigned over = __ballot_sync(0xffffffffu, n0 > cap || n1 > cap);
    const int c0 = min(n0, cap), c1 = min(n1, cap);
    int incl0 = c0, incl1 = c1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t0 = __shfl_up_sync(0xffffffffu, incl0, o), t1 = __shfl_up_sync(0xffffffffu, incl1, o);
      if (tid >= o) { incl0 += t0; incl1 += t1; }
    }
    const int half = __shfl_sync(0xffffffffu, incl0, 31);
    first_s[tid] = incl0 - c0;
    first_s[tid + 32] = half + incl1 - c1;
    if (tid == 31) {
      const int total = half + incl1;
      first_s[64] = total;
      slow_s = (over != 0u || total > FD_MAX_CAND) ? 1 : 0;
    }
  }
  __syncthreads();
  const int n_c = first_s[64];
  if (slow_s == 0) {
    // the row's candidates into shared memory (one round trip to memory for the whole block)
    for (int at = tid; at < n_c; at += FILTER_THREADS) {
      int lo_c = 0, hi_c = C - 1;             // the chunk whose list holds candidate `at`
      while (lo_c < hi_c) {
        const int mid = (lo_c + hi_c + 1) >> 1;
        if (first_s[mid] <= at) lo_c = mid; else hi_c = mid - 1;
      }
      const size_t src = ((size_t)r * C + lo_c) * cap + (at - first_s[lo_c]);
      cv[at] = cand_v[src];
      ci[at] = cand_i[src];
    }
    __syncthreads();
    // From here the first warp works alone (a block-wide barrier costs 0.3 us at 32 warps; a warp's costs
    // nothing to speak of).  The k-th largest candidate by bisection on the order key's bits; everything at
    // or above it survives (ties at the cutoff stay).
    if (tid < 32) {
      uint32_t cut = 0u;                      // invariant: at least top_k candidates have a key >= cut
      if (n_c > top_k && n_c <= 1024) {
        // (the usual case: the lane's keys in registers; a loop over shared memory per bit costs 13 us)
        uint32_t keys[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) keys[j] = lane + 32 * j < n_c ? order_key(cv[lane + 32 * j]) : 0u;
        for (int bit = 31; bit >= 0; --bit) {
          const uint32_t mid = cut | (1u << bit);
          int cnt = 0;
#pragma unroll
          for (int j = 0; j < 32; ++j) cnt += keys[j] >= mid ? 1 : 0;
          if (__reduce_add_sync(0xffffffffu, cnt) >= top_k) cut = mid;
        }
      } else if (n_c > top_k) {
        for (int bit = 31; bit >= 0; --bit) {
          const uint32_t mid = cut | (1u << bit);
          int cnt = 0;
          for (int i = lane; i < n_c; i += 32) cnt += order_key(cv[i]) >= mid ? 1 : 0;
          if (__reduce_add_sync(0xffffffffu, cnt) >= top_k) cut = mid;
        }
      }
      int n = 0;
      for (int g = 0; g < n_c; g += 32) {      // survivors, in the candidates' order
        const int i = g + lane;
        const bool in = i < n_c && order_key(cv[i]) >= cut;
        const unsigned mask = __ballot_sync(0xffffffffu, in);
        const int at = n + __popc(mask & ((1u << lane) - 1u));
        if (in && at < FILTER_CAP) { sv[at] = cv[i]; si[at] = ci[i]; }
        n += __popc(mask);
      }
      if (lane == 0) {
        n_s = n;
        if (n > FILTER_CAP) slow_s = 1;
      }
    }
    __syncthreads();
  }
  if (slow_s != 0) {
    // more ties than the lists hold: the whole row, one pass after another
    float* w = work + (size_t)r * V;
    filter_row(logits + (size_t)r * ld, V, w, inv_t, top_k, top_p, min_p, penalty,
               recent != nullptr ? recent + (size_t)r * n_recent : nullptr, n_recent);
    __syncthreads();
    sample_row(w, V, 1.0f, u, out + r);
    return;
  }
  if (tid >= 32) return;
  const int n = n_s;
  // by value, descending (ties by index, so that the order does not depend on which thread wrote first)
  warp_sort_by_value(sv, si, n, tv, ti);
  const float mx = sv[0];
  float total = 0.f;
  for (int i = lane; i < n; i += 32) {
    const float e = expf(sv[i] - mx);
    ev[i] = e;
    total += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  __syncwarp();
  // top-p: the shortest prefix of the descending order whose probabilities reach p
  int keep = n;
  if (top_p < 1.0f) {
    float run = 0.f;
    int found = -1;
    for (int g = 0; g < n && found < 0; g += 32) {
      const int i = g + lane;
      float incl = i < n ? ev[i] / total : 0.f;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, i < n && run + incl >= top_p);
      if (hit) found = g + __ffs(hit) - 1;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (found >= 0) keep = found + 1;
  }
  if (min_p > 0.f) {
    // prob_i < min_p * prob_max  <=>  exp(v_i - mx) < min_p; the list is sorted: a prefix stays
    int k2 = keep;
    for (int g = 0; g < keep; g += 32) {
      const int i = g + lane;
      const unsigned below = __ballot_sync(0xffffffffu, i < keep && ev[i] < min_p);
      if (below) { k2 = g + __ffs(below) - 1; break; }
    }
    keep = k2 < 1 ? 1 : k2;
  }
  // what is kept, by index (ascending): as (-index) descending with the same sort; then the draw: the first
  // kept index whose running sum of probabilities reaches u times their total, the last one with weight if
  // rounding leaves the target above the total (ops/sampling.go:167-181)
  for (int i = lane; i < keep; i += 32) {
    sv[i] = -(float)si[i];                    // (indices below 2^24 are exact in a float)
    si[i] = __float_as_int(ev[i]);
  }
  __syncwarp();
  warp_sort_by_value(sv, si, keep, tv, ti);
  float tot = 0.f;
  for (int i = lane; i < keep; i += 32) tot += __int_as_float(si[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
  const float target = u * tot;
  float run = 0.f;
  int pick = -1, last = -1;
  for (int g = 0; g < keep && pick < 0; g += 32) {
    const int i = g + lane;
    const float pr = i < keep ? __int_as_float(si[i]) : 0.f;
    float incl = pr;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const unsigned weighted = __ballot_sync(0xffffffffu, pr > 0.f);
    if (weighted) last = g + 31 - __clz(weighted);
    const unsigned hit = __ballot_sync(0xffffffffu, pr > 0.f && run + incl >= target);
    if (hit) pick = g + __ffs(hit) - 1;
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) out[r] = (int)(-sv[pick >= 0 ? pick : (last >= 0 ? last : 0)]);
}

// ---------------------------------------------------------------------------------------------
// The temperature draw for a large vocabulary in two kernels instead of one block per row that walks the row
// three times: (1) a block per chunk of FD_CHUNK entries leaves the chunk's maximum and its sum of
// exponentials against that maximum; (2) a block per row puts the chunks' sums on one scale, finds the chunk
// in which the running sum reaches u times the total, and walks that chunk alone, in index order.
__global__ void __launch_bounds__(FD_THREADS)
sample_chunks_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
                     float* __restrict__ part) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int r = blockIdx.x, c = blockIdx.y, C = gridDim.y, tid = threadIdx.x;
  const float* row = logits + (size_t)r * ld;
  const float inv_t = 1.0f / temperature[r];
  const int b = c * FD_CHUNK, n = min(V, b + FD_CHUNK) - b;
  float x[FD_PER_THREAD];
#pragma unroll
  for (int j = 0; j < FD_PER_THREAD; ++j) {
    const int i = tid + j * FD_THREADS;
    x[j] = i < n ? row[b + i] * inv_t : -INFINITY;
  }
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < FD_PER_THREAD; ++j) mx = fmaxf(mx, x[j]);
  mx = block_max(mx, red);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < FD_PER_THREAD; ++j) sum += x[j] == -INFINITY ? 0.f : expf(x[j] - mx);
  sum = block_sum(sum, red);
  if (tid == 0) {
    part[((size_t)r * C + c) * 2] = mx;
    part[((size_t)r * C + c) * 2 + 1] = sum;
  }
}

constexpr int SP_PER_THREAD = FD_CHUNK / SAMPLE_THREADS;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_pick_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
                   const float* __restrict__ part, int C, const int* __restrict__ request,
                   const int* __restrict__ draw, uint64_t seed, const unsigned long long* __restrict__ seed_dev,
                   int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  if (seed_dev != nullptr) seed = *seed_dev;
  __shared__ int chunk_s, pick_s, last_s;
  __shared__ float rest_s, max_s;
  __shared__ float wsum[SAMPLE_THREADS / 32];
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)r * ld;
  const float inv_t = 1.0f / temperature[r];
  if (tid < 32) {
    // chunks lane and lane + 32 (at most 64 chunks): their sums on the scale of the row's maximum, in order
    const float u = philox_uniform(seed, (uint32_t)draw[r], (uint32_t)request[r]);
    const float m0 = lane < C ? part[((size_t)r * C + lane) * 2] : -INFINITY;
    const float m1 = lane + 32 < C ? part[((size_t)r * C + lane + 32) * 2] : -INFINITY;
    float M = fmaxf(m0, m1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float s0 = (lane < C && m0 > -INFINITY) ? part[((size_t)r * C + lane) * 2 + 1] * expf(m0 - M) : 0.f;
    const float s1 = (lane + 32 < C && m1 > -INFINITY) ? part[((size_t)r * C + lane + 32) * 2 + 1] * expf(m1 - M) : 0.f;
    float i0 = s0, i1 = s1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t0 = __shfl_up_sync(0xffffffffu, i0, o), t1 = __shfl_up_sync(0xffffffffu, i1, o);
      if (lane >= o) { i0 += t0; i1 += t1; }
    }
    const float half = __shfl_sync(0xffffffffu, i0, 31);
    i1 += half;
    const float total = __shfl_sync(0xffffffffu, i1, 31);
    const float target = u * total;
    // the first chunk with weight whose running sum reaches the target
    const unsigned h0 = __ballot_sync(0xffffffffu, s0 > 0.f && i0 >= target);
    const unsigned h1 = __ballot_sync(0xffffffffu, s1 > 0.f && i1 >= target);
    const unsigned w0 = __ballot_sync(0xffffffffu, s0 > 0.f), w1 = __ballot_sync(0xffffffffu, s1 > 0.f);
    int chunk = -1;
    float before = 0.f;
    if (h0) {
      chunk = __ffs(h0) - 1;
      before = __shfl_sync(0xffffffffu, i0 - s0, chunk);
    } else if (h1) {
      chunk = __ffs(h1) - 1;
      before = __shfl_sync(0xffffffffu, i1 - s1, chunk);
      chunk += 32;
    }
    if (lane == 0) {
      if (chunk >= 0) {
        chunk_s = chunk;
        rest_s = target - before;
      } else {
        // rounding left the target above the total: the last entry with weight of the last chunk with weight
        chunk_s = w1 ? 63 - __clz(w1) : (w0 ? 31 - __clz(w0) : 0);
        rest_s = -1.f;
      }
      max_s = M;
      pick_s = 0x7fffffff;
      last_s = -1;
    }
  }
  __syncthreads();
  const int b = chunk_s * FD_CHUNK, n = min(V, b + FD_CHUNK) - b;
  const float rest = rest_s, M = max_s;
  // the chunk, SP_PER_THREAD consecutive entries per thread, and the threads' running sums in index order
  float pr[SP_PER_THREAD];
  float mine = 0.f;
#pragma unroll
  for (int j = 0; j < SP_PER_THREAD; ++j) {
    const int i = tid * SP_PER_THREAD + j;
    const float v = i < n ? row[b + i] * inv_t : -INFINITY;
    pr[j] = v == -INFINITY ? 0.f : expf(v - M);
    mine += pr[j];
  }
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  float run = incl - mine;
  for (int w = 0; w < warp; ++w) run += wsum[w];
  int first = 0x7fffffff, last = -1;
#pragma unroll
  for (int j = 0; j < SP_PER_THREAD; ++j) {
    run += pr[j];
    if (pr[j] > 0.f) {
      const int i = b + tid * SP_PER_THREAD + j;
      last = i;
      if (rest >= 0.f && run >= rest && first == 0x7fffffff) first = i;
    }
  }
  if (first != 0x7fffffff) atomicMin(&pick_s, first);
  if (last >= 0) atomicMax(&last_s, last);
  __syncthreads();
  if (tid == 0) out[r] = pick_s != 0x7fffffff ? pick_s : (last_s >= 0 ? last_s : b);
}

}  // namespace dlgo

using namespace dlgo;

// Chunks the vocabulary is cut into for `R` rows (1: one kernel, no scratch).
DLGO_EXPORT int dlgo_argmax_chunks(int R, int V) {
  if (V < 16384) return 1;
  int c = (V + 2047) / 2048;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 128;
  }
  const int want = (4 * sms + R - 1) / R;   // enough blocks for every SM
  if (c > want) c = want;
  return c < 1 ? 1 : (c > 64 ? 64 : c);
}

// logits[R, V] f32 (row stride ld) -> out[R] int32; scratch: R * chunks floats and as many ints
DLGO_EXPORT int dlgo_argmax(const float* logits, int R, int ld, int V, int* out, float* part_v, int* part_i,
                            cudaStream_t stream) {
  if (R <= 0) return DLGO_OK;
  if (V <= 0 || ld < V) return DLGO_ERR_SIZE;
  int nblk = dlgo_argmax_chunks(R, V);
  if (part_v == nullptr || part_i == nullptr) nblk = 1;
  const int threads = V / nblk >= 8192 ? 1024 : (V / nblk >= 1024 ? 256 : 64);
  launch_kernel(argmax_kernel, dim3(dim3(R, nblk)), dim3(threads), 0, stream, logits, ld, V, out, part_v, part_i);
  int st = launch_status();
  if (st != DLGO_OK || nblk == 1) return st;
  launch_kernel(argmax_finish_kernel, dim3(R), dim3(32), 0, stream, part_v, part_i, nblk, out);
  return launch_status();
}

// The same, and the ids brought to `host_out` (pinned host memory, R ints): returns when they are there.
DLGO_EXPORT int dlgo_argmax_host(const float* logits, int R, int ld, int V, int* out, float* part_v, int* part_i,
                                 int* host_out, cudaStream_t stream) {
  int st = dlgo_argmax(logits, R, ld, V, out, part_v, part_i, stream);
  if (st != DLGO_OK) return st;
  cudaError_t e = cudaMemcpyAsync(host_out, out, sizeof(int) * (size_t)R, cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize(stream);
}

// Greedy decoding of one batch for up to `max_steps` steps without returning to the caller.  The
// captured step (`graph_exec`) begins with the copy of its inputs (ids, positions, slots: `host_inputs`,
// pinned, [3][B]) to the device and ends with the argmax and the copy of the chosen ids into `host_ids`
// (pinned, [B]); a step here is one graph launch and a wait.  The ids become the next step's inputs at
// positions + 1.  Stops after the step in which a sequence chose one of `stop_ids`.  The ids of step s
// go to out_tokens[s * B ...]; returns the number of steps run (>= 1), or minus a CUDA error code.
// (The reference's loop is compiled code too: models/llm/generate.go:207-283.)
DLGO_EXPORT int dlgo_greedy_run_graph(int* host_inputs, int B, void* graph_exec,
                                      const int* host_ids, const int* stop_ids, int n_stop, int max_steps,
                                      int* out_tokens, cudaStream_t stream) {
  if (B <= 0 || max_steps <= 0) return 0;
  for (int step = 0; step < max_steps; ++step) {
    cudaError_t e = cudaGraphLaunch((cudaGraphExec_t)graph_exec, stream);
    if (e != cudaSuccess) return -(int)e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return -(int)e;
    bool stop = false;
    for (int b = 0; b < B; ++b) {
      const int id = ((const volatile int*)host_ids)[b];
      out_tokens[(size_t)step * B + b] = id;
      for (int k = 0; k < n_stop; ++k) stop |= stop_ids[k] == id;
      host_inputs[b] = id;
      host_inputs[B + b] += 1;
    }
    if (stop) return step + 1;
  }
  return max_steps;
}

// temperature[R] f32 (> 0), request[R] and draw[R] int32 key the uniform of each row
// seed_dev: null, or where the kernel reads the seed (then `seed` is ignored)
// part: null, or R * dlgo_sample_chunks(V) * 2 floats of scratch: a large vocabulary is then drawn from in two
// kernels over chunks of it
DLGO_EXPORT int dlgo_sample_chunks(int V) {
  const int C = (V + FD_CHUNK - 1) / FD_CHUNK;
  return (V >= 2 * FD_CHUNK && C <= 64) ? C : 0;
}

DLGO_EXPORT int dlgo_sample(const float* logits, int R, int ld, int V, const float* temperature, const int* request,
                            const int* draw, unsigned long long seed, const unsigned long long* seed_dev, int* out,
                            float* part, cudaStream_t stream) {
  if (R <= 0) return DLGO_OK;
  if (V <= 0 || ld < V) return DLGO_ERR_SIZE;
  if (((uintptr_t)seed_dev & 7) != 0) return DLGO_ERR_ALIGN;
  const int C = dlgo_sample_chunks(V);
  if (part != nullptr && C > 0 && R <= 65535) {
    launch_kernel(sample_chunks_kernel, dim3(R, C), dim3(FD_THREADS), 0, stream, logits, ld, V, temperature, part);
    int st = launch_status();
    if (st != DLGO_OK) return st;
    launch_kernel(sample_pick_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, temperature,
                  (const float*)part, C, request, draw, (uint64_t)seed, seed_dev, out);
    return launch_status();
  }
  const int threads = V >= 8192 ? 1024 : (V >= 1024 ? 256 : 64);
  launch_kernel(sample_kernel, dim3(R), dim3(threads), 0, stream, logits, ld, V, temperature, request, draw,
                (uint64_t)seed, seed_dev, out);
  return launch_status();
}

// The same loop for sampled decoding: the captured step (`graph_exec`) begins with the copies of its inputs
// and of the draw's inputs out of pinned memory and ends with the filters, the draw and the copy of the ids
// into `host_ids`.  `draw_inputs` (pinned int32): [2] seed, [B] request index, [B] index of the draw within
// the request, [B][W] the request's most recent tokens (-1: none), [B] how many tokens it has produced in
// all (the slot of the window that the next one takes is that count modulo W).  Per step every sequence's
// draw index advances and its token enters its window, as the loop above the engine would do it.
DLGO_EXPORT int dlgo_sampled_run_graph(int* host_inputs, int B, void* graph_exec, const int* host_ids,
                                       const int* stop_ids, int n_stop, int max_steps, int* out_tokens,
                                       int* draw_inputs, int W, cudaStream_t stream) {
  if (B <= 0 || max_steps <= 0) return 0;
  if (W <= 0 || draw_inputs == nullptr) return -(int)cudaErrorInvalidValue;
  int* draws = draw_inputs + 2 + B;
  int* recent = draw_inputs + 2 + 2 * B;
  int* counts = recent + (size_t)B * W;
  for (int step = 0; step < max_steps; ++step) {
    cudaError_t e = cudaGraphLaunch((cudaGraphExec_t)graph_exec, stream);
    if (e != cudaSuccess) return -(int)e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return -(int)e;
    bool stop = false;
    for (int b = 0; b < B; ++b) {
      const int id = ((const volatile int*)host_ids)[b];
      out_tokens[(size_t)step * B + b] = id;
      for (int k = 0; k < n_stop; ++k) stop |= stop_ids[k] == id;
      host_inputs[b] = id;
      host_inputs[B + b] += 1;
      draws[b] += 1;
      recent[(size_t)b * W + (counts[b] % W)] = id;
      counts[b] += 1;
    }
    if (stop) return step + 1;
  }
  return max_steps;
}

// the uniform a (seed, draw, request) triple yields, for tests and host-side twins
__global__ void uniform_kernel(uint64_t seed, const int* draw, const int* request, float* out, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = philox_uniform(seed, (uint32_t)draw[i], (uint32_t)request[i]);
}
DLGO_EXPORT int dlgo_uniform(unsigned long long seed, const int* draw, const int* request, float* out, int n,
                             cudaStream_t stream) {
  if (n <= 0) return DLGO_OK;
  launch_kernel(uniform_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, (uint64_t)seed, draw, request, out, n);
  return launch_status();
}

// logits[R, V] f32 (row stride ld) -> work[R, V] f32: penalty, temperature, top-k (0 or >= V: off; else at most
// 2048), top-p, min-p.
// recent[R, n_recent] int32 (-1 = none), n_recent <= 64, or null.
DLGO_EXPORT int dlgo_filter(const float* logits, int R, int ld, int V, float* work, float temperature, int top_k,
                            float top_p, float min_p, float penalty, const int* recent, int n_recent,
                            cudaStream_t stream) {
  if (R <= 0) return DLGO_OK;
  if (V <= 0 || ld < V || top_k < 0 || (top_k > FILTER_CAP && top_k < V) || n_recent < 0 ||
      n_recent > FILTER_RECENT || !(temperature > 0.f))
    return DLGO_ERR_SIZE;
  launch_kernel(filter_kernel, dim3(R), dim3(FILTER_THREADS), 0, stream, logits, ld, V, work, 1.0f / temperature,
                top_k, top_p, min_p, penalty, recent, n_recent);
  return launch_status();
}

// Chunks of the vocabulary and candidates per chunk that dlgo_filter_draw uses for this top_k, or 0 where it
// does not take the sizes (top_k off or above 256, or a vocabulary so large that a row's candidate lists would
// not fit the second kernel's shared memory): the caller then filters and draws with dlgo_filter / dlgo_sample.
DLGO_EXPORT int dlgo_filter_draw_chunks(int V, int top_k) {
  if (top_k <= 0 || top_k >= V || top_k > 256 || V > (1 << 24)) return 0;
  const int C = (V + FD_CHUNK - 1) / FD_CHUNK;
  if (C > 64 || C * (2 * top_k < top_k + 32 ? top_k + 32 : 2 * top_k) > FD_MAX_CAND) return 0;
  return C;
}
DLGO_EXPORT int dlgo_filter_draw_cap(int top_k) { return 2 * top_k < top_k + 32 ? top_k + 32 : 2 * top_k; }

// Filters (as dlgo_filter) and draw (as dlgo_sample, the temperature already applied) for a small top_k.
// cand_v / cand_i: R * chunks * cap floats / ints, cand_n: R * chunks ints; work[R, V] is written only by rows
// with more ties than the lists hold.
DLGO_EXPORT int dlgo_filter_draw(const float* logits, int R, int ld, int V, float* work, float temperature, int top_k,
                                 float top_p, float min_p, float penalty, const int* recent, int n_recent,
                                 float* cand_v, int* cand_i, int* cand_n, const int* request, const int* draw,
                                 unsigned long long seed, const unsigned long long* seed_dev, int* out,
                                 cudaStream_t stream) {
  if (R <= 0) return DLGO_OK;
  const int C = dlgo_filter_draw_chunks(V, top_k);
  if (C == 0 || ld < V || n_recent < 0 || n_recent > FILTER_RECENT || !(temperature > 0.f) || R > 65535)
    return DLGO_ERR_SIZE;
  if (((uintptr_t)seed_dev & 7) != 0) return DLGO_ERR_ALIGN;
  const int cap = dlgo_filter_draw_cap(top_k);
  constexpr int SMEM = FD_MAX_CAND * 8 + FILTER_CAP * 12;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(filter_draw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  launch_kernel(candidates_kernel, dim3(R, C), dim3(FD_THREADS), 0, stream, logits, ld, V, 1.0f / temperature, top_k,
                penalty, recent, n_recent, cap, cand_v, cand_i, cand_n);
  int st = launch_status();
  if (st != DLGO_OK) return st;
  launch_kernel(filter_draw_kernel, dim3(R), dim3(FILTER_THREADS), SMEM, stream, logits, ld, V, work,
                1.0f / temperature, top_k, top_p, min_p, penalty, recent, n_recent, C, cap, (const float*)cand_v,
                (const int*)cand_i, (const int*)cand_n, request, draw, (uint64_t)seed, seed_dev, out);
  return launch_status();
}
