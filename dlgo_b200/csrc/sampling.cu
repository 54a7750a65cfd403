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
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ request, const int* __restrict__ draw, uint64_t seed,
              const unsigned long long* __restrict__ seed_dev, int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  if (seed_dev != nullptr) seed = *seed_dev;   // (a captured step takes its seed from memory)
  __shared__ float scratch[32];
  __shared__ float wsum[SAMPLE_THREADS / 32];
  __shared__ int chosen;
  __shared__ float rest_s;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const float inv_t = 1.0f / temperature[r];
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
    const float u = philox_uniform(seed, (uint32_t)draw[r], (uint32_t)request[r]);
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
    if (lane == 0) out[r] = pick >= 0 ? pick : (last >= 0 ? last : b);
  }
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

__global__ void __launch_bounds__(FILTER_THREADS)
filter_kernel(const float* __restrict__ logits, int ld, int V, float* __restrict__ work, float inv_t, int top_k,
              float top_p, float min_p, float penalty, const int* __restrict__ recent, int n_recent) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int rec_s[FILTER_RECENT];
  __shared__ unsigned int count_s;
  __shared__ float sv[FILTER_CAP];
  __shared__ int si[FILTER_CAP];
  __shared__ float red[32];
  __shared__ float cut_s;
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * ld;
  float* out = work + (size_t)r * V;
  // recent tokens of this row, duplicates and out-of-range ids dropped
  if (tid < FILTER_RECENT) {
    int tok = (recent != nullptr && tid < n_recent) ? recent[(size_t)r * n_recent + tid] : -1;
    if (tok >= V) tok = -1;
    for (int j = 0; j < tid && tok >= 0; ++j)
      if (recent[(size_t)r * n_recent + j] == tok) tok = -1;
    rec_s[tid] = tok;
  }
  __syncthreads();
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
  // top-k: the k-th largest of the order-preserving keys, digit by digit from the top (11, 11 and 10
  // bits): a histogram of the digit over the keys that share the digits found so far, then the highest
  // bin at which the count from the top reaches what is still wanted.  Three passes over the row.
  uint32_t lo = 0u;                       // the digits found so far, in place
  {
    int* hist = si;                       // (the survivors' list is not in use yet: 2048 bins fit)
    __shared__ unsigned int want_s, digit_s;
    if (tid == 0) want_s = (unsigned int)top_k;
    for (int level = 0; level < 3; ++level) {
      const int shift = level == 0 ? 21 : (level == 1 ? 10 : 0);
      const int nb = level < 2 ? 2048 : 1024;
      const uint32_t above = level == 0 ? 0u : ~((1u << (shift + (level < 2 ? 11 : 10))) - 1u);
      for (int i = tid; i < nb; i += FILTER_THREADS) hist[i] = 0;
      __syncthreads();
      for (int i = tid; i < V; i += FILTER_THREADS) {
        const uint32_t key = order_key(out[i]);
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
        const int owner = owners ? __ffs(owners) - 1 : 31;         // (k <= V: some lane reaches it)
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
  }
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
    const float mx = sv[0];
    float total = 0.f;
    for (int i = 0; i < n; ++i) total += expf(sv[i] - mx);
    float cut = -INFINITY;                 // smallest value kept
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
    cut = keep < n ? (float)keep : -1.f;
    cut_s = cut;
  }
  __syncthreads();
  // positions keep .. n-1 of the sorted list are dropped (ties between kept and dropped values are
  // resolved by position in the sorted order, as the reference's sort does)
  const int keep = cut_s < 0.f ? n : (int)cut_s;
  for (int i = keep + tid; i < n; i += FILTER_THREADS) out[si[i]] = -INFINITY;
}

}  // namespace dlgo

using namespace dlgo;

// Chunks the vocabulary is cut into for `R` rows (1: one kernel, no scratch).
DLGO_EXPORT int dlgo_argmax_chunks(int R, int V) {
  if (V < 16384) return 1;
  int c = (V + 2047) / 2048;
  const int want = (4 * 148 + R - 1) / R;   // enough blocks for every SM
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
DLGO_EXPORT int dlgo_sample(const float* logits, int R, int ld, int V, const float* temperature, const int* request,
                            const int* draw, unsigned long long seed, const unsigned long long* seed_dev, int* out,
                            cudaStream_t stream) {
  if (R <= 0) return DLGO_OK;
  if (V <= 0 || ld < V) return DLGO_ERR_SIZE;
  if (((uintptr_t)seed_dev & 7) != 0) return DLGO_ERR_ALIGN;
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
