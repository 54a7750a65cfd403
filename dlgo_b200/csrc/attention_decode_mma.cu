// Decode attention in bfloat16 on the tensor cores (warp-level mma.sync, m16n8k16).
//
// Same formulas as attention_decode.cu (models/llm/forward.go:258-278): scores q.k * scale over the
// keys t <= pos (t > pos - window if windowed), softmax in fp32, weighted sum of the values.  The
// fp32-pipe kernel spends about 450 instructions per warp on 16 keys (a multiply-add per element and a
// shuffle tree per score); here a warp spends 16 tensor-core instructions on them, which is what
// counts once many sequences decode together.  A decode step has one query row per head, so the query
// heads of a kv head (up to 8 per block) are the rows of the 16-row MMA tile and rows 8-15 stay zero:
// the tensor cores are badly used and still several times faster than the fp32 pipes here.
//
// Nothing goes through shared memory on the way in: the k index of an MMA may be any permutation of
// the head's dimensions as long as q and k agree, and so may the order of the output dimensions.
// The permutations are chosen so that every lane's fragment registers are 16-byte pieces of rows as
// they lie in the cache pages:
//   * scores: lane (r = lane / 4, c = lane % 4) holds dimensions [c * HD/4, (c + 1) * HD/4) of query
//     head r and of key r of each 8-key n-tile; k-step kk takes 4 of them;
//   * values: the lane holds dimensions [r * HD/8, (r + 1) * HD/8) of keys 2c, 2c+1, 2c+8, 2c+9 of a
//     16-key k-step; a byte permute pairs two keys' elements into one B register.  Output column
//     nt * 8 + j of the MMA is dimension j * HD/8 + nt of the head.
// The probabilities go from the score accumulators straight into the A registers of the second MMA
// (rounded to bfloat16, as the prompt kernel does).
//
// A block takes one sequence, one kv head (8 of its query heads) and a slice of the pages; 2..8
// slices form a thread-block cluster and combine through distributed shared memory.
#include <cooperative_groups.h>
#include <math.h>

#include "attention_combine.cuh"
#include "attention_decode_tiles.cuh"
#include "common.cuh"

namespace dlgo {

constexpr int DM_THREADS = 128;
constexpr int DM_WARPS = DM_THREADS / 32;
constexpr int DM_GM = 8;   // query heads of a kv head per block

struct DecMmaParams {
  const __nv_bfloat16* q;
  int ldq;
  const __nv_bfloat16* kpages;
  const __nv_bfloat16* vpages;
  const int* page_table;
  int max_pages;
  const int* seq_slot;   // [B]
  const int* token_pos;  // [B] position of the new token (its key is already in the cache)
  __nv_bfloat16* out;
  int ldo;
  int Hq, Hkv, page_size, n_splits, n_gchunks, window;
  float scale;
  // optional: the projection's output comes in as unsummed fp32 K-slices and unrotated (q | k | v heads
  // per token); the kernel sums them, rotates q and k at the token's position and appends k and v to the
  // cache itself (one launch less per layer).  Whole-head rotation in the split-half pairing only.
  const float* parts;    // [S][B][ldq] or null
  int S;
  size_t part_stride;
  const float* cos_t;    // [positions][HD / 2]
  const float* sin_t;
  int write_cache;
  int clear_parts;       // S = 1 and `parts` is a sum that must be zero again for the next step: the block (or the
                         // cluster's first block) clears this (sequence, kv head)'s columns once all have read them
  float* part_acc;       // more than 8 slices: [B, Hq, n_splits, HD] and [B, Hq, n_splits, 2] scratch,
  float* part_ml;        // combined by a second kernel; else null (slices of a cluster combine on chip)
};

// NJ: 8-key n-tiles per warp iteration (2 or 4).  Heads of 128: two blocks per SM (255 registers a thread, nothing
// spilled); at three (170 registers) the tile's 128 registers of keys and values spill, and a decode step at the
// layer sizes of Llama 3.2 3B measured 2.12 ms against 2.06 ms at batch 8.
template <int HD, int NJ>
__global__ void __launch_bounds__(DM_THREADS, HD <= 64 ? 4 : 2) attention_decode_mma_kernel(DecMmaParams p) {
  using T = __nv_bfloat16;
  constexpr int TK = 8 * NJ;     // keys per warp iteration
  constexpr int KK = HD / 16;    // k-steps of the score MMA
  constexpr int NT = HD / 8;     // n-tiles of the output MMA
  constexpr int QV = HD / 32;    // 16-byte pieces of a lane's quarter of a key (or query) row
  constexpr int VV = HD / 64;    // 16-byte pieces of a lane's eighth of a value row
  __shared__ float sm_acc[DM_WARPS][DM_GM][HD];
  __shared__ float sm_ml[DM_WARPS][DM_GM][2];
  __shared__ float cl_acc[DM_GM][HD];   // this block's merged result, read by the cluster's first block
  __shared__ float cl_ml[DM_GM][2];

  pdl_launch_dependents();
  if (threadIdx.x == 0) TSTAMP(0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int b = blockIdx.x;
  const int kvh = blockIdx.y / p.n_gchunks, gc = blockIdx.y - kvh * p.n_gchunks;
  const int split = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int g0 = gc * DM_GM;
  const int GC = min(DM_GM, G - g0);
  const int PS = p.page_size;
  // the step's own inputs (in place before the step's first kernel starts)
  const int slot = p.seq_slot[b];
  const int pos = p.token_pos[b];
  const int t_end = pos + 1;
  const int t_begin = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int pg_first = t_begin / PS, pg_last = pos / PS;
  const int per = (pg_last - pg_first + 1 + p.n_splits - 1) / p.n_splits;
  const int pg_b = pg_first + split * per;
  const int pg_e = min(pg_last + 1, pg_b + per);
  const int tiles_per_page = PS / TK;
  const int n_tiles = max(0, pg_e - pg_b) * tiles_per_page;
  // page ids now (later loads of them hit L1), and a hint that pulls this block's rows into L2
  for (int tile = warp; tile < n_tiles; tile += DM_WARPS) {
    const int pg = pg_b + tile / tiles_per_page;
    const int key0 = (tile % tiles_per_page) * TK;
    if (pg * PS + key0 >= t_end) continue;
    const int page = p.page_table[(size_t)slot * p.max_pages + pg];
    const size_t base = (((size_t)page * p.Hkv + kvh) * PS + key0) * HD;
    constexpr int LINES = TK * HD * 2 / 128;
    // (only for short slices, at most four rounds a warp: measured on a B200, hinting a long slice all
    // at once makes decode at batch 64 and contexts near 4,000 17 % slower)
    if (n_tiles <= 4 * DM_WARPS) {
      for (int ln = lane; ln < LINES; ln += 32) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"((const char*)(p.kpages + base) + (size_t)ln * 128));
        asm volatile("prefetch.global.L2 [%0];" ::"l"((const char*)(p.vpages + base) + (size_t)ln * 128));
      }
    }
  }
  if (p.parts != nullptr && threadIdx.x < 2 * ((HD * 2 + 127) / 128)) {
    // the position's cos / sin row (a table nobody writes): on its way before the wait
    constexpr int LN = (HD * 2 + 127) / 128;
    const float* tbl = (threadIdx.x < LN ? p.cos_t : p.sin_t) + (size_t)pos * (HD / 2);
    asm volatile("prefetch.global.L1 [%0];" ::"l"((const char*)tbl + (size_t)(threadIdx.x % LN) * 128));
  }
  if (threadIdx.x == 0) TSTAMP(1);
  pdl_wait();
  if (threadIdx.x == 0) TSTAMP(2);

  // query fragments: head r of this block's chunk, this lane's quarter of the dimensions
  uint32_t qa[KK][2];
#pragma unroll
  for (int kk = 0; kk < KK; ++kk) qa[kk][0] = qa[kk][1] = 0u;
  if (p.parts == nullptr) {
    if (r < GC) {
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)b * p.ldq + (size_t)(kvh * G + g0 + r) * HD + c * (HD / 4));
#pragma unroll
      for (int v = 0; v < QV; ++v) {
        const uint4 u = src[v];
        qa[2 * v][0] = u.x; qa[2 * v][1] = u.y;
        qa[2 * v + 1][0] = u.z; qa[2 * v + 1][1] = u.w;
      }
    }
  } else {
    constexpr int RH = HD / 2;       // rotation pairs (i, i + HD/2)
    // The block whose pages hold the new position appends the token's key (rotated) and value first
    // (models/llm/forward.go:246-257): one warp, a lane per pair of dimensions.
    const int pg_new = pos / PS;
    if (p.write_cache && gc == 0 && pg_new >= pg_b && pg_new < pg_e) {   // block-uniform
      if (warp == 0) {
        const int page = p.page_table[(size_t)slot * p.max_pages + pg_new];
        const size_t row = (((size_t)page * p.Hkv + kvh) * PS + (pos % PS)) * HD;
        const float* kin = p.parts + (size_t)b * p.ldq + (size_t)(p.Hq + kvh) * HD;
        const float* vin = p.parts + (size_t)b * p.ldq + (size_t)(p.Hq + p.Hkv + kvh) * HD;
        for (int i = lane; i < RH; i += 32) {
          float k0 = 0.f, k1 = 0.f, v0 = 0.f, v1 = 0.f;
          for (int sl = 0; sl < p.S; ++sl) {          // slice order
            const size_t so = (size_t)sl * p.part_stride;
            k0 += __ldcg(kin + so + i); k1 += __ldcg(kin + so + i + RH);
            v0 += __ldcg(vin + so + i); v1 += __ldcg(vin + so + i + RH);
          }
          const float cs = p.cos_t[(size_t)pos * RH + i], sn = p.sin_t[(size_t)pos * RH + i];
          const_cast<T*>(p.kpages)[row + i] = __float2bfloat16_rn(k0 * cs - k1 * sn);
          const_cast<T*>(p.kpages)[row + i + RH] = __float2bfloat16_rn(k0 * sn + k1 * cs);
          const_cast<T*>(p.vpages)[row + i] = __float2bfloat16_rn(v0);
          const_cast<T*>(p.vpages)[row + i + RH] = __float2bfloat16_rn(v1);
        }
      }
      __threadfence_block();
      __syncthreads();   // the new row is in place before any warp of this block reads the page
    }
    // query head r, this lane's quarter of the dimensions: sum of the slices, rotation (the partner of a
    // dimension lies two quarters away: the lane with c ^ 2), rounding to bfloat16 as the separate
    // rope kernel does
    {      // (every lane takes part in the shuffles; lanes without a head carry zeros)
      constexpr int QN = HD / 4;      // dimensions per lane
      float x[QN];
#pragma unroll
      for (int k = 0; k < QN; ++k) x[k] = 0.f;
      if (r < GC) {
        const float* src = p.parts + (size_t)b * p.ldq + (size_t)(kvh * G + g0 + r) * HD + c * QN;
        // eight slices of two 16-byte pieces are in flight at a time (slices are added in order)
        for (int s0 = 0; s0 < p.S; s0 += 8) {
#pragma unroll
          for (int k4 = 0; k4 < QN / 4; k4 += 2) {
            float4 t[8][2];
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
              for (int e = 0; e < 2; ++e)
                t[j][e] = (s0 + j < p.S)
                              ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(s0 + j) * p.part_stride) + k4 + e)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                x[4 * (k4 + e)] += t[j][e].x; x[4 * (k4 + e) + 1] += t[j][e].y;
                x[4 * (k4 + e) + 2] += t[j][e].z; x[4 * (k4 + e) + 3] += t[j][e].w;
              }
          }
        }
      }
      const float* cs = p.cos_t + (size_t)pos * RH + (c & 1) * QN;
      const float* sn = p.sin_t + (size_t)pos * RH + (c & 1) * QN;
      float y[QN];
#pragma unroll
      for (int k = 0; k < QN; ++k) {
        const float other = __shfl_xor_sync(0xffffffffu, x[k], 2);
        const float ck = cs[k], sk = sn[k];
        y[k] = c < 2 ? (x[k] * ck - other * sk) : (other * sk + x[k] * ck);
      }
      if (r < GC) {
#pragma unroll
        for (int v = 0; v < QV; ++v) {
          qa[2 * v][0] = pack_bf16(y[8 * v], y[8 * v + 1]);
          qa[2 * v][1] = pack_bf16(y[8 * v + 2], y[8 * v + 3]);
          qa[2 * v + 1][0] = pack_bf16(y[8 * v + 4], y[8 * v + 5]);
          qa[2 * v + 1][1] = pack_bf16(y[8 * v + 6], y[8 * v + 7]);
        }
      }
    }
  }
  float o[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = 0.f;
  float m = -INFINITY, l = 0.f;   // of head r (l: this lane's share, summed over the quad at the end)

  decode_attend_tiles<HD, NJ>(p.kpages, p.vpages, p.page_table + (size_t)slot * p.max_pages, p.Hkv, kvh, PS, pg_b,
                              n_tiles, t_begin, t_end, p.scale, warp, DM_WARPS, lane, qa, o, m, l);
  if (threadIdx.x == 0) TSTAMP(3);

  // the quad's lanes share the maximum, so their sums add up
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (r < GC) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      // MMA column nt * 8 + 2c + e is dimension (2c + e) * HD/8 + nt of the head
      sm_acc[warp][r][(2 * c) * (HD / 8) + nt] = o[nt][0];
      sm_acc[warp][r][(2 * c + 1) * (HD / 8) + nt] = o[nt][1];
    }
    if (c == 0) {
      sm_ml[warp][r][0] = m;
      sm_ml[warp][r][1] = l;
    }
  }
  __syncthreads();
  // merge the warps: thread -> (head g, dim d)
  for (int idx = threadIdx.x; idx < GC * HD; idx += DM_THREADS) {
    const int g = idx / HD, d = idx - g * HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) mm = fmaxf(mm, sm_ml[w][g][0]);
    float a = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) {
      const float mw = sm_ml[w][g][0];
      if (mw != -INFINITY) {
        const float cw = expf(mw - mm);
        a = fmaf(cw, sm_acc[w][g][d], a);
        ll = fmaf(cw, sm_ml[w][g][1], ll);
      }
    }
    if (p.n_splits == 1) {
      p.out[(size_t)b * p.ldo + (size_t)(kvh * G + g0 + g) * HD + d] = __float2bfloat16_rn(a / ll);
    } else if (p.part_acc != nullptr) {
      const size_t o = ((size_t)b * p.Hq + (kvh * G + g0 + g)) * p.n_splits + split;
      p.part_acc[o * HD + d] = a;
      if (d == 0) {
        p.part_ml[o * 2] = mm;
        p.part_ml[o * 2 + 1] = ll;
      }
    } else {
      cl_acc[g][d] = a;
      if (d == 0) {
        cl_ml[g][0] = mm;
        cl_ml[g][1] = ll;
      }
    }
  }
  // the sums this (sequence, kv head) read: zero again for the next step's projection (every warp of the
  // block is past its reads: the merge above begins behind a block-wide barrier)
  auto clear_sums = [&]() {
    float* row = const_cast<float*>(p.parts) + (size_t)b * p.ldq;
    for (int i = threadIdx.x; i < GC * HD; i += DM_THREADS) row[(size_t)(kvh * G + g0) * HD + i] = 0.f;
    if (gc == 0)
      for (int i = threadIdx.x; i < HD; i += DM_THREADS) {
        row[(size_t)(p.Hq + kvh) * HD + i] = 0.f;
        row[(size_t)(p.Hq + p.Hkv + kvh) * HD + i] = 0.f;
      }
  };
  if (p.n_splits == 1 || p.part_acc != nullptr) {
    if (p.clear_parts) clear_sums();
    return;
  }
  // The slices of this (sequence, kv head, head chunk) are the blocks of one cluster: each leaves its
  // merged (max, sum, output) in its own shared memory; every block then finishes an equal share of
  // the outputs, reading all slices' values of them through distributed shared memory.
  namespace cg = cooperative_groups;
  cg::cluster_group cl = cg::this_cluster();
  if (threadIdx.x == 0) TSTAMP(4);
  cl.sync();
  if (threadIdx.x == 0) TSTAMP(5);
  const int NS = p.n_splits;
  const int me = (int)cl.block_rank();
  if (p.clear_parts && me == NS - 1) clear_sums();      // every slice of the cluster has read them
  const int total = GC * HD;
  const int share = (total + NS - 1) / NS;
  for (int idx = me * share + threadIdx.x; idx < min(total, (me + 1) * share); idx += DM_THREADS) {
    const int g = idx / HD, d = idx - g * HD;
    float ms[8], ls[8], as[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k < NS) {
        const float* rml = cl.map_shared_rank(&cl_ml[0][0], k);
        const float* racc = cl.map_shared_rank(&cl_acc[0][0], k);
        ms[k] = rml[g * 2];
        ls[k] = rml[g * 2 + 1];
        as[k] = racc[g * HD + d];
      } else {
        ms[k] = -INFINITY;
        ls[k] = 0.f;
        as[k] = 0.f;
      }
    }
    float mm = -INFINITY;
#pragma unroll
    for (int k = 0; k < 8; ++k) mm = fmaxf(mm, ms[k]);
    float a = 0.f, ll = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float ck = (ms[k] == -INFINITY) ? 0.f : expf(ms[k] - mm);
      a = fmaf(ck, as[k], a);
      ll = fmaf(ck, ls[k], ll);
    }
    p.out[(size_t)b * p.ldo + (size_t)(kvh * G + g0 + g) * HD + d] = __float2bfloat16_rn(a / ll);
  }
  if (threadIdx.x == 0) TSTAMP(6);
  cl.sync();   // nobody leaves while its shared memory may still be read
  if (threadIdx.x == 0) TSTAMP(7);
}

template <int HD, int NJ>
int launch_decode_mma(const DecMmaParams& p, int B, cudaStream_t stream) {
  dim3 grid(B, p.Hkv * p.n_gchunks, p.n_splits);
  if (p.n_splits > 1 && p.part_acc == nullptr) {
    launch_kernel_cluster(attention_decode_mma_kernel<HD, NJ>, grid, dim3(DM_THREADS), 0, stream,
                          dim3(1, 1, p.n_splits), p);
    return launch_status();
  }
  launch_kernel(attention_decode_mma_kernel<HD, NJ>, grid, dim3(DM_THREADS), 0, stream, p);
  int st = launch_status();
  if (st != DLGO_OK || p.n_splits == 1) return st;
  launch_kernel(attention_combine_kernel<__nv_bfloat16>, dim3(B, p.Hq), dim3(HD >= 128 ? 128 : 64), 0, stream,
                (const float*)p.part_acc, (const float*)p.part_ml, p.out, p.ldo, p.Hq, HD, p.n_splits);
  return launch_status();
}

}  // namespace dlgo

using namespace dlgo;

// 1 if the kernel takes these sizes: bfloat16 (implied), heads of 64 or 128, pages that hold whole tiles.
// 2..8 slices combine inside a thread-block cluster; more need scratch (B * Hq * n_splits * (hd + 2) floats)
// and a second kernel.
DLGO_EXPORT int dlgo_attention_decode_mma_takes(int hd, int page_size, int n_splits) {
  return (hd == 64 || hd == 128) && page_size % 32 == 0 && n_splits >= 1 && n_splits <= 65535;
}

// q[B, .] bf16 (row stride ldq, head h at column h * hd), one token per sequence at position
// token_pos[b] whose key and value are already in the cache; out[B, .] bf16 (row stride ldo).
// Or, with `parts` ([S][B][ldq] fp32, slice stride part_stride floats: the unsummed K-slices of the q | k | v
// projection) and cos/sin tables [positions][hd / 2]: q is null, the kernel sums, rotates (whole head,
// pairs (i, i + hd/2)) and, with write_cache, appends the token's key and value itself.
// keys_per_tile: 16 or 32 keys per warp iteration.
DLGO_EXPORT int dlgo_attention_decode_mma(const void* q, int B, int ldq, const void* kpages, const void* vpages,
                                          const int* page_table, int max_pages, const int* seq_slot,
                                          const int* token_pos, void* out, int ldo, int Hq, int Hkv, int hd,
                                          int page_size, int n_splits, int window, float scale, int keys_per_tile,
                                          float* scratch, const float* parts, int S, long long part_stride,
                                          const float* cos_t, const float* sin_t, int write_cache, int clear_parts,
                                          cudaStream_t stream) {
  if (B <= 0) return DLGO_OK;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return DLGO_ERR_SIZE;
  if (!dlgo_attention_decode_mma_takes(hd, page_size, n_splits)) return DLGO_ERR_SIZE;
  if (keys_per_tile != 16 && keys_per_tile != 32) return DLGO_ERR_SIZE;
  if (n_splits > 8 && scratch == nullptr) return DLGO_ERR_SIZE;
  if ((ldq & 7) || ((uintptr_t)kpages & 15) || ((uintptr_t)vpages & 15)) return DLGO_ERR_ALIGN;
  if (parts == nullptr) {
    if ((uintptr_t)q & 15) return DLGO_ERR_ALIGN;
  } else {
    // fused rotation and append: one head chunk per kv head, 16-byte slices, tables present
    if (Hq / Hkv > DM_GM || S <= 0 || (part_stride & 3) || ((uintptr_t)parts & 15) || cos_t == nullptr || sin_t == nullptr)
      return DLGO_ERR_SIZE;
    // clearing needs one sum whose readers meet: a single block or one cluster per (sequence, kv head)
    if (clear_parts && (S != 1 || n_splits > 8)) return DLGO_ERR_SIZE;
  }
  if (parts == nullptr && clear_parts) return DLGO_ERR_SIZE;
  const int G = Hq / Hkv;
  DecMmaParams p;
  p.q = (const __nv_bfloat16*)q; p.ldq = ldq;
  p.kpages = (const __nv_bfloat16*)kpages; p.vpages = (const __nv_bfloat16*)vpages;
  p.page_table = page_table; p.max_pages = max_pages; p.seq_slot = seq_slot; p.token_pos = token_pos;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size; p.n_splits = n_splits;
  p.n_gchunks = (G + DM_GM - 1) / DM_GM;
  p.window = window; p.scale = scale;
  p.parts = parts; p.S = S; p.part_stride = (size_t)part_stride; p.cos_t = cos_t; p.sin_t = sin_t;
  p.write_cache = write_cache;
  p.clear_parts = clear_parts;
  p.part_acc = n_splits > 8 ? scratch : nullptr;
  p.part_ml = n_splits > 8 ? scratch + (size_t)B * Hq * n_splits * hd : nullptr;
  if ((long long)Hkv * p.n_gchunks > 65535) return DLGO_ERR_SIZE;
  if (hd == 64) return keys_per_tile == 16 ? launch_decode_mma<64, 2>(p, B, stream) : launch_decode_mma<64, 4>(p, B, stream);
  return keys_per_tile == 16 ? launch_decode_mma<128, 2>(p, B, stream) : launch_decode_mma<128, 4>(p, B, stream);
}

DLGO_TIMES_EXPORT
