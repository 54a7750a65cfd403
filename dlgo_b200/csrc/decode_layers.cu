// A run of decoder layers for a decode step (one new token per sequence, at most 16 sequences) as ONE
// persistent kernel: a CTA per SM, phases handed over through grid-wide barriers in memory.
//
// What a layer computes is what the separate kernels compute (models/llm/forward.go:144-169, 207-317):
//   P1  q|k|v = Wqkv . (x * w1)          (the RMSNorm's per-token scale, ops/norm.go:10-32, is a scalar
//                                          that commutes with the product: it is applied to the sums in P2)
//   P2  rotation of q and k at the token's position, append of k and v to the cache pages, attention of
//       the new token over the cached keys and values (split over page slices, combined by the slice
//       that finishes last)
//   P3  residual += Wo . attention
//   P4  h = silu(s g) * (s u) with [g|u] = Wgu . (r * w2), s the RMSNorm scale of the residual r
//   P5  residual += Wd . h
// Contractions run on tcgen05 with the weight as the M operand (128 rows a tile) and the tokens as N = 16,
// fp32 accumulators in tensor memory; K is cut into slices so that every SM works on every product, and the
// slices add themselves into their fp32 target with reductions at the memory (no fixed order of the adds).
//
// Roles inside a CTA: warp 0 streams weight tiles by TMA into one ring of shared-memory stages that is
// shared by all products of all layers, so the stream runs ahead of the phases as far as the ring goes
// (weights depend on nothing); warp 1 issues the MMAs; warps 2-5 build the token operand in shared memory
// (norm, conversion to bf16, 128-byte swizzle), run the epilogues, the attention phase and the barriers.
//
// Every wait is bounded (mbarriers and the grid barrier alike): a wait that runs out sets the error word,
// every role leaves its loops, tensor memory is freed and the kernel returns.
#include <math.h>

#include "attention_decode_tiles.cuh"
#include "common.cuh"
#include "tcgen05.cuh"

namespace dlgo {

using namespace sm100;

constexpr int DL_THREADS = 192;
constexpr int DL_CT = 128;                 // compute threads (warps 2-5)
constexpr int DL_TILE_M = 128;
constexpr int DL_TILE_K = 64;
constexpr int DL_BN = 16;                  // tokens per step at most (the MMA's N)
constexpr int DL_A_BYTES = DL_TILE_M * DL_TILE_K * 2;
constexpr int DL_B_BYTES = DL_BN * DL_TILE_K * 2;     // the token operand, per K block
constexpr int DL_TMEM_COLS = 64;           // two accumulators of 32 columns (16 used)
constexpr int DL_GM = 8;                   // query heads of a kv head at most

__device__ int g_decode_layers_error = 0;

// Diagnostic build (-DDLGO_TIMING): compute thread 0 of every CTA stamps the global timer at the phase
// boundaries of the launch's second layer (16 stamps per CTA; dlgo_decode_layers_times fetches them).
#ifdef DLGO_TIMING
__device__ unsigned long long g_dl_times[256 * 16];
#define DL_STAMP(k)                                                        \
  do {                                                                     \
    if (li == 1 && ctid == 0 && cta < 256) {                               \
      unsigned long long t_;                                               \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));               \
      g_dl_times[cta * 16 + (k)] = t_;                                     \
    }                                                                      \
  } while (0)
#else
#define DL_STAMP(k) do {} while (0)
#endif

struct DlGemm {
  int rows, K, tiles, kblocks, splits, per;   // weight [rows, K]; tiles of 128 rows; K-slices of `per` K blocks
};

struct alignas(64) DlLayer {
  CUtensorMap w_qkv, w_o, w_gu, w_down;
  const float* norm1_w;
  const float* norm2_w;
  __nv_bfloat16* kpages;
  __nv_bfloat16* vpages;
  float eps1, eps2;
  int write_cache, pad_;
};

struct DlParams {
  const DlLayer* layers;
  int n_layers, T;
  int d, q_dim, kv_dim, F, Hq, Hkv;
  float scale;
  DlGemm qkv, o, gu, down;
  float* residual;            // [T][ld_res] fp32
  int ld_res;
  float* qkv_sum;             // [T][q_dim + 2 kv_dim] fp32, zero between uses
  float* scale1;              // [T]
  __nv_bfloat16* attn_out;    // [T][q_dim]
  __nv_bfloat16* h;           // [T][F]
  float* part_acc;            // [T][Hq][n_splits][hd]
  float* part_ml;             // [T][Hq][n_splits][2]
  int* tickets;               // [T][Hkv], zero between uses
  const int* page_table;
  int max_pages;
  const int* seq_slot;
  const int* token_pos;
  const float* cos_t;
  const float* sin_t;
  int page_size, n_splits, window;
  unsigned int* sync;         // [0] barrier arrivals of this launch, [1] CTAs that left; zero between launches
  int stages;
  int operand_bytes;
};

// ------------------------------------------------------------------------------------------- helpers
__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

constexpr uint32_t kGridWaitLimit = 1u << 22;   // polls of a few hundred ns each: seconds

// All CTAs of the grid meet (called by the 128 compute threads).  `target` = barriers so far * grid size.
__device__ __forceinline__ void grid_barrier(unsigned int* counter, unsigned int target, int ctid,
                                             volatile int* abort_flag) {
  cbar();
  if (ctid == 0 && !*abort_flag) {
    __threadfence();
    atomicAdd(counter, 1u);
    unsigned int v = 0;
    uint32_t spins = 0;
    for (;;) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
      if (v >= target) break;
      if (++spins >= kGridWaitLimit || *abort_flag) {
        *abort_flag = 1;
        break;
      }
      if (spins > 64) __nanosleep(64);
    }
    __threadfence();
  }
  cbar();
}

// byte offset of the 16-byte chunk `c8` (8 bf16) of row `t` in K block `j` of the token operand:
// rows of 128 bytes, 8-row groups of 1024 bytes, chunks XOR-swizzled by the row (what TMA's 128-byte
// swizzle writes and the UMMA descriptor expects)
__device__ __forceinline__ uint32_t operand_offset(int j, int t, int c8) {
  return (uint32_t)(j * DL_B_BYTES + (t >> 3) * 1024 + (t & 7) * 128 + ((c8 ^ (t & 7)) << 4));
}

// Token operand from fp32 rows times a weight vector (the norm without its per-token scale), K blocks
// [kb0, kb1).  With SS the CTA also gets every row's RMSNorm scale (rows read whole: kb0 = 0, kb1 = all).
// A thread takes the same four columns of every row; TM rows (8 or 16) times U column groups are in flight
// at once (32 loads of 16 bytes a thread: an SM needs that many to take 64 KB out of L2 in one round trip).
template <bool SS, int TM>
__device__ __forceinline__ void build_operand_f32(uint8_t* dst, const float* __restrict__ x, int ld,
                                                  const float* __restrict__ w, int K, int T, int kb0, int kb1,
                                                  int ctid, float eps, float* red /* [4][16] */,
                                                  float* scales /* [16] */) {
  constexpr int U = 32 / TM;
  const int n4 = (kb1 - kb0) * (DL_TILE_K / 4);
  const int k_base = kb0 * DL_TILE_K;
  float ss[TM];
#pragma unroll
  for (int t = 0; t < TM; ++t) ss[t] = 0.f;
  for (int j0 = ctid; j0 < n4; j0 += U * DL_CT) {
    float4 v[U][TM];
    float4 wv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j4 = j0 + u * DL_CT;
      const int k = k_base + 4 * j4;
      const bool in = j4 < n4 && k < K;        // K is a multiple of 8
#pragma unroll
      for (int t = 0; t < TM; ++t)
        v[u][t] = (in && t < T) ? __ldcg(reinterpret_cast<const float4*>(x + (size_t)t * ld + k))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
      wv[u] = in ? __ldg(reinterpret_cast<const float4*>(w + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j4 = j0 + u * DL_CT;
      if (j4 >= n4) break;
      const int kk = 4 * j4;
#pragma unroll
      for (int t = 0; t < TM; ++t) {
        if (t < T) {
          const float4 e = v[u][t];
          if (SS) ss[t] = fmaf(e.x, e.x, fmaf(e.y, e.y, fmaf(e.z, e.z, fmaf(e.w, e.w, ss[t]))));
          __nv_bfloat162 hh[2] = {__floats2bfloat162_rn(e.x * wv[u].x, e.y * wv[u].y),
                                  __floats2bfloat162_rn(e.z * wv[u].z, e.w * wv[u].w)};
          *reinterpret_cast<uint2*>(dst + operand_offset(kk >> 6, t, (kk & 63) >> 3) + ((kk & 7) << 1)) =
              *reinterpret_cast<uint2*>(hh);
        }
      }
    }
  }
  if (SS) {
#pragma unroll
    for (int t = 0; t < TM; ++t) {
      const float tot = warp_sum(ss[t]);
      if ((ctid & 31) == 0) red[(ctid >> 5) * 16 + t] = tot;
    }
    cbar();
    if (ctid < T) {
      const float tot = red[ctid] + red[16 + ctid] + red[32 + ctid] + red[48 + ctid];
      scales[ctid] = 1.0f / sqrtf(tot / (float)K + eps);
    }
  }
}

// The same for a K-slice of the rows (a few KB): a thread takes four columns of every row, all rows' loads in
// flight at once.
__device__ __forceinline__ void build_operand_slice(uint8_t* dst, const float* __restrict__ x, int ld,
                                                    const float* __restrict__ w, int K, int T, int kb0, int kb1,
                                                    int ctid) {
  const int n4 = (kb1 - kb0) * (DL_TILE_K / 4);
  const int k_base = kb0 * DL_TILE_K;
  for (int j4 = ctid; j4 < n4; j4 += DL_CT) {
    const int kk = 4 * j4, k = k_base + kk;
    const bool in = k < K;        // K is a multiple of 8
    float4 v[DL_BN];
#pragma unroll
    for (int t = 0; t < DL_BN; ++t)
      v[t] = (in && t < T) ? __ldcg(reinterpret_cast<const float4*>(x + (size_t)t * ld + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 wv = in ? __ldg(reinterpret_cast<const float4*>(w + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int t = 0; t < DL_BN; ++t) {
      if (t < T) {
        __nv_bfloat162 hh[2] = {__floats2bfloat162_rn(v[t].x * wv.x, v[t].y * wv.y),
                                __floats2bfloat162_rn(v[t].z * wv.z, v[t].w * wv.w)};
        *reinterpret_cast<uint2*>(dst + operand_offset(kk >> 6, t, (kk & 63) >> 3) + ((kk & 7) << 1)) =
            *reinterpret_cast<uint2*>(hh);
      }
    }
  }
}

// Token operand from bf16 rows, K blocks [kb0, kb1): 16-byte chunks, four loads in flight a thread.
__device__ __forceinline__ void build_operand_bf16(uint8_t* dst, const __nv_bfloat16* __restrict__ x, int ld, int K,
                                                   int T, int kb0, int kb1, int ctid) {
  const int n8 = (kb1 - kb0) * (DL_TILE_K / 8);
  const int k_base = kb0 * DL_TILE_K;
  const int total = T * n8;
  for (int i0 = ctid; i0 < total; i0 += 4 * DL_CT) {
    uint4 v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = i0 + e * DL_CT;
      v[e] = make_uint4(0u, 0u, 0u, 0u);
      if (idx < total) {
        const int t = idx / n8, ch = idx - t * n8;
        const int k = k_base + 8 * ch;
        if (k < K) v[e] = __ldcg(reinterpret_cast<const uint4*>(x + (size_t)t * ld + k));
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = i0 + e * DL_CT;
      if (idx < total) {
        const int t = idx / n8, ch = idx - t * n8;
        *reinterpret_cast<uint4*>(dst + operand_offset(ch >> 3, t, ch & 7)) = v[e];
      }
    }
  }
}

__device__ __forceinline__ float silu_mul2(float g, float u) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-g * 1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return g * u * r;
}

// What the three roles agree on: the units (tile, K-slice) of a product that this CTA works on are
// u = cta, cta + grid, ...; either the product has one K-slice (every unit reads the whole K range) or it has
// at most one unit per CTA.
struct UnitIter {
  int tiles, splits, per, kblocks;
  __device__ __forceinline__ UnitIter(const DlGemm& g) : tiles(g.tiles), splits(g.splits), per(g.per), kblocks(g.kblocks) {}
  __device__ __forceinline__ int count() const { return tiles * splits; }
  __device__ __forceinline__ void unit(int u, int& tile, int& kb0, int& kb1) const {
    tile = u % tiles;
    const int split = u / tiles;
    kb0 = split * per;
    kb1 = min(kblocks, kb0 + per);
  }
};

struct Shared {
  uint64_t* full;
  uint64_t* empty;
  uint64_t* bready;
  uint64_t* acc_full;    // [2]
  uint64_t* acc_empty;   // [2]
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  int* flag;             // broadcast word of the compute threads
  float* red;            // [4][16]
  float* scales;         // [16]
  uint8_t* ring;
  uint8_t* operand;
};

// ------------------------------------------------------------------------------ the attention phase
// One (sequence, kv head, page slice) by the 128 compute threads; `scratch` is the operand region.
template <int HD>
__device__ __forceinline__ void attention_item(const DlParams& p, const DlLayer& L, int b, int kvh, int split,
                                               int ctid, float* scratch, int* flag) {
  using T = __nv_bfloat16;
  constexpr int NJ = 4;
  constexpr int TK = 8 * NJ;
  constexpr int KK = HD / 16, NT = HD / 8, QV = HD / 32;
  constexpr int RH = HD / 2;
  constexpr int NW = DL_CT / 32;
  float* sm_acc = scratch;                              // [NW][8][HD]
  float* sm_ml = scratch + NW * DL_GM * HD;             // [NW][8][2]
  const int lane = ctid & 31, warp = ctid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int G = p.Hq / p.Hkv;
  const int PS = p.page_size;
  const int slot = p.seq_slot[b];
  const int pos = p.token_pos[b];
  const int t_end = pos + 1;
  const int t_begin = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int pg_first = t_begin / PS, pg_last = pos / PS;
  const int per = (pg_last - pg_first + 1 + p.n_splits - 1) / p.n_splits;
  const int pg_b = pg_first + split * per;
  const int pg_e = min(pg_last + 1, pg_b + per);
  const int n_tiles = max(0, pg_e - pg_b) * (PS / TK);
  const int* page_row = p.page_table + (size_t)slot * p.max_pages;
  const int ldq = p.q_dim + 2 * p.kv_dim;
  const float* sums = p.qkv_sum + (size_t)b * ldq;
  const float sc = __ldcg(p.scale1 + b);            // the norm's scale of this token, applied to the sums

  // the slice that holds the new position appends the token's key (rotated) and value first
  // (models/llm/forward.go:246-257); the rows are then read back from the page like every other key
  const int pg_new = pos / PS;
  if (L.write_cache && pg_new >= pg_b && pg_new < pg_e) {      // uniform over the compute threads
    if (warp == 0) {
      const int page = page_row[pg_new];
      if (page >= 0) {
        const size_t row = (((size_t)page * p.Hkv + kvh) * PS + (pos % PS)) * HD;
        const float* kin = sums + (size_t)(p.Hq + kvh) * HD;
        const float* vin = sums + (size_t)(p.Hq + p.Hkv + kvh) * HD;
        for (int i = lane; i < RH; i += 32) {
          const float k0 = __ldcg(kin + i) * sc, k1 = __ldcg(kin + i + RH) * sc;
          const float v0 = __ldcg(vin + i) * sc, v1 = __ldcg(vin + i + RH) * sc;
          const float cs = p.cos_t[(size_t)pos * RH + i], sn = p.sin_t[(size_t)pos * RH + i];
          L.kpages[row + i] = __float2bfloat16_rn(k0 * cs - k1 * sn);
          L.kpages[row + i + RH] = __float2bfloat16_rn(k0 * sn + k1 * cs);
          L.vpages[row + i] = __float2bfloat16_rn(v0);
          L.vpages[row + i + RH] = __float2bfloat16_rn(v1);
        }
      } else if (lane == 0) {
        atomicExch(&g_decode_layers_error, 2);      // no page for the position: nothing is written
      }
    }
    __threadfence_block();
    cbar();
  }
  // query head r, this lane's quarter of the dimensions: scale, rotation (the partner of a dimension lies
  // two quarters away: the lane with c ^ 2), rounding to bfloat16
  uint32_t qa[KK][2];
  {
    constexpr int QN = HD / 4;
    float x[QN];
#pragma unroll
    for (int k = 0; k < QN; ++k) x[k] = 0.f;
    if (r < G) {
      const float4* src = reinterpret_cast<const float4*>(sums + (size_t)(kvh * G + r) * HD + c * QN);
#pragma unroll
      for (int k4 = 0; k4 < QN / 4; ++k4) {
        const float4 v = __ldcg(src + k4);
        x[4 * k4] = v.x * sc; x[4 * k4 + 1] = v.y * sc; x[4 * k4 + 2] = v.z * sc; x[4 * k4 + 3] = v.w * sc;
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
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) qa[kk][0] = qa[kk][1] = 0u;
    if (r < G) {
#pragma unroll
      for (int v = 0; v < QV; ++v) {
        qa[2 * v][0] = pack_bf16(y[8 * v], y[8 * v + 1]);
        qa[2 * v][1] = pack_bf16(y[8 * v + 2], y[8 * v + 3]);
        qa[2 * v + 1][0] = pack_bf16(y[8 * v + 4], y[8 * v + 5]);
        qa[2 * v + 1][1] = pack_bf16(y[8 * v + 6], y[8 * v + 7]);
      }
    }
  }
  float o[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = 0.f;
  float m = -INFINITY, l = 0.f;
  decode_attend_tiles<HD, NJ>(L.kpages, L.vpages, page_row, p.Hkv, kvh, PS, pg_b, n_tiles, t_begin, t_end, p.scale,
                              warp, NW, lane, qa, o, m, l);
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (r < G) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      sm_acc[(warp * DL_GM + r) * HD + (2 * c) * (HD / 8) + nt] = o[nt][0];
      sm_acc[(warp * DL_GM + r) * HD + (2 * c + 1) * (HD / 8) + nt] = o[nt][1];
    }
    if (c == 0) {
      sm_ml[(warp * DL_GM + r) * 2] = m;
      sm_ml[(warp * DL_GM + r) * 2 + 1] = l;
    }
  }
  cbar();
  // merge the warps: thread -> (head g, dimension d)
  for (int idx = ctid; idx < G * HD; idx += DL_CT) {
    const int g = idx / HD, d = idx - g * HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) mm = fmaxf(mm, sm_ml[(w * DL_GM + g) * 2]);
    float a = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float mw = sm_ml[(w * DL_GM + g) * 2];
      if (mw != -INFINITY) {
        const float cw = expf(mw - mm);
        a = fmaf(cw, sm_acc[(w * DL_GM + g) * HD + d], a);
        ll = fmaf(cw, sm_ml[(w * DL_GM + g) * 2 + 1], ll);
      }
    }
    if (p.n_splits == 1) {
      p.attn_out[(size_t)b * p.q_dim + (size_t)(kvh * G + g) * HD + d] = __float2bfloat16_rn(a / ll);
    } else {
      const size_t oo = ((size_t)b * p.Hq + (kvh * G + g)) * p.n_splits + split;
      p.part_acc[oo * HD + d] = a;
      if (d == 0) {
        p.part_ml[oo * 2] = mm;
        p.part_ml[oo * 2 + 1] = ll;
      }
    }
  }
  if (p.n_splits == 1) {
    cbar();     // the scratch is free for the next item
    return;
  }
  // the slice that finishes last combines all slices of this (sequence, kv head)
  __threadfence();
  cbar();
  if (ctid == 0) {
    int* tk = p.tickets + b * p.Hkv + kvh;
    const int ticket = atomicAdd(tk, 1);
    const int last = ticket == p.n_splits - 1;
    if (last) *tk = 0;       // ready for the next layer
    *flag = last;
  }
  cbar();
  if (*flag) {
    __threadfence();
    const int NS = p.n_splits;
    for (int idx = ctid; idx < G * HD; idx += DL_CT) {
      const int g = idx / HD, d = idx - g * HD;
      const size_t o0 = ((size_t)b * p.Hq + (kvh * G + g)) * NS;
      float mm = -INFINITY;
      for (int s = 0; s < NS; ++s) mm = fmaxf(mm, __ldcg(p.part_ml + (o0 + s) * 2));
      float a = 0.f, ll = 0.f;
      for (int s = 0; s < NS; ++s) {
        const float ms = __ldcg(p.part_ml + (o0 + s) * 2);
        if (ms != -INFINITY) {
          const float cw = expf(ms - mm);
          a = fmaf(cw, __ldcg(p.part_acc + (o0 + s) * HD + d), a);
          ll = fmaf(cw, __ldcg(p.part_ml + (o0 + s) * 2 + 1), ll);
        }
      }
      p.attn_out[(size_t)b * p.q_dim + (size_t)(kvh * G + g) * HD + d] = __float2bfloat16_rn(a / ll);
    }
  }
  cbar();
}

// ------------------------------------------------------------------------------------- the kernel
// Epilogue kinds
enum { DL_EPI_RED = 0, DL_EPI_SWIGLU = 1 };

template <int HD>
__global__ void __launch_bounds__(DL_THREADS, 1) decode_layers_kernel(const __grid_constant__ DlParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int STAGES = p.stages;
  Shared sh;
  sh.ring = smem;
  sh.operand = smem + (size_t)STAGES * DL_A_BYTES;
  uint8_t* ctl = sh.operand + p.operand_bytes;
  sh.full = (uint64_t*)ctl;
  sh.empty = sh.full + STAGES;
  sh.bready = sh.empty + STAGES;
  sh.acc_full = sh.bready + 1;
  sh.acc_empty = sh.acc_full + 2;
  sh.tmem_slot = (uint32_t*)(sh.acc_empty + 2);
  sh.abort_flag = (volatile int*)(sh.tmem_slot + 1);
  sh.flag = (int*)(sh.tmem_slot + 2);
  sh.red = (float*)(sh.tmem_slot + 4);
  sh.scales = sh.red + 64;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, grid = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    mbar_init(sh.bready, 1);
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sh.acc_full[a], 1);
      mbar_init(&sh.acc_empty[a], DL_CT);
    }
    *sh.abort_flag = 0;
    *sh.flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(sh.tmem_slot, DL_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *sh.tmem_slot;
  volatile int* abort_flag = sh.abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ weights: one stream for all phases
    if (elect_one()) {
      uint32_t sc = 0;     // stages filled so far
      bool ok = true;
      for (int li = 0; ok && li < p.n_layers; ++li) {
        const DlLayer& L = p.layers[li];
        for (int ph = 0; ok && ph < 4; ++ph) {
          const DlGemm& g = ph == 0 ? p.qkv : (ph == 1 ? p.o : (ph == 2 ? p.gu : p.down));
          const CUtensorMap* map = ph == 0 ? &L.w_qkv : (ph == 1 ? &L.w_o : (ph == 2 ? &L.w_gu : &L.w_down));
          const UnitIter it(g);
          for (int u = cta; ok && u < it.count(); u += grid) {
            int tile, kb0, kb1;
            it.unit(u, tile, kb0, kb1);
            for (int kb = kb0; kb < kb1; ++kb, ++sc) {
              const uint32_t s = sc % (uint32_t)STAGES, phs = (sc / (uint32_t)STAGES) & 1u;
              if (!mbar_wait(&sh.empty[s], phs ^ 1u, abort_flag)) { ok = false; break; }
              mbar_expect_tx(&sh.full[s], DL_A_BYTES);
              tma_load_2d(sh.ring + (size_t)s * DL_A_BYTES, map, &sh.full[s], kb * DL_TILE_K, tile * DL_TILE_M);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------------------------------- MMAs
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(DL_TILE_M, DL_BN);
      uint32_t sc = 0, uc = 0, gph = 0;
      bool ok = true;
      for (int li = 0; ok && li < p.n_layers; ++li) {
        for (int ph = 0; ok && ph < 4; ++ph, ++gph) {
          const DlGemm& g = ph == 0 ? p.qkv : (ph == 1 ? p.o : (ph == 2 ? p.gu : p.down));
          const UnitIter it(g);
          if (!mbar_wait(sh.bready, gph & 1u, abort_flag)) { ok = false; break; }   // the operand is written
          tc_fence_after_sync();
          for (int u = cta; ok && u < it.count(); u += grid, ++uc) {
            int tile, kb0, kb1;
            it.unit(u, tile, kb0, kb1);
            const uint32_t a = uc & 1u;
            if (!mbar_wait(&sh.acc_empty[a], ((uc >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t tmem_d = tmem_base + a * 32u;
            for (int kb = kb0; kb < kb1; ++kb, ++sc) {
              const uint32_t s = sc % (uint32_t)STAGES, phs = (sc / (uint32_t)STAGES) & 1u;
              if (!mbar_wait(&sh.full[s], phs, abort_flag)) { ok = false; break; }
              tc_fence_after_sync();
              const uint64_t da = umma_desc_k_sw128(smem_u32(sh.ring + (size_t)s * DL_A_BYTES));
              const uint64_t db = umma_desc_k_sw128(smem_u32(sh.operand + (size_t)(kb - kb0) * DL_B_BYTES));
#pragma unroll
              for (int k = 0; k < DL_TILE_K / 16; ++k)
                umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb > kb0) || (k != 0));
              umma_commit(&sh.empty[s]);
            }
            if (ok) umma_commit(&sh.acc_full[a]);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------- operands, epilogues, attention, barriers
    const int ctid = threadIdx.x - 64;
    const int cw = ctid >> 5;               // 0..3
    const int quarter = warp & 3;           // the tensor-memory lanes this warp may read
    uint32_t uc = 0;                        // units so far
    unsigned int nbar = 0;                  // grid barriers so far
    const int ldq = p.q_dim + 2 * p.kv_dim;
    pdl_wait();                             // the residual comes from the kernel before this one

    // epilogue of this CTA's units of one product
    auto epilogue = [&](const DlGemm& g, int kind, float* dst, int ldd) {
      const UnitIter it(g);
      for (int u = cta; u < it.count(); u += grid, ++uc) {
        int tile, kb0, kb1;
        it.unit(u, tile, kb0, kb1);
        const uint32_t a = uc & 1u;
        const bool ok = __all_sync(0xffffffffu, mbar_wait(&sh.acc_full[a], (uc >> 1) & 1u, abort_flag));
        tc_fence_after_sync();
        float v[16];
        if (ok) {
          tmem_ld_32x16(tmem_base + a * 32u + ((uint32_t)(quarter * 32) << 16), v);
          tmem_ld_wait();
        }
        tc_fence_before_sync();
        mbar_arrive(&sh.acc_empty[a]);
        if (!ok) continue;
        const int row = tile * DL_TILE_M + quarter * 32 + lane;
        if (kind == DL_EPI_RED) {
          if (row < g.rows) {
#pragma unroll
            for (int j = 0; j < DL_BN; ++j)
              if (j < p.T) atomicAdd(dst + (size_t)j * ldd + row, v[j]);
          }
        } else {
          // rows come in blocks of 16 gate rows followed by their 16 up rows: lanes 0-15 hold gates
#pragma unroll
          for (int j = 0; j < DL_BN; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
            if (j < p.T && lane < 16 && row + 16 < g.rows) {
              const float s = sh.scales[j];
              const int feature = (row >> 5) * 16 + (row & 15);
              p.h[(size_t)j * p.F + feature] = __float2bfloat16_rn(silu_mul2(v[j] * s, other * s));
            }
          }
        }
      }
    };
    auto my_range = [&](const DlGemm& g, int& kb0, int& kb1) {
      // the K blocks this CTA's operand covers (see UnitIter: one range per product and CTA)
      const UnitIter it(g);
      int tile;
      kb0 = 0;
      kb1 = 0;
      if (cta < it.count()) it.unit(cta, tile, kb0, kb1);
    };
    auto operand_ready = [&]() {
      fence_proxy_async_smem();
      cbar();
      if (ctid == 0) mbar_arrive(sh.bready);
    };

    for (int li = 0; li < p.n_layers; ++li) {
      const DlLayer& L = p.layers[li];
      int kb0, kb1;
      DL_STAMP(0);
      // ---- P1: q|k|v sums
      my_range(p.qkv, kb0, kb1);
      build_operand_slice(sh.operand, p.residual, p.ld_res, L.norm1_w, p.d, p.T, kb0, kb1, ctid);
      operand_ready();
      DL_STAMP(1);
      if (cta < p.T) {        // this CTA computes the norm's scale of token `cta`
        float ss = 0.f;
        const float* row = p.residual + (size_t)cta * p.ld_res;
        for (int k = 4 * ctid; k < p.d; k += 4 * DL_CT) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(row + k));
          ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
        ss = warp_sum(ss);
        if (lane == 0) sh.red[cw] = ss;
        cbar();
        if (ctid == 0)
          p.scale1[cta] = 1.0f / sqrtf((sh.red[0] + sh.red[1] + sh.red[2] + sh.red[3]) / (float)p.d + L.eps1);
      }
      epilogue(p.qkv, DL_EPI_RED, p.qkv_sum, ldq);
      DL_STAMP(2);
      grid_barrier(p.sync, ++nbar * (unsigned)grid, ctid, abort_flag);
      DL_STAMP(3);
      if (li == 0 && ctid == 0) pdl_launch_dependents();   // every CTA of this grid is resident by now

      // ---- P2: rotation, append, attention
      {
        const int items = p.T * p.Hkv * p.n_splits;
        for (int it = cta; it < items; it += grid) {
          const int split = it % p.n_splits;
          const int bk = it / p.n_splits;
          attention_item<HD>(p, L, bk / p.Hkv, bk % p.Hkv, split, ctid, (float*)sh.operand, sh.flag);
        }
      }
      DL_STAMP(4);
      grid_barrier(p.sync, ++nbar * (unsigned)grid, ctid, abort_flag);
      DL_STAMP(5);

      // ---- P3: residual += Wo . attention
      my_range(p.o, kb0, kb1);
      build_operand_bf16(sh.operand, p.attn_out, p.q_dim, p.q_dim, p.T, kb0, kb1, ctid);
      operand_ready();
      DL_STAMP(6);
      {   // the sums were read by everyone: zero again for the next layer
        const int n4 = p.T * ldq / 4;
        float4* z = reinterpret_cast<float4*>(p.qkv_sum);
        for (int i = cta * DL_CT + ctid; i < n4; i += grid * DL_CT) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      epilogue(p.o, DL_EPI_RED, p.residual, p.ld_res);
      DL_STAMP(7);
      grid_barrier(p.sync, ++nbar * (unsigned)grid, ctid, abort_flag);
      DL_STAMP(8);

      // ---- P4: h = silu(s g) * (s u)
      my_range(p.gu, kb0, kb1);
      if (kb1 > kb0) {
        if (p.T <= 8)
          build_operand_f32<true, 8>(sh.operand, p.residual, p.ld_res, L.norm2_w, p.d, p.T, 0, p.gu.kblocks, ctid,
                                     L.eps2, sh.red, sh.scales);
        else
          build_operand_f32<true, 16>(sh.operand, p.residual, p.ld_res, L.norm2_w, p.d, p.T, 0, p.gu.kblocks, ctid,
                                      L.eps2, sh.red, sh.scales);
      }
      operand_ready();
      DL_STAMP(9);
      epilogue(p.gu, DL_EPI_SWIGLU, nullptr, 0);
      DL_STAMP(10);
      grid_barrier(p.sync, ++nbar * (unsigned)grid, ctid, abort_flag);
      DL_STAMP(11);

      // ---- P5: residual += Wd . h
      my_range(p.down, kb0, kb1);
      build_operand_bf16(sh.operand, p.h, p.F, p.F, p.T, kb0, kb1, ctid);
      operand_ready();
      DL_STAMP(12);
      epilogue(p.down, DL_EPI_RED, p.residual, p.ld_res);
      DL_STAMP(13);
      if (li + 1 < p.n_layers) grid_barrier(p.sync, ++nbar * (unsigned)grid, ctid, abort_flag);
      DL_STAMP(14);
    }
    // the barrier counters are zero again for the next launch once every CTA has left its last wait
    cbar();
    if (ctid == 0) {
      __threadfence();
      const unsigned int left = atomicAdd(p.sync + 1, 1u);
      if (left == (unsigned)grid - 1) {
        p.sync[0] = 0u;
        p.sync[1] = 0u;
        __threadfence();
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(&g_decode_layers_error, 1);
    // tile loads that may still be in flight land before shared memory is handed on
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, DL_TMEM_COLS);
  }
}

}  // namespace dlgo

using namespace dlgo;

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// weight [rows, K] bf16, row stride ld elements; box = 64 columns x 128 rows, 128-byte swizzle, zero fill
int weight_map(CUtensorMap* m, const void* base, int rows, int K, int ld) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return DLGO_ERR_DRIVER;
  if (((uintptr_t)base & 15) != 0 || (ld % 8) != 0 || K % 8 != 0) return DLGO_ERR_ALIGN;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)DL_TILE_K, (cuuint32_t)DL_TILE_M};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DLGO_OK : DLGO_ERR_DRIVER;
}

// K-slices of a product for `grid` CTAs: as many as give every CTA at most one unit (sum products), or one
// slice and units dealt out in turn (the gate/up product, whose epilogue needs whole sums).
DlGemm plan(int rows, int K, int grid, bool whole_k) {
  DlGemm g;
  g.rows = rows;
  g.K = K;
  g.tiles = (rows + DL_TILE_M - 1) / DL_TILE_M;
  g.kblocks = (K + DL_TILE_K - 1) / DL_TILE_K;
  int splits = 1;
  if (!whole_k && g.tiles <= grid) {
    splits = grid / g.tiles;
    if (splits > g.kblocks) splits = g.kblocks;
    if (splits < 1) splits = 1;
  }
  g.per = (g.kblocks + splits - 1) / splits;
  g.splits = (g.kblocks + g.per - 1) / g.per;      // no empty slices
  return g;
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

constexpr int kSmemBudget = 227 * 1024 - 2048;   // alignment slack and control words

// Bytes of the token operand region for these sizes and the ring's stages that fit beside it (0: refused).
int layout(const DlGemm& qkv, const DlGemm& o, const DlGemm& gu, const DlGemm& down, int hd, int* operand_bytes) {
  int kb = qkv.per;
  if (o.per > kb) kb = o.per;
  if (gu.kblocks > kb) kb = gu.kblocks;
  if (down.per > kb) kb = down.per;
  int bytes = kb * DL_B_BYTES;
  const int attn = (4 * DL_GM * hd + 4 * DL_GM * 2) * 4;      // the attention phase's merge buffers
  if (attn > bytes) bytes = attn;
  bytes = (bytes + 1023) & ~1023;
  *operand_bytes = bytes;
  int stages = (kSmemBudget - bytes - 1024) / DL_A_BYTES;
  if (stages > 12) stages = 12;
  return stages >= 4 ? stages : 0;
}

}  // namespace

// Number of CTAs the kernel runs with on the current device (one per SM).
DLGO_EXPORT int dlgo_decode_layers_grid() { return sm_count(); }

// 1 if the kernel takes these sizes: heads of 64 or 128, at most 8 query heads per kv head, pages of 64, at
// most 16 tokens, sizes in steps of 8, feed-forward rows in blocks of 32, and a token operand that leaves
// the weight ring at least four stages of shared memory.
DLGO_EXPORT int dlgo_decode_layers_takes(int T, int d, int Hq, int Hkv, int hd, int F, int page_size) {
  if (T < 1 || T > DL_BN || Hq <= 0 || Hkv <= 0 || Hq % Hkv || Hq / Hkv > DL_GM) return 0;
  if ((hd != 64 && hd != 128) || page_size != 64 || d % 8 || F % 16 || (Hq * hd) % 8) return 0;
  const int grid = sm_count();
  if (grid <= 0) return 0;
  const DlGemm qkv = plan((Hq + 2 * Hkv) * hd, d, grid, false), o = plan(d, Hq * hd, grid, false);
  const DlGemm gu = plan(2 * F, d, grid, true), down = plan(d, F, grid, false);
  int ob = 0;
  return layout(qkv, o, gu, down, hd, &ob) > 0 ? 1 : 0;
}

// Bytes of one layer's descriptor in the array `layers` (device memory) that dlgo_decode_layers reads.
DLGO_EXPORT int dlgo_decode_layers_desc_bytes() { return (int)sizeof(DlLayer); }

// Fills one layer's descriptor (host memory, 64-byte aligned): tensor maps of the four weights (bf16, row
// stride = K), norm weights, the layer's cache pages.  w_gu holds gate and up rows in blocks of 16 + 16.
DLGO_EXPORT int dlgo_decode_layers_describe(void* desc, const void* w_qkv, const void* w_o, const void* w_gu,
                                            const void* w_down, const float* norm1_w, const float* norm2_w,
                                            float eps1, float eps2, void* kpages, void* vpages, int write_cache, int d,
                                            int Hq, int Hkv, int hd, int F) {
  if (((uintptr_t)desc & 63) != 0) return DLGO_ERR_ALIGN;
  DlLayer* L = (DlLayer*)desc;
  const int qkv_n = (Hq + 2 * Hkv) * hd, q_dim = Hq * hd;
  int st = weight_map(&L->w_qkv, w_qkv, qkv_n, d, d);
  if (st == DLGO_OK) st = weight_map(&L->w_o, w_o, d, q_dim, q_dim);
  if (st == DLGO_OK) st = weight_map(&L->w_gu, w_gu, 2 * F, d, d);
  if (st == DLGO_OK) st = weight_map(&L->w_down, w_down, d, F, F);
  if (st != DLGO_OK) return st;
  if (((uintptr_t)norm1_w & 15) || ((uintptr_t)norm2_w & 15) || ((uintptr_t)kpages & 15) || ((uintptr_t)vpages & 15))
    return DLGO_ERR_ALIGN;
  L->norm1_w = norm1_w;
  L->norm2_w = norm2_w;
  L->kpages = (__nv_bfloat16*)kpages;
  L->vpages = (__nv_bfloat16*)vpages;
  L->eps1 = eps1;
  L->eps2 = eps2;
  L->write_cache = write_cache;
  L->pad_ = 0;
  return DLGO_OK;
}

// Floats of attention scratch (partial sums of the page slices) for T tokens.
DLGO_EXPORT long long dlgo_decode_layers_scratch_floats(int T, int Hq, int hd, int n_splits) {
  return n_splits > 1 ? (long long)T * Hq * n_splits * (hd + 2) : 0;
}

// Runs `n_layers` layers (descriptors in device memory) on the T tokens whose residual stream is
// residual[T][ld_res] fp32, in place.  qkv_sum [T][(Hq + 2 Hkv) hd] fp32 and tickets [T][Hkv] int32 must be
// zero and are left zero; sync: two zeroed unsigned ints, left zero; scale1 [T]; attn_out [T][Hq hd] bf16;
// h [T][F] bf16; scratch: dlgo_decode_layers_scratch_floats floats.  first: 1 if no kernel of the same step
// precedes it on the stream (it then starts only after all earlier work).
DLGO_EXPORT int dlgo_decode_layers(const void* layers, int n_layers, int T, int d, int Hq, int Hkv, int hd, int F,
                                   float scale, float* residual, int ld_res, float* qkv_sum, float* scale1,
                                   void* attn_out, void* h, float* scratch, int* tickets, const int* page_table,
                                   int max_pages, const int* seq_slot, const int* token_pos, const float* cos_t,
                                   const float* sin_t, int page_size, int n_splits, int window, unsigned int* sync,
                                   int first, cudaStream_t stream) {
  if (n_layers <= 0 || T <= 0) return DLGO_OK;
  if (!dlgo_decode_layers_takes(T, d, Hq, Hkv, hd, F, page_size)) return DLGO_ERR_SIZE;
  if (n_splits < 1 || n_splits > 1024 || (n_splits > 1 && scratch == nullptr)) return DLGO_ERR_SIZE;
  if (((uintptr_t)residual & 15) || (ld_res & 3) || ((uintptr_t)qkv_sum & 15) || ((uintptr_t)attn_out & 15) ||
      ((uintptr_t)h & 15) || ((uintptr_t)layers & 63))
    return DLGO_ERR_ALIGN;
  const int grid = sm_count();
  DlParams p;
  p.layers = (const DlLayer*)layers;
  p.n_layers = n_layers;
  p.T = T;
  p.d = d; p.q_dim = Hq * hd; p.kv_dim = Hkv * hd; p.F = F; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale;
  p.qkv = plan((Hq + 2 * Hkv) * hd, d, grid, false);
  p.o = plan(d, Hq * hd, grid, false);
  p.gu = plan(2 * F, d, grid, true);
  p.down = plan(d, F, grid, false);
  p.residual = residual; p.ld_res = ld_res;
  p.qkv_sum = qkv_sum; p.scale1 = scale1;
  p.attn_out = (__nv_bfloat16*)attn_out; p.h = (__nv_bfloat16*)h;
  p.part_acc = scratch;
  p.part_ml = scratch != nullptr ? scratch + (size_t)T * Hq * n_splits * hd : nullptr;
  p.tickets = tickets;
  p.page_table = page_table; p.max_pages = max_pages; p.seq_slot = seq_slot; p.token_pos = token_pos;
  p.cos_t = cos_t; p.sin_t = sin_t;
  p.page_size = page_size; p.n_splits = n_splits; p.window = window;
  p.sync = sync;
  p.stages = layout(p.qkv, p.o, p.gu, p.down, hd, &p.operand_bytes);
  if (p.stages <= 0) return DLGO_ERR_SIZE;
  const int smem = p.stages * DL_A_BYTES + p.operand_bytes + 1024 /* control */ + 1024 /* alignment */;
  auto kernel = hd == 64 ? decode_layers_kernel<64> : decode_layers_kernel<128>;
  static bool configured[2] = {false, false};
  if (!configured[hd == 128]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured[hd == 128] = true;
  }
  if (first)
    launch_kernel_first(kernel, dim3(grid), dim3(DL_THREADS), smem, stream, p);
  else
    launch_kernel(kernel, dim3(grid), dim3(DL_THREADS), smem, stream, p);
  return launch_status();
}

// 0, or what went wrong in a kernel of this library since the last call (clears the word): 1 a bounded wait
// ran out (the results are invalid; the caller must zero `sync`, `tickets` and `qkv_sum` again), 2 a
// token's position had no page in the table.
DLGO_EXPORT int dlgo_decode_layers_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_decode_layers_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_decode_layers_error, &zero, sizeof(int));
  return v;
}

#ifdef DLGO_TIMING
// Diagnostic build only: the phase stamps of the last launch's second layer, 16 per CTA for 256 CTAs.
DLGO_EXPORT int dlgo_decode_layers_times(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, dlgo::g_dl_times, sizeof(unsigned long long) * 256 * 16) == cudaSuccess ? 0 : -1;
}
#endif
