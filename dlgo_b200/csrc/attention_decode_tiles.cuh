// The inner loop of decode attention on the tensor cores (warp-level mma.sync, m16n8k16), shared by the
// kernels that run it: one warp walks tiles of TK = 8 NJ keys of one kv head and keeps, for up to eight
// query heads, a running maximum, sum and output (flash-style, fp32).  See attention_decode_mma.cu for the
// fragment permutations that let every lane load 16-byte pieces of rows straight from the cache pages.
#pragma once
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>

namespace dlgo {

// d (rows 0-7 only) += A (rows 0-7; rows 8-15 are zero) * B
__device__ __forceinline__ void mma_rows8(float& d0, float& d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  float x2, x3;
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %10, %10};"
      : "+f"(d0), "+f"(d1), "=f"(x2), "=f"(x3)
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t word_of(const uint4& u, int i) {   // i is a compile-time constant after unrolling
  return i == 0 ? u.x : (i == 1 ? u.y : (i == 2 ? u.z : u.w));
}
__device__ __forceinline__ float fast_exp(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}

// Tiles first_tile, first_tile + tile_step, ... of the slice's n_tiles tiles (tile i covers keys
// [(pg_b + i / tiles_per_page) * PS + (i % tiles_per_page) * TK, + TK) of the sequence whose page numbers are
// `page_row[]`), keys t in [t_begin, t_end) only.  Lane (r = lane / 4, c = lane % 4): `qa` holds head r's
// query fragments; `o` receives its output (MMA column nt * 8 + 2c + e is dimension (2c + e) * HD/8 + nt),
// `m` its running maximum and `l` this lane's share of the sum (to be added over the quad).
template <int HD, int NJ>
__device__ __forceinline__ void decode_attend_tiles(const __nv_bfloat16* kpages, const __nv_bfloat16* vpages,
                                                    const int* __restrict__ page_row, int Hkv, int kvh, int PS,
                                                    int pg_b, int n_tiles, int t_begin, int t_end, float scale,
                                                    int first_tile, int tile_step, int lane,
                                                    const uint32_t (&qa)[HD / 16][2], float (&o)[HD / 8][2], float& m,
                                                    float& l) {
  using T = __nv_bfloat16;
  constexpr int TK = 8 * NJ;     // keys per warp iteration
  constexpr int KK = HD / 16;    // k-steps of the score MMA
  constexpr int NT = HD / 8;     // n-tiles of the output MMA
  constexpr int QV = HD / 32;    // 16-byte pieces of a lane's quarter of a key (or query) row
  constexpr int VV = HD / 64;    // 16-byte pieces of a lane's eighth of a value row
  const int r = lane >> 2, c = lane & 3;
  const int tiles_per_page = PS / TK;
  for (int tile = first_tile; tile < n_tiles; tile += tile_step) {
    const int pg = pg_b + tile / tiles_per_page;
    const int key0 = (tile % tiles_per_page) * TK;
    if (pg * PS + key0 >= t_end) continue;                       // wholly beyond the sequence (warp-uniform)
    const int page = page_row[pg];
    const size_t base = ((size_t)page * Hkv + kvh) * PS * HD;
    const T* kp = kpages + base;
    const T* vp = vpages + base;
    const int t0 = pg * PS + key0;
    // every load of the tile is requested before any arithmetic: one memory round trip
    uint4 ku[NJ][QV];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int key = key0 + j * 8 + r;
      const bool live = t0 + j * 8 + r < t_end && t0 + j * 8 + r >= t_begin;   // (dead rows may hold anything: skip them)
#pragma unroll
      for (int v = 0; v < QV; ++v)
        ku[j][v] = live ? *reinterpret_cast<const uint4*>(kp + (size_t)key * HD + c * (HD / 4) + v * 8)
                        : make_uint4(0u, 0u, 0u, 0u);
    }
    uint4 vu[NJ / 2][4][VV];
#pragma unroll
    for (int ks = 0; ks < NJ / 2; ++ks) {
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int kin = ks * 16 + 2 * c + (q4 & 1) + (q4 >> 1) * 8;   // keys 2c, 2c+1, 2c+8, 2c+9 of the k-step
        const int t = t0 + kin;
        const bool live = t < t_end && t >= t_begin;
#pragma unroll
        for (int v = 0; v < VV; ++v)
          vu[ks][q4][v] = live ? *reinterpret_cast<const uint4*>(vp + (size_t)(key0 + kin) * HD + r * (HD / 8) + v * 8)
                               : make_uint4(0u, 0u, 0u, 0u);        // zero: its probability is zero as well
      }
    }
    // scores of head r against keys j * 8 + 2c, 2c + 1
    float s[NJ][2];
    float tmax = -INFINITY;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      s[j][0] = s[j][1] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
        const uint32_t b0 = word_of(ku[j][kk >> 1], (kk & 1) * 2);
        const uint32_t b1 = word_of(ku[j][kk >> 1], (kk & 1) * 2 + 1);
        mma_rows8(s[j][0], s[j][1], qa[kk][0], qa[kk][1], b0, b1);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int t = t0 + j * 8 + 2 * c + e;
        s[j][e] = (t < t_end && t >= t_begin) ? s[j][e] * scale : -INFINITY;
        tmax = fmaxf(tmax, s[j][e]);
      }
    }
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    const float m_new = fmaxf(m, tmax);
    const float corr = (m == -INFINITY) ? 0.f : fast_exp(m - m_new);
    m = m_new;
    l *= corr;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { o[nt][0] *= corr; o[nt][1] *= corr; }
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float pr = (s[j][e] == -INFINITY) ? 0.f : fast_exp(s[j][e] - m_new);
        s[j][e] = pr;
        l += pr;
      }
    // output: probabilities (A) times values (B)
#pragma unroll
    for (int ks = 0; ks < NJ / 2; ++ks) {
      const uint32_t a0 = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
      const uint32_t a2 = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
#pragma unroll
      for (int w = 0; w < NT / 2; ++w) {          // 32-bit word w of the lane's piece holds n-tiles 2w and 2w + 1
        const uint32_t wa = word_of(vu[ks][0][w >> 2], w & 3), wb = word_of(vu[ks][1][w >> 2], w & 3);
        const uint32_t wc = word_of(vu[ks][2][w >> 2], w & 3), wd = word_of(vu[ks][3][w >> 2], w & 3);
        mma_rows8(o[2 * w][0], o[2 * w][1], a0, a2, __byte_perm(wa, wb, 0x5410), __byte_perm(wc, wd, 0x5410));
        mma_rows8(o[2 * w + 1][0], o[2 * w + 1][1], a0, a2, __byte_perm(wa, wb, 0x7632), __byte_perm(wc, wd, 0x7632));
      }
    }
  }
}

}  // namespace dlgo
