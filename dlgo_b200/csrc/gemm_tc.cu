// bfloat16 contraction on the Blackwell tensor cores: D[Ra, Rb] = A[Ra, K] . B[Rb, K]^T with fp32
// accumulation in tensor memory.
//
// Both operands are K-major ([rows, K] row-major), which is how the reference keeps weights
// ([out x in], models/llm/model.go:64-80) and how activations are packed.  One CTA computes a
// 128 x BN tile (optionally one K-slice of it):
//   warp 0    one thread issues TMA tile loads (128-byte swizzle) into a ring of shared-memory stages
//   warp 1    allocates tensor memory; one thread issues tcgen05.mma (128 x BN x 16 per instruction) and
//             commits each stage back to the loader and the finished accumulator to the epilogue
//   warps 2-5 read the accumulator from tensor memory (each warp its own 32 lanes) and run the epilogue
// Rows and columns beyond the matrices are zero-filled by TMA on the way in and masked on the way out,
// so any Ra, Rb and any K that is a multiple of 8 are taken.
//
// Which operand is the weight is the caller's choice.  For many tokens A is the activations and the
// output is written row-major (`transposed` = 0).  For few tokens (decode) A is the WEIGHT, so its
// 128 rows fill the tensor core's M while the tokens sit in N = 16..64, and the tile is written
// transposed: out[col * ldo + row].
//
// Epilogues: store bf16, store fp32 (logits), add into an fp32 residual in place
// (models/llm/forward.go:163,169), or SwiGLU (ops/activation.go:8-38) over a weight whose rows come
// in blocks of 16 gate rows followed by their 16 up rows, writing h = silu(g) * u.
//
// Few tokens also have: partials (every K-slice leaves its fp32 tile for the reader to add) and an atomic add
// of every K-slice into an fp32 residual (no pass over partial results at all; the order of the adds,
// hence the last bits of the sum, is not fixed).
//
// Split-K (decode): `splits` CTAs share an output tile.  Each writes its fp32 partial to a
// workspace; the CTA that arrives last adds the partials in slice order (so the sum does not
// depend on which one was last) and runs the epilogue.
#include <math.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace dlgo {

using namespace sm100;

enum { TC_STORE = 0, TC_STORE_F32 = 1, TC_ADD_F32 = 2, TC_SWIGLU = 3, TC_PARTIAL = 4, TC_RED_F32 = 5, TC_ROPE_QKV = 6 };

constexpr int TILE_M = 128;
constexpr int TILE_K = 64;  // 128 bytes of bf16: one swizzle row
constexpr int UMMA_K = 16;
constexpr int TC_THREADS = 192;

__device__ int g_gemm_tc_error = 0;  // set when a bounded wait ran out

// What the q | k | v projection's epilogue needs to finish the job of the rotation kernel (models/llm/
// forward.go:246-257): rotate every q and k head at its token's position (pairs (i, i + hd/2), the whole
// head) and put k and v where the cache keeps them.  Pages of 64 positions, heads of 64 or 128.
struct TcRope {
  const float* cos_t;       // [positions][hd / 2]
  const float* sin_t;
  const int* token_pos;     // [tokens]
  const int* token_seq;     // [tokens] index of the token's sequence in the batch
  const int* seq_slot;      // [sequences]
  const int* page_table;    // [slots][max_pages]
  int max_pages;
  __nv_bfloat16* kpages;    // [pages][Hkv][64][hd]
  __nv_bfloat16* vpages;
  int Hq, Hkv, hd, write_cache;
};

struct TcParams {
  TcRope rope;        // TC_ROPE_QKV only
  int Ra, Rb, K;      // rows of A, rows of B, contraction length
  void* out;
  int ldo;
  int transposed;     // 0: out[row * ldo + col]; 1: out[col * ldo + row]
  int epilogue;
  int splits;
  float* workspace;   // [splits][tiles][BN][128] fp32, when splits > 1
  int* counters;      // [tiles], zero before the first launch; left zero
  int stages;         // shared-memory ring size
  int staged;         // many-token kernels: epilogue through shared memory and TMA stores
  int static_operand; // 0: none; 1: A, 2: B holds weights no earlier kernel writes (loaded before pdl_wait)
};

template <int BN> struct TcConfig {
  static constexpr int MAX_STAGES = BN >= 256 ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int A_BYTES = TILE_M * TILE_K * 2;
  static constexpr int B_BYTES = BN * TILE_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  static constexpr int smem_bytes(int stages) {
    return stages * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
  }
};

// silu(g) * u = g * u / (1 + exp(-g)) (models/llm/forward.go:298-303) for a result that is rounded to
// bfloat16: exp and the reciprocal as one approximate instruction each (relative error ~1e-6, far
// below the rounding).  The exact expf and division cost some thirty dependent instructions per value,
// which an epilogue with one warp per scheduler cannot hide.
__device__ __forceinline__ float silu_mul(float g, float u) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-g * 1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return g * u * r;
}

// One row's 32 consecutive columns (or 16 when NV == 16) -> memory, per epilogue.
template <int NV>
__device__ __forceinline__ void epilogue_store(const TcParams& p, const float* v, int row, int col0, int lane) {
  if (p.epilogue == TC_SWIGLU) {
    if (!p.transposed) {
      // columns are weight rows: [16 gate | 16 up] per 32 columns -> 16 outputs at column col0 / 2
      static_assert(NV == 32 || NV == 16, "");
      if (NV == 32 && row < p.Ra) {
        __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)row * p.ldo + col0 / 2;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (col0 + 16 + j < p.Rb) {
            const float g = v[j], u = v[16 + j];
            o[j] = __float2bfloat16_rn(silu_mul(g, u));
          }
        }
      }
    } else {
      // rows are weight rows: lanes 0-15 hold gate rows, lanes 16-31 their up rows
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
        const int col = col0 + j;
        if (lane < 16 && row + 16 < p.Ra && col < p.Rb) {
          const float g = v[j];
          const int feature = (row >> 5) * 16 + (row & 15);
          ((__nv_bfloat16*)p.out)[(size_t)col * p.ldo + feature] = __float2bfloat16_rn(silu_mul(g, other));
        }
      }
    }
    return;
  }
  if (!p.transposed) {
    if (row >= p.Ra) return;
    const size_t base = (size_t)row * p.ldo + col0;
    if (col0 + NV <= p.Rb && (p.ldo & 7) == 0) {
      // whole, aligned run of columns: 16-byte accesses
      if (p.epilogue == TC_STORE) {
        uint4* o = reinterpret_cast<uint4*>((__nv_bfloat16*)p.out + base);
#pragma unroll
        for (int j = 0; j < NV / 8; ++j) {
          __nv_bfloat162 h[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(v[8 * j + 2 * q], v[8 * j + 2 * q + 1]);
          o[j] = *reinterpret_cast<uint4*>(h);
        }
      } else {
        float4* o = reinterpret_cast<float4*>((float*)p.out + base);
#pragma unroll
        for (int j = 0; j < NV / 4; ++j) {
          float4 x = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          if (p.epilogue == TC_ADD_F32) {
            const float4 y = o[j];
            x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
          }
          o[j] = x;
        }
      }
      return;
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (col0 + j < p.Rb) {
        if (p.epilogue == TC_STORE) ((__nv_bfloat16*)p.out)[base + j] = __float2bfloat16_rn(v[j]);
        else if (p.epilogue == TC_STORE_F32) ((float*)p.out)[base + j] = v[j];
        else ((float*)p.out)[base + j] += v[j];
      }
    }
  } else {
    if (row >= p.Ra) return;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int col = col0 + j;
      if (col < p.Rb) {
        const size_t o = (size_t)col * p.ldo + row;
        if (p.epilogue == TC_STORE) ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v[j]);
        else if (p.epilogue == TC_STORE_F32) ((float*)p.out)[o] = v[j];
        else ((float*)p.out)[o] += v[j];
      }
    }
  }
}

template <int BN>
__device__ __forceinline__ void gemm_tc_body(const CUtensorMap& map_a, const CUtensorMap& map_b,
                                             const CUtensorMap& map_red, const TcParams& p) {
  using C = TcConfig<BN>;
  constexpr int STAGE = C::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  // tiles want 1024-byte alignment for the 128-byte swizzle
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int STAGES = p.stages;  // ring size (<= 8): as many as the K range needs, fewer to let two CTAs share an SM
  uint64_t* full = (uint64_t*)(smem + STAGES * STAGE);
  uint64_t* empty = full + STAGES;
  uint64_t* accum = empty + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(accum + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* last_flag = (int*)(tmem_slot + 2);

  pdl_launch_dependents();
  if (threadIdx.x == 0) TSTAMP(0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_a = blockIdx.x, tile_b = blockIdx.y, split = blockIdx.z;
  const int kblocks_total = (p.K + TILE_K - 1) / TILE_K;
  const int per = (kblocks_total + p.splits - 1) / p.splits;
  const int kb0 = split * per;
  const int kb1 = min(kblocks_total, kb0 + per);
  const int nkb = max(0, kb1 - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      // Weights do not depend on earlier kernels: their tiles for the first ring of stages are
      // requested before waiting for the predecessor, the activations' tiles after.
      const int npre = min(nkb, STAGES);
      const uint32_t tx = STAGE;
      for (int i = 0; i < npre; ++i) {
        uint8_t* a_dst = smem + i * STAGE;
        mbar_expect_tx(&full[i], tx);
        if (p.static_operand == 1) tma_load_2d(a_dst, &map_a, &full[i], (kb0 + i) * TILE_K, tile_a * TILE_M);
        if (p.static_operand == 2) tma_load_2d(a_dst + C::A_BYTES, &map_b, &full[i], (kb0 + i) * TILE_K, tile_b * BN);
      }
      TSTAMP(1);
      pdl_wait();
      TSTAMP(2);
      for (int i = 0; i < npre; ++i) {
        uint8_t* a_dst = smem + i * STAGE;
        if (p.static_operand != 1) tma_load_2d(a_dst, &map_a, &full[i], (kb0 + i) * TILE_K, tile_a * TILE_M);
        if (p.static_operand != 2)
          tma_load_2d(a_dst + C::A_BYTES, &map_b, &full[i], (kb0 + i) * TILE_K, tile_b * BN);
      }
      for (int i = npre; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) break;
        uint8_t* a_dst = smem + s * STAGE;
        uint8_t* b_dst = a_dst + C::A_BYTES;
        mbar_expect_tx(&full[s], tx);
        tma_load_2d(a_dst, &map_a, &full[s], (kb0 + i) * TILE_K, tile_a * TILE_M);
        tma_load_2d(b_dst, &map_b, &full[s], (kb0 + i) * TILE_K, tile_b * BN);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, BN < 16 ? 16 : BN);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&full[s], ph, abort_flag)) break;
        if (i == 0) TSTAMP(3);
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(smem + s * STAGE);
        const uint64_t da = umma_desc_k_sw128(a_addr);
        const uint64_t db = umma_desc_k_sw128(a_addr + C::A_BYTES);
#pragma unroll
        for (int k = 0; k < TILE_K / UMMA_K; ++k) {
          // inside a 128-byte swizzle row, the next K = 16 slice starts 32 bytes on (2 in 16-byte units)
          umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
        }
        umma_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
      }
      umma_commit(accum);        // the accumulator is complete
      TSTAMP(4);
    }
  } else {
    // epilogue warps: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31
    const int quarter = warp & 3;
    const int row = tile_a * TILE_M + quarter * 32 + lane;
    pdl_wait();  // the output, the workspace and the counters may still be in use by the predecessor
    bool ok = true;
    if (nkb > 0) ok = mbar_wait(accum, 0, abort_flag);
    if (warp == 2 && lane == 0) TSTAMP(5);
    tc_fence_after_sync();
    constexpr int NV = BN >= 32 ? 32 : 16;
    const int ntiles = gridDim.x * gridDim.y;
    const int tile_lin = tile_b * gridDim.x + tile_a;
    if (p.epilogue == TC_PARTIAL) {
      // every K-slice leaves its fp32 partial in out[split][col][row] (transposed tiles only); whoever
      // reads the result next adds the slices in order.  No ticket, no second pass here.
      float* dst = (float*)p.out + (size_t)split * p.Rb * p.ldo;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += NV) {
        float v[NV];
        if (ok && nkb > 0) {
          const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
          if (NV == 32) tmem_ld_32x32(taddr, v); else tmem_ld_32x16(taddr, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < NV; ++j) v[j] = 0.f;
        }
        if (row < p.Ra) {
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            const int col = tile_b * BN + c0 + j;
            if (col < p.Rb) dst[(size_t)col * p.ldo + row] = v[j];
          }
        }
      }
    } else if (p.epilogue == TC_RED_F32 && p.staged) {
      // every K-slice adds its tile into out[col][row] (fp32, transposed tiles only) with ONE bulk reduction:
      // the tile is laid out in shared memory as it lies in memory ([BN tokens][128 rows] fp32; the ring is
      // idle by now, every load of it having been consumed) and leaves as a TMA add-reduce, clipped at the
      // tensor's bounds.  One instruction in place of 128 x BN reductions of four bytes each.
      if (ok && nkb > 0) {
        float* stage = (float*)smem;
        const int r_in = quarter * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += NV) {
          float v[NV];
          const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
          if (NV == 32) tmem_ld_32x32(taddr, v); else tmem_ld_32x16(taddr, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < NV; ++j) stage[(c0 + j) * TILE_M + r_in] = v[j];
        }
        fence_proxy_async_smem();
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ok && nkb > 0 && warp == 2 && lane == 0) {
        tma_reduce_add_2d(&map_red, smem, tile_a * TILE_M, tile_b * BN);
        tma_store_commit();
        tma_store_wait_all();
      }
    } else if (p.epilogue == TC_RED_F32) {
      // (without a tensor map of the target: a reduction at the memory per element)
      float* dst = (float*)p.out;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += NV) {
        if (!(ok && nkb > 0)) break;
        float v[NV];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
        if (NV == 32) tmem_ld_32x32(taddr, v); else tmem_ld_32x16(taddr, v);
        tmem_ld_wait();
        if (row < p.Ra) {
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            const int col = tile_b * BN + c0 + j;
            if (col < p.Rb) atomicAdd(dst + (size_t)col * p.ldo + row, v[j]);
          }
        }
      }
    } else if (p.splits == 1 && p.epilogue == TC_SWIGLU && p.transposed && BN >= 32 && (p.ldo & 1) == 0) {
      // Many tokens per tile: the 64 outputs of a token (silu(gate) * up of this tile's 128 weight
      // rows) are gathered in shared memory (the ring is idle by now) and leave as one 128-byte row
      // per token, instead of 32 bytes per warp and token.
      __nv_bfloat16* stage = (__nv_bfloat16*)smem;                 // [BN tokens][64 outputs]
      if (ok) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += NV) {
          float v[NV];
          const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
          if (NV == 32) tmem_ld_32x32(taddr, v); else tmem_ld_32x16(taddr, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
            if (lane < 16) stage[(c0 + j) * 64 + quarter * 16 + lane] = __float2bfloat16_rn(silu_mul(v[j], other));
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ok) {
        const int feat0 = tile_a * 64 + 2 * lane;                  // this lane's two outputs of a token
        const int n_feat = p.Ra / 2;
        for (int c = quarter; c < BN; c += 4) {
          const int col = tile_b * BN + c;
          if (col >= p.Rb) break;
          __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)col * p.ldo + feat0;
          if (feat0 + 1 < n_feat) *reinterpret_cast<uint32_t*>(o) = *reinterpret_cast<const uint32_t*>(&stage[c * 64 + 2 * lane]);
          else if (feat0 < n_feat) o[0] = stage[c * 64 + 2 * lane];
        }
      }
    } else if (p.splits == 1) {
      if (ok) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += NV) {
          float v[NV];
          const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
          if (NV == 32) tmem_ld_32x32(taddr, v); else tmem_ld_32x16(taddr, v);
          tmem_ld_wait();
          epilogue_store<NV>(p, v, row, tile_b * BN + c0, lane);
        }
      }
    } else {
      // partial tile -> workspace [split][tile][col][128 rows] (rows innermost: coalesced)
      float* ws = p.workspace + ((size_t)split * ntiles + tile_lin) * (size_t)(BN * TILE_M);
      const int r_in = quarter * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += NV) {
        float v[NV];
        if (ok && nkb > 0) {
          const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
          if (NV == 32) tmem_ld_32x32(taddr, v); else tmem_ld_32x16(taddr, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < NV; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) ws[(size_t)(c0 + j) * TILE_M + r_in] = v[j];
      }
      __threadfence();
      // the 128 epilogue threads meet, one of them takes a ticket
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        const int ticket = atomicAdd(&p.counters[tile_lin], 1);
        *last_flag = (ticket == p.splits - 1);
        if (ticket == p.splits - 1) p.counters[tile_lin] = 0;  // ready for the next launch
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*last_flag && ok) {
        __threadfence();
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += NV) {
          float v[NV];
#pragma unroll
          for (int j = 0; j < NV; ++j) v[j] = 0.f;
          // partials are added in slice order (the sum does not depend on which CTA came last), but
          // four slices' loads are in flight at a time so the L2 round trips overlap
          const size_t stride = (size_t)ntiles * (size_t)(BN * TILE_M);
          const float* src0 = p.workspace + (size_t)tile_lin * (size_t)(BN * TILE_M) + (size_t)c0 * TILE_M + r_in;
          int s = 0;
          for (; s + 4 <= p.splits; s += 4) {
            float t0[NV], t1[NV], t2[NV], t3[NV];
#pragma unroll
            for (int j = 0; j < NV; ++j) {
              t0[j] = __ldcg(src0 + (size_t)(s + 0) * stride + (size_t)j * TILE_M);
              t1[j] = __ldcg(src0 + (size_t)(s + 1) * stride + (size_t)j * TILE_M);
              t2[j] = __ldcg(src0 + (size_t)(s + 2) * stride + (size_t)j * TILE_M);
              t3[j] = __ldcg(src0 + (size_t)(s + 3) * stride + (size_t)j * TILE_M);
            }
#pragma unroll
            for (int j = 0; j < NV; ++j) v[j] = (((v[j] + t0[j]) + t1[j]) + t2[j]) + t3[j];
          }
          for (; s < p.splits; ++s) {
#pragma unroll
            for (int j = 0; j < NV; ++j) v[j] += __ldcg(src0 + (size_t)s * stride + (size_t)j * TILE_M);
          }
          epilogue_store<NV>(p, v, row, tile_b * BN + c0, lane);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) TSTAMP(6);
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(&g_gemm_tc_error, 1);
    // give tile loads that may still be in flight time to land before shared memory is handed on
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_red, const __grid_constant__ TcParams p) {
  gemm_tc_body<BN>(map_a, map_b, map_red, p);
}

// Epilogue of the many-token kernels: one accumulator tile (128 rows x BN fp32 columns in tensor
// memory) goes through two 16 KB staging buffers in shared memory, 128 bytes per row in the
// 128-byte swizzle, and from there to global memory with TMA: a tile store (bf16, fp32, SwiGLU) or
// an fp32 add-reduce for the residual (the residual is never read by the SM).  Rows are written
// whole and coalesced, and rows or columns beyond the matrix are clipped by the tensor map.
// Called by the 128 epilogue threads together; `chunk` counts staging buffers used so far.
constexpr int STAGING_BYTES = 2 * 16384;

// 32 accumulator columns of a row as bfloat16 into four 16-byte pieces of a swizzled 128-byte staging row
__device__ __forceinline__ void stage_bf16_32(uint8_t* row, int r, int first_piece, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 b2[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) b2[q] = __floats2bfloat162_rn(v[8 * j + 2 * q], v[8 * j + 2 * q + 1]);
    *reinterpret_cast<uint4*>(row + (((first_piece + j) ^ (r & 7)) << 4)) = *reinterpret_cast<uint4*>(b2);
  }
}
// ... and straight to memory (16-byte aligned)
__device__ __forceinline__ void store_bf16_32(__nv_bfloat16* dst, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 b2[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) b2[q] = __floats2bfloat162_rn(v[8 * j + 2 * q], v[8 * j + 2 * q + 1]);
    *reinterpret_cast<uint4*>(dst + 8 * j) = *reinterpret_cast<uint4*>(b2);
  }
}

// The epilogue of the q | k | v projection of a prompt step: a head at a time (64 or 128 accumulator columns of
// the thread's token), q and k heads rotated in fp32 and rounded once; q goes to the output through the staging
// buffers and TMA stores as TC_STORE does, k and v go straight to the token's row of its cache page.
// What a thread of the rotating epilogue knows about its token before the accumulator is ready: where its k and
// v rows go and, for heads of 64, the token's 32 cosines and 32 sines (they stay in registers for all heads of
// the tile: beside a ring of 200 KB the SM's L1 holds 28 KB, so re-read per head they would come from L2 every
// time).  Fetched while the tile's MMAs still run.
struct RopeRow {
  const float* cs;
  const float* sn;
  __nv_bfloat16* krow;
  __nv_bfloat16* vrow;
  float4 c4[8], s4[8];
  bool table_held;
};

__device__ __forceinline__ void rope_prepare(const TcParams& p, int row0, int r, RopeRow& rr) {
  const TcRope& R = p.rope;
  const int hd = R.hd, half = hd >> 1;
  const int t = row0 + r;
  const bool live = t < p.Ra;
  const int pos = live ? R.token_pos[t] : 0;
  rr.cs = R.cos_t + (size_t)pos * half;
  rr.sn = R.sin_t + (size_t)pos * half;
  rr.krow = rr.vrow = nullptr;
  rr.table_held = half == 32;
  if (rr.table_held) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      rr.c4[i] = __ldg(reinterpret_cast<const float4*>(rr.cs) + i);
      rr.s4[i] = __ldg(reinterpret_cast<const float4*>(rr.sn) + i);
    }
  }
  if (live && R.write_cache) {
    const int slot = R.seq_slot[R.token_seq[t]];
    const int page = R.page_table[(size_t)slot * R.max_pages + (pos >> 6)];
    if (page >= 0) {
      const size_t base = ((size_t)page * R.Hkv * 64 + (size_t)(pos & 63)) * hd;
      rr.krow = R.kpages + base;
      rr.vrow = R.vpages + base;
    } else {
      atomicExch(&g_gemm_tc_error, 1);        // a page that was never reserved: nothing is written
    }
  }
}

template <int BN>
__device__ __forceinline__ void rope_qkv_epilogue(const TcParams& p, const CUtensorMap* map_out, uint8_t* staging,
                                                  uint32_t lane_addr, int row0, int col0, int r, bool issuer,
                                                  int& chunk, RopeRow& rr) {
  const TcRope& R = p.rope;
  const int hd = R.hd, half = hd >> 1;
  const float* cs = rr.cs;
  const float* sn = rr.sn;
  __nv_bfloat16* krow = rr.krow;
  __nv_bfloat16* vrow = rr.vrow;
  float4 (&c4)[8] = rr.c4;
  float4 (&s4)[8] = rr.s4;
  const bool table_held = rr.table_held;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += hd) {
    const int head = (col0 + c0) / hd;                       // the same for the whole CTA
    if (head >= R.Hq + 2 * R.Hkv) break;                     // (columns beyond the projection's rows)
    const bool is_q = head < R.Hq, is_k = !is_q && head < R.Hq + R.Hkv;
    const int bufs = hd >> 6;                                // staging buffers a q head takes: 64 columns each
    if (is_q) {
      if (issuer) { if (bufs == 2) tma_store_wait_read<0>(); else tma_store_wait_read<1>(); }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const int kvh = is_k ? head - R.Hq : head - R.Hq - R.Hkv;
    __nv_bfloat16* dst = is_q ? nullptr : ((is_k ? krow : vrow) == nullptr ? nullptr
                                           : (is_k ? krow : vrow) + (size_t)kvh * 64 * hd);
#pragma unroll 1
    for (int g = 0; g < half; g += 32) {
      // dimensions [g, g + 32) and their partners [g + half, g + half + 32); the 16 loads of the token's
      // cosines and sines are all on their way before anything waits for one (one round trip, not eight)
      if (!table_held && (is_q || is_k)) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          c4[i] = __ldg(reinterpret_cast<const float4*>(cs + g) + i);
          s4[i] = __ldg(reinterpret_cast<const float4*>(sn + g) + i);
        }
      }
      float a[32], b[32];
      tmem_ld_32x32(lane_addr + c0 + g, a);
      tmem_ld_32x32(lane_addr + c0 + half + g, b);
      tmem_ld_wait();
      if (is_q || is_k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float cc[4] = {c4[i].x, c4[i].y, c4[i].z, c4[i].w}, ss[4] = {s4[i].x, s4[i].y, s4[i].z, s4[i].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float x0 = a[4 * i + e], x1 = b[4 * i + e];
            a[4 * i + e] = x0 * cc[e] - x1 * ss[e];
            b[4 * i + e] = x0 * ss[e] + x1 * cc[e];
          }
        }
      }
      if (is_q) {
        // column c of the head lies in staging buffer c / 64, 16-byte piece (c % 64) / 8
        uint8_t* b0 = staging + ((chunk + (g >> 6)) & 1) * 16384 + r * 128;
        uint8_t* b1 = staging + ((chunk + ((half + g) >> 6)) & 1) * 16384 + r * 128;
        stage_bf16_32(b0, r, (g & 63) >> 3, a);
        stage_bf16_32(b1, r, ((half + g) & 63) >> 3, b);
      } else if (dst != nullptr) {
        store_bf16_32(dst + g, a);
        store_bf16_32(dst + half + g, b);
      }
    }
    if (is_q) {
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (issuer) {
        for (int j = 0; j < bufs; ++j)
          tma_store_2d(map_out, staging + ((chunk + j) & 1) * 16384, col0 + c0 + 64 * j, row0);
        tma_store_commit();
      }
      chunk += bufs;
    }
  }
}

template <int BN>
__device__ __forceinline__ void staged_epilogue(const TcParams& p, const CUtensorMap* map_out, uint8_t* staging,
                                                uint32_t acc_addr, int row0, int col0, int quarter, int lane,
                                                bool issuer, int& chunk, RopeRow* rope_row = nullptr) {
  const int r = quarter * 32 + lane;
  const uint32_t lane_addr = acc_addr + ((uint32_t)(quarter * 32) << 16);
  if (p.epilogue == TC_ROPE_QKV) {
    rope_qkv_epilogue<BN>(p, map_out, staging, lane_addr, row0, col0, r, issuer, chunk, *rope_row);
    return;
  }
  // accumulator columns that make one 128-byte output row chunk
  const int step = p.epilogue == TC_STORE ? 64 : (p.epilogue == TC_SWIGLU ? 128 : 32);
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += step, ++chunk) {
    uint8_t* buf = staging + (chunk & 1) * 16384;
    if (issuer) tma_store_wait_read<1>();     // the store that last used this buffer has read it
    asm volatile("bar.sync 1, 128;" ::: "memory");
    uint8_t* row = buf + r * 128;
    if (p.epilogue == TC_STORE) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v[32];
        tmem_ld_32x32(lane_addr + c0 + 32 * h, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 b2[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) b2[q] = __floats2bfloat162_rn(v[8 * j + 2 * q], v[8 * j + 2 * q + 1]);
          *reinterpret_cast<uint4*>(row + (((4 * h + j) ^ (r & 7)) << 4)) = *reinterpret_cast<uint4*>(b2);
        }
      }
    } else if (p.epilogue == TC_SWIGLU) {
      // per 32 accumulator columns: 16 gate values then their 16 up values -> 16 outputs
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        float v[32];
        tmem_ld_32x32(lane_addr + c0 + 32 * h, v);
        tmem_ld_wait();
        __nv_bfloat162 b2[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float g0 = v[2 * q], g1 = v[2 * q + 1], u0 = v[16 + 2 * q], u1 = v[16 + 2 * q + 1];
          b2[q] = __floats2bfloat162_rn(silu_mul(g0, u0), silu_mul(g1, u1));
        }
        *reinterpret_cast<uint4*>(row + (((2 * h) ^ (r & 7)) << 4)) = *reinterpret_cast<uint4*>(&b2[0]);
        *reinterpret_cast<uint4*>(row + (((2 * h + 1) ^ (r & 7)) << 4)) = *reinterpret_cast<uint4*>(&b2[4]);
      }
    } else {
      float v[32];
      tmem_ld_32x32(lane_addr + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float4*>(row + ((j ^ (r & 7)) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (issuer) {
      const int x = p.epilogue == TC_SWIGLU ? (col0 + c0) / 2 : col0 + c0;
      if (p.epilogue == TC_ADD_F32) tma_reduce_add_2d(map_out, buf, x, row0);
      else tma_store_2d(map_out, buf, x, row0);
      tma_store_commit();
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Many tokens: one persistent CTA per SM walks over output tiles.  Two accumulators live in tensor
// memory (2 x BN columns), so the epilogue of tile i (tensor memory -> registers -> global) runs
// while the tensor core already works on tile i+1; the shared-memory ring keeps streaming across
// tile boundaries.  Tiles are taken in an order that keeps the CTAs running at the same time on
// the same few weight tiles (all row tiles of one column tile are neighbours), so the weights are
// read from L2.
template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          const __grid_constant__ CUtensorMap map_out, TcParams p) {
  using C = TcConfig<BN>;
  const int STAGES = p.stages;
  constexpr uint32_t TMEM_COLS = 2 * C::TMEM_COLS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + STAGES * C::STAGE_BYTES;
  uint64_t* full = (uint64_t*)(staging + STAGING_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;     // 2
  uint64_t* acc_empty = acc_full + 2;      // 2
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_a = (p.Ra + TILE_M - 1) / TILE_M, tiles_b = (p.Rb + BN - 1) / BN;
  const int n_tiles = tiles_a * tiles_b;
  const int nkb = (p.K + TILE_K - 1) / TILE_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      pdl_wait();
      int it = 0;  // K blocks issued so far, over all tiles
      for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const int tile_a = t % tiles_a, tile_b = t / tiles_a;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { t = n_tiles; break; }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          mbar_expect_tx(&full[s], C::STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, &full[s], kb * TILE_K, tile_a * TILE_M);
          tma_load_2d(a_dst + C::A_BYTES, &map_b, &full[s], kb * TILE_K, tile_b * BN);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, BN);
      int it = 0, local = 0;
      for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++local) {
        const int buf = local & 1;
        // the epilogue must have emptied this accumulator (two tiles ago)
        if (local >= 2 && !mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * C::TMEM_COLS;
        bool ok = true;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full[s], (it / STAGES) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint64_t da = umma_desc_k_sw128(a_addr);
          const uint64_t db = umma_desc_k_sw128(a_addr + C::A_BYTES);
#pragma unroll
          for (int k = 0; k < TILE_K / UMMA_K; ++k) umma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          umma_commit(&empty[s]);
        }
        umma_commit(&acc_full[buf]);
        if (!ok) break;
      }
    }
  } else {
    const int quarter = warp & 3;
    const bool issuer = warp == 2 && lane == 0;
    const bool staged = p.staged != 0;
    pdl_wait();
    constexpr int NV = 32;
    int local = 0, chunk = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++local) {
      const int tile_a = t % tiles_a, tile_b = t / tiles_a;
      const int buf = local & 1;
      const int row = tile_a * TILE_M + quarter * 32 + lane;
      RopeRow rope_row;
      if (p.epilogue == TC_ROPE_QKV) rope_prepare(p, tile_a * TILE_M, quarter * 32 + lane, rope_row);
      if (!mbar_wait(&acc_full[buf], (local >> 1) & 1, abort_flag)) break;
      tc_fence_after_sync();
      if (staged) {
        staged_epilogue<BN>(p, &map_out, staging, tmem_base + buf * C::TMEM_COLS, tile_a * TILE_M, tile_b * BN, quarter,
                            lane, issuer, chunk, &rope_row);
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += NV) {
          float v[NV];
          tmem_ld_32x32(tmem_base + buf * C::TMEM_COLS + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
          tmem_ld_wait();
          epilogue_store<NV>(p, v, row, tile_b * BN + c0, lane);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[buf]);
    }
    if (issuer) tma_store_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(&g_gemm_tc_error, 1);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// Many tokens, CTA pairs: two CTAs of a cluster share one 256 x BN tile through cta_group::2.  Each
// CTA loads 128 rows of A and HALF of the tile's B rows; the leader's MMAs read both halves from both
// CTAs' shared memory and write 128 accumulator rows into each CTA's tensor memory.  Per CTA and
// K block that is 16 KB + BN/2 x 128 B of shared-memory fill for the work a single CTA would need
// 16 KB + BN x 128 B for, which is what lets the tensor pipe run near its peak.  Persistent, two
// accumulators per CTA, no multicast loads (each CTA fetches its own halves).
template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_out, TcParams p) {
  constexpr int HALF_N = BN / 2;
  constexpr int A_BYTES = TILE_M * TILE_K * 2;
  constexpr int B_BYTES = HALF_N * TILE_K * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t ACC_COLS = BN;                 // fp32 columns of one accumulator
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;      // 512 for BN = 256, 256 for BN = 128
  const int STAGES = p.stages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + STAGES * STAGE_BYTES;
  uint64_t* full = (uint64_t*)(staging + STAGING_BYTES);       // used in the leader only
  uint64_t* empty = full + STAGES;                             // local in each CTA
  uint64_t* acc_full = empty + STAGES;                         // 2, local in each CTA
  uint64_t* acc_empty = acc_full + 2;                          // 2, used in the leader only (256 arrivals)
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_a = (p.Ra + 2 * TILE_M - 1) / (2 * TILE_M), tiles_b = (p.Rb + BN - 1) / BN;
  const int n_tiles = tiles_a * tiles_b;
  const int nkb = (p.K + TILE_K - 1) / TILE_K;
  // K-slices (add-reduce epilogue only: every slice adds its tile into the target by TMA): unit u is tile
  // u % n_tiles, K blocks [(u / n_tiles) * kper, ...)
  const int ksplits = p.splits > 1 ? p.splits : 1;
  const int kper = (nkb + ksplits - 1) / ksplits;
  const int n_units = n_tiles * ksplits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 256);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers exist before anything arrives on them remotely
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      pdl_wait();
      int it = 0;
      for (int u = pair; u < n_units; u += n_pairs) {
        const int t = u % n_tiles;
        const int tile_a = t % tiles_a, tile_b = t / tiles_a;
        const int kb0 = (u / n_tiles) * kper, kb1 = min(nkb, kb0 + kper);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { u = n_units; break; }
          uint8_t* a_dst = smem + s * STAGE_BYTES;
          // the leader's barrier counts the bytes of both CTAs' loads
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
          tma_load_2d_pair(a_dst, &map_a, bar, kb * TILE_K, tile_a * 2 * TILE_M + (int)rank * TILE_M);
          tma_load_2d_pair(a_dst + A_BYTES, &map_b, bar, kb * TILE_K, tile_b * BN + (int)rank * HALF_N);
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * TILE_M, BN);
      int it = 0, local = 0;
      for (int u = pair; u < n_units; u += n_pairs, ++local) {
        const int buf = local & 1;
        if (local >= 2 && !mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
        bool ok = true;
        const int kb0 = (u / n_tiles) * kper, kb1 = min(nkb, kb0 + kper);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full[s], (it / STAGES) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = umma_desc_k_sw128(a_addr);
          const uint64_t db = umma_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < TILE_K / UMMA_K; ++k)
            umma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0) || (k != 0));
          umma_commit_pair(&empty[s]);     // both CTAs may refill the stage
        }
        umma_commit_pair(&acc_full[buf]);  // both CTAs' epilogues may read the accumulator
        if (!ok) break;
      }
    }
  } else {
    const int quarter = warp & 3;
    const bool issuer = warp == 2 && lane == 0;
    const bool staged = p.staged != 0;
    pdl_wait();
    constexpr int NV = 32;
    int local = 0, chunk = 0;
    for (int u = pair; u < n_units; u += n_pairs, ++local) {
      const int t = u % n_tiles;
      const int tile_a = t % tiles_a, tile_b = t / tiles_a;
      const int buf = local & 1;
      const int row0 = tile_a * 2 * TILE_M + (int)rank * TILE_M;
      const int row = row0 + quarter * 32 + lane;
      RopeRow rope_row;               // (fetched while the tile's MMAs still run)
      if (p.epilogue == TC_ROPE_QKV) rope_prepare(p, row0, quarter * 32 + lane, rope_row);
      if (!mbar_wait(&acc_full[buf], (local >> 1) & 1, abort_flag)) break;
      tc_fence_after_sync();
      if (staged) {
        staged_epilogue<BN>(p, &map_out, staging, tmem_base + buf * ACC_COLS, row0, tile_b * BN, quarter, lane, issuer,
                            chunk, &rope_row);
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += NV) {
          float v[NV];
          tmem_ld_32x32(tmem_base + buf * ACC_COLS + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
          tmem_ld_wait();
          epilogue_store<NV>(p, v, row, tile_b * BN + c0, lane);
        }
      }
      tc_fence_before_sync();
      mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
    }
    if (issuer) tma_store_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();          // nobody leaves while the other CTA may still signal or be read
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(&g_gemm_tc_error, 1);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
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
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// [rows, K] bf16, row stride ld elements; box = 64 columns x box_rows rows, 128-byte swizzle, zero fill
int make_map(CUtensorMap* m, const void* base, int rows, int K, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return DLGO_ERR_DRIVER;
  if (((uintptr_t)base & 15) != 0 || (ld % 8) != 0) return DLGO_ERR_ALIGN;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DLGO_OK : DLGO_ERR_DRIVER;
}

// Output tensor map of the staged epilogue: rows of 128 bytes (64 bf16 or 32 fp32), 128 rows, swizzled.
// Returns DLGO_ERR_ALIGN where the output cannot be described (then the direct epilogue is used).
int make_out_map(CUtensorMap* m, const TcParams& p) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return DLGO_ERR_DRIVER;
  const bool bf16 = p.epilogue == TC_STORE || p.epilogue == TC_SWIGLU || p.epilogue == TC_ROPE_QKV;
  const int esize = bf16 ? 2 : 4;
  const long long cols = p.epilogue == TC_SWIGLU ? p.Rb / 2 : p.Rb;
  if (((uintptr_t)p.out & 15) != 0 || ((long long)p.ldo * esize) % 16 != 0) return DLGO_ERR_ALIGN;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)p.Ra};
  cuuint64_t strides[1] = {(cuuint64_t)p.ldo * esize};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esize), (cuuint32_t)TILE_M};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, p.out, dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DLGO_OK : DLGO_ERR_DRIVER;
}

// Tensor map of a transposed fp32 target out[Rb][ldo] for the few-token kernel's add-reduce: boxes of 128
// rows (inner) x bn tokens, no swizzle.  DLGO_ERR_ALIGN where TMA cannot describe it.
int make_red_map(CUtensorMap* m, void* out, int Ra, int Rb, int ldo, int bn) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return DLGO_ERR_DRIVER;
  if (((uintptr_t)out & 15) != 0 || (ldo % 4) != 0) return DLGO_ERR_ALIGN;
  cuuint64_t dims[2] = {(cuuint64_t)Ra, (cuuint64_t)Rb};
  cuuint64_t strides[1] = {(cuuint64_t)ldo * 4};
  cuuint32_t box[2] = {(cuuint32_t)TILE_M, (cuuint32_t)bn};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DLGO_OK : DLGO_ERR_DRIVER;
}

template <int BN>
int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, cudaStream_t stream) {
  using C = TcConfig<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::smem_bytes(C::MAX_STAGES));
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((p.Ra + TILE_M - 1) / TILE_M, (p.Rb + BN - 1) / BN, p.splits);
  if (grid.y > 65535 || grid.z > 65535) return DLGO_ERR_SIZE;
  TcParams q = p;
  const int kblocks = (p.K + TILE_K - 1) / TILE_K;
  const int per_split = (kblocks + p.splits - 1) / p.splits;
  int stages = C::MAX_STAGES;
  if (p.transposed) {
    // few tokens: keep the footprint under half an SM so that two CTAs (of this kernel or of the next
    // one, launched early) share it and one's start-up hides behind the other's streaming
    // (more than 16 tokens: one CTA per SM, and the whole of shared memory for its ring: 1.205 -> 1.190 ms a step
    // at batch 64, 0.950 -> 0.946 at batch 32 at Llama 3.2 1B sizes; at batch 8 the deep ring costs 10 %)
    static const int ring_kb = [] { const char* e = getenv("DLGO_TC_RING_KB"); return e ? atoi(e) : 110; }();
    static const int ring_kb_wide = [] { const char* e = getenv("DLGO_TC_RING_KB_WIDE"); return e ? atoi(e) : 200; }();
    const int kb = BN >= 32 ? ring_kb_wide : ring_kb;
    while (stages > 2 && C::smem_bytes(stages) > kb * 1024) --stages;
  }
  if (stages > per_split) stages = per_split < 2 ? 2 : per_split;
  q.stages = stages;
  q.staged = 0;
  CUtensorMap mr = ma;   // a valid map even when unused
  if (p.epilogue == TC_RED_F32 && BN >= 32 && BN <= 64 && stages * C::STAGE_BYTES >= BN * TILE_M * 4) {
    // more than 16 tokens: the add-reduce as one TMA instruction per tile instead of 128 x BN reductions of
    // four bytes.  Measured on a B200 (Llama 3.2 1B sizes, ms a step): 1.209 against 1.300 at batch 64, 0.949
    // against 0.993 at batch 32; at batch 8 the detour through shared memory costs more than the 1,024
    // reductions it saves (0.775 against 0.763).  DLGO_TC_RED_TMA=0 switches it off.
    static const bool use_tma = [] { const char* e = getenv("DLGO_TC_RED_TMA"); return e == nullptr || e[0] != '0'; }();
    if (use_tma && make_red_map(&mr, p.out, p.Ra, p.Rb, p.ldo, BN) == DLGO_OK) q.staged = 1;
  }
  launch_kernel(gemm_tc_kernel<BN>, dim3(grid), dim3(TC_THREADS), C::smem_bytes(stages), stream, ma, mb, mr, q);
  return launch_status();
}

template <int BN>
int launch_tc_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, cudaStream_t stream) {
  using C = TcConfig<BN>;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::smem_bytes(C::MAX_STAGES) + STAGING_BYTES);
    if (e != cudaSuccess) { sms = 0; return (int)e; }
  }
  const int tiles = ((p.Ra + TILE_M - 1) / TILE_M) * ((p.Rb + BN - 1) / BN);
  TcParams q = p;
  // one CTA per SM with as deep a ring as shared memory allows beside the epilogue's staging buffers
  int ctas_per_sm = 1;
  q.stages = C::MAX_STAGES;
  const int slots = sms * ctas_per_sm;
  CUtensorMap mo = ma;   // a valid map even when unused
  q.staged = (getenv("DLGO_TC_DIRECT_EPILOGUE") == nullptr && make_out_map(&mo, q) == DLGO_OK) ? 1 : 0;
  launch_kernel(gemm_tc_persistent_kernel<BN>, dim3(tiles < slots ? tiles : slots), dim3(TC_THREADS),
                C::smem_bytes(q.stages) + STAGING_BYTES, stream, ma, mb, mo, q);
  return launch_status();
}

template <int BN>
int launch_tc_pair(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, cudaStream_t stream) {
  constexpr int STAGE_BYTES = TILE_M * TILE_K * 2 + (BN / 2) * TILE_K * 2;
  constexpr int STAGES = BN >= 256 ? 6 : 8;
  constexpr int SMEM = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 + 256;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) { sms = 0; return (int)e; }
  }
  const int tiles = ((p.Ra + 2 * TILE_M - 1) / (2 * TILE_M)) * ((p.Rb + BN - 1) / BN);
  int pairs = sms / 2;
  TcParams q = p;
  q.stages = STAGES;
  CUtensorMap mo = ma;
  q.staged = (getenv("DLGO_TC_DIRECT_EPILOGUE") == nullptr && make_out_map(&mo, q) == DLGO_OK) ? 1 : 0;
  // Fewer tiles than CTA pairs (prompts of a few hundred tokens against a long K): a product whose epilogue
  // adds into its target by TMA reduction is cut into K-slices, so that every pair works; each slice adds its
  // own tile.  Slices of at least 8 K blocks.
  q.splits = 1;
  if (q.staged && p.epilogue == TC_ADD_F32 && tiles < pairs) {
    const int kblocks = (p.K + TILE_K - 1) / TILE_K;
    int ks = pairs / tiles;
    if (ks > kblocks / 8) ks = kblocks / 8;
    if (ks > 1) {
      const int per = (kblocks + ks - 1) / ks;
      q.splits = (kblocks + per - 1) / per;      // no empty slices
    }
  } else if (q.staged && p.epilogue == TC_ADD_F32) {
    // A few more tiles than pairs (96 tiles are two rounds of 74 pairs, the second a third full): K-slices
    // where they shorten the rounds by more than their extra epilogues cost (a tenth of a tile's time each).
    static const int max_ks = [] { const char* e = getenv("DLGO_TC_PAIR_KSPLIT_MAX"); return e ? atoi(e) : 4; }();
    const int kblocks = (p.K + TILE_K - 1) / TILE_K;
    float best = (float)((tiles + pairs - 1) / pairs);
    int best_ks = 1;
    for (int ks = 2; ks <= max_ks && ks <= kblocks / 8; ++ks) {
      const float cost = (float)((tiles * ks + pairs - 1) / pairs) / ks * (1.0f + 0.1f * (ks - 1) * 32.0f / kblocks);
      if (cost < 0.9f * best) { best = cost; best_ks = ks; }
    }
    if (best_ks > 1) {
      const int per = (kblocks + best_ks - 1) / best_ks;
      q.splits = (kblocks + per - 1) / per;
    }
  }
  if (tiles * q.splits < pairs) pairs = tiles * q.splits;
  launch_kernel_cluster(gemm_tc_pair_kernel<BN>, dim3(2 * pairs), dim3(TC_THREADS), SMEM, stream, dim3(2, 1, 1), ma, mb,
                        mo, q);
  return launch_status();
}

}  // namespace

// Floats of workspace and ints of counters a call with `splits` > 1 needs.
DLGO_EXPORT long long dlgo_gemm_tc_workspace_floats(int Ra, int Rb, int bn, int splits) {
  if (splits <= 1) return 0;
  const long long tiles = (long long)((Ra + TILE_M - 1) / TILE_M) * ((Rb + bn - 1) / bn);
  return tiles * splits * bn * TILE_M;
}
DLGO_EXPORT int dlgo_gemm_tc_tiles(int Ra, int Rb, int bn) {
  return ((Ra + TILE_M - 1) / TILE_M) * ((Rb + bn - 1) / bn);
}

// A[Ra, K] (row stride lda) and B[Rb, K] (row stride ldb) in bf16; out per `transposed` and `epilogue`
// (0 store bf16, 1 store f32, 2 add into f32, 3 SwiGLU to bf16, 4 partials: out is fp32
// [splits][Rb][ldo] and slice s writes out[s][col][row], transposed only; 5 every K-slice adds itself into
// f32 out atomically, transposed only, no workspace); bn in {16, 32, 64, 128, 256}.
// static_operand: 1 if A, 2 if B holds weights that no kernel launched before this one writes (their
// tiles are then requested before the kernel waits for its predecessor), else 0.
// pair_tile: 0, or 128 / 256 to compute 256 x pair_tile tiles with pairs of CTAs (cta_group::2; many
// tokens only: not transposed, one K-slice; bn is then ignored).
DLGO_EXPORT int dlgo_gemm_tc(const void* A, int Ra, int lda, const void* B, int Rb, int ldb, int K, void* out,
                             int ldo, int transposed, int epilogue, int bn, int splits, float* workspace,
                             int* counters, int static_operand, int pair_tile, cudaStream_t stream) {
  if (Ra <= 0 || Rb <= 0) return DLGO_OK;
  if (K <= 0 || K % 8 || lda < K || ldb < K || splits < 1) return DLGO_ERR_SIZE;
  if (epilogue < 0 || epilogue > 5) return DLGO_ERR_SIZE;
  if (splits > (K + TILE_K - 1) / TILE_K) return DLGO_ERR_SIZE;
  if ((epilogue == TC_PARTIAL || epilogue == TC_RED_F32) && !transposed) return DLGO_ERR_SIZE;
  if (splits > 1 && epilogue != TC_PARTIAL && epilogue != TC_RED_F32 &&
      (workspace == nullptr || counters == nullptr))
    return DLGO_ERR_SIZE;
  if (epilogue == TC_SWIGLU) {
    const int weight_rows = transposed ? Ra : Rb;
    if (weight_rows % 32 || (!transposed && bn < 32)) return DLGO_ERR_SIZE;
  }
  CUtensorMap ma, mb;
  int st = make_map(&ma, A, Ra, K, lda, TILE_M);
  if (st != DLGO_OK) return st;
  st = make_map(&mb, B, Rb, K, ldb, bn);
  if (st != DLGO_OK) return st;
  TcParams p = {};
  p.Ra = Ra; p.Rb = Rb; p.K = K; p.out = out; p.ldo = ldo; p.transposed = transposed; p.epilogue = epilogue;
  p.splits = splits; p.workspace = workspace; p.counters = counters;
  p.static_operand = (static_operand == 1 || static_operand == 2) ? static_operand : 0;
  if (!transposed && splits == 1 && pair_tile != 0) {
    // many tokens, CTA pairs: A's box is 128 rows, B's box is half the tile's width
    if (pair_tile != 128 && pair_tile != 256) return DLGO_ERR_SIZE;
    st = make_map(&mb, B, Rb, K, ldb, pair_tile / 2);
    if (st != DLGO_OK) return st;
    return pair_tile == 256 ? launch_tc_pair<256>(ma, mb, p, stream) : launch_tc_pair<128>(ma, mb, p, stream);
  }
  if (!transposed && splits == 1 && (bn == 128 || bn == 256)) {
    // many tokens: persistent CTAs with two accumulators in tensor memory
    return bn == 256 ? launch_tc_persistent<256>(ma, mb, p, stream) : launch_tc_persistent<128>(ma, mb, p, stream);
  }
  switch (bn) {
    case 16: return launch_tc<16>(ma, mb, p, stream);
    case 32: return launch_tc<32>(ma, mb, p, stream);
    case 64: return launch_tc<64>(ma, mb, p, stream);
    case 128: return launch_tc<128>(ma, mb, p, stream);
    case 256: return launch_tc<256>(ma, mb, p, stream);
    default: return DLGO_ERR_SIZE;
  }
}

// The q | k | v projection of a prompt step with the rotation and the cache append in its epilogue:
// qkv[T, Rb] (bf16, row stride ldo) receives the rotated q heads (its k and v columns are left alone), the
// rotated k heads and the v heads go to their tokens' rows of the pages [pages][Hkv][64][hd].  x[T, K] and
// w[Rb, K] bf16 with Rb = (Hq + 2 Hkv) * hd; hd 64 or 128, whole-head rotation in the split-half pairing,
// cos / sin tables [positions][hd / 2]; pages of 64 positions.  Tiles of 256 columns: pair_tile 256 (CTA
// pairs) or 0 (single CTAs).  DLGO_ERR_ALIGN where the output cannot go through TMA stores.
struct DlgoRopeArgs {
  const float* cos_t;
  const float* sin_t;
  const int* token_pos;
  const int* token_seq;
  const int* seq_slot;
  const int* page_table;
  int max_pages;
  void* kpages;
  void* vpages;
  int Hq, Hkv, hd, write_cache;
};

DLGO_EXPORT int dlgo_gemm_tc_rope_takes(int Rb, int K, int Hq, int Hkv, int hd, int page_size) {
  return (hd == 64 || hd == 128) && page_size == 64 && Hq > 0 && Hkv > 0 && Rb == (Hq + 2 * Hkv) * hd && Rb >= 256 &&
         K > 0 && K % 8 == 0;
}

DLGO_EXPORT int dlgo_gemm_tc_rope(const void* x, int T, int ldx, const void* w, int Rb, int ldw, int K, void* qkv,
                                  int ldo, int pair_tile, const DlgoRopeArgs* rope, cudaStream_t stream) {
  if (T <= 0) return DLGO_OK;
  if (rope == nullptr || !dlgo_gemm_tc_rope_takes(Rb, K, rope->Hq, rope->Hkv, rope->hd, 64) || ldx < K || ldw < K ||
      (pair_tile != 0 && pair_tile != 256))
    return DLGO_ERR_SIZE;
  if (rope->cos_t == nullptr || rope->sin_t == nullptr || rope->token_pos == nullptr ||
      (rope->write_cache && (rope->token_seq == nullptr || rope->seq_slot == nullptr || rope->page_table == nullptr ||
                             rope->kpages == nullptr || rope->vpages == nullptr)))
    return DLGO_ERR_SIZE;
  if (((uintptr_t)rope->cos_t & 15) || ((uintptr_t)rope->sin_t & 15) || ((uintptr_t)rope->kpages & 15) ||
      ((uintptr_t)rope->vpages & 15))
    return DLGO_ERR_ALIGN;
  CUtensorMap ma, mb;
  int st = make_map(&ma, x, T, K, ldx, TILE_M);
  if (st != DLGO_OK) return st;
  st = make_map(&mb, w, Rb, K, ldw, pair_tile ? pair_tile / 2 : 256);
  if (st != DLGO_OK) return st;
  TcParams p = {};
  p.Ra = T; p.Rb = Rb; p.K = K; p.out = qkv; p.ldo = ldo; p.transposed = 0; p.epilogue = TC_ROPE_QKV;
  p.splits = 1; p.workspace = nullptr; p.counters = nullptr; p.static_operand = 2;
  p.rope.cos_t = rope->cos_t; p.rope.sin_t = rope->sin_t; p.rope.token_pos = rope->token_pos;
  p.rope.token_seq = rope->token_seq; p.rope.seq_slot = rope->seq_slot; p.rope.page_table = rope->page_table;
  p.rope.max_pages = rope->max_pages;
  p.rope.kpages = (__nv_bfloat16*)rope->kpages; p.rope.vpages = (__nv_bfloat16*)rope->vpages;
  p.rope.Hq = rope->Hq; p.rope.Hkv = rope->Hkv; p.rope.hd = rope->hd; p.rope.write_cache = rope->write_cache;
  // this epilogue exists in the staged form only
  CUtensorMap probe;
  if (getenv("DLGO_TC_DIRECT_EPILOGUE") != nullptr || make_out_map(&probe, p) != DLGO_OK) return DLGO_ERR_ALIGN;
  return pair_tile ? launch_tc_pair<256>(ma, mb, p, stream) : launch_tc_persistent<256>(ma, mb, p, stream);
}

// 1 if a kernel of this library gave up a bounded wait since the last call (clears the flag).
DLGO_EXPORT int dlgo_gemm_tc_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_gemm_tc_error, &zero, sizeof(int));
  return v;
}

DLGO_TIMES_EXPORT
