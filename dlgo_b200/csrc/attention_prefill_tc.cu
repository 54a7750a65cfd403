// Causal grouped-query attention for prompts on the Blackwell tensor cores (bfloat16, head size 64
// or 128).
//
// Same formulas as attention.cu (models/llm/forward_batch.go:188-207: every prompt position attends
// the keys t <= its position, read back from the cache; softmax in fp32).  A CTA takes up to 128
// consecutive tokens of one sequence and one query head, and walks the sequence's pages one page
// (64 keys) at a time; blocks this small leave room for three CTAs on an SM (two at head size 128),
// whose softmax phases, bound by the SM's 16 exponentials a clock, interleave with one another's MMAs:
//   warp 0     TMA: the query tile once, then key and value pages into a two-stage ring
//   warp 1     tcgen05.mma: S = Q K^T (128 x 64, fp32 in tensor memory), then O += P V, the output
//              accumulating in tensor memory over all key blocks
//   warps 2-5  one thread per query row: reads its 64 scores from tensor memory once, masks,
//              keeps a reference maximum and the sum (fp32, exp2 on pre-scaled scores) and writes
//              P as bf16 into shared memory in the swizzled layout the tensor core reads.  The
//              reference maximum follows the true one lazily: only when a block's maximum exceeds
//              it by more than 2^8 is the row's output in tensor memory rescaled (read, multiplied,
//              written back); otherwise probabilities are simply up to 256 times larger than with
//              the true maximum, which fp32 sums and bf16 probabilities carry without loss, and
//              the final division by the sum (taken against the same reference) cancels it
// Values are read as the MN-major operand straight from the page layout [key][head_dim].
// Keys that were never written (the tail of the last page, pages a window has given back) get
// probability zero; their value rows are zeroed in shared memory so that 0 * garbage cannot
// become NaN.
#include <math.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace dlgo {

using namespace sm100;

constexpr int PF_THREADS = 192;
constexpr int PF_ROWS = 128;   // query rows per CTA
constexpr int PF_KEYS = 64;    // keys per step (one page)

__device__ int g_attention_tc_error = 0;

struct PfParams {
  const int* tiles;       // [n_tiles][3]: sequence, first packed token, count (<= 128)
  const int* seq_slot;
  const int* token_pos;
  const int* page_table;
  int max_pages;
  __nv_bfloat16* out;
  int ldo;
  int Hq, Hkv, window;
  float scale_log2e;      // score scale times log2(e)
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Diagnostic build: cycles of the first softmax thread per phase, summed over the key blocks of a tile
// (slot 0..6: wait for scores, read them, maximum, wait for P V, rescale, exponentials and P, hand-over;
// slot 7: key blocks)
#ifdef DLGO_TIMING
#define PF_CLK_DECL long long clk_sum[7] = {0, 0, 0, 0, 0, 0, 0}; long long clk_t = clock64()
#define PF_CLK(k) do { const long long n_ = clock64(); clk_sum[k] += n_ - clk_t; clk_t = n_; } while (0)
#define PF_CLK_WRITE(nblk)                                                        \
  do {                                                                            \
    const int c_ = blockIdx.y * gridDim.x + blockIdx.x;                           \
    if (threadIdx.x == 64 && c_ < 1024) {                                         \
      for (int k_ = 0; k_ < 7; ++k_) g_times[c_ * 8 + k_] = (unsigned long long)clk_sum[k_]; \
      g_times[c_ * 8 + 7] = (unsigned long long)(nblk);                           \
    }                                                                             \
  } while (0)
#else
#define PF_CLK_DECL do {} while (0)
#define PF_CLK(k) do {} while (0)
#define PF_CLK_WRITE(nblk) do {} while (0)
#endif

// MN-major operand (rows of 128 bytes = 64 contiguous N elements, 8 K-rows per 1024-byte group),
// 128-byte swizzle; `lbo_bytes` is the distance between 64-element N blocks.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <int HD>
__global__ void __launch_bounds__(PF_THREADS, HD <= 64 ? 3 : 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PfParams p) {
  constexpr int NCH = HD / 64;                 // 64-wide chunks of the head
  constexpr int QBYTES = NCH * 16384;          // [128 rows][HD]
  constexpr int KVBYTES = NCH * 8192;          // [64 keys][HD] per stage
  constexpr int PBYTES = 16384;                // [128 rows][64 keys]
  constexpr uint32_t O_COL = PF_KEYS;          // scores in columns [0, 64), the output behind them
  constexpr uint32_t TMEM_COLS = HD <= 64 ? 128 : 256;
  // the swizzled tiles want 1024-byte alignment; the kernel has no static shared memory, so the
  // dynamic window starts aligned (checked: a misaligned start ends the kernel with the error word set)
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(&g_attention_tc_error, 1);
    return;
  }
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + QBYTES;                 // 2 stages
  uint8_t* v_s = k_s + 2 * KVBYTES;            // 2 stages
  uint8_t* p_s = v_s + 2 * KVBYTES;
  uint64_t* bars = (uint64_t*)(p_s + PBYTES);
  uint64_t* qfull = bars;          // 1
  uint64_t* kfull = bars + 1;      // 2
  uint64_t* vfull = bars + 3;      // 2
  uint64_t* kempty = bars + 5;     // 2: the scores that read this stage's keys have completed
  uint64_t* vempty = bars + 7;     // 2: the P V that read this stage's values has completed
  uint64_t* s_full = bars + 9;
  uint64_t* s_free = bars + 10;    // the scores of a block are in registers: the next block's may overwrite them
  uint64_t* p_full = bars + 11;    // P of a block is written and O is rescaled if need be
  uint64_t* pv_done = bars + 12;   // a block's P V has completed: P may be overwritten, O touched
  uint32_t* tmem_slot = (uint32_t*)(bars + 14);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x;   // heads fastest: the heads of a group, which read the same keys, start together
  const int G = p.Hq / p.Hkv;
  const int kvh = head / G;

  if (threadIdx.x == 0) {
    mbar_init(qfull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kfull[s], 1);
      mbar_init(&vfull[s], 1);
      mbar_init(&kempty[s], 1);
      mbar_init(&vempty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 4);
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait();
  const int tile = blockIdx.y;   // in table order: the caller lists the tiles that see most keys first
  const int seq = p.tiles[3 * tile], tok0 = p.tiles[3 * tile + 1], ntok = p.tiles[3 * tile + 2];
  const int slot = p.seq_slot[seq];
  const int pos0 = p.token_pos[tok0];
  const int t_end = pos0 + ntok;                                  // one past the last key any row sees
  const int t_begin = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int first_live_page = t_begin / 64;                       // pages before it may have been given back
  const int kb_first = t_begin / PF_KEYS, kb_last = (t_end - 1) / PF_KEYS;
  const int nblk = kb_last - kb_first + 1;
  const int last_page = (t_end - 1) / 64;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(qfull, QBYTES);
      for (int j = 0; j < NCH; ++j) tma_load_2d(q_s + j * 16384, &map_q, qfull, head * HD + j * 64, tok0);
      // keys run one block ahead of values: a stage's keys are free once their scores have completed,
      // its values only after the P V that follows a whole softmax later
      auto page_of = [&](int it) {
        const int pg = kb_first + it;
        return (pg >= first_live_page && pg <= last_page) ? p.page_table[(size_t)slot * p.max_pages + pg] : -1;
      };
      auto load_k = [&](int it) {
        const int st = it & 1;
        if (it >= 2 && !mbar_wait(&kempty[st], ((it >> 1) - 1) & 1, abort_flag)) return false;
        const int page = page_of(it);
        mbar_expect_tx(&kfull[st], page >= 0 ? NCH * 8192 : 0);
        if (page >= 0)
          for (int j = 0; j < NCH; ++j)
            tma_load_2d(k_s + st * KVBYTES + j * 8192, &map_k, &kfull[st], j * 64, (page * p.Hkv + kvh) * 64);
        return true;
      };
      auto load_v = [&](int it) {
        const int st = it & 1;
        if (it >= 2 && !mbar_wait(&vempty[st], ((it >> 1) - 1) & 1, abort_flag)) return false;
        const int page = page_of(it);
        mbar_expect_tx(&vfull[st], page >= 0 ? NCH * 8192 : 0);
        if (page >= 0)
          for (int j = 0; j < NCH; ++j)
            tma_load_2d(v_s + st * KVBYTES + j * 8192, &map_v, &vfull[st], j * 64, (page * p.Hkv + kvh) * 64);
        return true;
      };
      bool ok = load_k(0);
      for (int it = 0; ok && it < nblk; ++it) {
        if (it + 1 < nblk) ok = load_k(it + 1);
        if (ok) ok = load_v(it);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(PF_ROWS, PF_KEYS);
      constexpr uint32_t idesc_o = umma_idesc_bf16(PF_ROWS, HD) | (1u << 16);   // B is MN-major
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      bool ok = mbar_wait(qfull, 0, abort_flag) && mbar_wait(&kfull[0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(k_s);
#pragma unroll
        for (int j = 0; j < NCH; ++j)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base, umma_desc_k_sw128(q_addr + j * 16384) + 2 * k,
                      umma_desc_k_sw128(k_addr + j * 8192) + 2 * k, idesc_s, (j | k) != 0);
        umma_commit(s_full);
      }
      if (ok) umma_commit(&kempty[0]);
      for (int it = 0; ok && it < nblk; ++it) {
        const int st = it & 1;
        if (it + 1 < nblk) {
          // the next block's scores as soon as this block's are in registers: they are computed while
          // the softmax threads work on this block
          const int st2 = (it + 1) & 1;
          ok = mbar_wait(s_free, it & 1, abort_flag) && mbar_wait(&kfull[st2], ((it + 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t k_addr = smem_u32(k_s + st2 * KVBYTES);
#pragma unroll
          for (int j = 0; j < NCH; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16(tmem_base, umma_desc_k_sw128(q_addr + j * 16384) + 2 * k,
                        umma_desc_k_sw128(k_addr + j * 8192) + 2 * k, idesc_s, (j | k) != 0);
          umma_commit(s_full);
          umma_commit(&kempty[st2]);
        }
        ok = mbar_wait(p_full, it & 1, abort_flag) && mbar_wait(&vfull[st], (it >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(v_s + st * KVBYTES);
#pragma unroll
        for (int kk = 0; kk < PF_KEYS / 16; ++kk)
          umma_bf16(tmem_base + O_COL, umma_desc_k_sw128(p_addr) + 2 * kk,
                    umma_desc_mn_sw128(v_addr + kk * 2048, 8192), idesc_o, (it | kk) != 0);
        umma_commit(&vempty[st]);
        umma_commit(pv_done);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;            // query row of the tile and key row of a stage
    const int pos_r = pos0 + r;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float m = -INFINITY, l = 0.f;                 // reference maximum (lazy) and sum against it
    bool ok = true;
    PF_CLK_DECL;
    for (int it = 0; ok && it < nblk; ++it) {
      const int st = it & 1;
      const int k0 = (kb_first + it) * PF_KEYS;
      PF_CLK(6);
      // value rows of keys that were never written, or whose page was not loaded, must be zero
      {
        const int t = k0 + r;                      // threads 0..63 stand for the stage's key rows
        if (r < PF_KEYS && (t >= t_end || (t >> 6) < first_live_page)) {
          ok = mbar_wait(&vfull[st], (it >> 1) & 1, abort_flag);
          uint8_t* row = v_s + st * KVBYTES + r * 128;
#pragma unroll
          for (int j = 0; j < NCH; ++j)
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(row + j * 8192 + c * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      // the scores of this block, into registers; then the tensor core may write the next block's
      if (ok) ok = mbar_wait(s_full, it & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      PF_CLK(0);
      float v[PF_KEYS];
#pragma unroll
      for (int c0 = 0; c0 < PF_KEYS; c0 += 32) tmem_ld_32x32(lane_addr + c0, v + c0);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      PF_CLK(1);
      const int lo = p.window > 0 ? pos_r - p.window : -1;        // keys t > lo and t <= pos_r are seen
      // blocks that lie wholly inside every row's range need no mask (all but the diagonal ones)
      const bool full_block = (k0 + PF_KEYS - 1 <= pos0) && (p.window <= 0 || k0 > pos0 + ntok - 1 - p.window);
      if (!full_block) {
#pragma unroll
        for (int j = 0; j < PF_KEYS; ++j) {
          const int t = k0 + j;
          if (!(t <= pos_r && t > lo)) v[j] = -INFINITY;
        }
      }
      // (four independent chains: one chain of 128 dependent maxima would cost its latency 128 times)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < PF_KEYS; j += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) mx4[e] = fmaxf(mx4[e], v[j + e]);
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= p.scale_log2e;                                       // the scale is positive: max commutes with it
      // Lazy reference: move it (and rescale the row's output) only when this block's maximum exceeds
      // it by more than 8 (a factor of 256); tensor-memory accesses are warp-wide, so the warp goes
      // through the rescaling together and rows that need none multiply by one.
      const bool move = mx > m + 8.0f || (m == -INFINITY && mx > -INFINITY);
      // P of the block before must have been consumed, and O be at rest, before either is touched
      // (its P V was issued when this iteration began: it has completed by now as a rule)
      PF_CLK(2);
      if (it > 0) {
        ok = mbar_wait(pv_done, (it - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
      }
      PF_CLK(3);
      if (__any_sync(0xffffffffu, move)) {
        const float corr = move ? ((m == -INFINITY) ? 0.f : fast_exp2(m - mx)) : 1.0f;
        if (move) {
          m = mx;
          l *= corr;
        }
        if (it > 0) {
#pragma unroll 1
          for (int c0 = 0; c0 < HD; c0 += 16) {     // (small pieces: the row's scores stay in registers meanwhile)
            float o[16];
            tmem_ld_32x16(lane_addr + O_COL + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] *= corr;
            tmem_st_32x16(lane_addr + O_COL + c0, o);
          }
          tmem_st_wait();
        }
      }
      PF_CLK(4);
      const float mref = (m == -INFINITY) ? 0.f : m;
      // probabilities, their sum, and P as bf16 in the swizzled K-major layout
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c0 = 0; c0 < PF_KEYS; c0 += 8) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // (masked scores are -inf: exp2 gives zero)
          const float p0 = fast_exp2(fmaf(v[c0 + 2 * e], p.scale_log2e, -mref));
          const float p1 = fast_exp2(fmaf(v[c0 + 2 * e + 1], p.scale_log2e, -mref));
          sum4[e] += p0 + p1;
          h[e] = __floats2bfloat162_rn(p0, p1);
        }
        const int ch = c0 >> 3;                                   // 8-key chunk index 0..7
        uint8_t* dst = p_s + r * 128 + ((ch ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(h);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      PF_CLK(5);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P (and zeroed V rows) -> tensor core
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);   // one arrival per warp stands for its 32 rows
    }
    PF_CLK_WRITE(nblk);
    // the finished output: out of tensor memory once, divided by the sum
    if (ok) ok = mbar_wait(pv_done, (nblk - 1) & 1, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.0f / l;
      __nv_bfloat16* o = p.out + (size_t)(tok0 + r) * p.ldo + (size_t)head * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float acc[32];
        tmem_ld_32x32(lane_addr + O_COL + c0, acc);
        tmem_ld_wait();
        if (r < ntok) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(acc[c * 8 + 2 * e] * inv, acc[c * 8 + 2 * e + 1] * inv);
            *reinterpret_cast<uint4*>(o + c0 + c * 8) = *reinterpret_cast<uint4*>(h);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(&g_attention_tc_error, 1);
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
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

int make_map(CUtensorMap* m, const void* base, long long rows, int cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return DLGO_ERR_DRIVER;
  if (((uintptr_t)base & 15) != 0 || (ld % 8) != 0) return DLGO_ERR_ALIGN;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DLGO_OK : DLGO_ERR_DRIVER;
}

template <int HD>
int launch_pf(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PfParams& p, int n_tiles,
              cudaStream_t stream) {
  constexpr int SMEM = (HD / 64) * (16384 + 4 * 8192) + 16384 + 256;   // Q, 2 stages of K and of V, P, barriers
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM);
    if (e != cudaSuccess) return (int)e;
    // With heads of 64 three CTAs fit an SM (3 x 64 KB of shared memory, 3 x 128 columns of tensor
    // memory), with heads of 128 two: one's softmax runs beside the others' MMAs and maxima.  That
    // needs the largest carve-out.
    cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         (int)cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  launch_kernel(attention_prefill_tc_kernel<HD>, dim3(p.Hq, n_tiles), dim3(PF_THREADS), SMEM, stream, mq, mk, mv, p);
  return launch_status();
}

}  // namespace

// 1 if the tensor-core kernel takes these sizes (bf16, head size 64 or 128, pages of 64 keys)
DLGO_EXPORT int dlgo_attention_prefill_tc_takes(int dtype, int hd, int page_size) {
  return dtype == DLGO_BF16 && (hd == 64 || hd == 128) && page_size == 64;
}

// q[T, .] bf16 with row stride ldq (head h at column h*hd); pages [n_pages, Hkv, 64, hd] bf16;
// tiles[n_tiles][3] of at most 128 tokens each; out[T, Hq*hd] bf16 with row stride ldo.
DLGO_EXPORT int dlgo_attention_prefill_tc(const void* q, int T, int ldq, const void* kpages, const void* vpages,
                                          int n_pages, const int* page_table, int max_pages, const int* tiles,
                                          int n_tiles, const int* seq_slot, const int* token_pos, void* out, int ldo,
                                          int Hq, int Hkv, int hd, int window, float scale, cudaStream_t stream) {
  if (T <= 0 || n_tiles <= 0) return DLGO_OK;
  if (n_tiles > 65535) return DLGO_ERR_SIZE;   // tiles are the grid's second dimension
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || !(hd == 64 || hd == 128) || Hq > 65535) return DLGO_ERR_SIZE;
  if (ldo % 8 || ((uintptr_t)out & 15)) return DLGO_ERR_ALIGN;
  CUtensorMap mq, mk, mv;
  int st = make_map(&mq, q, T, Hq * hd, ldq, 128);
  if (st != DLGO_OK) return st;
  st = make_map(&mk, kpages, (long long)n_pages * Hkv * 64, hd, hd, 64);
  if (st != DLGO_OK) return st;
  st = make_map(&mv, vpages, (long long)n_pages * Hkv * 64, hd, hd, 64);
  if (st != DLGO_OK) return st;
  PfParams p;
  p.tiles = tiles; p.seq_slot = seq_slot; p.token_pos = token_pos; p.page_table = page_table; p.max_pages = max_pages;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo; p.Hq = Hq; p.Hkv = Hkv; p.window = window;
  p.scale_log2e = scale * 1.4426950408889634f;
  if (hd == 64) return launch_pf<64>(mq, mk, mv, p, n_tiles, stream);
  return launch_pf<128>(mq, mk, mv, p, n_tiles, stream);
}

DLGO_EXPORT int dlgo_attention_tc_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_attention_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_attention_tc_error, &zero, sizeof(int));
  return v;
}

DLGO_TIMES_EXPORT
