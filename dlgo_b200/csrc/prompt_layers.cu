// The layer loop of a prompt step as native calls.
//
// A prompt step of the usual pre-norm block is eight launches a layer: norm, q/k/v projection, rotation and
// cache append, attention, output projection, norm, gate/up projection with SwiGLU, down projection.  Issued
// one by one from Python, each costs about 19 us of host time (argument checks, temporaries, the foreign
// call), 2.6 ms for a 16-layer model whatever the prompt's length, which is more than the GPU needs for a
// prompt of 1,000 tokens.  Here the same entry points, with the same arguments, are called from one native
// loop.  (The reference's forward pass is compiled code throughout: models/llm/forward_batch.go:78-215.)
//
// This file has no kernel and no policy of its own: the entry points come in as addresses (they live in this
// package's other libraries), and tile shapes, sizes and constants come from the parts the model was built
// from.
#include <cuda_runtime.h>

#include "common.cuh"

extern "C" {

typedef int (*RmsNormFn)(const float* x, const float* w, void* out, int out_dtype, const int* rows, int R, int d,
                         float eps, cudaStream_t stream);
typedef int (*GemmTcFn)(const void* A, int Ra, int lda, const void* B, int Rb, int ldb, int K, void* out, int ldo,
                        int transposed, int epilogue, int bn, int splits, float* workspace, int* counters,
                        int static_operand, int pair_tile, cudaStream_t stream);
typedef int (*RopeAppendFn)(void* qkv, int dtype, int T, int ld, const float* cos_t, const float* sin_t,
                            const int* token_pos, const int* token_seq, const int* seq_slot, const int* page_table,
                            int max_pages, void* kpages, void* vpages, int Hq, int Hkv, int hd, int rot,
                            int page_size, int interleaved, int write_cache, const float* parts, int S,
                            long long part_stride, int clear_parts, cudaStream_t stream);
typedef int (*AttentionFn)(const void* q, int T, int ldq, const void* kpages, const void* vpages, int n_pages,
                           const int* page_table, int max_pages, const int* tiles, int n_tiles, const int* seq_slot,
                           const int* token_pos, void* out, int ldo, int Hq, int Hkv, int hd, int window, float scale,
                           cudaStream_t stream);

// as in gemm_tc.cu
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
typedef int (*GemmTcRopeFn)(const void* x, int T, int ldx, const void* w, int Rb, int ldw, int K, void* qkv, int ldo,
                            int pair_tile, const DlgoRopeArgs* rope, cudaStream_t stream);

// Entry points of the kernel libraries.
struct DlgoPromptEntryPoints {
  RmsNormFn rmsnorm;
  GemmTcFn gemm_tc;
  RopeAppendFn rope_append;
  AttentionFn attention;
  GemmTcRopeFn gemm_tc_rope;
};

// What the layers of a run share.
struct DlgoPromptShape {
  int hidden, heads, kv_heads, head_dim, ffn;   // ffn: width of the SwiGLU (the gate/up weight has 2 * ffn rows)
  int rotary_dim, interleaved, window, page_size;
  float scale;
};

// One layer: weights (bfloat16; gate and up rows interleaved in blocks of 16), norm weights (fp32), its pages.
struct DlgoPromptLayer {
  const void* w_qkv;
  const void* w_o;
  const void* w_gate_up;
  const void* w_down;
  const float* norm1_w;
  const float* norm2_w;
  float eps1, eps2;
  void* kpages;
  void* vpages;
  int n_pages;
  int write_cache;
};

// One step: the residual stream, buffers for the layers' intermediates, the batch's tables, and the tile
// shapes that the contraction's planner chose for this many tokens.
struct DlgoPromptStep {
  int tokens;
  float* residual;        // [tokens, hidden] fp32, added into
  void* x;                // [tokens, hidden] bf16
  void* qkv;              // [tokens, (heads + 2 kv_heads) * head_dim] bf16
  void* attn_out;         // [tokens, heads * head_dim] bf16
  void* h;                // [tokens, ffn] bf16
  const float* cos_t;
  const float* sin_t;
  const int* token_pos;
  const int* token_seq;
  const int* seq_slot;
  const int* page_table;
  int max_pages;
  const int* tiles;       // attention tiles, heaviest first
  int n_tiles;
  int bn[4];              // tile width of qkv, o, gate_up, down
  int pair[4];            // their CTA-pair tile (0: none)
  int fuse_rope;          // the q/k/v projection's epilogue rotates and appends: no launch for that
};

}  // extern "C"

namespace {
constexpr int TC_STORE = 0, TC_ADD_F32 = 2, TC_SWIGLU = 3;   // epilogue codes of dlgo_gemm_tc
}

// Runs `n_layers` layers.  Returns 0, or the first non-zero status with *failed_call = 8 * layer + call
// (calls in the order of the list above).
DLGO_EXPORT int dlgo_prompt_layers(const DlgoPromptEntryPoints* fn, const DlgoPromptShape* s,
                                   const DlgoPromptLayer* layers, int n_layers, const DlgoPromptStep* p,
                                   int* failed_call, cudaStream_t stream) {
  if (fn == nullptr || s == nullptr || layers == nullptr || p == nullptr) return DLGO_ERR_SIZE;
  if (fn->rmsnorm == nullptr || fn->gemm_tc == nullptr || fn->rope_append == nullptr || fn->attention == nullptr ||
      fn->gemm_tc_rope == nullptr)
    return DLGO_ERR_DRIVER;
  const int T = p->tokens, d = s->hidden;
  const int q_dim = s->heads * s->head_dim, n_cols = (s->heads + 2 * s->kv_heads) * s->head_dim;
  if (T <= 0 || n_layers <= 0) return DLGO_OK;
  int st = DLGO_OK, call = 0;
#define DLGO_STEP(expr)                           \
  do {                                            \
    st = (expr);                                  \
    if (st != DLGO_OK) {                          \
      if (failed_call) *failed_call = call;       \
      return st;                                  \
    }                                             \
    ++call;                                       \
  } while (0)
  for (int l = 0; l < n_layers; ++l) {
    const DlgoPromptLayer& L = layers[l];
    call = 8 * l;
    DLGO_STEP(fn->rmsnorm(p->residual, L.norm1_w, p->x, DLGO_BF16, nullptr, T, d, L.eps1, stream));
    if (p->fuse_rope) {
      const DlgoRopeArgs rope = {p->cos_t, p->sin_t, p->token_pos, p->token_seq, p->seq_slot, p->page_table,
                                 p->max_pages, L.kpages, L.vpages, s->heads, s->kv_heads, s->head_dim, L.write_cache};
      DLGO_STEP(fn->gemm_tc_rope(p->x, T, d, L.w_qkv, n_cols, d, d, p->qkv, n_cols, p->pair[0], &rope, stream));
      ++call;
    } else {
      DLGO_STEP(fn->gemm_tc(p->x, T, d, L.w_qkv, n_cols, d, d, p->qkv, n_cols, 0, TC_STORE, p->bn[0], 1, nullptr,
                            nullptr, 2, p->pair[0], stream));
      DLGO_STEP(fn->rope_append(p->qkv, DLGO_BF16, T, n_cols, p->cos_t, p->sin_t, p->token_pos, p->token_seq,
                                p->seq_slot, p->page_table, p->max_pages, L.kpages, L.vpages, s->heads, s->kv_heads,
                                s->head_dim, s->rotary_dim, s->page_size, s->interleaved, L.write_cache, nullptr, 0, 0,
                                0, stream));
    }
    DLGO_STEP(fn->attention(p->qkv, T, n_cols, L.kpages, L.vpages, L.n_pages, p->page_table, p->max_pages, p->tiles,
                            p->n_tiles, p->seq_slot, p->token_pos, p->attn_out, q_dim, s->heads, s->kv_heads,
                            s->head_dim, s->window, s->scale, stream));
    DLGO_STEP(fn->gemm_tc(p->attn_out, T, q_dim, L.w_o, d, q_dim, q_dim, p->residual, d, 0, TC_ADD_F32, p->bn[1], 1,
                          nullptr, nullptr, 2, p->pair[1], stream));
    DLGO_STEP(fn->rmsnorm(p->residual, L.norm2_w, p->x, DLGO_BF16, nullptr, T, d, L.eps2, stream));
    DLGO_STEP(fn->gemm_tc(p->x, T, d, L.w_gate_up, 2 * s->ffn, d, d, p->h, s->ffn, 0, TC_SWIGLU, p->bn[2], 1, nullptr,
                          nullptr, 2, p->pair[2], stream));
    DLGO_STEP(fn->gemm_tc(p->h, T, s->ffn, L.w_down, d, s->ffn, s->ffn, p->residual, d, 0, TC_ADD_F32, p->bn[3], 1,
                          nullptr, nullptr, 2, p->pair[3], stream));
  }
#undef DLGO_STEP
  return DLGO_OK;
}

// Launches per layer, for the caller's count.
DLGO_EXPORT int dlgo_prompt_layers_launches(int fuse_rope) { return fuse_rope ? 7 : 8; }
