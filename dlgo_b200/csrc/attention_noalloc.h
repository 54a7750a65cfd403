// dlgo_attention_noalloc: attention over the paged cache for callers that cannot allocate.
//
// This entry point has no counterpart in computerex/dlgo.  It exists for callers of this library
// that must not (or cannot) obtain device memory themselves at the time of the call: code running
// inside a host callback or another library's hook where cudaMalloc is off limits, an embedding
// runtime whose memory budget is fixed and handed out once at start-up, or a C program that links
// the library without PyTorch's allocator.  The split-KV form of the attention kernel needs
// scratch (per-slice partial sums that a second kernel combines); the ordinary entry point,
// dlgo_attention, takes that scratch from its caller.  This variant keeps the scratch in a
// file-scope device array inside the library instead, so the caller passes only inputs and outputs.
//
// Limits and rules:
//   * The scratch holds DLGO_ATTENTION_NOALLOC_FLOATS floats (8 MiB).  Every GPU that loads the
//     library holds that much until the process exits.  A call needs
//     T * Hq * n_splits * (hd + 2) floats when n_splits > 1 (none when n_splits == 1); a call that
//     needs more is refused with DLGO_ERR_SIZE and launches nothing.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and remembers it per device.  Make that first call outside any stream
//     capture.
//   * All calls share the one array and it keeps whatever the last call left in it.  Nothing in it
//     has to start at zero: every (token, head, slice) entry that the combine kernel reads is
//     written by the first kernel of the same call, PROVIDED the tiles cover every token 0 .. T-1
//     exactly once (as the engine's tile tables do).  The combine runs over all T tokens: a token
//     that no tile covers would be combined from whatever an earlier, possibly foreign, call left
//     in the array.  The tile table lives in device memory, so the entry point cannot check this.
//     Two calls that overlap on the GPU (different streams, or the same stream from different
//     threads without ordering) race on the array: order them.
//   * It calls no cudaMalloc, cudaFree or any allocating routine, of CUDA or of PyTorch.
//
// Arguments are those of dlgo_attention without `scratch`; the result is the same.
#pragma once
#include <cuda_runtime.h>

#define DLGO_ATTENTION_NOALLOC_FLOATS (2u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

int dlgo_attention_noalloc(const void* q, int dtype, int T, int ldq, const void* kpages, const void* vpages,
                           const int* page_table, int max_pages, const int* tiles, int n_tiles, int tile_tokens_max,
                           const int* seq_slot, const int* token_pos, void* out, int ldo, int Hq, int Hkv, int hd,
                           int page_size, int n_splits, int gchunk, int window, float scale, cudaStream_t stream);

// Floats of scratch a call with these sizes would need (0 for one slice); compare with the limit above.
long long dlgo_attention_noalloc_needs(int T, int Hq, int hd, int n_splits);

#ifdef __cplusplus
}
#endif
