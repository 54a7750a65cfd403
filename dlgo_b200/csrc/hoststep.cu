// Host side of a decode step as native calls.
//
// Between "the next token ids are known" and "the step's graph runs" lie a copy of the step's inputs
// (ids, positions, slots) out of one pinned buffer, an event that says when that buffer may be written
// again, and the launch of the captured graph: three runtime calls that, made one by one from Python,
// cost more host time than the GPU idles for comfortably at these step times.  Here they are one call.
// (The reference's generation loop is compiled code throughout, models/llm/generate.go:91-283.)
#include <cuda_runtime.h>

#include "common.cuh"

namespace {
struct HostStep {
  cudaEvent_t copied;
};
}  // namespace

DLGO_EXPORT void* dlgo_hoststep_create() {
  HostStep* h = new HostStep();
  if (cudaEventCreateWithFlags(&h->copied, cudaEventDisableTiming) != cudaSuccess) {
    delete h;
    return nullptr;
  }
  return h;
}

DLGO_EXPORT void dlgo_hoststep_destroy(void* handle) {
  HostStep* h = (HostStep*)handle;
  if (h == nullptr) return;
  cudaEventDestroy(h->copied);
  delete h;
}

// Returns once the last launch's copy out of the pinned buffer has finished (at once if there was none).
DLGO_EXPORT int dlgo_hoststep_wait(void* handle) {
  return (int)cudaEventSynchronize(((HostStep*)handle)->copied);
}

// pinned host buffer -> device inputs, mark the buffer free, launch the step's graph
DLGO_EXPORT int dlgo_hoststep_launch(void* handle, void* dev_inputs, const void* host_inputs, long long nbytes,
                                     void* graph_exec, cudaStream_t stream) {
  HostStep* h = (HostStep*)handle;
  cudaError_t e = cudaMemcpyAsync(dev_inputs, host_inputs, (size_t)nbytes, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return (int)e;
  e = cudaEventRecord(h->copied, stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGraphLaunch((cudaGraphExec_t)graph_exec, stream);
}
