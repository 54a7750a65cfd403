// Combining the per-slice partial results of split-KV attention (shared by the attention kernels).
#pragma once
#include <math.h>

#include "common.cuh"

namespace dlgo {

// out[token, head, :] = sum_s w_s acc_s / sum_s w_s l_s with w_s = exp(m_s - max m)
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                         T* __restrict__ out, int ldo, int Hq, int hd, int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int token = blockIdx.x, head = blockIdx.y;
  const size_t o = ((size_t)token * Hq + head) * n_splits;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(o + s) * 2]);
  float denom = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = part_ml[(o + s) * 2];
    if (ms != -INFINITY) denom += expf(ms - m) * part_ml[(o + s) * 2 + 1];
  }
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = part_ml[(o + s) * 2];
      if (ms != -INFINITY) a = fmaf(expf(ms - m), part_acc[(o + s) * hd + d], a);
    }
    out[(size_t)token * ldo + (size_t)head * hd + d] = from_float<T>(a / denom);
  }
}

}  // namespace dlgo
