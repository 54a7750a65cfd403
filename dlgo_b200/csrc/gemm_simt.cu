// y[M, N] = x[M, K] . W[N, K]^T on the fp32 pipes (FFMA), for every size.
//
// This is the contraction of the true 32-bit path (no tensor cores, no
// reduced-precision matrix mode), the plain counterpart the tensor-core kernel
// is checked against, and the stand-in where the tensor-core kernel refuses a
// size.  The reference contracts one weight row with the activation vector per
// output (blas/blas.go:152-196, models/llm/forward.go:224,286,296-298); here
// each output is one running fp32 sum over k in index order, so a row's
// result does not depend on the other rows of the launch.
//
// Epilogues: store in the activation type, store fp32 (logits), or add into an
// fp32 residual in place (models/llm/forward.go:163,169).
#include "common.cuh"

namespace dlgo {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
enum { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2 };

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, void* __restrict__ out, int M, int N, int K,
                 int lda, int ldw, int ldo) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int ty = tid / 16, tx = tid % 16;
  // loading: thread -> (row = tid / 4, k offset = (tid % 4) * 4 .. +3)
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      const int gm = m0 + lrow;
      const T* ap = A + (size_t)gm * lda + k0 + lk;
#pragma unroll
      for (int j = 0; j < 4; ++j) As[lk + j][lrow] = (gm < M && k0 + lk + j < K) ? to_float(ap[j]) : 0.f;
      const int gn = n0 + lrow;
      const T* wp = W + (size_t)gn * ldw + k0 + lk;
#pragma unroll
      for (int j = 0; j < 4; ++j) Ws[lk + j][lrow] = (gn < N && k0 + lk + j < K) ? to_float(wp[j]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      const size_t o = (size_t)gm * ldo + gn;
      if (EPI == EPI_STORE) ((T*)out)[o] = from_float<T>(acc[i][j]);
      else if (EPI == EPI_STORE_F32) ((float*)out)[o] = acc[i][j];
      else ((float*)out)[o] += acc[i][j];
    }
  }
}

template <typename T>
int launch_gemm_simt(const void* A, const void* W, void* out, int M, int N, int K, int lda, int ldw, int ldo,
                     int epilogue, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return DLGO_ERR_SIZE;
  const T* a = (const T*)A;
  const T* w = (const T*)W;
  switch (epilogue) {
    case EPI_STORE: launch_kernel(gemm_simt_kernel<T, EPI_STORE>, dim3(grid), dim3(256), 0, stream, a, w, out, M, N, K, lda, ldw, ldo); break;
    case EPI_STORE_F32:
      launch_kernel(gemm_simt_kernel<T, EPI_STORE_F32>, dim3(grid), dim3(256), 0, stream, a, w, out, M, N, K, lda, ldw, ldo);
      break;
    case EPI_ADD_F32:
      launch_kernel(gemm_simt_kernel<T, EPI_ADD_F32>, dim3(grid), dim3(256), 0, stream, a, w, out, M, N, K, lda, ldw, ldo);
      break;
    default: return DLGO_ERR_SIZE;
  }
  return launch_status();
}

}  // namespace dlgo

// A[M, K] (row stride lda), W[N, K] (row stride ldw), both of element type `dtype`;
// out[M, N] (row stride ldo): epilogue 0 stores `dtype`, 1 stores f32, 2 adds into f32.
DLGO_EXPORT int dlgo_gemm_simt(const void* A, const void* W, void* out, int dtype, int M, int N, int K, int lda,
                               int ldw, int ldo, int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return DLGO_OK;
  if (K <= 0 || lda < K || ldw < K || ldo < N) return DLGO_ERR_SIZE;
  if (dtype == DLGO_F32) return dlgo::launch_gemm_simt<float>(A, W, out, M, N, K, lda, ldw, ldo, epilogue, stream);
  if (dtype == DLGO_BF16)
    return dlgo::launch_gemm_simt<__nv_bfloat16>(A, W, out, M, N, K, lda, ldw, ldo, epilogue, stream);
  return DLGO_ERR_DTYPE;
}
