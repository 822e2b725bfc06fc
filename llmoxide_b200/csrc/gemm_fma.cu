// Matrix product on the FMA units: Y[M,N] = X[M,K] * W[N,K]^T with float32
// accumulation and no reduced-precision mode of any kind.  It is the matrix
// product of the true 32-bit path, and the fallback of the bfloat16 path for
// shapes the tensor-core kernel refuses (K not a multiple of 8) and for
// weights that the checkpoint stores in 32-bit.
//
// y[t,o] = sum_i W[o,i] x[t,i], W row-major [out, in]
// (crates/model/src/ops.rs:83-101).  Every output element is accumulated by
// one thread in the order i = 0..K-1, so a row's result does not depend on M,
// on the tile it falls into or on what else is in the batch.
#include "common.cuh"

#define FMA_BM 64
#define FMA_BN 64
#define FMA_BK 16

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
gemm_fma_kernel(const TX* __restrict__ X, const TW* __restrict__ W, TY* __restrict__ Y, int M, int N, int K,
                long long ldx, long long ldw, long long ldy) {
  __shared__ float Xs[FMA_BK][FMA_BM + 4];
  __shared__ float Ws[FMA_BK][FMA_BN + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * FMA_BM, n0 = blockIdx.x * FMA_BN;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += FMA_BK) {
    {
      const int m = m0 + lrow, n = n0 + lrow;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int k = k0 + lk + c;
        Xs[lk + c][lrow] = (m < M && k < K) ? to_f32(X[(size_t)m * ldx + k]) : 0.f;
        Ws[lk + c][lrow] = (n < N && k < K) ? to_f32(W[(size_t)n * ldw + k]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < FMA_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = Xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) Y[(size_t)m * ldy + n] = from_f32<TY>(acc[i][j]);
    }
  }
}

LLMX_API int llmx_gemm_fma(const void* X, int x_dtype, const void* W, int w_dtype, void* Y, int y_dtype, int M,
                           int N, int K, long long ldx, long long ldw, long long ldy, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || ldx < K || ldw < K || ldy < N) return LLMX_REFUSED(1);
  dim3 grid((N + FMA_BN - 1) / FMA_BN, (M + FMA_BM - 1) / FMA_BM);
  if (grid.y > 65535) return LLMX_REFUSED(3);
#define CASE(TX, TW, TY) \
  launch_pdl(gemm_fma_kernel<TX, TW, TY>, grid, dim3(256), 0, stream, (const TX*)X, (const TW*)W, (TY*)Y, M, N, K, ldx, ldw, ldy)
  const int key = x_dtype * 4 + w_dtype * 2 + y_dtype;
  switch (key) {
    case 0: CASE(float, float, float); break;
    case 1: CASE(float, float, bf16); break;
    case 2: CASE(float, bf16, float); break;
    case 3: CASE(float, bf16, bf16); break;
    case 4: CASE(bf16, float, float); break;
    case 5: CASE(bf16, float, bf16); break;
    case 6: CASE(bf16, bf16, float); break;
    case 7: CASE(bf16, bf16, bf16); break;
    default: return LLMX_REFUSED(2);
  }
#undef CASE
  return LLMX_LAUNCH_STATUS();
}
