// Generic linear layer on the CUDA cores, true 32-bit arithmetic:
//   C[M,N] = epilogue(A[M,K] . W[N,K]^T + bias[N]) (+ residual[M,N])
// A, W and the residual are float32 or bfloat16 (one dtype for the three);
// products and sums are float32 FMAs; C is that dtype or float32.
// Every output element is one accumulator that adds k = 0..K-1 in order, so
// a row's result does not depend on how many other rows the call has.
// This is the whole matrix path of the float32 engine, and the fallback of
// the bfloat16 engine for shapes its tensor-core kernels refuse.
//
// Tile 64x64, K step 16, 256 threads with a 4x4 micro-tile each.  Any M, N, K.
#include "activations.cuh"

MLXB_DEFINE_LAST_ERROR()

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T, typename TO, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, const float* __restrict__ bias,
                 const T* residual, TO* C, int M, int N, int K,
                 int lda, int ldc) {
  __shared__ float sA[BK][BM + 4];
  __shared__ float sW[BK][BN + 4];
  pdl_trigger();
  pdl_wait();
  A = after_wait(A);
  residual = after_wait(residual);
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads; thread owns rows ty*4.., cols tx*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // loading: 64 rows x 16 k per tile = 1024 elements, 4 per thread;
  // thread loads row lr = tid / 4, k = (tid % 4) * 4 + {0..3}
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int m = m0 + lr, n = n0 + lr;
      sA[lk + i][lr] = (m < M && k < K) ? to_f(A[(size_t)m * lda + k]) : 0.f;
      sW[lk + i][lr] = (n < N && k < K) ? to_f(W[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sW[kk][tx * 4 + j];
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
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      v = activate<EPI, false>(v);
      if (residual) v += to_f(residual[(size_t)m * ldc + n]);
      C[(size_t)m * ldc + n] = from_f<TO>(v);
    }
  }
}

template <typename T, typename TO>
static int launch(const void* A, const void* W, const float* bias, const void* residual, void* C, int M, int N,
                  int K, int lda, int ldc, int epi, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  return dispatch_activation(epi, [&](auto e) {
    launch_pdl(gemm_simt_kernel<T, TO, decltype(e)::value>, grid, dim3(256), 0, stream, (const T*)A, (const T*)W, bias,
               (const T*)residual, (TO*)C, M, N, K, lda, ldc);
    return mlxb_check_launch("linear (generic)");
  });
}

// dtype: dtype of A, W, residual.  out_f32 != 0: C is float32 whatever dtype is.
// lda: row stride of A in elements (>= K); ldc: row stride of C and residual.
// bias (float32[N]) and residual may be null.
MLXB_EXPORT int mlxb_linear_simt(int dtype, int out_f32, const void* A, const void* W, const float* bias,
                                 const void* residual, void* C, int M, int N, int K, int lda, int ldc, int epi,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || lda < K || ldc < N) return mlxb_fail(MLXB_BAD_ARG, "linear: K %d lda %d ldc %d N %d", K, lda, ldc, N);
  if ((M + BM - 1) / BM > 65535) return mlxb_fail(MLXB_BAD_ARG, "linear: %d rows are too many for one call", M);
  if (dtype == MLXB_F32) return launch<float, float>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, stream);
  if (dtype == MLXB_BF16) {
    if (out_f32) return launch<__nv_bfloat16, float>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, stream);
    return launch<__nv_bfloat16, __nv_bfloat16>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, stream);
  }
  return mlxb_fail(MLXB_BAD_DTYPE, "linear: dtype code %d", dtype);
}
