// The few-rows linear layer (gemm_smallm.cuh) as it is: plain, and with the cache write of a fused
// [q | k | v] projection in its epilogue.
#include "gemm_smallm.cuh"

MLXB_DEFINE_LAST_ERROR()

// A: bfloat16 [M, K] at row stride lda (elements, multiple of 8, base 16-byte aligned);
// W: bfloat16 [N, K] contiguous; bias float32[N] or null; residual bfloat16 [M, N] at row stride ldc or null;
// C: bfloat16 or float32 (out_f32) [M, N] at row stride ldc.  1 <= M <= 64, K % 8 == 0.
MLXB_EXPORT int mlxb_linear_smallm(int out_f32, const void* A, const void* W, const float* bias, const void* residual,
                                   void* C, int M, int N, int K, int lda, int ldc, int epi, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (int e = check_args(M, N, K, lda, ldc, epi, A, W)) return e;
  const KvScatter none = {};
  if (out_f32) return launch<float, false, false>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, none, NormFold{}, stream);
  return launch<__nv_bfloat16, false, false>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, none, NormFold{}, stream);
}

// The fused [q | k | v] projection of an attention layer with the cache write in its epilogue:
// columns [0, q_width) go to C (bfloat16, row stride ldc); the Hkv*Dh key columns and the Hkv*Dh value
// columns after them go into k_pool / v_pool [n_pages, Hkv, page, Dh] at each token's page and row.
// N must equal q_width + 2*Hkv*Dh.  Rows with token_req < 0 (padding) write no keys or values.
MLXB_EXPORT int mlxb_linear_smallm_qkv(const void* A, const void* W, const float* bias, void* C, int M, int N, int K,
                                       int lda, int ldc, const int* positions, const int* token_req,
                                       const int* block_table, int max_pages, int n_pages, int page, int Hkv, int Dh,
                                       int q_width, void* k_pool, void* v_pool, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (int e = check_args(M, N, K, lda, ldc, EPI_NONE, A, W)) return e;
  if (Hkv <= 0 || Dh <= 0 || page <= 0 || q_width < 0 || N != q_width + 2 * Hkv * Dh)
    return mlxb_fail(MLXB_BAD_ARG, "linear (q|k|v): %d outputs for %d query columns and 2 x %d x %d", N, q_width, Hkv, Dh);
  KvScatter kv = {positions, token_req, block_table, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, status,
                  max_pages, n_pages, page, Hkv, Dh, q_width};
  return launch<__nv_bfloat16, true, false>(A, W, bias, nullptr, C, M, N, K, lda, ldc, EPI_NONE, kv, NormFold{}, stream);
}
