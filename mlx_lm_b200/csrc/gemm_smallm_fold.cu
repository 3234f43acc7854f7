// The few-rows linear layer (gemm_smallm.cuh) with the LayerNorm before it folded in: W is the folded weight
// W . diag(gain), bias the folded bias, colsum[n] = sum_k W[n,k] (float32), eps the norm's; A holds the rows
// before the norm.  See NormFold in gemm_smallm.cuh.  Otherwise as the entry points of gemm_smallm.cu.
#include "gemm_smallm.cuh"

MLXB_DEFINE_LAST_ERROR()

MLXB_EXPORT int mlxb_linear_smallm_fold(int out_f32, const void* A, const void* W, const float* bias,
                                        const void* residual, void* C, int M, int N, int K, int lda, int ldc, int epi,
                                        const float* colsum, float eps, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (int e = check_args(M, N, K, lda, ldc, epi, A, W)) return e;
  if (colsum == nullptr) return mlxb_fail(MLXB_BAD_ARG, "linear (folded norm): column sums missing");
  const KvScatter none = {};
  const NormFold fold = {colsum, eps};
  if (out_f32) return launch<float, false, true>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, none, fold, stream);
  return launch<__nv_bfloat16, false, true>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, none, fold, stream);
}

MLXB_EXPORT int mlxb_linear_smallm_qkv_fold(const void* A, const void* W, const float* bias, void* C, int M, int N,
                                            int K, int lda, int ldc, const int* positions, const int* token_req,
                                            const int* block_table, int max_pages, int n_pages, int page, int Hkv,
                                            int Dh, int q_width, void* k_pool, void* v_pool, int* status,
                                            const float* colsum, float eps, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (int e = check_args(M, N, K, lda, ldc, EPI_NONE, A, W)) return e;
  if (colsum == nullptr) return mlxb_fail(MLXB_BAD_ARG, "linear (folded norm): column sums missing");
  if (Hkv <= 0 || Dh <= 0 || page <= 0 || q_width < 0 || N != q_width + 2 * Hkv * Dh)
    return mlxb_fail(MLXB_BAD_ARG, "linear (q|k|v): %d outputs for %d query columns and 2 x %d x %d", N, q_width, Hkv, Dh);
  KvScatter kv = {positions, token_req, block_table, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, status,
                  max_pages, n_pages, page, Hkv, Dh, q_width};
  const NormFold fold = {colsum, eps};
  return launch<__nv_bfloat16, true, true>(A, W, bias, nullptr, C, M, N, K, lda, ldc, EPI_NONE, kv, fold, stream);
}
