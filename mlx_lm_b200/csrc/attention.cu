// Attention over the paged key/value cache: generic kernels, 32-bit math.
//
// Cache layout of one layer: K and V are [n_pages][n_kv_heads][page][head_dim];
// a request's position p lives in page block_table[req][p / page], row p % page.
// A negative block-table entry means "no page" (never written, or already
// given back because a window has passed it).
//
// kv_write   copies this step's key and value rows from the fused projection
//            output into the pages.
// attention  one warp per (token, query head): the query at position p of its
//            request attends keys max(0, p-window+1) .. p through the block
//            table, this step's own tokens included (kv_write runs first).
//            Scores, running maximum, sum and the weighted sum of values are
//            float32; keys are visited in order 32 at a time, so the result
//            for a token does not depend on what else is in the batch or on
//            how the request's tokens were cut into steps.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

// qkv row of token t: [q (Hq*Dh) | k (Hkv*Dh) | v (Hkv*Dh)] at row stride ld.
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src, int ld,
                                const int* __restrict__ positions, const int* __restrict__ token_req,
                                const int* __restrict__ block_table, int max_pages, int n_pages, int page,
                                int Hkv, int Dh, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                int* __restrict__ status) {
  const int t = blockIdx.x;
  const int p = positions[t];
  const int r = token_req[t];
  if (r < 0) return;  // padding token of a fixed-shape batch
  const int lp = p / page;
  if (p < 0 || lp >= max_pages) {
    if (threadIdx.x == 0) atomicOr(status, MLXB_ST_POSITION_RANGE);
    return;
  }
  const int pg = block_table[(size_t)r * max_pages + lp];
  if (pg < 0) return;  // padding entry of a fixed-shape batch: nothing to store
  if (pg >= n_pages) {
    if (threadIdx.x == 0) atomicOr(status, MLXB_ST_PAGE_RANGE);
    return;
  }
  const int row = p % page;
  const int n = Hkv * Dh;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int h = i / Dh, d = i - h * Dh;
    const size_t dst = (((size_t)pg * Hkv + h) * page + row) * Dh + d;
    k_pool[dst] = k_src[(size_t)t * ld + i];
    v_pool[dst] = v_src[(size_t)t * ld + i];
  }
}

constexpr int MAX_DPL = 8;  // head_dim <= 256: up to 8 output dims per lane

template <typename T>
__global__ void __launch_bounds__(128)
attention_generic_kernel(const T* __restrict__ q, int ldq, const int* __restrict__ positions,
                         const int* __restrict__ token_req, const int* __restrict__ block_table,
                         int max_pages, int n_pages, int page, int Hq, int Hkv, int Dh, int window,
                         float scale, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         T* __restrict__ out, int ldo, int n_tokens, int* __restrict__ status) {
  extern __shared__ float sq[];  // [warps][Dh]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int w = blockIdx.x * (blockDim.x >> 5) + warp;
  if (w >= n_tokens * Hq) return;
  const int t = w / Hq, h = w - t * Hq;
  const int hk = h / (Hq / Hkv);
  const int p = positions[t];
  const int r = token_req[t];
  if (r < 0) return;  // padding token of a fixed-shape batch: its output row is never read
  const int* bt = block_table + (size_t)r * max_pages;
  float* myq = sq + warp * Dh;
  for (int d = lane; d < Dh; d += 32) myq[d] = to_f(q[(size_t)t * ldq + h * Dh + d]) * scale;
  __syncwarp();

  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  float m = -INFINITY, l = 0.f;
  float o[MAX_DPL];
#pragma unroll
  for (int i = 0; i < MAX_DPL; ++i) o[i] = 0.f;

  for (int j0 = lo; j0 <= p; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    int pg = -1;
    if (j <= p) {
      const int lp = j / page;
      pg = lp < max_pages ? bt[lp] : -1;
      if (pg >= n_pages) { atomicOr(status, MLXB_ST_PAGE_RANGE); pg = -1; }
      if (pg >= 0) {
        const T* kp = k_pool + (((size_t)pg * Hkv + hk) * page + (j % page)) * Dh;
        float a = 0.f;
        for (int d = 0; d < Dh; ++d) a = fmaf(myq[d], to_f(kp[d]), a);
        s = a;
      } else {
        atomicOr(status, MLXB_ST_POSITION_RANGE);  // a key inside the range has no page
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float pj = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) o[i] *= corr;
    m = m_new;
    const int nk = min(32, p - j0 + 1);
    for (int jj = 0; jj < nk; ++jj) {
      const float pw = __shfl_sync(0xffffffffu, pj, jj);
      const int pgj = __shfl_sync(0xffffffffu, pg, jj);
      if (pgj < 0) continue;
      const T* vp = v_pool + (((size_t)pgj * Hkv + hk) * page + ((j0 + jj) % page)) * Dh;
#pragma unroll
      for (int i = 0; i < MAX_DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < Dh) o[i] = fmaf(pw, to_f(vp[d]), o[i]);
      }
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < Dh) out[(size_t)t * ldo + h * Dh + d] = from_f<T>(o[i] * inv);
  }
}

static int check_common(const char* what, int page, int Hq, int Hkv, int Dh) {
  if (page <= 0 || (page & (page - 1))) return mlxb_fail(MLXB_BAD_ARG, "%s: page size %d is not a power of two", what, page);
  if (Hkv <= 0 || Hq <= 0 || Hq % Hkv) return mlxb_fail(MLXB_BAD_ARG, "%s: %d query heads over %d key/value heads", what, Hq, Hkv);
  if (Dh <= 0 || Dh > 32 * MAX_DPL) return mlxb_fail(MLXB_BAD_ARG, "%s: head size %d is outside 1..%d", what, Dh, 32 * MAX_DPL);
  return 0;
}

MLXB_EXPORT int mlxb_kv_write(int dtype, const void* k_src, const void* v_src, int ld, const int* positions,
                              const int* token_req, const int* block_table, int max_pages, int n_pages, int page,
                              int Hkv, int Dh, void* k_pool, void* v_pool, int n_tokens, int* status,
                              cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (int e = check_common("kv_write", page, Hkv, Hkv, Dh)) return e;
  const int threads = Hkv * Dh >= 512 ? 256 : 128;
  if (dtype == MLXB_F32)
    kv_write_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)k_src, (const float*)v_src, ld, positions,
                                                            token_req, block_table, max_pages, n_pages, page, Hkv, Dh,
                                                            (float*)k_pool, (float*)v_pool, status);
  else if (dtype == MLXB_BF16)
    kv_write_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)k_src, (const __nv_bfloat16*)v_src, ld, positions, token_req, block_table, max_pages,
        n_pages, page, Hkv, Dh, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, status);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "kv_write: dtype code %d", dtype);
  return mlxb_check_launch("kv_write");
}

// q: [n_tokens, >= Hq*Dh] at row stride ldq; out: [n_tokens, Hq*Dh] at row stride ldo.
// window <= 0: all keys 0..p.
MLXB_EXPORT int mlxb_attention_generic(int dtype, const void* q, int ldq, const int* positions, const int* token_req,
                                       const int* block_table, int max_pages, int n_pages, int page, int Hq, int Hkv,
                                       int Dh, int window, float scale, const void* k_pool, const void* v_pool,
                                       void* out, int ldo, int n_tokens, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (int e = check_common("attention", page, Hq, Hkv, Dh)) return e;
  const int warps = 4;
  const long long total = (long long)n_tokens * Hq;
  const int blocks = (int)((total + warps - 1) / warps);
  const size_t smem = (size_t)warps * Dh * sizeof(float);
  if (dtype == MLXB_F32)
    attention_generic_kernel<float><<<blocks, warps * 32, smem, stream>>>(
        (const float*)q, ldq, positions, token_req, block_table, max_pages, n_pages, page, Hq, Hkv, Dh, window, scale,
        (const float*)k_pool, (const float*)v_pool, (float*)out, ldo, n_tokens, status);
  else if (dtype == MLXB_BF16)
    attention_generic_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, ldq, positions, token_req, block_table, max_pages, n_pages, page, Hq, Hkv, Dh, window,
        scale, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, ldo, n_tokens, status);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "attention: dtype code %d", dtype);
  return mlxb_check_launch("attention (generic)");
}
