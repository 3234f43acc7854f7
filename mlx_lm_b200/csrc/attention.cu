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
//
// attention_decode / attention_combine  (single-token rows: decode steps)
//            A row has one query but hundreds of keys, and a small batch has too
//            few (row, head) pairs to fill 148 SMs, so the keys are cut into
//            chunks of a fixed number of positions.  One CTA per (chunk, head,
//            row) streams its keys and values once with 16-byte loads (Dh/8
//            threads side by side on one key, so a warp reads contiguous
//            runs), keeps a running (max, sum, weighted values) per thread
//            group, merges the groups, and writes one partial (m, l, o[Dh]) to
//            scratch memory.  The CTA that finishes last for a (row, head) —
//            found with a ticket counter that it resets to zero afterwards —
//            folds that row's partials in chunk order and writes the output.
//            The chunk length is a constant of the engine, not of the batch,
//            so a row's result does not depend on its neighbours.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

// qkv row of token t: [q (Hq*Dh) | k (Hkv*Dh) | v (Hkv*Dh)] at row stride ld.
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src, int ld,
                                const int* __restrict__ positions, const int* __restrict__ token_req,
                                const int* __restrict__ block_table, int max_pages, int n_pages, int page,
                                int Hkv, int Dh, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  k_src = after_wait(k_src);
  v_src = after_wait(v_src);
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
  if ((Dh & 7) == 0 && (ld & 7) == 0 && (((uintptr_t)k_src | (uintptr_t)v_src | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0) {
    // 8 elements at a time (16 bytes of bfloat16, 32 of float32): a head's row is contiguous in the page
    for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {
      const int h = i / Dh, d = i - h * Dh;
      const size_t dst = (((size_t)pg * Hkv + h) * page + row) * Dh + d;
      const size_t src = (size_t)t * ld + i;
      if (sizeof(T) == 2) {
        *reinterpret_cast<uint4*>(k_pool + dst) = *reinterpret_cast<const uint4*>(k_src + src);
        *reinterpret_cast<uint4*>(v_pool + dst) = *reinterpret_cast<const uint4*>(v_src + src);
      } else {
#pragma unroll
        for (int e = 0; e < 8; e += 4) {
          *reinterpret_cast<float4*>(k_pool + dst + e) = *reinterpret_cast<const float4*>(k_src + src + e);
          *reinterpret_cast<float4*>(v_pool + dst + e) = *reinterpret_cast<const float4*>(v_src + src + e);
        }
      }
    }
    return;
  }
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
                         T* __restrict__ out, int ldo, const int* __restrict__ rows, int n_tokens,
                         int* __restrict__ status) {
  extern __shared__ float sq[];  // [warps][Dh]
  pdl_trigger();
  pdl_wait();
  q = after_wait(q);
  k_pool = after_wait(k_pool);
  v_pool = after_wait(v_pool);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int w = blockIdx.x * (blockDim.x >> 5) + warp;
  if (w >= n_tokens * Hq) return;
  const int ti = w / Hq, h = w - ti * Hq;
  const int t = rows ? rows[ti] : ti;
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
  const int threads = Hkv * Dh >= 2048 ? 256 : (Hkv * Dh >= 1024 ? 128 : 64);
  if (dtype == MLXB_F32)
    launch_pdl(kv_write_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)k_src,
               (const float*)v_src, ld, positions, token_req, block_table, max_pages, n_pages, page, Hkv, Dh,
               (float*)k_pool, (float*)v_pool, status);
  else if (dtype == MLXB_BF16)
    launch_pdl(kv_write_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream,
               (const __nv_bfloat16*)k_src, (const __nv_bfloat16*)v_src, ld, positions, token_req, block_table,
               max_pages, n_pages, page, Hkv, Dh, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, status);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "kv_write: dtype code %d", dtype);
  return mlxb_check_launch("kv_write");
}

// q: [*, >= Hq*Dh] at row stride ldq; out: [*, Hq*Dh] at row stride ldo; rows: int32[n_tokens] token indices to
// process, or null for tokens 0..n_tokens-1.  window <= 0: all keys 0..p.
MLXB_EXPORT int mlxb_attention_generic(int dtype, const void* q, int ldq, const int* positions, const int* token_req,
                                       const int* block_table, int max_pages, int n_pages, int page, int Hq, int Hkv,
                                       int Dh, int window, float scale, const void* k_pool, const void* v_pool,
                                       void* out, int ldo, const int* rows, int n_tokens, int* status,
                                       cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (int e = check_common("attention", page, Hq, Hkv, Dh)) return e;
  const int warps = 4;
  const long long total = (long long)n_tokens * Hq;
  const int blocks = (int)((total + warps - 1) / warps);
  const size_t smem = (size_t)warps * Dh * sizeof(float);
  if (dtype == MLXB_F32)
    launch_pdl(attention_generic_kernel<float>, dim3(blocks), dim3(warps * 32), smem, stream,
        (const float*)q, ldq, positions, token_req, block_table, max_pages, n_pages, page, Hq, Hkv, Dh, window, scale,
        (const float*)k_pool, (const float*)v_pool, (float*)out, ldo, rows, n_tokens, status);
  else if (dtype == MLXB_BF16)
    launch_pdl(attention_generic_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, stream,
        (const __nv_bfloat16*)q, ldq, positions, token_req, block_table, max_pages, n_pages, page, Hq, Hkv, Dh, window,
        scale, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, ldo, rows, n_tokens,
        status);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "attention: dtype code %d", dtype);
  return mlxb_check_launch("attention (generic)");
}


// ---------------------------------------------------------------- single-token rows

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}


// Raw 8-element rows as they come from memory; converted to float only when used, so that many
// keys can be in flight per thread.
template <typename T> struct Raw8;
template <> struct Raw8<__nv_bfloat16> {
  uint4 u;
  // keys and values are read once: they need no place in L1 (16 and 32 rows: a step 2-3 % faster)
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p));
  }
  // past L1: for a row whose cache line may have been fetched before its last writer finished
  __device__ __forceinline__ void load_fresh(const __nv_bfloat16* p) { u = __ldcg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void zero() { u = make_uint4(0u, 0u, 0u, 0u); }
  __device__ __forceinline__ void get(float (&v)[8]) const {
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <> struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = *reinterpret_cast<const float4*>(p);
    b = *reinterpret_cast<const float4*>(p + 4);
  }
  __device__ __forceinline__ void load_fresh(const float* p) {
    a = __ldcg(reinterpret_cast<const float4*>(p));
    b = __ldcg(reinterpret_cast<const float4*>(p + 4));
  }
  __device__ __forceinline__ void zero() { a = make_float4(0.f, 0.f, 0.f, 0.f); b = a; }
  __device__ __forceinline__ void get(float (&v)[8]) const {
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};

// partial: float [n_rows][Hq][n_chunks_max][Dh + 2] = (m, l, o[Dh]) per chunk.
// DEC_THREADS: 512 when there are no more (row, head) pairs than SMs (one CTA streams a whole row's keys with
// many loads in flight), 256 when there are more (two CTAs per SM, so that one CTA's merge overlaps the
// other's loads; a third CTA per SM would need 80 registers a thread, and the spills cost more than it gains).
template <typename T, int TPK, int DEC_THREADS>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(const T* __restrict__ q, int ldq, const int* __restrict__ rows,
                        const int* __restrict__ positions, const int* __restrict__ token_req,
                        const int* __restrict__ block_table, int max_pages, int n_pages, int page, int Hq, int Hkv,
                        int Dh, int window, float scale, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                        float* partial, int* counters, int n_chunks_max, int chunk, T* __restrict__ out, int ldo,
                        int* __restrict__ status) {
  constexpr int GROUPS = DEC_THREADS / TPK;
  constexpr int U = sizeof(T) == 2 ? 8 : 4;   // keys in flight per thread
  extern __shared__ float sm[];               // per warp: m | l | o[Dh]
  __shared__ int s_last;
  // The kernel before this one wrote the queries and, into the pages, the key and value of each row's own
  // position.  Everything else this kernel reads is older: the step's inputs (requests, positions, block
  // tables) and the keys and values of earlier positions.  So the chain of dependent loads (request ->
  // page ids -> first batch of keys and values) goes out before the wait for that kernel, and only the
  // query and the row's own key and value are fetched after it.
  pdl_trigger();
  const int c = blockIdx.x, h = blockIdx.y, ri = blockIdx.z;
  const int t = rows ? rows[ri] : ri;
  const int grp = threadIdx.x / TPK, j = threadIdx.x % TPK;
  const int d0 = 8 * j;
  const bool active = d0 < Dh;
  const int r = token_req[t];
  const int p = positions[t];
  if (r < 0) return;
  // A position the chunks do not cover has no CTA for its last chunk: the merge below would wait for a
  // ticket that never comes.  Every CTA of such a row reports it and leaves before any ticket is taken, so
  // the row's counter stays zero (the row's output is not written).
  if (p < 0 || p / chunk >= n_chunks_max) {
    if (threadIdx.x == 0) atomicOr(status, MLXB_ST_POSITION_RANGE);
    return;
  }
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int k_begin = max(lo, c * chunk), k_end = min(p + 1, (c + 1) * chunk);
  if (k_begin >= k_end) return;
  const int c0 = lo / chunk, c1 = p / chunk;   // the chunks of this row that hold keys
  const int hk = h / (Hq / Hkv);
  const int* bt = block_table + (size_t)r * max_pages;
  const int shift = __ffs(page) - 1;

  float m = -INFINITY, l = 0.f, o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = 0.f;

  const int n_keys = k_end - k_begin;
  const int iters = (n_keys + GROUPS * U - 1) / (GROUPS * U);
  int pg_next[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int key = k_begin + u * GROUPS + grp;
    const int lp = key >> shift;
    pg_next[u] = (key < k_end && lp < max_pages) ? bt[lp] : -1;
  }
  Raw8<T> kr[U], vr[U];
  bool ok[U];
  // All key and value rows of batch `it`; the page ids were fetched one batch ahead.  With `early`, the
  // row's own position is left for fetch_own(): it is not in memory yet.
  auto fetch = [&](int it, bool early) {
    int pg[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int key = k_begin + (it * U + u) * GROUPS + grp;
      ok[u] = key < k_end;
      pg[u] = pg_next[u];
      const int nkey = key + U * GROUPS, nlp = nkey >> shift;
      pg_next[u] = (nkey < k_end && nlp < max_pages) ? bt[nlp] : -1;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int key = k_begin + (it * U + u) * GROUPS + grp;
      if (ok[u] && (pg[u] < 0 || pg[u] >= n_pages)) {
        if (j == 0) atomicOr(status, pg[u] < 0 ? MLXB_ST_POSITION_RANGE : MLXB_ST_PAGE_RANGE);
        ok[u] = false;
      }
      if (ok[u] && active && !(early && key == p)) {
        const size_t off = (((size_t)pg[u] * Hkv + hk) * page + (key & (page - 1))) * Dh + d0;
        kr[u].load(k_pool + off);
        vr[u].load(v_pool + off);
      } else {
        kr[u].zero();
        vr[u].zero();
      }
    }
  };
  fetch(0, true);
  int own_pg = -1;   // page of the row's own position, if it belongs to this chunk's first batch
  if (p >= k_begin && p < k_end && p - k_begin < GROUPS * U) {
    const int lp = p >> shift;
    own_pg = lp < max_pages ? bt[lp] : -1;
  }
  pdl_wait();
  const T* q_now = after_wait(q);
  const T* k_now = after_wait(k_pool);
  const T* v_now = after_wait(v_pool);
  float qv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) qv[i] = 0.f;
  if (active) load8<T>(q_now + (size_t)t * ldq + h * Dh + d0, qv);
  if (own_pg >= 0 && own_pg < n_pages && active && (p - k_begin) % GROUPS == grp) {
    const int u_own = (p - k_begin) / GROUPS;
    const size_t off = (((size_t)own_pg * Hkv + hk) * page + (p & (page - 1))) * Dh + d0;
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (u == u_own) {
        kr[u].load_fresh(k_now + off);
        vr[u].load_fresh(v_now + off);
      }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) qv[i] *= scale;

  for (int it = 0; it < iters; ++it) {
    if (it > 0) fetch(it, false);   // these rows are older than this step, whichever pointer they are read through
    float sc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[8];
      kr[u].get(kf);
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s = fmaf(qv[i], kf[i], s);
#pragma unroll
      for (int w = TPK / 2; w > 0; w >>= 1) s += __shfl_xor_sync(0xffffffffu, s, w);
      sc[u] = ok[u] ? s : -INFINITY;
    }
    float m_new = m;
#pragma unroll
    for (int u = 0; u < U; ++u) m_new = fmaxf(m_new, sc[u]);
    if (m_new != -INFINITY) {               // one rescale per batch instead of one per key
      const float corr = expf(m - m_new);   // exp(-inf) = 0 for the first batch
      l *= corr;
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] *= corr;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float pw = expf(sc[u] - m_new);   // 0 for keys that are not there
        float vf[8];
        vr[u].get(vf);
        l += pw;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = fmaf(pw, vf[i], o[i]);
      }
      m = m_new;
    }
  }

  // Merge the thread groups: first the groups of a warp with shuffles (lanes that hold the same
  // dims of different groups are TPK apart), then the warps through shared memory.
#pragma unroll
  for (int w = TPK; w < 32; w <<= 1) {
    const float m_o = __shfl_xor_sync(0xffffffffu, m, w);
    const float l_o = __shfl_xor_sync(0xffffffffu, l, w);
    const float m_n = fmaxf(m, m_o);
    const float wa = m == -INFINITY ? 0.f : expf(m - m_n), wb = m_o == -INFINITY ? 0.f : expf(m_o - m_n);
    l = l * wa + l_o * wb;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float o_o = __shfl_xor_sync(0xffffffffu, o[i], w);
      o[i] = o[i] * wa + o_o * wb;
    }
    m = m_n;
  }
  constexpr int NWARP = DEC_THREADS / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* sm_m = sm;                 // [NWARP]
  float* sm_l = sm + NWARP;         // [NWARP]
  float* sm_o = sm + 2 * NWARP;     // [NWARP][Dh]
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
  if (lane < TPK && active) {
#pragma unroll
    for (int i = 0; i < 8; ++i) sm_o[warp * Dh + d0 + i] = o[i];
  }
  __syncthreads();
  if (c0 == c1 && threadIdx.x >= Dh) return;   // single chunk: only Dh threads have work left
  float M = -INFINITY;
#pragma unroll
  for (int w2 = 0; w2 < NWARP; ++w2) M = fmaxf(M, sm_m[w2]);
  float wgt[NWARP];
  float L = 0.f;
#pragma unroll
  for (int w2 = 0; w2 < NWARP; ++w2) {
    wgt[w2] = sm_m[w2] == -INFINITY ? 0.f : expf(sm_m[w2] - M);
    L = fmaf(sm_l[w2], wgt[w2], L);
  }

  if (c0 == c1) {   // the only chunk of this row: no partial results, no ticket
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int d = threadIdx.x; d < Dh; d += DEC_THREADS) {
      float acc = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < NWARP; ++w2) acc = fmaf(wgt[w2], sm_o[w2 * Dh + d], acc);
      out[(size_t)t * ldo + h * Dh + d] = from_f<T>(acc * inv);
    }
    return;
  }

  float* dst = partial + (((size_t)ri * Hq + h) * n_chunks_max + c) * (Dh + 2);
  for (int d = threadIdx.x; d < Dh; d += DEC_THREADS) {
    float acc = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < NWARP; ++w2) acc = fmaf(wgt[w2], sm_o[w2 * Dh + d], acc);
    dst[2 + d] = acc;
  }
  if (threadIdx.x == 0) {
    dst[0] = M;
    dst[1] = L;
  }

  // The last CTA of this (row, head) to get here combines all chunks, in chunk order.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&counters[ri * Hq + h], 1);
    s_last = (ticket == c1 - c0);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* src = partial + ((size_t)ri * Hq + h) * n_chunks_max * (Dh + 2);
  float Mx = -INFINITY;
  for (int cc = c0; cc <= c1; ++cc) Mx = fmaxf(Mx, __ldcg(src + (size_t)cc * (Dh + 2)));   // independent loads
  float Ls = 0.f;
  for (int cc = c0; cc <= c1; ++cc)
    Ls += __ldcg(src + (size_t)cc * (Dh + 2) + 1) * expf(__ldcg(src + (size_t)cc * (Dh + 2)) - Mx);
  const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
  for (int d = threadIdx.x; d < Dh; d += DEC_THREADS) {
    float acc = 0.f;
    for (int cc = c0; cc <= c1; ++cc)
      acc = fmaf(expf(__ldcg(src + (size_t)cc * (Dh + 2)) - Mx), __ldcg(src + (size_t)cc * (Dh + 2) + 2 + d), acc);
    out[(size_t)t * ldo + h * Dh + d] = from_f<T>(acc * inv);
  }
  if (threadIdx.x == 0) counters[ri * Hq + h] = 0;   // ready for the next call
}

template <typename T>
static int launch_decode(const void* q, int ldq, const int* rows, const int* positions, const int* token_req,
                         const int* block_table, int max_pages, int n_pages, int page, int Hq, int Hkv, int Dh,
                         int window, float scale, const void* k_pool, const void* v_pool, float* partial,
                         int* counters, int n_chunks_max, int chunk, void* out, int ldo, int n_rows, int* status,
                         cudaStream_t stream) {
  const int chunks8 = (Dh + 7) / 8;
  int tpk = 2;
  while (tpk < chunks8) tpk <<= 1;
  const dim3 grid(n_chunks_max, Hq, n_rows);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  // more (row, head, chunk) CTAs than SMs: several smaller CTAs per SM
  const bool many = (long long)n_rows * Hq * n_chunks_max > sms;
#define DEC2(TPK_, TH_)                                                                                              \
  {                                                                                                                  \
    const size_t smem = (size_t)(TH_ / 32) * (Dh + 2) * sizeof(float);                                               \
    launch_pdl(attention_decode_kernel<T, TPK_, TH_>, grid, dim3(TH_), smem, stream, (const T*)q, ldq, rows,         \
               positions, token_req, block_table, max_pages, n_pages, page, Hq, Hkv, Dh, window, scale,              \
               (const T*)k_pool, (const T*)v_pool, partial, counters, n_chunks_max, chunk, (T*)out, ldo, status);    \
  }
#define DEC(TPK_) { if (many) DEC2(TPK_, 256) else DEC2(TPK_, 512) }
  if (tpk == 2) DEC(2) else if (tpk == 4) DEC(4) else if (tpk == 8) DEC(8) else if (tpk == 16) DEC(16) else DEC(32)
#undef DEC
#undef DEC2
  return mlxb_check_launch("attention (single-token rows)");
}

// Floats of scratch that n_rows rows need.
MLXB_EXPORT long long mlxb_attention_decode_scratch(int n_rows, int Hq, int Dh, int n_chunks_max) {
  return (long long)n_rows * Hq * n_chunks_max * (Dh + 2);
}

// Rows with one query each.  rows: int32[n_rows] token indices or null (tokens 0..n_rows-1).
// n_chunks_max * chunk should cover every position a row may have: a row whose position lies beyond gets no
// output and sets MLXB_ST_POSITION_RANGE in *status (its counter stays zero).  partial: float32 scratch of
// mlxb_attention_decode_scratch() floats, contents need not be initialised; counters: int32[n_rows * Hq]
// that must be ZERO before the first call and are left zero by every call.
// Dh must be a multiple of 8 (16 for bfloat16 alignment is implied by pages); q rows 16-byte aligned.
MLXB_EXPORT int mlxb_attention_decode(int dtype, const void* q, int ldq, const int* rows, const int* positions,
                                      const int* token_req, const int* block_table, int max_pages, int n_pages,
                                      int page, int Hq, int Hkv, int Dh, int window, float scale, const void* k_pool,
                                      const void* v_pool, float* partial, int* counters, int n_chunks_max, int chunk,
                                      void* out, int ldo, int n_rows, int* status, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (int e = check_common("attention (single-token rows)", page, Hq, Hkv, Dh)) return e;
  if (Dh % 8) return mlxb_fail(MLXB_BAD_ARG, "attention (single-token rows): head size %d is not a multiple of 8", Dh);
  if (chunk <= 0 || n_chunks_max <= 0 || n_chunks_max > 65535 || n_rows > 65535 || Hq > 65535)
    return mlxb_fail(MLXB_BAD_ARG, "attention (single-token rows): chunk %d x %d, %d rows, %d heads", chunk,
                     n_chunks_max, n_rows, Hq);
  const int esz = dtype == MLXB_F32 ? 4 : 2;
  if (((uintptr_t)q & 15) || ((size_t)ldq * esz) % 16 || ((size_t)Dh * esz) % 16)
    return mlxb_fail(MLXB_BAD_ARG, "attention (single-token rows): query rows and heads must be 16-byte aligned");
  if (dtype == MLXB_F32)
    return launch_decode<float>(q, ldq, rows, positions, token_req, block_table, max_pages, n_pages, page, Hq, Hkv,
                                Dh, window, scale, k_pool, v_pool, partial, counters, n_chunks_max, chunk, out, ldo,
                                n_rows, status, stream);
  if (dtype == MLXB_BF16)
    return launch_decode<__nv_bfloat16>(q, ldq, rows, positions, token_req, block_table, max_pages, n_pages, page, Hq,
                                        Hkv, Dh, window, scale, k_pool, v_pool, partial, counters, n_chunks_max, chunk,
                                        out, ldo, n_rows, status, stream);
  return mlxb_fail(MLXB_BAD_DTYPE, "attention (single-token rows): dtype code %d", dtype);
}

// ---------------------------------------------------------------- no-allocation variant
// Declared and documented in attention_noalloc.h.
#include "attention_noalloc.h"

// Scratch for the per-chunk partial results, owned by the library.  In host code this name is only
// a handle for the runtime: the address kernels can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_partial[MLXB_NOALLOC_SCRATCH_FLOATS];

// Ticket counters of the kernel, one per (row, head); zero when the library is loaded and left zero by every call.
static __device__ __align__(256) int g_noalloc_counters[MLXB_NOALLOC_COUNTERS];

static float* g_noalloc_partial_ptr[64];   // device addresses of the arrays, per device ordinal
static int* g_noalloc_counters_ptr[64];

MLXB_EXPORT int mlxb_attention_decode_noalloc(int dtype, const void* q, int ldq, const int* rows,
                                              const int* positions, const int* token_req, const int* block_table,
                                              int max_pages, int n_pages, int page, int n_q_heads, int n_kv_heads,
                                              int head_dim, int window, float scale, const void* k_pool,
                                              const void* v_pool, int n_chunks_max, int chunk, void* out, int ldo,
                                              int n_rows, int* status, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (n_q_heads <= 0 || head_dim <= 0 || n_chunks_max <= 0)
    return mlxb_fail(MLXB_BAD_ARG, "attention (no allocation): %d heads of %d, %d chunks", n_q_heads, head_dim,
                     n_chunks_max);
  const long long need = mlxb_attention_decode_scratch(n_rows, n_q_heads, head_dim, n_chunks_max);
  if (need > (long long)MLXB_NOALLOC_SCRATCH_FLOATS)
    return mlxb_fail(MLXB_BAD_ARG,
                     "attention (no allocation): %d rows x %d heads x %d chunks x (%d + 2) = %lld floats of scratch, "
                     "the built-in array holds %d",
                     n_rows, n_q_heads, n_chunks_max, head_dim, need, (int)MLXB_NOALLOC_SCRATCH_FLOATS);
  if ((long long)n_rows * n_q_heads > (long long)MLXB_NOALLOC_COUNTERS)
    return mlxb_fail(MLXB_BAD_ARG, "attention (no allocation): %d rows x %d heads, the built-in counters hold %d",
                     n_rows, n_q_heads, (int)MLXB_NOALLOC_COUNTERS);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return mlxb_fail((int)e, "attention (no allocation): cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return mlxb_fail(MLXB_BAD_ARG, "attention (no allocation): device ordinal %d", dev);
  if (g_noalloc_partial_ptr[dev] == nullptr) {   // first call on this device (it is current): look the address up
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_partial);
    if (e != cudaSuccess || p == nullptr)
      return mlxb_fail(e != cudaSuccess ? (int)e : MLXB_BAD_ARG,
                       "attention (no allocation): cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    int* cnt = nullptr;
    e = cudaGetSymbolAddress((void**)&cnt, g_noalloc_counters);
    if (e != cudaSuccess || cnt == nullptr)
      return mlxb_fail(e != cudaSuccess ? (int)e : MLXB_BAD_ARG,
                       "attention (no allocation): cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_noalloc_counters_ptr[dev] = cnt;
    g_noalloc_partial_ptr[dev] = p;
  }
  return mlxb_attention_decode(dtype, q, ldq, rows, positions, token_req, block_table, max_pages, n_pages, page,
                               n_q_heads, n_kv_heads, head_dim, window, scale, k_pool, v_pool,
                               g_noalloc_partial_ptr[dev], g_noalloc_counters_ptr[dev], n_chunks_max, chunk, out, ldo,
                               n_rows, status, stream);
}
