// A whole decode step in one persistent kernel.
//
// A step in which every request brings one token is a chain of some hundred and seventy small
// dependent kernels; each link costs a launch gap and a cold start (index arithmetic, first loads)
// of several microseconds, an order of magnitude more than streaming its weights takes.  Here the
// chain is data: a table of phases (embedding, norm, linear layer, attention over the pages), built
// on the host from the very launches a step issues, and one kernel with one CTA per SM walks the
// table.  Between phases the CTAs meet at a barrier in global memory (about 1.4 us on 148 SMs);
// while a phase runs, every CTA asks L2 for its share of the next phase's weights, so the weight
// stream from HBM does not stop at phase boundaries.
//
// What a phase does:
//   embed      x[m] = wte[token[m]] * scale + wpe[position[m]]
//   norm       y[m] = LayerNorm(x[rows[m]])
//   linear     C = epilogue(LayerNorm?(A) . W^T + bias) (+ residual); the norm of the input rows, when
//              asked for, is applied while the activation fragments are loaded (its statistics are
//              computed by every CTA for itself: a few rows, cheaper than one more barrier); an output
//              that is a fused [q | k | v] projection scatters k and v into the pages
//   attention  one query per row over the row's pages, keys split over the threads of a CTA and, for
//              long rows, over chunks that the last CTA to finish merges
// Arithmetic and orders of summation follow the single kernels of the chain (gemm_smallm.cu,
// norm.cu, attention.cu): bfloat16 operands, float32 accumulation, statistics, softmax and sums.
//
// Every CTA must be resident at once, so the kernel is launched cooperatively (the launch fails
// rather than deadlocks if it does not fit).  Every wait is bounded: a CTA that waits too long sets
// MLXB_ST_WAIT_TIMEOUT in the status word and returns, and so do the others when their own waits
// run out.  After such an abort the three synchronisation words must be zeroed before the next launch.
//
// Activations written in one phase and read in the next by other SMs are read with ld.global.cg
// (L2 only); weights, gains and biases, which nothing writes, go through the read-only path.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

#ifndef MLXB_DP_TPK
#define MLXB_DP_TPK 8        // threads that share one key in the attention phase: the power of two >= head_dim / 8
#endif

enum { DP_EMBED = 1, DP_NORM = 2, DP_LINEAR = 3, DP_ATTENTION = 4 };
enum { DPF_LN = 1, DPF_GELU = 2, DPF_OUT_F32 = 4, DPF_SCATTER = 8 };

constexpr int DP_THREADS = 512;
constexpr int DP_WARPS = DP_THREADS / 32;

// One entry of the table.  The Python side mirrors this layout field by field
// (mlx_lm_b200/ops/program.py); mlxb_decode_program_phase_bytes() lets it check the size.
struct Phase {
  const void* A;            // embed: wte; norm: x; linear: input rows; attention: q
  const void* W;            // embed: wpe or null; linear: weight [N, K]
  const float* bias;        // linear: bias or null; norm: bias or null
  const float* ln_gain;     // norm / linear with DPF_LN
  const float* ln_bias;     // may be null
  const int* rows;          // norm / linear with DPF_LN: input row of output row m, or null; attention: token rows or null
  const void* residual;     // linear: bfloat16 [M, ldc] or null
  void* C;                  // output
  void* k_pool;             // [n_pages, Hkv, page, Dh]
  void* v_pool;
  const int* block_table;   // [*, max_pages]
  const int* tokens;        // embed
  const int* positions;     // embed, scatter, attention
  const int* token_req;     // scatter, attention
  float* partial;           // attention scratch
  int* counters;            // attention tickets
  const void* next_w;       // weights to ask L2 for while this phase runs
  long long next_bytes;
  int op, flags, M, N, K, lda, ldc;
  int max_pages, n_pages, page, Hq, Hkv, Dh, window, q_width;
  int n_chunks_max, chunk, vocab, n_pos;
  float eps, scale, embed_scale;
  int pad_;
};

struct Header {
  const Phase* phases;
  int n_phases;
  unsigned* sync;   // [0] arrivals, never reset; [1] value of [0] when this launch began; [2] exit tickets
  int* status;
  unsigned long long* trace;   // null, or 2 * n_phases words: CTA 0's clock (ns) when each phase began and ended
};

// ------------------------------------------------------------------------------------------ memory helpers
__device__ __forceinline__ uint4 ld_w(const void* p) {     // weights: read-only path, no L1 allocation
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_act(const void* p) {   // activations and pages: L2 is the point of coherence
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ int ld_act_i32(const int* p) {
  int v;
  asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_act_bf16(const __nv_bfloat16* p) {
  unsigned short v;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return __uint_as_float((unsigned)v << 16);
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_inc(unsigned* p) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ------------------------------------------------------------------------------------------ the barrier
// All CTAs of the grid; `target` is the value the arrival counter has once everybody has arrived.
// False when the wait gave up (status bit set): the caller returns at once.
constexpr unsigned DP_SPIN_FAST = 1u << 14, DP_SPIN_LIMIT = 1u << 21;   // about a second in all

__device__ __forceinline__ bool grid_barrier(unsigned* arrivals, unsigned target, int* status, int* s_flag) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    red_release_inc(arrivals);
    unsigned spins = 0;
    int good = 1;
    while ((int)(ld_acquire_u32(arrivals) - target) < 0) {
      if (++spins > DP_SPIN_LIMIT) {
        atomicOr(status, MLXB_ST_WAIT_TIMEOUT);
        good = 0;
        break;
      }
      if (spins > DP_SPIN_FAST) __nanosleep(256);
    }
    __threadfence();
    *s_flag = good;
  }
  __syncthreads();
  return *s_flag != 0;
}

// Ask L2 for this CTA's share of [p, p + bytes).
__device__ __forceinline__ void prefetch_share(const void* p, long long bytes) {
  if (p == nullptr || bytes <= 0) return;
  const long long lines = (bytes + 127) >> 7;
  const long long per = (lines + gridDim.x - 1) / gridDim.x;
  const long long l0 = (long long)blockIdx.x * per, l1 = min(lines, l0 + per);
  const char* base = reinterpret_cast<const char*>(p);
  for (long long l = l0 + threadIdx.x; l < l1; l += DP_THREADS)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(base + (l << 7)));
}

// ------------------------------------------------------------------------------------------ norm statistics
__device__ __forceinline__ void row_stats(const __nv_bfloat16* xr, int D, float eps, int lane, float& mean,
                                          float& rstd) {
  row_stats_bf16(xr, D, eps, lane, mean, rstd, [](const __nv_bfloat16* p) { return ld_act(p); });
}

// ------------------------------------------------------------------------------------------ phases
__device__ __forceinline__ void embed_phase(const Phase* ph, int* status) {
  const int M = ph->M, D = ph->N, V = ph->vocab, P = ph->n_pos;
  const __nv_bfloat16* wte = (const __nv_bfloat16*)ph->A;
  const __nv_bfloat16* wpe = (const __nv_bfloat16*)ph->W;
  __nv_bfloat16* out = (__nv_bfloat16*)ph->C;
  const float scale = ph->embed_scale;
  for (int m = blockIdx.x; m < M; m += gridDim.x) {
    const int id = ld_act_i32(ph->tokens + m);
    const int p = wpe ? ld_act_i32(ph->positions + m) : 0;
    bool ok = true;
    if (id < 0 || id >= V) { ok = false; if (threadIdx.x == 0) atomicOr(status, MLXB_ST_TOKEN_RANGE); }
    if (wpe && (p < 0 || p >= P)) { ok = false; if (threadIdx.x == 0) atomicOr(status, MLXB_ST_POSITION_RANGE); }
    for (int d = threadIdx.x * 8; d < D; d += DP_THREADS * 8) {
      float o[8];
      if (ok) {
        float e[8];
        unpack8(ld_w(wte + (size_t)id * D + d), e);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = e[i] * scale;
        if (wpe) {
          float q[8];
          unpack8(ld_w(wpe + (size_t)p * D + d), q);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += q[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = 0.f;
      }
      *reinterpret_cast<uint4*>(out + (size_t)m * D + d) = pack8(o);
    }
  }
}

__device__ __forceinline__ void norm_phase(const Phase* ph) {
  const int R = ph->M, D = ph->K;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* x = (const __nv_bfloat16*)ph->A;
  __nv_bfloat16* y = (__nv_bfloat16*)ph->C;
  for (int r = blockIdx.x * DP_WARPS + warp; r < R; r += gridDim.x * DP_WARPS) {
    const __nv_bfloat16* xr = x + (size_t)(ph->rows ? ld_act_i32(ph->rows + r) : r) * D;
    float mean, rstd;
    row_stats(xr, D, ph->eps, lane, mean, rstd);
    for (int d = lane * 8; d < D; d += 256)
      *reinterpret_cast<uint4*>(y + (size_t)r * D + d) = normalise8(ld_act(xr + d), mean, rstd, ph->ln_gain, ph->ln_bias, d);
  }
}

// MT: 16-row token tiles; NW: 8-column weight tiles of one pass.  A CTA owns a contiguous range of the
// 8-column tiles of the output and walks it in passes of NW; its 16 warps share the K blocks of a pass.
template <int MT, int NW>
__device__ __forceinline__ void linear_phase(const Phase* ph, float* smem, int* status) {
  constexpr int PER = MT * NW * 4;
  float* part = smem;                          // [DP_WARPS][PER][32]
  float* s_mean = smem + DP_WARPS * PER * 32;  // [16 * MT]
  float* s_rstd = s_mean + 16 * MT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int M = ph->M, N = ph->N, K = ph->K, lda = ph->lda, ldc = ph->ldc, flags = ph->flags;
  const __nv_bfloat16* A = (const __nv_bfloat16*)ph->A;
  const __nv_bfloat16* W = (const __nv_bfloat16*)ph->W;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const int tiles = (N + 7) >> 3;
  const int t_begin = (int)((long long)blockIdx.x * tiles / gridDim.x);
  const int t_end = (int)((long long)(blockIdx.x + 1) * tiles / gridDim.x);
  if (t_begin >= t_end) return;
  const bool ln = flags & DPF_LN;
  const float* gain = ph->ln_gain;
  const float* lbias = ph->ln_bias;

  const int n_blocks = (K + 31) >> 5;
  constexpr int UNROLL = (MT * NW >= 8) ? 1 : 2;   // K blocks per warp and iteration
  constexpr int STEP = DP_WARPS * UNROLL;

  const __nv_bfloat16* wrow[NW];
  bool wok[NW];
  auto set_pass = [&](int t0) {
#pragma unroll
    for (int j = 0; j < NW; ++j) {
      const int n = (t0 + j) * 8 + g;
      wok[j] = (t0 + j) < t_end && n < N;
      wrow[j] = W + (size_t)(wok[j] ? n : 0) * K + 8 * q;
    }
  };
  auto load_w = [&](int kb, uint4 (&dst)[UNROLL][NW]) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb + u * DP_WARPS) * 32;
      const bool kin = (kb + u * DP_WARPS) < n_blocks && (k + 8 * q) < K;   // K % 8 == 0: a chunk is all in or all out
#pragma unroll
      for (int j = 0; j < NW; ++j) dst[u][j] = (kin && wok[j]) ? ld_w(wrow[j] + k) : zero;
    }
  };
  // the first weight fragments do not depend on the activations: they go out before the statistics
  uint4 wv[UNROLL][NW];
  set_pass(t_begin);
  load_w(warp, wv);

  if (ln) {
    for (int m = warp; m < M; m += DP_WARPS) {
      const __nv_bfloat16* xr = A + (size_t)(ph->rows ? ld_act_i32(ph->rows + m) : m) * lda;
      float mean, rstd;
      row_stats(xr, K, ph->eps, lane, mean, rstd);
      if (lane == 0) { s_mean[m] = mean; s_rstd[m] = rstd; }
    }
    __syncthreads();
  }
  const __nv_bfloat16* arow[MT][2];
  bool aok[MT][2];
  float mu[MT][2], rs[MT][2];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = i * 16 + h * 8 + g;
      aok[i][h] = m < M;
      const int mm = aok[i][h] ? m : 0;
      arow[i][h] = A + (size_t)((ln && ph->rows) ? ld_act_i32(ph->rows + mm) : mm) * lda + 8 * q;
      mu[i][h] = ln ? s_mean[mm] : 0.f;
      rs[i][h] = ln ? s_rstd[mm] : 1.f;
    }
  auto load_a = [&](int kb, uint4 (&dst)[UNROLL][MT][2]) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb + u * DP_WARPS) * 32;
      const bool kin = (kb + u * DP_WARPS) < n_blocks && (k + 8 * q) < K;
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (kin && aok[i][h]) {
            const uint4 raw = ld_act(arow[i][h] + k);
            dst[u][i][h] = ln ? normalise8(raw, mu[i][h], rs[i][h], gain, lbias, k + 8 * q) : raw;
          } else {
            dst[u][i][h] = zero;
          }
        }
    }
  };

  for (int t0 = t_begin; t0 < t_end; t0 += NW) {
    float acc[MT][NW][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NW; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

    for (int kb = warp; kb < n_blocks; kb += STEP) {
      uint4 av[UNROLL][MT][2], wn[UNROLL][NW];
      load_a(kb, av);
      load_w(kb + STEP, wn);          // the next iteration's weights are in flight while this one multiplies
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int j = 0; j < NW; ++j) {
            mma_bf16(acc[i][j], av[u][i][0].x, av[u][i][1].x, av[u][i][0].y, av[u][i][1].y, wv[u][j].x, wv[u][j].y);
            mma_bf16(acc[i][j], av[u][i][0].z, av[u][i][1].z, av[u][i][0].w, av[u][i][1].w, wv[u][j].z, wv[u][j].w);
          }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
#pragma unroll
        for (int j = 0; j < NW; ++j) wv[u][j] = wn[u][j];
    }
    const int n0 = t0 * 8;
    const int n_pass = min(NW, t_end - t0) * 8;   // columns of this pass
    if (t0 + NW < t_end) {                        // the next pass's first weights go out before the reduction
      set_pass(t0 + NW);
      load_w(warp, wv);
    }
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NW; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) part[(warp * PER + (i * NW + j) * 4 + c) * 32 + lane] = acc[i][j][c];
    __syncthreads();
    for (int e = threadIdx.x; e < PER * 32; e += DP_THREADS) {
      const int idx = e >> 5, l2 = e & 31;
      const int c = idx & 3, j = (idx >> 2) % NW, i = (idx >> 2) / NW;
      const int m = i * 16 + (l2 >> 2) + ((c & 2) ? 8 : 0);
      const int nl = j * 8 + 2 * (l2 & 3) + (c & 1);
      const int n = n0 + nl;
      if (m >= M || nl >= n_pass || n >= N) continue;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < DP_WARPS; ++w) v += part[w * PER * 32 + e];
      if (ph->bias) v += __ldg(ph->bias + n);
      if (flags & DPF_GELU) v = gelu_new_fast(v);
      if (ph->residual) v += ld_act_bf16((const __nv_bfloat16*)ph->residual + (size_t)m * ldc + n);
      if ((flags & DPF_SCATTER) && n >= ph->q_width) {
        const int r = ld_act_i32(ph->token_req + m);
        if (r >= 0) {
          const int pos = ld_act_i32(ph->positions + m);
          const int lp = pos / ph->page;
          const int pg = (pos >= 0 && lp < ph->max_pages) ? ld_act_i32(ph->block_table + (size_t)r * ph->max_pages + lp) : -2;
          if (pg == -2) {
            atomicOr(status, MLXB_ST_POSITION_RANGE);
          } else if (pg >= ph->n_pages) {
            atomicOr(status, MLXB_ST_PAGE_RANGE);
          } else if (pg >= 0) {
            const int kvw = ph->Hkv * ph->Dh;
            int c2 = n - ph->q_width;
            __nv_bfloat16* pool = (__nv_bfloat16*)ph->k_pool;
            if (c2 >= kvw) { c2 -= kvw; pool = (__nv_bfloat16*)ph->v_pool; }
            const int hh = c2 / ph->Dh, d = c2 - hh * ph->Dh;
            pool[(((size_t)pg * ph->Hkv + hh) * ph->page + (pos % ph->page)) * ph->Dh + d] = __float2bfloat16_rn(v);
          }
        }
      } else if (flags & DPF_OUT_F32) {
        ((float*)ph->C)[(size_t)m * ldc + n] = v;
      } else {
        ((__nv_bfloat16*)ph->C)[(size_t)m * ldc + n] = __float2bfloat16_rn(v);
      }
    }
    __syncthreads();
  }
}

// One (chunk, head, row) of the attention phase: attention_decode_kernel of attention.cu for bfloat16 and
// 512 threads, with loads that see what the phase before wrote.
template <int TPK>
__device__ __forceinline__ void attention_item(const Phase* ph, int c, int h, int ri, float* sm, int* s_last,
                                               int* status) {
  constexpr int GROUPS = DP_THREADS / TPK;
  constexpr int U = 8;   // keys in flight per thread
  constexpr int NWARP = DP_WARPS;
  const int Dh = ph->Dh, Hq = ph->Hq, Hkv = ph->Hkv, page = ph->page, max_pages = ph->max_pages;
  const int n_pages = ph->n_pages, window = ph->window, chunk = ph->chunk, n_chunks_max = ph->n_chunks_max;
  const int ldq = ph->lda, ldo = ph->ldc;
  const __nv_bfloat16* q = (const __nv_bfloat16*)ph->A;
  const __nv_bfloat16* k_pool = (const __nv_bfloat16*)ph->k_pool;
  const __nv_bfloat16* v_pool = (const __nv_bfloat16*)ph->v_pool;
  __nv_bfloat16* out = (__nv_bfloat16*)ph->C;
  const int t = ph->rows ? ld_act_i32(ph->rows + ri) : ri;
  const int grp = threadIdx.x / TPK, j = threadIdx.x % TPK;
  const int d0 = 8 * j;
  const bool active = d0 < Dh;
  float qv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) qv[i] = 0.f;
  if (active) unpack8(ld_act(q + (size_t)t * ldq + h * Dh + d0), qv);
  const int r = ld_act_i32(ph->token_req + t);
  const int p = ld_act_i32(ph->positions + t);
  if (r < 0) return;
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int k_begin = max(lo, c * chunk), k_end = min(p + 1, (c + 1) * chunk);
  if (k_begin >= k_end) return;
  const int c0 = lo / chunk, c1 = p / chunk;   // the chunks of this row that hold keys
  const int hk = h / (Hq / Hkv);
  const int* bt = ph->block_table + (size_t)r * max_pages;
  const int shift = __ffs(page) - 1;
  const float scale = ph->scale;
#pragma unroll
  for (int i = 0; i < 8; ++i) qv[i] *= scale;

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
    pg_next[u] = (key < k_end && lp < max_pages) ? ld_act_i32(bt + lp) : -1;
  }
  for (int it = 0; it < iters; ++it) {
    int pg[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int key = k_begin + (it * U + u) * GROUPS + grp;
      ok[u] = key < k_end;
      pg[u] = pg_next[u];
      const int nkey = key + U * GROUPS, nlp = nkey >> shift;
      pg_next[u] = (nkey < k_end && nlp < max_pages) ? ld_act_i32(bt + nlp) : -1;
    }
    uint4 kr[U], vr[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int key = k_begin + (it * U + u) * GROUPS + grp;
      if (ok[u] && (pg[u] < 0 || pg[u] >= n_pages)) {
        if (j == 0) atomicOr(status, pg[u] < 0 ? MLXB_ST_POSITION_RANGE : MLXB_ST_PAGE_RANGE);
        ok[u] = false;
      }
      if (ok[u] && active) {
        const size_t off = (((size_t)pg[u] * Hkv + hk) * page + (key & (page - 1))) * Dh + d0;
        kr[u] = ld_act(k_pool + off);
        vr[u] = ld_act(v_pool + off);
      } else {
        kr[u] = make_uint4(0u, 0u, 0u, 0u);
        vr[u] = kr[u];
      }
    }
    float sc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[8];
      unpack8(kr[u], kf);
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
    if (m_new != -INFINITY) {
      const float corr = expf(m - m_new);
      l *= corr;
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] *= corr;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float pw = expf(sc[u] - m_new);
        float vf[8];
        unpack8(vr[u], vf);
        l += pw;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = fmaf(pw, vf[i], o[i]);
      }
      m = m_new;
    }
  }

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
  float Mx = -INFINITY;
#pragma unroll
  for (int w2 = 0; w2 < NWARP; ++w2) Mx = fmaxf(Mx, sm_m[w2]);
  float wgt[NWARP];
  float L = 0.f;
#pragma unroll
  for (int w2 = 0; w2 < NWARP; ++w2) {
    wgt[w2] = sm_m[w2] == -INFINITY ? 0.f : expf(sm_m[w2] - Mx);
    L = fmaf(sm_l[w2], wgt[w2], L);
  }
  if (c0 == c1) {
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int d = threadIdx.x; d < Dh; d += DP_THREADS) {
      float acc = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < NWARP; ++w2) acc = fmaf(wgt[w2], sm_o[w2 * Dh + d], acc);
      out[(size_t)t * ldo + h * Dh + d] = __float2bfloat16_rn(acc * inv);
    }
    return;
  }

  float* dst = ph->partial + (((size_t)ri * Hq + h) * n_chunks_max + c) * (Dh + 2);
  for (int d = threadIdx.x; d < Dh; d += DP_THREADS) {
    float acc = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < NWARP; ++w2) acc = fmaf(wgt[w2], sm_o[w2 * Dh + d], acc);
    dst[2 + d] = acc;
  }
  if (threadIdx.x == 0) {
    dst[0] = Mx;
    dst[1] = L;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&ph->counters[ri * Hq + h], 1);
    *s_last = (ticket == c1 - c0);
  }
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  const float* src = ph->partial + ((size_t)ri * Hq + h) * n_chunks_max * (Dh + 2);
  float Mt = -INFINITY;
  for (int cc = c0; cc <= c1; ++cc) Mt = fmaxf(Mt, __ldcg(src + (size_t)cc * (Dh + 2)));
  float Ls = 0.f;
  for (int cc = c0; cc <= c1; ++cc)
    Ls += __ldcg(src + (size_t)cc * (Dh + 2) + 1) * expf(__ldcg(src + (size_t)cc * (Dh + 2)) - Mt);
  const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
  for (int d = threadIdx.x; d < Dh; d += DP_THREADS) {
    float acc = 0.f;
    for (int cc = c0; cc <= c1; ++cc)
      acc = fmaf(expf(__ldcg(src + (size_t)cc * (Dh + 2)) - Mt), __ldcg(src + (size_t)cc * (Dh + 2) + 2 + d), acc);
    out[(size_t)t * ldo + h * Dh + d] = __float2bfloat16_rn(acc * inv);
  }
  if (threadIdx.x == 0) ph->counters[ri * Hq + h] = 0;   // ready for the next step
}

// ------------------------------------------------------------------------------------------ the kernel
template <int MT>
__global__ void __launch_bounds__(DP_THREADS, 1) decode_program_kernel(Header hd) {
  constexpr int NW = MT == 4 ? 2 : 4;
  extern __shared__ float smem[];
  __shared__ int s_flag;
  __shared__ unsigned s_base;
  __shared__ __align__(16) Phase s_phase;
  static_assert(sizeof(Phase) % 16 == 0, "the phase record is copied in 16-byte pieces");
  if (threadIdx.x == 0) s_base = *reinterpret_cast<volatile unsigned*>(hd.sync + 1);
  if (threadIdx.x < sizeof(Phase) / 16)
    reinterpret_cast<uint4*>(&s_phase)[threadIdx.x] = __ldg(reinterpret_cast<const uint4*>(hd.phases) + threadIdx.x);
  __syncthreads();
  const unsigned base = s_base;
  const Phase* ph = &s_phase;
  for (int p = 0; p < hd.n_phases; ++p) {
    if (hd.trace && blockIdx.x == 0 && threadIdx.x == 0) hd.trace[2 * p] = global_ns();
    prefetch_share(ph->next_w, ph->next_bytes);
    const int op = ph->op;
    if (op == DP_EMBED) {
      embed_phase(ph, hd.status);
    } else if (op == DP_NORM) {
      norm_phase(ph);
    } else if (op == DP_LINEAR) {
      linear_phase<MT, NW>(ph, smem, hd.status);
    } else if (op == DP_ATTENTION) {
      const int per_row = ph->Hq * ph->n_chunks_max;
      const int items = ph->M * per_row;
      for (int it = blockIdx.x; it < items; it += gridDim.x) {
        const int ri = it / per_row, rem = it - ri * per_row;
        __syncthreads();   // the item before may still be read from shared memory
        attention_item<MLXB_DP_TPK>(ph, rem % ph->n_chunks_max, rem / ph->n_chunks_max, ri, smem, &s_flag, hd.status);
      }
    }
    if (hd.trace && blockIdx.x == 0) {
      __syncthreads();
      if (threadIdx.x == 0) hd.trace[2 * p + 1] = global_ns();
    }
    if (p + 1 == hd.n_phases) break;
    // the next record is fetched while the others arrive
    uint4 rec = make_uint4(0u, 0u, 0u, 0u);
    if (threadIdx.x < sizeof(Phase) / 16)
      rec = __ldg(reinterpret_cast<const uint4*>(hd.phases + p + 1) + threadIdx.x);
    __syncthreads();   // everybody is done with the current record
    if (threadIdx.x < sizeof(Phase) / 16) reinterpret_cast<uint4*>(&s_phase)[threadIdx.x] = rec;
    if (!grid_barrier(hd.sync, base + (unsigned)(p + 1) * gridDim.x, hd.status, &s_flag)) return;
  }
  // the last CTA out moves the base on for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned tk = atomicAdd(hd.sync + 2, 1u);
    if (tk == gridDim.x - 1) {
      hd.sync[1] = base + (unsigned)(hd.n_phases - 1) * gridDim.x;
      hd.sync[2] = 0u;
    }
  }
}

MLXB_EXPORT int mlxb_decode_program_phase_bytes() { return (int)sizeof(Phase); }
MLXB_EXPORT int mlxb_decode_program_tpk() { return MLXB_DP_TPK; }

// Profiling aid: launches made after this call write CTA 0's clock at the begin and end of every phase to
// `words` (2 * n_phases 64-bit words on the device); null switches it off again.
static unsigned long long* g_trace = nullptr;
MLXB_EXPORT void mlxb_decode_program_trace(void* words) { g_trace = (unsigned long long*)words; }

template <int MT>
static int launch_program(const Header& hd, int grid, cudaStream_t stream) {
  constexpr int NW = MT == 4 ? 2 : 4;
  const size_t smem = ((size_t)DP_WARPS * MT * NW * 4 * 32 + 2 * 16 * MT) * sizeof(float);
  static bool raised = false;
  auto kern = decode_program_kernel<MT>;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return mlxb_fail((int)e, "decode program: shared memory of %zu bytes: %s", smem, cudaGetErrorString(e));
    raised = true;
  }
  int per_sm = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, DP_THREADS, smem);
  if (e != cudaSuccess || per_sm < 1)
    return mlxb_fail(e != cudaSuccess ? (int)e : MLXB_BAD_ARG, "decode program: a CTA of %d threads and %zu bytes does not fit an SM",
                     DP_THREADS, smem);
  Header h = hd;
  void* args[] = {&h};
  e = cudaLaunchCooperativeKernel((void*)kern, dim3(grid), dim3(DP_THREADS), args, smem, stream);
  if (e != cudaSuccess) return mlxb_fail((int)e, "decode program: cooperative launch: %s", cudaGetErrorString(e));
  return 0;
}

// phases: device array of n_phases entries (see Phase); max_rows: the largest M of any phase (<= 64);
// head_dim: of the attention phases (all alike; 0 if there is none); sync: three zeroed 32-bit words on the
// device that belong to this program; status: the engine's status word.
MLXB_EXPORT int mlxb_decode_program(const void* phases, int n_phases, int max_rows, int head_dim, void* sync,
                                    int* status, cudaStream_t stream) {
  if (n_phases <= 0) return 0;
  if (max_rows <= 0 || max_rows > 64) return mlxb_fail(MLXB_BAD_ARG, "decode program: %d rows, at most 64", max_rows);
  if (head_dim > 0) {
    int tpk = 2;
    while (tpk * 8 < head_dim) tpk <<= 1;
    if (tpk != MLXB_DP_TPK || head_dim % 8 || head_dim > 256)
      return mlxb_fail(MLXB_BAD_ARG, "decode program: built for heads of up to %d (more than %d), got %d",
                       8 * MLXB_DP_TPK, MLXB_DP_TPK == 2 ? 0 : 4 * MLXB_DP_TPK, head_dim);
  }
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess || sms <= 0) return mlxb_fail((int)e, "decode program: device query: %s", cudaGetErrorString(e));
  Header hd = {(const Phase*)phases, n_phases, (unsigned*)sync, status, g_trace};
  if (max_rows <= 16) return launch_program<1>(hd, sms, stream);
  if (max_rows <= 32) return launch_program<2>(hd, sms, stream);
  return launch_program<4>(hd, sms, stream);
}
