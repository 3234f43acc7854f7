// Linear layer for few rows (decode steps): M <= 64 tokens against a weight
// that has to be streamed from HBM once.
//   C[M,N] = epilogue(A[M,K] . W[N,K]^T + bias[N]) (+ residual[M,N])
// A, W, residual bfloat16; float32 accumulation; C bfloat16 or float32.
//
// The kernel is bound by reading W, so it is organised around that stream:
// a CTA owns 8*NW output features (rows of W) over the whole K; its 8 (or 16) warps
// take the 32-wide K blocks round robin, so the CTA reads 8 consecutive
// blocks (512 contiguous bytes of each row) at a time, every thread with one
// 16-byte load per row block straight into registers (no shared-memory
// staging), several blocks in flight.  Products run on the tensor cores
// (mma.sync m16n8k16, tokens on the 16-side, weight rows on the 8-side).
// Both operands are loaded with the same trick: the thread that owns logical
// k-slots (2q, 2q+1, 2q+8, 2q+9) of two consecutive MMAs loads the 8
// physically consecutive values 8q..8q+7 of the block, and since a dot product
// does not care about the order of its terms, activation and weight fragments
// agree as long as both use this mapping.
// The partial sums of a CTA's warps are added in warp order through shared memory;
// the order of additions depends on K and on the size class of M (up to 16, 32, 64
// rows), never on which rows share the call.
// K must be a multiple of 8 (16-byte loads); other K go to the generic kernel.
//
// Launch gaps: the kernel is launched as a programmatic dependent (common.cuh).  Before it
// waits for its predecessor it asks L2 for its whole slab of W and loads its first weight
// fragments, so the weight stream of one layer overlaps the tail of the kernel before it.
//
// Fused cache write: with a KvScatter argument the output is the fused [q | k | v] projection of an
// attention layer; q columns go to C as usual, k and v columns go straight into the request's
// pages (the element for token m, head h, dim d lands in page block_table[req][pos / page], row
// pos % page), which saves the separate cache-write kernel of a decode step.
#pragma once

#include "activations.cuh"


__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#include "kv_scatter.cuh"

// A LayerNorm folded into the linear layer that follows it.  With W' = W . diag(gain) (rounded to bfloat16 once,
// when the weights are bound), colsum[n] = sum_k W'[n,k] and bias' = bias + W . norm_bias,
//   LayerNorm(x) . W^T + bias  =  rstd * (x . W'^T - mean * colsum) + bias'
// so the products run on the rows as they are, with no pass over them beforehand, and the rows' mean and
// 1/std are only needed in the epilogue.  Every thread adds up x and x^2 of the activation fragments it loads
// anyway; the sums are completed across the CTA together with the partial products.
// Accuracy: the variance comes from one pass, E[x^2] - mean^2 in float32, whose relative error grows like
// 1e-7 (mean/std)^2; and the epilogue's difference sum - mean * colsum amplifies the rounding of the
// accumulation by about |mean|/std as well.  Both stay below bfloat16 resolution while |mean| is not more
// than a hundred times the row's spread, which bfloat16 rows can hardly exceed (three significant digits)
// and the inputs of a transformer's norms do not come near.  (Taking the variance about the row's first
// element instead was measured: 6 % more time per decode step for accuracy the difference above does not keep.)
struct NormFold {
  const float* colsum;   // [N], null: no fold
  float eps;
};

// MT: 16-row token tiles (M <= 16*MT); NW: 8-row weight tiles per CTA; WARPS: warps that share the K blocks.
// The second launch bound (at least one CTA per SM, which says nothing new) is there for the register
// allocator: without it the compiler keeps these kernels at 76 registers for the sake of occupancy; with it they
// get 116 and run a decode step of 124 kernels 2-7 % faster (fewer, faster CTAs per SM, and room beside them for
// the CTAs of the next kernel, which fetch their weights while they wait).
// Except where the output is float32 at up to 16 rows: that is a vocabulary-sized output head, thousands of
// short-lived CTAs in ten waves and more, where a third CTA per SM (80 registers) counts for more than a faster
// CTA: 24.6 against 26.6 microseconds (four CTAs, 64 registers: 28.7).
template <int MT, int NW, int WARPS, typename TO, int EPI, bool SCATTER, bool FOLD>
__global__ void __launch_bounds__(WARPS * 32, (sizeof(TO) == 4 && MT == 1 && WARPS == 8) ? 3 : 1)
gemm_smallm_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                   const float* __restrict__ bias, const __nv_bfloat16* residual, TO* C, int M, int N, int K,
                   int lda, int ldc, KvScatter kv, NormFold fold) {
  extern __shared__ float part[];   // [WARPS][MT*NW*4][32], then with FOLD [WARPS][16*MT][2] sums of x and x^2
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * (8 * NW);
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  float acc[MT][NW][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NW; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

  const __nv_bfloat16* wrow[NW];
  bool wok[NW];
#pragma unroll
  for (int j = 0; j < NW; ++j) {
    const int n = n0 + j * 8 + g;
    wok[j] = n < N;
    wrow[j] = W + (size_t)(wok[j] ? n : 0) * K + 8 * q;
  }
  const __nv_bfloat16* arow[MT][2];
  bool aok[MT][2];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = i * 16 + h * 8 + g;
      aok[i][h] = m < M;
      arow[i][h] = A + (size_t)(aok[i][h] ? m : 0) * lda + 8 * q;
    }

  const int n_blocks = (K + 31) >> 5;
  constexpr int UNROLL = (MT * NW >= 8) ? 1 : (MT * NW >= 2 ? 2 : 4);   // K blocks per warp and iteration
  constexpr int STEP = WARPS * UNROLL;

  auto load_w = [&](int kb, uint4 (&dst)[UNROLL][NW]) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb + u * WARPS) * 32;
      const bool kin = (kb + u * WARPS) < n_blocks && (k + 8 * q) < K;   // K % 8 == 0: a chunk is all in or all out
#pragma unroll
      for (int j = 0; j < NW; ++j) dst[u][j] = (kin && wok[j]) ? ldg_stream(wrow[j] + k) : zero;
    }
  };

  // Before waiting for the previous kernel: everything that touches only W and the step's inputs.
  pdl_trigger();
  {
    const int lines_per_row = (K * 2 + 127) >> 7;
    for (int i = threadIdx.x; i < 8 * NW * lines_per_row; i += WARPS * 32) {
      const int rrow = i / lines_per_row, n = n0 + rrow;
      if (n < N) {
        const char* p = reinterpret_cast<const char*>(W + (size_t)n * K) + (size_t)(i - rrow * lines_per_row) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
      }
    }
  }
  uint4 wv[UNROLL][NW];
  load_w(warp, wv);
  // What the epilogue needs besides the sums comes from memory too (bias; for the fused cache write the
  // token's request, position and page: three loads that depend on one another).  With few elements per
  // thread these are fetched here, where their latency hides behind the weight stream, instead of after
  // the reduction.  None of it is written by a kernel: bias is a weight, the rest are the step's inputs.
  constexpr int PER = MT * NW * 4;
  constexpr int EPT = (PER + WARPS - 1) / WARPS;     // output elements per thread
  constexpr bool HOIST = EPT <= 2;
  float e_bias[HOIST ? EPT : 1];
  float e_colsum[HOIST ? EPT : 1];
  __nv_bfloat16* e_dst[HOIST ? EPT : 1];             // where a key or value element goes (null: nowhere)
  float e_res[HOIST ? EPT : 1];
  auto elem_mn = [&](int e, int& m, int& n) {
    const int idx = e >> 5, ln = e & 31;
    const int c = idx & 3, j = (idx >> 2) % NW, i = (idx >> 2) / NW;
    m = i * 16 + (ln >> 2) + ((c & 2) ? 8 : 0);
    n = n0 + j * 8 + 2 * (ln & 3) + (c & 1);
  };
  if (HOIST) {
#pragma unroll
    for (int x = 0; x < EPT; ++x) {
      const int e = threadIdx.x + x * WARPS * 32;
      int m, n;
      elem_mn(e, m, n);
      const bool in = e < PER * 32 && m < M && n < N;
      e_bias[x] = (in && bias) ? bias[n] : 0.f;
      e_colsum[x] = (FOLD && in) ? fold.colsum[n] : 0.f;
      e_dst[x] = nullptr;
      if (SCATTER && in && n >= kv.q_width) e_dst[x] = kv_slot(kv, m, n);
    }
  }
  // With more elements per thread only the rows' part of the cache addresses is looked up here (one thread per
  // row walks request -> position -> page); the epilogue adds the column's part.
  __shared__ long long s_row_base[(SCATTER && !HOIST) ? 16 * MT : 1];
  if (SCATTER && !HOIST && threadIdx.x < 16 * MT)
    s_row_base[threadIdx.x] = (int)threadIdx.x < M ? kv_row_base(kv, threadIdx.x) : -1;
  pdl_wait();
  A = after_wait(A);
  residual = after_wait(residual);
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) arow[i][h] = after_wait(arow[i][h]);
  if (HOIST) {
#pragma unroll
    for (int x = 0; x < EPT; ++x) {
      const int e = threadIdx.x + x * WARPS * 32;
      int m, n;
      elem_mn(e, m, n);
      e_res[x] = (residual && e < PER * 32 && m < M && n < N) ? __bfloat162float(residual[(size_t)m * ldc + n]) : 0.f;
    }
  }

  auto load_a = [&](int kb, uint4 (&dst)[UNROLL][MT][2]) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb + u * WARPS) * 32;
      const bool kin = (kb + u * WARPS) < n_blocks && (k + 8 * q) < K;
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int h = 0; h < 2; ++h) dst[u][i][h] = (kin && aok[i][h]) ? ldg_cached(arow[i][h] + k) : zero;
    }
  };
  // With more than 32 rows the activation fragments are fetched an iteration ahead as well (their L2
  // latency would otherwise sit in every iteration); with few rows that only costs registers.
  constexpr bool AHEAD = MT >= 4;
  uint4 av[UNROLL][MT][2];
  if (AHEAD) load_a(warp, av);

  float sx[MT][2], sq[MT][2];      // FOLD: this thread's share of sum x and sum x^2 of rows g and g + 8 of each tile
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) sx[i][h] = sq[i][h] = 0.f;

  for (int kb = warp; kb < n_blocks; kb += STEP) {
    uint4 wn[UNROLL][NW], an[UNROLL][MT][2];
    if (!AHEAD) load_a(kb, av);
    load_w(kb + STEP, wn);          // the next iteration's operands are in flight while this one multiplies
    if (AHEAD) load_a(kb + STEP, an);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NW; ++j) {
          mma_bf16(acc[i][j], av[u][i][0].x, av[u][i][1].x, av[u][i][0].y, av[u][i][1].y, wv[u][j].x, wv[u][j].y);
          mma_bf16(acc[i][j], av[u][i][0].z, av[u][i][1].z, av[u][i][0].w, av[u][i][1].w, wv[u][j].z, wv[u][j].w);
        }
    if (FOLD) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float v[8];
            unpack8(av[u][i][h], v);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              sx[i][h] += v[e];
              sq[i][h] = fmaf(v[e], v[e], sq[i][h]);
            }
          }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
      for (int j = 0; j < NW; ++j) wv[u][j] = wn[u][j];
      if (AHEAD) {
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int h = 0; h < 2; ++h) av[u][i][h] = an[u][i][h];
      }
    }
  }

#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NW; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) part[(warp * PER + (i * NW + j) * 4 + c) * 32 + lane] = acc[i][j][c];
  float* stat = part + WARPS * PER * 32;   // [WARPS][16 * MT][2]
  if (FOLD) {
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h) {   // the four lanes of a row hold different k: add them up
        sx[i][h] += __shfl_xor_sync(0xffffffffu, sx[i][h], 1);
        sx[i][h] += __shfl_xor_sync(0xffffffffu, sx[i][h], 2);
        sq[i][h] += __shfl_xor_sync(0xffffffffu, sq[i][h], 1);
        sq[i][h] += __shfl_xor_sync(0xffffffffu, sq[i][h], 2);
        if (q == 0) {
          stat[(warp * 16 * MT + i * 16 + h * 8 + g) * 2] = sx[i][h];
          stat[(warp * 16 * MT + i * 16 + h * 8 + g) * 2 + 1] = sq[i][h];
        }
      }
  }
  __syncthreads();
  // FOLD: rstd * (sum - mean * colsum[n]) in place of the sum, from the warps' shares of sum x and sum x^2
  auto unfold = [&](float v, int m, int n, float colsum) {
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      s1 += stat[(w * 16 * MT + m) * 2];
      s2 += stat[(w * 16 * MT + m) * 2 + 1];
    }
    const float mean = s1 / (float)K;
    const float var = fmaxf(s2 / (float)K - mean * mean, 0.f);
    return rsqrtf(var + fold.eps) * (v - mean * colsum);
  };
  if (HOIST) {
#pragma unroll
    for (int x = 0; x < EPT; ++x) {
      const int e = threadIdx.x + x * WARPS * 32;
      if (e >= PER * 32) break;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += part[w * PER * 32 + e];
      int m, n;
      elem_mn(e, m, n);
      if (m < M && n < N) {
        if (FOLD) v = unfold(v, m, n, e_colsum[x]);
        v += e_bias[x];
        v = activate<EPI, true>(v);
        v += e_res[x];
        if (SCATTER && n >= kv.q_width) {
          if (e_dst[x]) *e_dst[x] = __float2bfloat16_rn(v);
        } else {
          C[(size_t)m * ldc + n] = from_f<TO>(v);
        }
      }
    }
  } else {
    // the same, with the loads of all the thread's elements asked for together, after the products
    float l_bias[EPT], l_colsum[EPT], l_res[EPT];
#pragma unroll
    for (int x = 0; x < EPT; ++x) {
      const int e = threadIdx.x + x * WARPS * 32;
      int m, n;
      elem_mn(e, m, n);
      const bool in = e < PER * 32 && m < M && n < N;
      l_bias[x] = (in && bias) ? bias[n] : 0.f;
      l_colsum[x] = (FOLD && in) ? fold.colsum[n] : 0.f;
      l_res[x] = (in && residual) ? __bfloat162float(residual[(size_t)m * ldc + n]) : 0.f;
    }
#pragma unroll
    for (int x = 0; x < EPT; ++x) {
      const int e = threadIdx.x + x * WARPS * 32;
      if (e >= PER * 32) break;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += part[w * PER * 32 + e];
      int m, n;
      elem_mn(e, m, n);
      if (m < M && n < N) {
        if (FOLD) v = unfold(v, m, n, l_colsum[x]);
        v += l_bias[x];
        v = activate<EPI, true>(v);
        v += l_res[x];
        if (SCATTER && n >= kv.q_width) {
          __nv_bfloat16* dst = kv_slot_at(kv, s_row_base[m], n);
          if (dst) *dst = __float2bfloat16_rn(v);
        } else {
          C[(size_t)m * ldc + n] = from_f<TO>(v);
        }
      }
    }
  }
}

template <int MT, int NW, int WARPS, typename TO, bool SCATTER, bool FOLD>
static int launch_epi(const void* A, const void* W, const float* bias, const void* residual, void* C, int M, int N,
                      int K, int lda, int ldc, int epi, const KvScatter& kv, const NormFold& fold,
                      cudaStream_t stream) {
  const dim3 grid((N + 8 * NW - 1) / (8 * NW));
  const size_t smem = ((size_t)WARPS * MT * NW * 4 * 32 + (FOLD ? (size_t)WARPS * 16 * MT * 2 : 0)) * sizeof(float);
  // The fused cache write has no activation: only the plain epilogue is built for it.
  return dispatch_activation(SCATTER ? (int)EPI_NONE : epi, [&](auto e) {
    constexpr int EPI = SCATTER ? (int)EPI_NONE : (int)decltype(e)::value;
    auto kern = gemm_smallm_kernel<MT, NW, WARPS, TO, EPI, SCATTER, FOLD>;
    static bool raised = false;   // once per instantiation, and never for the first time inside a stream capture
    if (smem > 48 * 1024 && !raised) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      raised = true;
    }
    launch_pdl(kern, grid, dim3(WARPS * 32), smem, stream, (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias,
               (const __nv_bfloat16*)residual, (TO*)C, M, N, K, lda, ldc, kv, fold);
    return mlxb_check_launch("linear (few rows)");
  });
}

template <typename TO, bool SCATTER, bool FOLD>
static int launch(const void* A, const void* W, const float* bias, const void* residual, void* C, int M, int N, int K,
                  int lda, int ldc, int epi, const KvScatter& kv, const NormFold& fold, cudaStream_t stream) {
  // Weight tiles (of 8 outputs) per CTA.  Two things pull apart.  Every CTA reads all M rows of the activations from
  // L2, so with many rows and many CTAs that traffic (M x K x 2 bytes per CTA) exceeds the weight stream itself; and
  // a launch with more CTAs than the SMs hold at once runs in waves, of which only the first can fetch its weights
  // while the kernel before still runs.  Measured on 1024-, 1280- and 1600-wide models: at up to 16 rows two tiles
  // wherever one-tile CTAs would be more than one per SM (1024-wide, 8 rows: 3072 outputs 3.9 against 5.6
  // microseconds, 4096 outputs 4.0 against 5.4, a decode step 0.59 against 0.65 ms; a vocabulary-sized output 26.6
  // against 36.8; four tiles are slower everywhere, and so are two for outputs that fit one CTA per SM; three tiles
  // where two would still be more CTAs than fit at once: 1280-wide, 5120 outputs, a step 1.18 against 1.28 ms; 1600-wide
  // 2.05 against 2.12; three tiles where two fit are slower); four tiles
  // for wide outputs at 17 to 32 rows (a step of 32 rows 1.14 against 1.20 ms) and at 33 to 64 rows (a quarter
  // faster than one).
  const int tiles = (N + 7) / 8;
  const int mt = M <= 16 ? 1 : (M <= 32 ? 2 : 4);
  int nw = 1;
  if (mt == 4) nw = tiles >= 384 ? 4 : (tiles >= 2 * 148 ? 2 : 1);
  else if (mt == 2) nw = tiles >= 2 * 148 ? 4 : 1;
  else {
    const int sms = mlxb_sm_count();
    nw = tiles > sms ? 2 : 1;
    if (tiles < 2048 && (tiles + 1) / 2 > 2 * sms) nw = 3;   // two tiles would still leave more CTAs than fit at once
  }

  // K blocks are shared by 8 warps; a long K with few output tiles gets 16 so that a warp's chain of
  // dependent loads stays short, and so do more than 32 rows with one weight tile per CTA (a 1024-wide output at
  // 64 rows: 4.6 against 5.8 microseconds).
#define GO(MT_, NW_)                                                                                              \
  {                                                                                                               \
    if ((K >= 2048 || MT_ == 4) && NW_ == 1)                                                                      \
      return launch_epi<MT_, NW_, 16, TO, SCATTER, FOLD>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, kv, fold, \
                                                         stream);                                               \
    return launch_epi<MT_, NW_, 8, TO, SCATTER, FOLD>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, kv, fold,  \
                                                      stream);                                                  \
  }
  if (mt == 1) { if (nw == 3) GO(1, 3); if (nw == 2) GO(1, 2); GO(1, 1); }
  if (mt == 2) { if (nw == 4) GO(2, 4); GO(2, 1); }
  if (nw == 4) GO(4, 4);
  if (nw == 2) GO(4, 2);
  GO(4, 1);
#undef GO
}

static int check_args(int M, int N, int K, int lda, int ldc, int epi, const void* A, const void* W) {
  if (M > 64) return mlxb_fail(MLXB_BAD_ARG, "linear (few rows): %d rows, at most 64", M);
  if (K <= 0 || (K & 7) || (lda & 7) || lda < K || ldc < N)
    return mlxb_fail(MLXB_BAD_ARG, "linear (few rows): K %d and row stride %d must be multiples of 8 (ldc %d, N %d)",
                     K, lda, ldc, N);
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15))
    return mlxb_fail(MLXB_BAD_ARG, "linear (few rows): operands must be 16-byte aligned");
  if (!activation_known(epi)) return mlxb_fail(MLXB_BAD_ARG, "linear: epilogue code %d", epi);
  return 0;
}

