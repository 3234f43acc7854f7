// Linear layer for up to 16 rows (decode steps) against a WIDE weight that has to be streamed from HBM once, such
// as an output head over a vocabulary:
//   C[M,N] = epilogue(A[M,K] . W[N,K]^T + bias[N]) (+ residual[M,N])
// A, W, residual bfloat16; float32 accumulation; C bfloat16 or float32.  (The second of two few-rows kernels:
// gemm_smallm.cuh stages weights in registers and is the faster one for the narrower layers inside a block;
// `preferred()` below says which runs.)
//
// The kernel is bound by reading W, so it is organised around the weight stream, which must never stop:
//
//   * One CTA per SM (at most) owns a contiguous range of 8*NW-row tiles of W.  A producer warp copies the CTA's
//     slab into a ring of shared-memory stages with bulk asynchronous copies (cp.async.bulk, completion counted
//     on an mbarrier per stage), running as far ahead as the ring allows: a stage holds 8*NW rows x 1024/NW
//     columns, about 16 KB, so the five stages of a CTA hold the whole slab of a layer of GPT-2 medium.  Two such
//     CTAs fit an SM, so the CTA of the NEXT kernel of the step is resident while this one computes, and since
//     weights do not depend on the kernel before, its producer fills its ring BEFORE the wait for that kernel
//     (programmatic dependent launch, common.cuh): when the wait returns, the weights are in shared memory.
//   * Eight compute warps share the 32-wide K blocks of a stage round robin.  Products run on the tensor cores
//     (mma.sync m16n8k16, tokens on the 16-side, weight rows on the 8-side).  Both operands use the same
//     permutation of K inside a block: the thread that owns logical k-slots (2q, 2q+1, 2q+8, 2q+9) of two
//     consecutive MMAs takes the 8 physically consecutive values 8q..8q+7, one 16-byte access, and since a dot
//     product does not care about the order of its terms the fragments of A and W agree.  W fragments come from
//     shared memory (rows padded by 64 bytes: the eight lanes of a quarter warp hit distinct banks), A fragments
//     from global memory (L2); with one token tile and K <= 1024 a warp meets the same K blocks in every tile of
//     the CTA and keeps its A fragments in registers for all of them.
//   * The partial sums of the warps are added in warp order through shared memory (one named barrier for the
//     tiles of a CTA, up to four at a time): the order of additions depends on K and on the size class of M (up to 16, 32, 64 rows),
//     never on which rows share the call.  Bias, the activation, the residual add and, for the fused
//     [q | k | v] projection, the write of keys and values into the pages (kv_scatter.cuh) follow.
//
// A LayerNorm folded into the layer (FOLD): with W' = W . diag(gain) (rounded to bfloat16 once, when the weights
// are bound), colsum[n] = sum_k W'[n,k] and bias' = bias + W . norm_bias,
//   LayerNorm(x) . W^T + bias  =  rstd * (x . W'^T - mean * colsum) + bias'
// so the products run on the rows as they are and mean and 1/std are only needed in the epilogue; every thread
// adds up x and x^2 of the A fragments of the CTA's first tile, which together cover each row exactly once.
// Accuracy: the variance comes from one pass, E[x^2] - mean^2 in float32, whose relative error grows like
// 1e-7 (mean/std)^2, and the epilogue's difference amplifies the rounding of the accumulation by about
// |mean|/std; both stay below bfloat16 resolution while |mean| is not more than a hundred times the row's spread.
//
// Every wait on a barrier is bounded.  A wait that gives up sets a flag all roles see: the compute warps skip
// the rest of their work but still meet at every barrier, the producer waits (bounded) for the copies it
// has in flight, nothing more is stored, and the kernel reports MLXB_ST_WAIT_TIMEOUT in the status word.
// K must be a multiple of 8 (16-byte rows); other K go to the generic kernel.
#pragma once

#include "activations.cuh"
#include "kv_scatter.cuh"

namespace gs {

constexpr int CW = 8;                       // compute warps
constexpr int THREADS = (CW + 1) * 32;      // + the producer warp
constexpr int ROW_PAD = 64;                 // bytes between the rows of a stage beyond their data
constexpr uint32_t SPIN_LIMIT = 1u << 22;   // polls before a wait gives up (about a second)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait of a whole warp with one answer for all its lanes; false after SPIN_LIMIT polls or when another
// role has given up.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  bool ok = false;
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
    if (mbar_try(bar, parity)) { ok = true; break; }
    if ((i & 255u) == 255u && *abort_flag) break;
  }
  ok = __all_sync(0xffffffffu, ok);
  if (!ok) *abort_flag = 1;
  return ok;
}
// 16-byte aligned global -> shared bulk copy of a multiple of 16 bytes; completion is counted on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint4 lds128(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
  return v;
}
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void compute_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory"); }

struct NormFold {
  const float* colsum;   // [N], null: no fold
  float eps;
};

template <int NW>
struct Geo {
  static constexpr int ROWS = 8 * NW;                    // weight rows of a stage (and of a tile)
  static constexpr int KS = 1024 / NW;                   // columns of a stage
  static constexpr int ROW_BYTES = KS * 2 + ROW_PAD;     // = 64 mod 128: conflict-free 16-byte reads by row
  static constexpr int STAGE_BYTES = ROWS * ROW_BYTES;
  static constexpr int KB = KS / 32;                     // 32-wide K blocks of a stage
};

// MT: 16-row token tiles (M <= 16*MT); NW: 8-row weight tiles per stage; STAGES: depth of the ring; TG: tiles
// whose epilogues run together.
// RESIDENT: one token tile and K <= 1024: a warp's A fragments stay in registers for all the CTA's tiles.
template <int MT, int NW, int STAGES, int TG, bool RESIDENT, typename TO, int EPI, bool SCATTER, bool FOLD>
__global__ void __launch_bounds__(THREADS, MT <= 2 ? 2 : 1)
gemm_stream_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                   const float* __restrict__ bias, const __nv_bfloat16* residual, TO* C, int M, int N, int K, int lda,
                   int ldc, KvScatter kv, NormFold fold, int* __restrict__ status) {
  using G = Geo<NW>;
  constexpr int PER = MT * NW * 4;                 // accumulators of a thread
  constexpr int PART = CW * PER * 32;              // floats of a tile's partial sums
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* stages = smem;                                                  // [STAGES][STAGE_BYTES]
  float* part = reinterpret_cast<float*>(smem + STAGES * G::STAGE_BYTES);  // [TG][CW][PER][32]
  float* stat = part + TG * PART;                                          // [CW][16 * MT][2] sums of x, x^2
  __shared__ uint64_t full[STAGES], empty[STAGES];
  __shared__ long long s_row_base[SCATTER ? 16 * MT : 1];
  __shared__ int s_abort;
  volatile int* abort_flag = &s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int n_tiles = (N + G::ROWS - 1) / G::ROWS;
  const int t_begin = (int)(((long long)blockIdx.x * n_tiles) / gridDim.x);
  const int t_end = (int)(((long long)(blockIdx.x + 1) * n_tiles) / gridDim.x);
  const int n_ks = (K + G::KS - 1) / G::KS;        // stages per tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CW); }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_trigger();

  if (warp == CW) {
    // ---------------------------------------------------------------- producer: the weight stream
    // Weights are written by no kernel, so the stream starts at once and never looks at the wait for the
    // kernel before.
    int it = 0;
    bool ok = true;
    for (int tile = t_begin; tile < t_end && ok; ++tile) {
      const int n0 = tile * G::ROWS;
      const int rows = min(G::ROWS, N - n0);
      for (int ks = 0; ks < n_ks; ++ks, ++it) {
        const int s = it % STAGES;
        if (it >= STAGES && !(ok = mbar_wait_warp(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag))) break;
        const int k0 = ks * G::KS;
        const uint32_t row_bytes = (uint32_t)(min(G::KS, K - k0) * 2);
        if (lane == 0) mbar_expect_tx(&full[s], row_bytes * (uint32_t)rows);
        __syncwarp();
        for (int r = lane; r < rows; r += 32)
          bulk_load(stages + (size_t)s * G::STAGE_BYTES + (size_t)r * G::ROW_BYTES, W + (size_t)(n0 + r) * K + k0,
                    row_bytes, &full[s]);
      }
    }
    if (*abort_flag) {   // somebody gave up: let the copies already issued land before the CTA exits
      for (int i = it > STAGES ? it - STAGES : 0; i < it; ++i)
        for (uint32_t p = 0; p < (1u << 20); ++p)
          if (mbar_try(&full[i % STAGES], (uint32_t)((i / STAGES) & 1))) break;
    }
  } else {
    // ---------------------------------------------------------------- compute warps
    // Before the wait: what depends only on the step's inputs (for the fused cache write each row's request,
    // position and page, three loads that depend on one another).
    if (SCATTER && threadIdx.x < 16 * MT)
      s_row_base[threadIdx.x] = (int)threadIdx.x < M ? kv_row_base(kv, threadIdx.x) : -1;
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
    pdl_wait();
    residual = after_wait(residual);
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h) arow[i][h] = after_wait(arow[i][h]);

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    constexpr int KBW = (G::KB + CW - 1) / CW;        // K blocks of a stage a warp takes
    auto load_a = [&](int k, uint4 (&dst)[MT][2]) {   // the thread's 8 values of block column k (k + 8q < K checked here)
      const bool kin = k + 8 * q < K;
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int h = 0; h < 2; ++h) dst[i][h] = (kin && aok[i][h]) ? gs::ldg_cached(arow[i][h] + k) : zero;
    };
    uint4 a_res[RESIDENT ? KBW : 1][MT][2];
    if constexpr (RESIDENT) {
#pragma unroll
      for (int b = 0; b < KBW; ++b) load_a((warp + b * CW) * 32, a_res[b]);
    }
    float sx[MT][2], sq[MT][2];      // FOLD: this thread's share of sum x and sum x^2 of rows g and g + 8 of each tile
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h) sx[i][h] = sq[i][h] = 0.f;

    // A fragments of a stage's blocks are asked for before the wait for the stage's weights (they do not depend
    // on them); with one token tile there are registers to ask for the next stage's as well while this one
    // multiplies.
    constexpr bool AHEAD = !RESIDENT && MT == 1;
    auto load_stage_a = [&](int ks, uint4 (&dst)[KBW][MT][2]) {
#pragma unroll
      for (int b = 0; b < KBW; ++b) {
        const int kb = warp + b * CW;
        const int k = ks * G::KS + kb * 32;
        if (kb < G::KB && k < K) load_a(k, dst[b]);
        else {
#pragma unroll
          for (int i = 0; i < MT; ++i) dst[b][i][0] = dst[b][i][1] = zero;
        }
      }
    };
    // two sets of fragments used in turns (no copies between them: a copy would wait for the loads it copies)
    uint4 a_ping[RESIDENT ? 1 : KBW][MT][2], a_pong[AHEAD ? KBW : 1][MT][2];
    bool flip = false;     // AHEAD: the current stage's fragments are in a_pong
    if constexpr (AHEAD) load_stage_a(0, a_ping);

    // The products of one block of a stage: the thread's W fragments of the tile's NW row groups from shared memory
    // against its A fragments, added to acc; with `stats` the sums of x and x^2 on the way.
    auto block_products = [&](const uint8_t* st, int kb, int k, int n0, const uint4 (&af)[MT][2], float (&acc)[MT][NW][4],
                              bool stats) {
      const bool kin = k + 8 * q < K;
      uint4 wv[NW];
#pragma unroll
      for (int j = 0; j < NW; ++j)
        wv[j] = (kin && n0 + j * 8 + g < N) ? gs::lds128(st + (size_t)(j * 8 + g) * G::ROW_BYTES + (kb * 32 + 8 * q) * 2)
                                            : zero;
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const uint4 a0 = af[i][0], a1 = af[i][1];
#pragma unroll
        for (int j = 0; j < NW; ++j) {
          gs::mma_bf16(acc[i][j], a0.x, a1.x, a0.y, a1.y, wv[j].x, wv[j].y);
          gs::mma_bf16(acc[i][j], a0.z, a1.z, a0.w, a1.w, wv[j].z, wv[j].w);
        }
        if (stats) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float v[8];
            unpack8(h == 0 ? a0 : a1, v);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              sx[i][h] += v[e];
              sq[i][h] = fmaf(v[e], v[e], sq[i][h]);
            }
          }
        }
      }
    };
    auto store_partials = [&](int tg, const float (&acc)[MT][NW][4]) {
      float* buf = part + tg * PART;
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NW; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) buf[(warp * PER + (i * NW + j) * 4 + c) * 32 + lane] = acc[i][j][c];
    };

    // The CTA's tiles are worked off in groups of TG: the products of all tiles of a group first (their partial
    // sums go to shared memory, a buffer per tile), then ONE barrier and one epilogue for the whole group, whose
    // operands (bias, column sums: weights; residual: asked for right behind the wait for the kernel before) are in
    // registers by then.  A CTA of a layer of GPT-2 medium has one group, so the work after the wait is: A
    // fragments, products from shared memory, one barrier, sums, store.
    constexpr int TILE_E = PER * 32;                                // elements (row, column) of a tile
    constexpr int EPT = (TG * TILE_E + CW * 32 - 1) / (CW * 32);    // elements of a group a thread finishes
    auto elem = [&](int e, int tile0, int& tg, int& m, int& n) {
      tg = e / TILE_E;
      const int r = e - tg * TILE_E, idx = r >> 5, ln = r & 31;
      const int c = idx & 3, j = (idx >> 2) % NW, i = (idx >> 2) / NW;
      m = i * 16 + (ln >> 2) + ((c & 2) ? 8 : 0);
      n = (tile0 + tg) * G::ROWS + j * 8 + 2 * (ln & 3) + (c & 1);
    };

    int it = 0;
    bool ok = true;
    for (int tile0 = t_begin; tile0 < t_end; tile0 += TG) {
      float e_bias[EPT], e_colsum[EPT], e_res[EPT];
#pragma unroll
      for (int x = 0; x < EPT; ++x) {
        int tg, m, n;
        elem(threadIdx.x + x * CW * 32, tile0, tg, m, n);
        const bool in = threadIdx.x + x * CW * 32 < TG * TILE_E && tile0 + tg < t_end && m < M && n < N;
        e_bias[x] = (in && bias) ? bias[n] : 0.f;
        e_colsum[x] = (FOLD && in) ? fold.colsum[n] : 0.f;
        e_res[x] = (in && residual) ? __bfloat162float(residual[(size_t)m * ldc + n]) : 0.f;
      }
      const bool first = tile0 == t_begin;
      if constexpr (RESIDENT) {
        // One stage per tile: the tiles of the group are worked on side by side, a block of all of them at a
        // time, so that their chains of dependent products overlap.
        const int n_group = min(TG, t_end - tile0);
        float acc[TG][MT][NW][4];
#pragma unroll
        for (int tg = 0; tg < TG; ++tg)
#pragma unroll
          for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < NW; ++j)
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[tg][i][j][c] = 0.f;
        for (int tg = 0; tg < n_group && ok; ++tg)
          ok = mbar_wait_warp(&full[(it + tg) % STAGES], (uint32_t)(((it + tg) / STAGES) & 1), abort_flag);
        if (ok) {
#pragma unroll
          for (int b = 0; b < KBW; ++b) {
            const int kb = warp + b * CW, k = kb * 32;
            if (kb < G::KB && k < K) {
#pragma unroll
              for (int tg = 0; tg < TG; ++tg)
                if (tg < n_group)
                  block_products(stages + (size_t)((it + tg) % STAGES) * G::STAGE_BYTES, kb, k, (tile0 + tg) * G::ROWS,
                                 a_res[b], acc[tg], FOLD && first && tg == 0);
            }
          }
          __syncwarp();
          if (lane == 0)
            for (int tg = 0; tg < n_group; ++tg) mbar_arrive(&empty[(it + tg) % STAGES]);
        }
        it += n_group;
#pragma unroll
        for (int tg = 0; tg < TG; ++tg)
          if (tg < n_group) store_partials(tg, acc[tg]);
      } else {
#pragma unroll 1
        for (int tg = 0; tg < TG; ++tg) {
          const int tile = tile0 + tg;
          if (tile >= t_end) break;
          const int n0 = tile * G::ROWS;
          const bool stats = FOLD && first && tg == 0;
          float acc[MT][NW][4];
#pragma unroll
          for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < NW; ++j)
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
          // one stage: its A fragments are in `use`; with AHEAD the next stage's (or the next tile's first) go to `fill`
          auto stage = [&](int ks, uint4 (&use)[KBW][MT][2], uint4 (&fill)[AHEAD ? KBW : 1][MT][2]) {
            const int s = it % STAGES;
            if constexpr (!AHEAD) load_stage_a(ks, use);
            if constexpr (AHEAD) load_stage_a(ks + 1 < n_ks ? ks + 1 : 0, fill);
            if (!(ok = mbar_wait_warp(&full[s], (uint32_t)((it / STAGES) & 1), abort_flag))) return;
            const uint8_t* st = stages + (size_t)s * G::STAGE_BYTES;
#pragma unroll
            for (int b = 0; b < KBW; ++b) {
              const int kb = warp + b * CW, k = ks * G::KS + kb * 32;
              if (kb < G::KB && k < K) block_products(st, kb, k, n0, use[b], acc, stats);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            ++it;
          };
          for (int ks = 0; ks < n_ks && ok; ++ks) {
            if constexpr (AHEAD) {
              if (!flip) stage(ks, a_ping, a_pong);
              else stage(ks, a_pong, a_ping);
              flip = !flip;
            } else {
              stage(ks, a_ping, a_pong);
            }
          }
          store_partials(tg, acc);
        }
      }
      if (FOLD && first) {
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
      compute_barrier();
      if (!*abort_flag) {
#pragma unroll
        for (int x = 0; x < EPT; ++x) {
          const int e = threadIdx.x + x * CW * 32;
          int tg, m, n;
          elem(e, tile0, tg, m, n);
          if (e < TG * TILE_E && tile0 + tg < t_end && m < M && n < N) {
            const float* buf = part + tg * PART + (e - tg * TILE_E);
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < CW; ++w) v += buf[w * TILE_E];
            if (FOLD) {   // the row's statistics: the warps' shares, added in warp order
              float s1 = 0.f, s2 = 0.f;
#pragma unroll
              for (int w = 0; w < CW; ++w) {
                s1 += stat[(w * 16 * MT + m) * 2];
                s2 += stat[(w * 16 * MT + m) * 2 + 1];
              }
              const float mean = s1 / (float)K;
              const float var = fmaxf(s2 / (float)K - mean * mean, 0.f);
              v = rsqrtf(var + fold.eps) * (v - mean * e_colsum[x]);
            }
            v += e_bias[x];
            v = activate<EPI, true>(v);
            v += e_res[x];
            if (SCATTER && n >= kv.q_width) {
              __nv_bfloat16* dst = kv_slot_at(kv, s_row_base[m], n);
              if (dst) *dst = __float2bfloat16_rn(v);
            } else {
              C[(size_t)m * ldc + n] = from_f<TO>(v);
            }
          }
        }
      }
      if (tile0 + TG < t_end) compute_barrier();   // the buffers are written again by the next group
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_abort && status) atomicOr(status, MLXB_ST_WAIT_TIMEOUT);
}

static inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

template <int MT, int NW, int STAGES, int TG, bool RESIDENT, typename TO, bool SCATTER, bool FOLD>
static int launch_cfg(const void* A, const void* W, const float* bias, const void* residual, void* C, int M, int N,
                      int K, int lda, int ldc, int epi, const KvScatter& kv, const NormFold& fold, int* status,
                      cudaStream_t stream) {
  using G = Geo<NW>;
  const int n_tiles = (N + G::ROWS - 1) / G::ROWS;
  const dim3 grid(n_tiles < sm_count() ? n_tiles : sm_count());
  constexpr int PER = MT * NW * 4;
  const size_t smem = (size_t)STAGES * G::STAGE_BYTES + (size_t)TG * CW * PER * 32 * sizeof(float) +
                      (size_t)CW * 16 * MT * 2 * sizeof(float);
  // The fused cache write has no activation: only the plain epilogue is built for it.
  return dispatch_activation(SCATTER ? (int)EPI_NONE : epi, [&](auto e) {
    constexpr int EPI = SCATTER ? (int)EPI_NONE : (int)decltype(e)::value;
    auto kern = gemm_stream_kernel<MT, NW, STAGES, TG, RESIDENT, TO, EPI, SCATTER, FOLD>;
    static bool raised = false;   // once per instantiation, and never for the first time inside a stream capture
    if (!raised) {
      cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess)
        return mlxb_fail((int)err, "linear (few rows): %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      raised = true;
    }
    launch_pdl(kern, grid, dim3(THREADS), smem, stream, (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias,
               (const __nv_bfloat16*)residual, (TO*)C, M, N, K, lda, ldc, kv, fold, status);
    return mlxb_check_launch("linear (few rows)");
  });
}

template <typename TO, bool SCATTER, bool FOLD>
static int launch(const void* A, const void* W, const float* bias, const void* residual, void* C, int M, int N, int K,
                  int lda, int ldc, int epi, const KvScatter& kv, const NormFold& fold, int* status,
                  cudaStream_t stream) {
#define GS_GO(MT_, NW_, ST_, TG_, RES_) \
  return launch_cfg<MT_, NW_, ST_, TG_, RES_, TO, SCATTER, FOLD>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, kv, fold, status, stream)
  if (K <= 1024) GS_GO(1, 1, 5, 4, true);
  GS_GO(1, 1, 5, 4, false);
#undef GS_GO
}

// Where this kernel is the faster one of the two few-rows kernels (measured on a B200 with the widths of GPT-2
// medium, large and XL): up to 16 rows against an output as wide as a vocabulary.  Each CTA then streams dozens
// of tiles and the ring never runs dry.  For the layers inside a block (a few tiles per CTA) the kernel that
// stages weights in registers (gemm_smallm.cuh) is as fast or faster: there a launch is bounded by what follows
// the wait for the kernel before (A fragments, a chain of products, a barrier, the epilogue), not by the stream.
static inline bool preferred(int M, int N) { return M <= 16 && N >= 8192; }

static int check_args(int M, int N, int K, int lda, int ldc, int epi, const void* A, const void* W) {
  if (M > 16) return mlxb_fail(MLXB_BAD_ARG, "linear (few rows, streamed): %d rows, at most 16", M);
  if (K <= 0 || (K & 7) || (lda & 7) || lda < K || ldc < N)
    return mlxb_fail(MLXB_BAD_ARG, "linear (few rows): K %d and row stride %d must be multiples of 8 (ldc %d, N %d)",
                     K, lda, ldc, N);
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15))
    return mlxb_fail(MLXB_BAD_ARG, "linear (few rows): operands must be 16-byte aligned");
  if (!activation_known(epi)) return mlxb_fail(MLXB_BAD_ARG, "linear: epilogue code %d", epi);
  return 0;
}

}  // namespace gs
