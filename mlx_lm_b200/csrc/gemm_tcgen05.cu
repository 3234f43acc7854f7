// Linear layer for many rows (prompt portions) on the 5th-generation tensor cores:
//   C[M,N] = epilogue(A[M,K] . W[N,K]^T + bias[N]) (+ residual[M,N])
// A, W, residual bfloat16 (both operands K-major: the K index is contiguous), C bfloat16 or float32.
//
// The kernel is persistent: one CTA per SM walks over the 128 x BN output tiles (BN = 128, 192 or 256,
// chosen so that the last wave of tiles is as full as possible).  Warp 0 is the TMA producer: it fills a
// ring of shared-memory stages with 128x64 tiles of A and BNx64 tiles of W (cp.async.bulk.tensor,
// 128-byte swizzle, completion counted on an mbarrier per stage; rows and columns outside the
// matrices arrive as zeros).  Warp 1 allocates tensor memory and issues tcgen05.mma (kind::f16, bf16
// inputs, float32 accumulator of 128 lanes x BN columns in TMEM), four K=16 steps per stage, and
// releases each stage with tcgen05.commit.  There are two accumulators in TMEM: while warps 2-17 (the
// epilogue, four warps per quadrant of 32 TMEM lanes, each a quarter of the columns) read a finished one
// with tcgen05.ld, add the bias, apply gelu_new, add the residual and store, the MMA warp already
// fills the other with the next tile.
// No multicast copy anywhere: every CTA fetches its own tiles.
//
// Pairs (template parameter CG = 2).  The main loop of one CTA is bound by its SM's shared memory: per K step
// 128 rows of A and BN rows of W go in and the tensor core reads the same rows out again, more cycles than the
// products take.  With many rows the kernel therefore runs as thread-block clusters of two CTAs on a
// 256 x BN tile (tcgen05 with .cta_group::2): each CTA fetches its own 128 rows of A and only its half of the
// W rows, the CTA of cluster rank 0 (the leader) issues one product per K step for both, which reads A from
// each CTA's own shared memory and the two halves of W from both, and leaves each CTA's 128 rows of the
// result in that CTA's tensor memory.  The copies of both CTAs are counted on the leader's barrier of the stage
// (.cta_group::2 copies may name a barrier of the peer), a stage is released to both producers by one
// tcgen05.commit that arrives in both CTAs, a finished accumulator is announced to both CTAs' epilogue warps
// the same way, and the epilogue warps of both hand an accumulator back on the leader's barrier.  The tensor
// memory is allocated and freed by warp 1 of both CTAs with the .cta_group::2 forms.  The two CTAs meet at a
// cluster barrier after set-up (so that nobody signals a barrier that is not initialised yet) and before the
// tensor memory is freed (so that nobody frees or leaves while the peer still reads, signals or copies).
//
// Every wait on an mbarrier is bounded: after a limit of polls the waiter raises an abort flag in
// shared memory and a bit in the caller's status word; all roles then fall through to the common
// exit, where the tensor memory is freed.  A timeout therefore ends the kernel with an error code
// instead of a hang.
//
// K and the row strides must be multiples of 8 elements (16 bytes), base addresses 16-byte aligned.
// The accumulation order over K is fixed (stage by stage, four steps per stage), independent of M.
#include <cuda.h>

#include "activations.cuh"
#include "kv_scatter.cuh"

MLXB_DEFINE_LAST_ERROR()

constexpr int BM = 128, BK = 64;
constexpr int EPI_WARPS = 16;                     // four per quadrant of TMEM lanes, each a quarter of the columns
constexpr int THREADS = 64 + 32 * EPI_WARPS;
// Polls of a barrier before a wait gives up (about a second).  A test builds this file with
// MLXB_TEST_WAIT_TIMEOUT defined: the limit is then short, and mlxb_test_withhold_arrival(1) makes the MMA thread
// leave out the arrival that tells the epilogue warps that a CTA's first accumulator is complete, so that their
// wait runs out and the abort path below is taken: every role leaves its loop, the CTA waits (bounded) for
// what it has in flight, reports MLXB_ST_WAIT_TIMEOUT, frees its tensor memory and returns.  Nothing else differs.
#ifdef MLXB_TEST_WAIT_TIMEOUT
constexpr uint32_t SPIN_LIMIT = 1u << 12;
__device__ int g_test_withhold_arrival = 0;
#else
constexpr uint32_t SPIN_LIMIT = 1u << 22;
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false after SPIN_LIMIT polls or when another role gave up.
// peer_abort: the shared::cluster address of the peer CTA's flag in a pair (0: none), raised together with this one.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t peer_abort = 0) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (peer_abort) asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer_abort), "r"(1) : "memory");
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor, K-major operand in 128-byte swizzled rows: start address / 16,
// leading-dimension offset 1 (unused with swizzle), stride between 8-row groups 1024 bytes,
// descriptor version 1 (bit 46), layout type SWIZZLE_128B (2) in bits 61-63.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor for kind::f16: float32 accumulator (bits 4-5 = 1), A and B bfloat16
// (bits 7-9 and 10-12 = 1), both K-major (bits 15, 16 = 0), N/8 in bits 17-22, M/16 in bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---- pairs of CTAs (.cta_group::2)
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the shared::cluster address of the same variable in the CTA of the given rank
__device__ __forceinline__ uint32_t peer_addr(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
// a copy into this CTA's shared memory whose bytes are counted on a barrier given by its shared::cluster address
// (the leader's barrier of the stage)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
// one product over the pair: M = 256 (128 rows in each CTA), issued by the leader only
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the pair's products issued so far have completed, on the barrier at this offset in both CTAs
__device__ __forceinline__ void umma_commit_both(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
// ... on this CTA's barrier only
__device__ __forceinline__ void umma_commit_pair_local(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

template <int BN, int STAGES, int CG>
struct Smem {
  alignas(1024) __nv_bfloat16 a[STAGES][BM * BK];
  alignas(1024) __nv_bfloat16 b[STAGES][(BN / CG) * BK];   // in a pair: this CTA's half of the W rows
  alignas(8) uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t drained;       // abort path only: every tensor-core operation issued so far has completed
  uint32_t tmem_base;
  int abort_flag;
  alignas(16) uint4 stage[EPI_WARPS][32 * 4];   // per epilogue warp: 32 rows x 32 bfloat16 results on their way out
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// A LayerNorm folded into the weights (see NormFold in gemm_smallm.cuh): the epilogue turns the product of the
// rows as they are into rstd * (sum - mean * colsum[n]).  stats[m] = (mean, rstd) of row m, from row_stats.
struct NormFoldRows {
  const float* colsum;    // [N], null: no fold
  const float2* stats;    // [M]
};

__device__ __forceinline__ void unfold8(float (&v)[8], int n8, int N, const float* __restrict__ colsum, float mean,
                                        float rstd) {
  if (n8 + 8 <= N && (((uintptr_t)(colsum + n8)) & 15) == 0) {   // the same 32 bytes for every lane: two broadcast loads
    const float4 c0 = *reinterpret_cast<const float4*>(colsum + n8), c1 = *reinterpret_cast<const float4*>(colsum + n8 + 4);
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float nm = -mean * rstd;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = fmaf(nm, cs[i], rstd * v[i]);
    return;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (n8 + i < N) v[i] = rstd * (v[i] - mean * colsum[n8 + i]);
}

// One 8-column group of an output row: the folded norm's correction, bias, activation, residual; the eight
// float32 results stay in v.
template <int EPI>
__device__ __forceinline__ void finish8(float (&v)[8], const uint32_t* r, int n8, int N, size_t row,
                                        const float* __restrict__ bias, bool bias_vec, const __nv_bfloat16* residual,
                                        bool have_fetched, uint4 fetched, const float* __restrict__ colsum, float mean,
                                        float rstd) {
  const bool whole = n8 + 8 <= N;
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
  if (colsum) unfold8(v, n8, N, colsum, mean, rstd);
  if (bias) {
    if (whole && bias_vec) {   // the same 32 bytes for every lane of the warp: two broadcast loads
      const float4 b0 = *reinterpret_cast<const float4*>(bias + n8), b1 = *reinterpret_cast<const float4*>(bias + n8 + 4);
      v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
      v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (n8 + i < N) v[i] += bias[n8 + i];
    }
  }
  if (EPI != EPI_NONE) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = activate<EPI, true>(v[i]);
  }
  if (residual) {
    if (have_fetched || (whole && ((row + n8) & 7) == 0)) {
      const uint4 u = have_fetched ? fetched : *reinterpret_cast<const uint4*>(residual + row + n8);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] += __uint_as_float(w[i] << 16);
        v[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (n8 + i < N) v[i] += __bfloat162float(residual[row + n8 + i]);
    }
  }
}

// float32 results go out as they are: 32 bytes a lane and group, a whole sector.
__device__ __forceinline__ void store8_f32(const float (&v)[8], int n8, int N, size_t row, float* C) {
  float* out = C + row + n8;
  if (n8 + 8 <= N && ((row + n8) & 3) == 0) {
    *reinterpret_cast<float4*>(out) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(out + 4) = make_float4(v[4], v[5], v[6], v[7]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (n8 + i < N) out[i] = v[i];
  }
}

// bfloat16 results are 16 bytes a lane and group.  Written by the lane that holds them (one lane per row) they
// would be half sectors 32 rows apart; so a warp first puts its 32 rows x 32 columns into shared memory (64 bytes
// a row, the 16-byte pieces of a row XORed with bits of the row number against bank conflicts) and writes them out
// from there with four lanes on the 64 contiguous bytes of a row: whole sectors, half as many.
__device__ __forceinline__ int stage_index(int row, int piece) { return row * 4 + (piece ^ ((row >> 1) & 3)); }

// Eight bfloat16 of row `row` (an element offset) at column n8, from a staged piece.
__device__ __forceinline__ void store_piece(uint4 u, int n8, int N, size_t row, __nv_bfloat16* C) {
  __nv_bfloat16* out = C + row + n8;
  if (n8 + 8 <= N && ((row + n8) & 7) == 0) {
    *reinterpret_cast<uint4*>(out) = u;
  } else {
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (n8 + i < N) out[i] = e[i];
  }
}

// Eight key or value columns n8..n8+7 (n8 >= q_width, a multiple of 8; N = q_width + 2*Hkv*Dh with Dh a
// multiple of 8, so the eight stay inside one head and all of them exist) of one token into the token's page:
// one 16-byte store.  slot: the page's element offset, in_page: the token's row in it.
__device__ __forceinline__ void scatter_piece(uint4 u, int n8, const KvScatter& kv, long long slot, int in_page) {
  const int kvw = kv.Hkv * kv.Dh;
  int c2 = n8 - kv.q_width;
  __nv_bfloat16* pool = kv.k_pool;
  if (c2 >= kvw) { c2 -= kvw; pool = kv.v_pool; }
  const int hh = c2 / kv.Dh, d = c2 - hh * kv.Dh;
  *reinterpret_cast<uint4*>(pool + ((size_t)slot + (size_t)hh * kv.page + in_page) * kv.Dh + d) = u;
}

template <int BN, int STAGES, typename TO, int EPI, bool SCATTER, int CG>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, const __nv_bfloat16* residual, TO* C, int M, int N, int K,
                    int ldc, int* __restrict__ status, KvScatter kv, NormFoldRows fold) {
  extern __shared__ uint8_t smem_raw[];
  Smem<BN, STAGES, CG>& sm = *reinterpret_cast<Smem<BN, STAGES, CG>*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (K + BK - 1) / BK;
  // A tile is (CG * 128) x BN; in a pair the CTA of rank r takes rows 128 r .. 128 r + 127 of it and fetches rows
  // (BN / 2) r .. of the tile's W rows.  Pair (or CTA) c takes tiles c, c + step, ...
  const int rank = CG == 2 ? (int)cluster_rank() : 0;
  const bool leader = rank == 0;
  const int tiles_m = (M + CG * BM - 1) / (CG * BM), tiles_n = (N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int first_tile = (int)blockIdx.x / CG, tile_step = (int)gridDim.x / CG;
  auto tile_m0 = [&](int t) { return (t % tiles_m) * (CG * BM) + rank * BM; };      // this CTA's first row
  auto tile_n0 = [&](int t) { return (t / tiles_m) * BN; };                          // the tile's first column
  constexpr int W_ROWS = BN / CG;                          // W rows per copy
  constexpr uint32_t STAGE_BYTES = CG * (BM + W_ROWS) * BK * sizeof(__nv_bfloat16);   // counted on a stage's barrier
  constexpr uint32_t TMEM_COLS = BN <= 128 ? 256 : 512;   // two accumulators; a power of two

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&sm.acc_full[b], 1); mbar_init(&sm.acc_empty[b], CG * 32 * EPI_WARPS); }
    mbar_init(&sm.drained, 1);
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
  }
  if (warp == 1) {   // the MMA warp owns the tensor memory (in a pair: warp 1 of both CTAs, the same columns in both)
    if (CG == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                   "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                   "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  volatile int* abort_flag = &sm.abort_flag;
  // In a pair: the leader's barriers as the peer names them, and the peer's abort flag.
  const uint32_t peer_abort = CG == 2 ? peer_addr(&sm.abort_flag, (uint32_t)(rank ^ 1)) : 0u;
  pdl_trigger();
  // The weights do not come from the previous kernel: the W rows of the first tile's first stages are asked
  // for before the wait, so that after it only the rows of A are missing.  The barriers of these stages are armed
  // before the two CTAs of a pair meet, the copies follow after.
  int early = 0;
  if (first_tile < n_tiles) early = k_tiles < STAGES ? k_tiles : STAGES;
  if (threadIdx.x == 0 && leader)
    for (int s = 0; s < early; ++s) mbar_expect_tx(&sm.full[s], STAGE_BYTES);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (CG == 2) cluster_sync();   // the peer's barriers are initialised, the leader's first stages armed
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sm.tmem_base;
  // this CTA's copies of a stage: its rows of A, its rows of W
  auto load_a = [&](int s, int kt, int m0) {
    if (CG == 2) tma_load_2d_pair(sm.a[s], &map_a, kt * BK, m0, peer_addr(&sm.full[s], 0));
    else tma_load_2d(sm.a[s], &map_a, kt * BK, m0, &sm.full[s]);
  };
  auto load_w = [&](int s, int kt, int n0) {
    if (CG == 2) tma_load_2d_pair(sm.b[s], &map_w, kt * BK, n0 + rank * W_ROWS, peer_addr(&sm.full[s], 0));
    else tma_load_2d(sm.b[s], &map_w, kt * BK, n0, &sm.full[s]);
  };
  if (threadIdx.x == 0)
    for (int s = 0; s < early; ++s) load_w(s, s, tile_n0(first_tile));
  pdl_wait();   // A (and the residual) come from the previous kernel
  residual = after_wait(residual);

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;   // stages filled so far, over all tiles
      bool ok = true;
      for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step) {
        const int m0 = tile_m0(tile), n0 = tile_n0(tile);
        for (int kt = 0; kt < k_tiles; ++kt, ++issued) {
          const int s = issued % STAGES;
          const uint32_t ph = (issued / STAGES) & 1;
          if (issued < early) {   // a fresh stage, armed, whose W rows are on their way already
            load_a(s, kt, m0);
            continue;
          }
          // free once the products that read it have completed (in a pair: the commit arrives in both CTAs)
          if (!mbar_wait(&sm.empty[s], ph ^ 1, abort_flag, peer_abort)) { ok = false; break; }
          if (leader) mbar_expect_tx(&sm.full[s], STAGE_BYTES);
          load_a(s, kt, m0);
          load_w(s, kt, n0);
        }
      }
      if (*abort_flag && leader) {   // gave up: let the copies already issued land before the CTA exits
        for (int i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i) {
          const uint32_t addr = smem_u32(&sm.full[i % STAGES]);
          for (uint32_t p = 0; p < (1u << 20); ++p) {
            uint32_t done;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                         "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(addr), "r"((uint32_t)((i / STAGES) & 1))
                         : "memory");
            if (done) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {   // one thread issues the products, for both CTAs of a pair
      constexpr uint32_t idesc = umma_idesc(CG * BM, BN);
      int consumed = 0, it = 0;
      bool ok = true;
      for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step, ++it) {
        const int b = it & 1;
        // the epilogue (of both CTAs) must have drained this accumulator (its previous use was tile it-2)
        ok = mbar_wait(&sm.acc_empty[b], ((it >> 1) & 1) ^ 1, abort_flag, peer_abort);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_acc = tmem_base + (uint32_t)(b * BN);
        for (int kt = 0; kt < k_tiles; ++kt, ++consumed) {
          const int s = consumed % STAGES;
          const uint32_t ph = (consumed / STAGES) & 1;
          ok = mbar_wait(&sm.full[s], ph, abort_flag, peer_abort);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          // the same offsets in both CTAs of a pair: the descriptors name them in each CTA's own shared memory
          const uint64_t da = umma_desc(smem_u32(sm.a[s])), db = umma_desc(smem_u32(sm.b[s]));
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {   // 16 bf16 = 32 bytes = 2 units of the descriptor's start address
            if (CG == 2) umma_bf16_pair(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
            else umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
          }
          // the stage is free once these MMAs have read it
          if (CG == 2) umma_commit_both(&sm.empty[s]);
          else umma_commit(&sm.empty[s]);
        }
#ifdef MLXB_TEST_WAIT_TIMEOUT
        if (g_test_withhold_arrival && it == 0) continue;   // the test's missing arrival
#endif
        if (ok) {   // arrives when every MMA of this tile has completed
          if (CG == 2) umma_commit_both(&sm.acc_full[b]);
          else umma_commit(&sm.acc_full[b]);
        }
      }
    }
  } else {
    // epilogue: warps 2..17; warp w may touch TMEM lanes 32*(w%4) .. +31; the four warps of a quadrant
    // split the tile's columns
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;          // which slice of the columns (0 .. EPI_WARPS/4 - 1)
    constexpr int HALF_COLS = BN / (EPI_WARPS / 4);   // 32, 48 or 64 columns per warp
    const bool bias_vec = bias && (((uintptr_t)bias & 15) == 0);
    const uint32_t acc_empty_leader[2] = {CG == 2 ? peer_addr(&sm.acc_empty[0], 0) : 0u,
                                          CG == 2 ? peer_addr(&sm.acc_empty[1], 0) : 0u};
    int it = 0;
    for (int tile = first_tile; tile < n_tiles; tile += tile_step, ++it) {
      const int b = it & 1;
      const int m0 = tile_m0(tile), n0 = tile_n0(tile);
      const int m = m0 + q * 32 + lane;
      const size_t row = (size_t)m * ldc;
      // The residual of this lane's row, 32 columns at a time (64 contiguous bytes), is fetched a chunk ahead:
      // the first chunk while the tile's products are still running, each further one while the chunk before
      // it is worked on.  Bit g of `have` says that group g of the chunk was fetched (whole and aligned).
      float mean = 0.f, rstd = 1.f;
      if (fold.colsum != nullptr && m < M) {
        const float2 st = fold.stats[m];
        mean = st.x;
        rstd = st.y;
      }
      uint4 res0, res1, res2, res3, nx0, nx1, nx2, nx3;
      res0 = res1 = res2 = res3 = nx0 = nx1 = nx2 = nx3 = make_uint4(0u, 0u, 0u, 0u);
      unsigned have = 0, have_next = 0;
#define FETCH_RESIDUAL(C0, D0, D1, D2, D3, HAVE)                                                        \
      {                                                                                                   \
        HAVE = 0;                                                                                         \
        if (residual != nullptr && m < M) {                                                               \
          const int nb = n0 + half * HALF_COLS + (C0);                                                    \
          const __nv_bfloat16* rp = residual + row + nb;                                                  \
          const bool al = ((row + nb) & 7) == 0;                                                          \
          if (al && (C0) + 0 < HALF_COLS && nb + 8 <= N) { D0 = *reinterpret_cast<const uint4*>(rp); HAVE |= 1u; }          \
          if (al && (C0) + 8 < HALF_COLS && nb + 16 <= N) { D1 = *reinterpret_cast<const uint4*>(rp + 8); HAVE |= 2u; }     \
          if (al && (C0) + 16 < HALF_COLS && nb + 24 <= N) { D2 = *reinterpret_cast<const uint4*>(rp + 16); HAVE |= 4u; }   \
          if (al && (C0) + 24 < HALF_COLS && nb + 32 <= N) { D3 = *reinterpret_cast<const uint4*>(rp + 24); HAVE |= 8u; }   \
        }                                                                                                 \
      }
      FETCH_RESIDUAL(0, res0, res1, res2, res3, have)
      if (!mbar_wait(&sm.acc_full[b], (it >> 1) & 1, abort_flag, peer_abort)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // fused cache write: this row's slot in its page (an element offset before the head and dim are added);
      // -1 for a padding row or an index out of range
      long long slot = -1;
      int in_page = 0;
      if (SCATTER && m < M && n0 + BN > kv.q_width) {
        const int r = kv.token_req[m];
        if (r >= 0) {
          const int pos = kv.positions[m];
          const int lp = pos / kv.page;
          const int pg = (pos >= 0 && lp < kv.max_pages) ? kv.block_table[(size_t)r * kv.max_pages + lp] : -2;
          if (pg == -2) atomicOr(kv.status, MLXB_ST_POSITION_RANGE);
          else if (pg >= kv.n_pages) atomicOr(kv.status, MLXB_ST_PAGE_RANGE);
          else if (pg >= 0) { slot = (long long)pg * kv.Hkv * kv.page; in_page = pos % kv.page; }
        }
      }
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BN + half * HALF_COLS);
#pragma unroll 1
      for (int c0 = 0; c0 < HALF_COLS; c0 += 32) {
        uint32_t r[32];
        if (c0 + 32 <= HALF_COLS) {
          tmem_ld32(taddr + (uint32_t)c0, r);   // every lane takes part
        } else {                                // 48 columns per warp (BN = 192): the last 16
          tmem_ld16(taddr + (uint32_t)c0, r);
        }
        if (c0 + 32 < HALF_COLS) FETCH_RESIDUAL(c0 + 32, nx0, nx1, nx2, nx3, have_next)
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 + 32 >= HALF_COLS) {   // this warp's part of the accumulator is in registers: hand it back
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          if (CG == 2) mbar_arrive_cluster(acc_empty_leader[b]);   // the leader issues the products into both halves
          else mbar_arrive(&sm.acc_empty[b]);
        }
        if (sizeof(TO) == 4) {
          if (m < M) {
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              const int n8 = n0 + half * HALF_COLS + c0 + g8 * 8;
              if (c0 + g8 * 8 < HALF_COLS && n8 < N) {
                float v[8];
                finish8<EPI>(v, r + g8 * 8, n8, N, row, bias, bias_vec, residual, (have >> g8) & 1,
                             g8 == 0 ? res0 : (g8 == 1 ? res1 : (g8 == 2 ? res2 : res3)), fold.colsum, mean, rstd);
                store8_f32(v, n8, N, row, reinterpret_cast<float*>(C));
              }
            }
          }
        } else {
          uint4* stg = sm.stage[warp - 2];
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            const int n8 = n0 + half * HALF_COLS + c0 + g8 * 8;
            uint4 u = make_uint4(0u, 0u, 0u, 0u);
            if (m < M && c0 + g8 * 8 < HALF_COLS && n8 < N) {
              float v[8];
              if (SCATTER && n8 >= kv.q_width)   // keys and values: no activation, no residual
                finish8<EPI_NONE>(v, r + g8 * 8, n8, N, row, bias, bias_vec, nullptr, false, u, fold.colsum, mean, rstd);
              else
                finish8<EPI>(v, r + g8 * 8, n8, N, row, bias, bias_vec, residual, (have >> g8) & 1,
                             g8 == 0 ? res0 : (g8 == 1 ? res1 : (g8 == 2 ? res2 : res3)), fold.colsum, mean, rstd);
              u = pack8(v);
            }
            stg[stage_index(lane, g8)] = u;
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j) {   // four lanes on a row's 64 bytes, eight rows an instruction
            const int rr = 8 * j + (lane >> 2), piece = lane & 3;
            const uint4 u = stg[stage_index(rr, piece)];
            const int mm = m0 + q * 32 + rr;
            const int n8 = n0 + half * HALF_COLS + c0 + piece * 8;
            long long slot_r = -1;
            int in_page_r = 0;
            if (SCATTER) {   // the row's page, from the lane that looked it up
              slot_r = __shfl_sync(0xffffffffu, slot, rr);
              in_page_r = __shfl_sync(0xffffffffu, in_page, rr);
            }
            if (mm < M && c0 + piece * 8 < HALF_COLS && n8 < N) {
              if (SCATTER && n8 >= kv.q_width) {
                if (slot_r >= 0) scatter_piece(u, n8, kv, slot_r, in_page_r);
              } else {
                store_piece(u, n8, N, (size_t)mm * ldc, reinterpret_cast<__nv_bfloat16*>(C));
              }
            }
          }
          __syncwarp();   // the pieces are read before the next chunk overwrites them
        }
        res0 = nx0; res1 = nx1; res2 = nx2; res3 = nx3;
        have = have_next;
      }
#undef FETCH_RESIDUAL
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // In a pair nobody goes on alone: the peer's epilogue may still read its tensor memory, and arrivals, copies
  // counted on the leader's barriers and a raised abort flag may still be on their way.
  if (CG == 2) cluster_sync();
  const bool aborted = sm.abort_flag != 0;     // the same in both CTAs of a pair from here on
  if (threadIdx.x == 0 && aborted) atomicOr(status, MLXB_ST_WAIT_TIMEOUT);
  if (warp == 1 && leader) {
    if (lane == 0 && aborted) {
      // Somebody gave up.  Products this thread issued may still be running on the tensor memory that is freed
      // below: one more commit arrives when all of them have completed; wait for it, bounded.
      if (CG == 2) umma_commit_pair_local(&sm.drained);
      else umma_commit(&sm.drained);
      const uint32_t addr = smem_u32(&sm.drained);
      for (uint32_t p = 0; p < (1u << 20); ++p) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(addr), "r"(0u) : "memory");
        if (done) break;
      }
    }
    __syncwarp();
  }
  if (CG == 2 && aborted) cluster_sync();   // the peer frees its half only after the leader's products have drained
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (CG == 2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- host side

#ifdef MLXB_TEST_WAIT_TIMEOUT
// Test builds only: switch the withheld arrival on or off for the launches that follow on this device.
MLXB_EXPORT int mlxb_test_withhold_arrival(int on) {
  const cudaError_t e = cudaMemcpyToSymbol(g_test_withhold_arrival, &on, sizeof(int));
  if (e != cudaSuccess) return mlxb_fail((int)e, "withhold_arrival: %s", cudaGetErrorString(e));
  return 0;
}
#endif

static int make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(__nv_bfloat16)};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                                            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    const char* msg = nullptr;
    cuGetErrorString(r, &msg);
    return mlxb_fail(MLXB_BAD_ARG, "linear (tensor cores): cuTensorMapEncodeTiled(%d x %d, ld %d): %s", rows, cols, ld,
                     msg ? msg : "?");
  }
  return 0;
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

template <int BN, int STAGES, typename TO, bool SCATTER = false, int CG = 1>
static int launch(const void* A, const void* W, const float* bias, const void* residual, void* C, int M, int N, int K,
                  int lda, int ldc, int epi, int* status, cudaStream_t stream, const KvScatter& kv = KvScatter{},
                  const NormFoldRows& fold = NormFoldRows{}) {
  static_assert((BN / CG) % 8 == 0 && BN % (16 * CG) == 0, "a CTA's W rows are whole 8-row swizzle groups");
  static_assert(sizeof(Smem<BN, STAGES, CG>) + 1024 <= 227 * 1024, "stages and staging buffers fit a CTA's shared memory");
  CUtensorMap ma, mw;
  if (int e = make_map(&ma, A, M, K, lda, BM)) return e;
  if (int e = make_map(&mw, W, N, K, K, BN / CG)) return e;      // a copy brings this CTA's rows of the tile
  const size_t smem = sizeof(Smem<BN, STAGES, CG>) + 1024;
  const int n_tiles = ((M + CG * BM - 1) / (CG * BM)) * ((N + BN - 1) / BN);
  const int units = sm_count() / CG;                              // CTAs, or pairs of them
  const dim3 grid(CG * (n_tiles < units ? n_tiles : units));
  // The fused cache write has no activation: only the plain epilogue is built for it.
  return dispatch_activation(SCATTER ? (int)EPI_NONE : epi, [&](auto e) {
    constexpr int EPI = SCATTER ? (int)EPI_NONE : (int)decltype(e)::value;
    auto kern = gemm_tcgen05_kernel<BN, STAGES, TO, EPI, SCATTER, CG>;
    static bool raised = false;   // once per instantiation, and never for the first time inside a stream capture
    if (!raised) {
      cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return mlxb_fail((int)err, "linear (tensor cores): %zu bytes of shared memory: %s", smem,
                                               cudaGetErrorString(err));
      raised = true;
    }
    if (CG == 1) {
      launch_pdl(kern, grid, dim3(THREADS), smem, stream, ma, mw, bias, (const __nv_bfloat16*)residual, (TO*)C, M, N, K,
                 ldc, status, kv, fold);
    } else {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = grid;
      cfg.blockDim = dim3(THREADS);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = stream;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = CG;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = mlxb_pdl_enabled() ? 2 : 1;
      cudaLaunchKernelEx(&cfg, kern, ma, mw, bias, (const __nv_bfloat16*)residual, (TO*)C, M, N, K, ldc, status, kv, fold);
    }
    return mlxb_check_launch("linear (tensor cores)");
  });
}

// Tile shape.  The width is the one whose waves of tiles over the SMs cost least, a tile's cost being the rows it
// streams per K step (128 rows of A plus BN rows of W).  Pairs of CTAs on 256 x BN tiles are taken where they were
// measured faster: long inner dimensions (their gain is in the main loop: 8192 x 8192 x 8192 runs at 1.50 against
// 1.39 PFLOP/s) with at least three waves of tiles to work on; with short inner dimensions or few tiles the pair's
// set-up and its hand-overs across the cluster cost more than the main loop gains (2048 x 4096 x 1024: 31.7 against
// 29.7 us).
struct TileChoice { int bn, cg; };
static TileChoice tile_choice(int M, int N, int K, bool pairs_built) {
  const int sms = sm_count();
  const char* want_pair = getenv("MLXB_TC_PAIR");   // experiments and tests: 0 = never, 1 = wherever a pair has two row tiles
  int cg = 1;
  if (pairs_built && M > BM) {
    if (want_pair) cg = want_pair[0] == '1' ? 2 : 1;
    else if (K >= 2048 && (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256) >= 3 * (sms / 2)) cg = 2;
  }
  const int tiles_m = (M + cg * BM - 1) / (cg * BM), units = sms / cg;
  TileChoice best = {128, cg};
  long long best_cost = -1;
  for (int bn : {256, 192, 128}) {
    const long long tiles = (long long)tiles_m * ((N + bn - 1) / bn);
    const long long cost = ((tiles + units - 1) / units) * (cg * BM + bn);
    if (best_cost < 0 || cost < best_cost) { best = {bn, cg}; best_cost = cost; }
  }
  if (const char* force = getenv("MLXB_TC_BN")) best.bn = atoi(force);   // experiments and tests
  return best;
}

// A: bfloat16 [M, K] at row stride lda; W: bfloat16 [N, K] contiguous; bias float32[N] or null; residual bfloat16
// [M, N] at row stride ldc or null (may alias C); C bfloat16 or float32 (out_f32) [M, N] at row stride ldc.
// K, lda multiples of 8; A and W 16-byte aligned.  status: int32 word that receives MLXB_ST_WAIT_TIMEOUT if a
// bounded wait inside the kernel gives up.
static int linear_tcgen05(int out_f32, const void* A, const void* W, const float* bias, const void* residual, void* C,
                          int M, int N, int K, int lda, int ldc, int epi, int* status, const NormFoldRows& fold,
                          cudaStream_t stream);

MLXB_EXPORT int mlxb_linear_tcgen05(int out_f32, const void* A, const void* W, const float* bias, const void* residual,
                                    void* C, int M, int N, int K, int lda, int ldc, int epi, int* status,
                                    cudaStream_t stream) {
  return linear_tcgen05(out_f32, A, W, bias, residual, C, M, N, K, lda, ldc, epi, status, NormFoldRows{}, stream);
}

// The same with a folded LayerNorm: W and bias are the folded ones, colsum float32[N], stats float32[M][2]
// (mean, rstd of the rows of A, from mlxb_row_stats).
MLXB_EXPORT int mlxb_linear_tcgen05_fold(int out_f32, const void* A, const void* W, const float* bias,
                                         const void* residual, void* C, int M, int N, int K, int lda, int ldc, int epi,
                                         int* status, const float* colsum, const void* stats, cudaStream_t stream) {
  if (colsum == nullptr || stats == nullptr) return mlxb_fail(MLXB_BAD_ARG, "linear (folded norm): column sums or row statistics missing");
  return linear_tcgen05(out_f32, A, W, bias, residual, C, M, N, K, lda, ldc, epi, status,
                        NormFoldRows{colsum, (const float2*)stats}, stream);
}

static int linear_tcgen05(int out_f32, const void* A, const void* W, const float* bias, const void* residual, void* C,
                          int M, int N, int K, int lda, int ldc, int epi, int* status, const NormFoldRows& fold,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (lda & 7) || lda < K || ldc < N)
    return mlxb_fail(MLXB_BAD_ARG, "linear (tensor cores): K %d and row stride %d must be multiples of 8 (ldc %d, N %d)",
                     K, lda, ldc, N);
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15))
    return mlxb_fail(MLXB_BAD_ARG, "linear (tensor cores): operands must be 16-byte aligned");
  if (!activation_known(epi)) return mlxb_fail(MLXB_BAD_ARG, "linear: epilogue code %d", epi);
  const TileChoice best = tile_choice(M, N, K, !out_f32);   // pairs are built for bfloat16 results
#define GO(BN_, ST_)                                                                                              \
  {                                                                                                               \
    if (out_f32)                                                                                                  \
      return launch<BN_, ST_, float>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, status, stream, KvScatter{}, \
                                     fold);                                                                       \
    return launch<BN_, ST_, __nv_bfloat16>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, status, stream,        \
                                           KvScatter{}, fold);                                                    \
  }
#define GO2(BN_, ST_)                                                                                             \
  return launch<BN_, ST_, __nv_bfloat16, false, 2>(A, W, bias, residual, C, M, N, K, lda, ldc, epi, status, stream, \
                                                   KvScatter{}, fold);
  if (best.cg == 2) {
    if (best.bn == 256) GO2(256, 6)
    if (best.bn == 192) GO2(192, 6)
    GO2(128, 8)
  }
  if (best.bn == 256) GO(256, 4)
  if (best.bn == 192) GO(192, 4)
  GO(128, 6)
#undef GO
#undef GO2
}


// The fused [q | k | v] projection with the cache write in its epilogue, for many rows: columns [0, q_width) go
// to C (bfloat16, row stride ldc); key and value columns go into k_pool / v_pool [n_pages, Hkv, page, Dh] at each
// token's page and row.  N = q_width + 2*Hkv*Dh; q_width and Dh multiples of 8.  Rows with token_req < 0 write
// no keys or values.
static int linear_tcgen05_qkv(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int lda,
                              int ldc, const int* positions, const int* token_req, const int* block_table,
                              int max_pages, int n_pages, int page, int Hkv, int Dh, int q_width, void* k_pool,
                              void* v_pool, int* status, const NormFoldRows& fold, cudaStream_t stream);

MLXB_EXPORT int mlxb_linear_tcgen05_qkv(const void* A, const void* W, const float* bias, void* C, int M, int N, int K,
                                        int lda, int ldc, const int* positions, const int* token_req,
                                        const int* block_table, int max_pages, int n_pages, int page, int Hkv, int Dh,
                                        int q_width, void* k_pool, void* v_pool, int* status, cudaStream_t stream) {
  return linear_tcgen05_qkv(A, W, bias, C, M, N, K, lda, ldc, positions, token_req, block_table, max_pages, n_pages,
                            page, Hkv, Dh, q_width, k_pool, v_pool, status, NormFoldRows{}, stream);
}

// The same with a folded LayerNorm (see mlxb_linear_tcgen05_fold).
MLXB_EXPORT int mlxb_linear_tcgen05_qkv_fold(const void* A, const void* W, const float* bias, void* C, int M, int N,
                                             int K, int lda, int ldc, const int* positions, const int* token_req,
                                             const int* block_table, int max_pages, int n_pages, int page, int Hkv,
                                             int Dh, int q_width, void* k_pool, void* v_pool, int* status,
                                             const float* colsum, const void* stats, cudaStream_t stream) {
  if (colsum == nullptr || stats == nullptr) return mlxb_fail(MLXB_BAD_ARG, "linear (folded norm): column sums or row statistics missing");
  return linear_tcgen05_qkv(A, W, bias, C, M, N, K, lda, ldc, positions, token_req, block_table, max_pages, n_pages,
                            page, Hkv, Dh, q_width, k_pool, v_pool, status, NormFoldRows{colsum, (const float2*)stats},
                            stream);
}

static int linear_tcgen05_qkv(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, int lda,
                              int ldc, const int* positions, const int* token_req, const int* block_table,
                              int max_pages, int n_pages, int page, int Hkv, int Dh, int q_width, void* k_pool,
                              void* v_pool, int* status, const NormFoldRows& fold, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (lda & 7) || lda < K || ldc < N)
    return mlxb_fail(MLXB_BAD_ARG, "linear (tensor cores): K %d and row stride %d must be multiples of 8 (ldc %d, N %d)",
                     K, lda, ldc, N);
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15))
    return mlxb_fail(MLXB_BAD_ARG, "linear (tensor cores): operands must be 16-byte aligned");
  if (Hkv <= 0 || Dh <= 0 || (Dh & 7) || page <= 0 || q_width < 0 || (q_width & 7) || N != q_width + 2 * Hkv * Dh)
    return mlxb_fail(MLXB_BAD_ARG, "linear (q|k|v): %d outputs for %d query columns and 2 x %d x %d", N, q_width, Hkv, Dh);
  const KvScatter kv = {positions, token_req, block_table, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, status,
                        max_pages, n_pages, page, Hkv, Dh, q_width};
  const TileChoice best = tile_choice(M, N, K, true);
  if (best.cg == 2) {
    if (best.bn == 256)
      return launch<256, 6, __nv_bfloat16, true, 2>(A, W, bias, nullptr, C, M, N, K, lda, ldc, EPI_NONE, status, stream, kv, fold);
    if (best.bn == 192)
      return launch<192, 6, __nv_bfloat16, true, 2>(A, W, bias, nullptr, C, M, N, K, lda, ldc, EPI_NONE, status, stream, kv, fold);
    return launch<128, 8, __nv_bfloat16, true, 2>(A, W, bias, nullptr, C, M, N, K, lda, ldc, EPI_NONE, status, stream, kv, fold);
  }
  if (best.bn == 256)
    return launch<256, 4, __nv_bfloat16, true>(A, W, bias, nullptr, C, M, N, K, lda, ldc, EPI_NONE, status, stream, kv, fold);
  if (best.bn == 192)
    return launch<192, 4, __nv_bfloat16, true>(A, W, bias, nullptr, C, M, N, K, lda, ldc, EPI_NONE, status, stream, kv, fold);
  return launch<128, 6, __nv_bfloat16, true>(A, W, bias, nullptr, C, M, N, K, lda, ldc, EPI_NONE, status, stream, kv, fold);
}
