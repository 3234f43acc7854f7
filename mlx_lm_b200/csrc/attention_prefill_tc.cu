// Causal attention of prompt portions over the paged key/value cache on the tcgen05 tensor cores, for heads
// of 64 (128-byte rows, one swizzle span).
//
// One CTA handles a tile of up to 128 queries of one head and walks the request's keys in blocks of 128
// positions.  Warp 8 is the producer and the MMA issuer (one elected thread), warps 0-7 do the softmax, two
// threads per query row (the row is the thread's lane of tensor memory; warps 0-3 take the block's first 64 keys
// and the first 32 output dims, warps 4-7 the others; the two exchange their maxima through shared memory):
//   TMA        Q tile once; per block the pages of K and of V (one box of [page x 64] per page, straight from
//              the pool [n_pages * Hkv * page, 64] through the block table) into 128-byte-swizzled shared memory
//   S = Q K^T  tcgen05.mma, M 128 x N 128 x K 64, both operands K-major, accumulator in tensor memory
//   softmax    tcgen05.ld of the row, mask (causal, window), running maximum and sum in float32 with exp2 of
//              scores pre-multiplied by scale * log2(e); P rounded to bfloat16 into shared memory in the
//              K-major swizzled layout of an A operand
//   O_b = P V  tcgen05.mma, M 128 x N 64 x K 128; V is used as it lies in the pages, [key][dim], i.e. as an
//              MN-major B operand; a fresh accumulator per block
//   O          kept in registers by the softmax threads: O = O * correction + O_b, so nothing is ever
//              written back to tensor memory
// K of the next block is requested as soon as S has been computed, V of the next block as soon as P V has, so
// the loads overlap the softmax; two CTAs fit an SM (80 KB of shared memory, 256 of 512 tensor-memory
// columns each) and overlap one another's phases.  The order in which a query's keys are added depends only
// on its position (blocks of 128 positions from block 0 or the window's first block upward).
//
// Every mbarrier wait is bounded; a wait that gives up sets an abort flag that all roles see, the CTA frees
// its tensor memory and reports MLXB_ST_WAIT_TIMEOUT.  TMA coordinates: x is always 0 or a multiple of 64
// elements (128 bytes).  Pages that a block covers but the request does not have (beyond its last position)
// are loaded from the request's first page instead: their scores are masked, and the values they are
// multiplied with (by zero) must be finite.
#include <cuda.h>

#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

constexpr int TQ = 128;          // queries per tile
constexpr int TK = 128;          // keys per block
constexpr int HD = 64;           // head size
constexpr int AT_SOFTMAX = 256;  // softmax threads: 8 warps
constexpr int AT_THREADS = AT_SOFTMAX + 32;  // + 1 producer / MMA warp
constexpr int MMA_WARP = AT_SOFTMAX / 32;
constexpr uint32_t AT_SPIN_LIMIT = 1u << 20;
constexpr uint32_t AT_TMEM_COLS = 256;   // S: columns 0..127, O_b: 128..191

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
// Bounded wait for the phase with the given parity; false after AT_SPIN_LIMIT polls or when another role gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < AT_SPIN_LIMIT; ++i) {
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
  return false;
}
// The same for a whole warp, with one answer for all its lanes: the warp stays together whatever happens, so
// that it can meet in __syncwarp afterwards.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// Shared-memory matrix descriptors for 128-byte-swizzled tiles whose rows are 128 bytes and whose groups of 8
// rows are 1024 bytes apart: start address / 16, the stride between 8-row groups (1024 bytes) in bits 32-45,
// descriptor version 1 (bit 46), layout SWIZZLE_128B (2) in bits 61-63.  For a K-major operand (rows = M or N
// index, the 128 bytes run along K) the other offset (bits 16-29) is unused; for an MN-major operand (rows = K
// index, the 128 bytes run along M or N) it is the distance between 64-element spans along M/N, of which there
// is one here.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::f16: float32 accumulator, A and B bfloat16, A K-major, B K-major or
// MN-major (bit 16), N/8 in bits 17-22, M/16 in bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
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
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AtSmem {
  alignas(1024) __nv_bfloat16 q[TQ * HD];        // [query][dim], 128-byte rows, swizzled (TMA)
  alignas(1024) __nv_bfloat16 k[TK * HD];        // [key][dim]
  alignas(1024) __nv_bfloat16 v[TK * HD];        // [key][dim]
  alignas(1024) __nv_bfloat16 p[2 * TQ * 64];    // two spans of 64 keys: [span][query][64 keys], swizzled by hand
  alignas(8) uint64_t q_full, k_full, v_full, s_full, p_full, o_full;
  uint64_t x_full;                               // the softmax threads' exchange of row maxima (and, at the end, sums)
  float row_max[2][TQ];                          // the two halves' maxima of the current block, per row
  uint32_t tmem_base;
  int abort_flag;
};

// tiles: int32 [n_tiles][4] = (row of the tile's first token among the step's tokens, queries in the tile
// (1..128), block-table row of the request, position of the tile's first query).
__global__ void __launch_bounds__(AT_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int4* __restrict__ tiles,
                            const int* __restrict__ block_table, int max_pages, int n_pages, int page, int Hq, int Hkv,
                            int window, float scale_log2e, __nv_bfloat16* out, int ldo, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  AtSmem& sm = *reinterpret_cast<AtSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (tiles[blockIdx.x].y <= 0) return;   // a tile without queries pads the list to a size seen before: nothing to do

  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 1);
    mbar_init(&sm.k_full, 1);
    mbar_init(&sm.v_full, 1);
    mbar_init(&sm.s_full, 1);
    mbar_init(&sm.p_full, AT_SOFTMAX / 32);   // one arrival per softmax warp
    mbar_init(&sm.o_full, 1);
    mbar_init(&sm.x_full, AT_SOFTMAX / 32);
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == MMA_WARP) {   // the MMA warp owns the tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(AT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sm.tmem_base;
  volatile int* abort_flag = &sm.abort_flag;
  pdl_trigger();
  pdl_wait();   // queries, keys and values of this step come from the kernel before

  const int4 tile = tiles[blockIdx.x];
  const int row0 = tile.x, n_rows = tile.y, req = tile.z, pos0 = tile.w;
  const int h = blockIdx.y, hk = h / (Hq / Hkv);
  const int last_pos = pos0 + n_rows - 1;
  const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int kb_lo = first_key / TK, kb_hi = last_pos / TK;
  const int n_blocks = kb_hi - kb_lo + 1;

  if (warp == MMA_WARP) {
    // The whole warp takes part in the loads: lane s looks up the page of slot s of a block (one round of
    // global loads for all pages at once, a block ahead of its use) and issues that page's TMA copy; lane 0
    // alone arms the barriers and issues the MMAs.  Waits are done by every lane with one answer for the warp.
    const int* bt = block_table + (size_t)req * max_pages;
    const int shift = __ffs(page) - 1;
    const int pages_per_block = TK / page;
    int first_page = bt[0];
    if (first_page < 0 || first_page >= n_pages) {
      if (lane == 0) atomicOr(status, first_page < 0 ? MLXB_ST_POSITION_RANGE : MLXB_ST_PAGE_RANGE);
      first_page = 0;
    }
    auto page_of = [&](int kb) {   // the page this lane copies for block kb (lanes >= pages_per_block: unused)
      const int key0 = kb * TK + lane * page;
      int pg = first_page;
      if (lane < pages_per_block && kb <= kb_hi && key0 <= last_pos) {
        const int lp = key0 >> shift;
        const int id = lp < max_pages ? bt[lp] : -1;
        if (id < 0 || id >= n_pages) atomicOr(status, id < 0 ? MLXB_ST_POSITION_RANGE : MLXB_ST_PAGE_RANGE);
        else pg = id;
      }
      return pg;
    };
    auto load_pages = [&](const CUtensorMap* map, __nv_bfloat16* dst, uint64_t* bar, int pg) {
      if (lane == 0) mbar_expect_tx(bar, TK * HD * (uint32_t)sizeof(__nv_bfloat16));
      __syncwarp();
      if (lane < pages_per_block) tma_load_2d(dst + (size_t)lane * page * HD, map, 0, (pg * Hkv + hk) * page, bar);
    };
    int pg_now = page_of(kb_lo);
    if (lane == 0) {
      mbar_expect_tx(&sm.q_full, TQ * HD * (uint32_t)sizeof(__nv_bfloat16));
      tma_load_2d(sm.q, &map_q, h * HD, row0, &sm.q_full);
    }
    load_pages(&map_k, sm.k, &sm.k_full, pg_now);
    load_pages(&map_v, sm.v, &sm.v_full, pg_now);
    int pg_next = page_of(kb_lo + 1);

    constexpr uint32_t idesc_s = umma_idesc(TQ, TK, false);
    constexpr uint32_t idesc_o = umma_idesc(TQ, HD, true);
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;
    // S of a block needs only its keys and the S columns, which the softmax threads give back with P; so
    // S(i + 1) is issued right behind P V(i) and is ready when the softmax threads come back from accumulating O.
    auto issue_s = [&]() {
      if (lane == 0) {
        const uint64_t da = umma_desc(smem_u32(sm.q), 16), db = umma_desc(smem_u32(sm.k), 16);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)   // 16 bf16 = 32 bytes = 2 units of the descriptor's start address
          umma_bf16(tmem_s, da + 2 * k, db + 2 * k, idesc_s, k > 0 ? 1u : 0u);
        umma_commit(&sm.s_full);
      }
      __syncwarp();
    };
    bool ok = mbar_wait_warp(&sm.q_full, 0, abort_flag) && mbar_wait_warp(&sm.k_full, 0, abort_flag);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_s();
    }
    for (int i = 0; i < n_blocks && ok; ++i) {
      const uint32_t ph = (uint32_t)(i & 1);
      const bool more = i + 1 < n_blocks;
      if (!(ok = mbar_wait_warp(&sm.s_full, ph, abort_flag))) break;    // S(i) is there: the K block is free
      if (more) load_pages(&map_k, sm.k, &sm.k_full, pg_next);
      if (!(ok = mbar_wait_warp(&sm.v_full, ph, abort_flag))) break;
      if (!(ok = mbar_wait_warp(&sm.p_full, ph, abort_flag))) break;    // P(i) is written, S(i) has been read
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < TK / 16; ++j) {   // 16 keys per step: A advances inside and across the two spans of P,
                                              // B by 16 rows of V
          const uint64_t da = umma_desc(smem_u32(sm.p) + (uint32_t)(j >> 2) * (TQ * 64 * 2), 16) + 2 * (j & 3);
          const uint64_t db = umma_desc(smem_u32(sm.v) + (uint32_t)j * (16 * HD * 2), TK * HD * 2);
          umma_bf16(tmem_o, da, db, idesc_o, j > 0 ? 1u : 0u);
        }
        umma_commit(&sm.o_full);
      }
      __syncwarp();
      if (more) {
        if (!(ok = mbar_wait_warp(&sm.k_full, ph ^ 1u, abort_flag))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_s();
      }
      const int pg_after = page_of(kb_lo + i + 2);                 // its latency hides behind the wait below
      if (!(ok = mbar_wait_warp(&sm.o_full, ph, abort_flag))) break;    // O_b(i) is there: V and P are free
      if (more) load_pages(&map_v, sm.v, &sm.v_full, pg_next);
      pg_next = pg_after;
    }
  } else {
    // softmax: thread (half, r) owns keys [64 half, 64 half + 64) of every block and output dims
    // [32 half, 32 half + 32) of query row r, which is lane r of tensor memory (warp w may touch lanes 32 (w % 4) ..)
    const int half = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int pos = pos0 + r;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t t_s = t_row + (uint32_t)(half * 64), t_o = t_row + 128u + (uint32_t)(half * 32);
    float o[HD / 2];
#pragma unroll
    for (int d = 0; d < HD / 2; ++d) o[d] = 0.f;
    float m = -INFINITY, l = 0.f;   // running maximum of the row in units of the exponent; this half's running sum
    uint8_t* p_row = reinterpret_cast<uint8_t*>(sm.p) + half * (TQ * 64 * 2) + (r >> 3) * 1024 + (r & 7) * 128;
    bool ok = true;
    for (int i = 0; i < n_blocks && ok; ++i) {
      const uint32_t ph = (uint32_t)(i & 1);
      const int key_base = (kb_lo + i) * TK + half * 64;
      if (!(ok = mbar_wait_warp(&sm.s_full, ph, abort_flag))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // blocks that lie wholly before the tile's first query and after every row's window floor need no mask
      const bool open = (kb_lo + i) * TK + TK - 1 <= pos0 && (window <= 0 || (kb_lo + i) * TK >= last_pos - window + 1);
      uint32_t s0[32], s1[32];
      tmem_ld32(t_s, s0);
      tmem_ld32(t_s + 32u, s1);
      tmem_wait_ld();
      float mx = -INFINITY;
      if (open) {
#pragma unroll
        for (int e = 0; e < 32; ++e) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[e]), __uint_as_float(s1[e])));
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int k0 = key_base + e, k1 = key_base + 32 + e;
          if (!(k0 <= pos && k0 >= lo)) s0[e] = 0xff800000u;   // -inf: masked here once, exp2 gives 0 below
          if (!(k1 <= pos && k1 >= lo)) s1[e] = 0xff800000u;
          mx = fmaxf(mx, fmaxf(__uint_as_float(s0[e]), __uint_as_float(s1[e])));
        }
      }
      sm.row_max[half][r] = mx;                         // a bounded wait, not bar.sync: a role may have given up
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.x_full);
      if (!(ok = mbar_wait_warp(&sm.x_full, ph, abort_flag))) break;
      mx = fmaxf(mx, sm.row_max[half ^ 1][r]);
      const float m_new = fmaxf(m, mx * scale_log2e);   // scale > 0
      const float base = m_new == -INFINITY ? 0.f : m_new;
      const float corr = fast_exp2(m - base);           // 2^-inf = 0
      m = m_new;
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float a0 = __uint_as_float(c == 0 ? s0[e] : s1[e]), a1 = __uint_as_float(c == 0 ? s0[e + 1] : s1[e + 1]);
          const float p0 = fast_exp2(fmaf(a0, scale_log2e, -base)), p1 = fast_exp2(fmaf(a1, scale_log2e, -base));
          sum += p0 + p1;
          const __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
          packed[e >> 1] = *reinterpret_cast<const uint32_t*>(&pr);
        }
        // 32 keys = four 16-byte chunks of this row's 64-key span, swizzled with the row
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = c * 4 + q4;
          *reinterpret_cast<uint4*>(p_row + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
        }
      }
      l = l * corr + sum;
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P was written by ordinary stores; the MMA reads it
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.p_full);
      if (!(ok = mbar_wait_warp(&sm.o_full, ph, abort_flag))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      {
        uint32_t ob[32];
        tmem_ld32(t_o, ob);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = fmaf(o[e], corr, __uint_as_float(ob[e]));
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    // the row's sum is the two halves' sums
    if (ok) {
      sm.row_max[half][r] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.x_full);
      ok = mbar_wait_warp(&sm.x_full, (uint32_t)(n_blocks & 1), abort_flag);
      l += sm.row_max[half ^ 1][r];
    }
    if (ok && r < n_rows) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = out + (size_t)(row0 + r) * ldo + h * HD + half * (HD / 2);
#pragma unroll
      for (int d = 0; d < HD / 2; d += 8) {
        float v8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v8[e] = o[d + e] * inv;
        *reinterpret_cast<uint4*>(dst + d) = pack8(v8);
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && sm.abort_flag) atomicOr(status, MLXB_ST_WAIT_TIMEOUT);
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(AT_TMEM_COLS) : "memory");
  }
}

static int make_map(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_rows,
                    const char* what) {
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(__nv_bfloat16)};
  const cuuint32_t box[2] = {(cuuint32_t)HD, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                                            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    const char* msg = nullptr;
    cuGetErrorString(r, &msg);
    return mlxb_fail(MLXB_BAD_ARG, "attention (portions, tcgen05): tensor map of %s (%lld x %d, ld %lld): %s", what,
                     rows, cols, ld, msg ? msg : "?");
  }
  return 0;
}

// bfloat16, heads of 64.  q: [n_tokens, >= Hq*64] at row stride ldq (a multiple of 8, base 16-byte aligned);
// out: [*, Hq*64] at row stride ldo (a multiple of 8, 16-byte aligned); tiles: int32 [n_tiles][4], see the kernel
// (tiles of at most 128 queries; a tile of 0 queries is skipped); pools [n_pages, Hkv, page, 64], page a power of two from 8 to 128.
MLXB_EXPORT int mlxb_attention_prefill_tc(const void* q, int ldq, int n_tokens, const int* tiles, int n_tiles,
                                          const int* block_table, int max_pages, int n_pages, int page, int Hq,
                                          int Hkv, int Dh, int window, float scale, const void* k_pool,
                                          const void* v_pool, void* out, int ldo, int* status, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (Dh != HD) return mlxb_fail(MLXB_BAD_ARG, "attention (portions, tcgen05): head size %d, this kernel takes %d", Dh, HD);
  if (page < 8 || page > TK || (page & (page - 1)))
    return mlxb_fail(MLXB_BAD_ARG, "attention (portions, tcgen05): page size %d (a power of two from 8 to %d)", page, TK);
  if (Hkv <= 0 || Hq <= 0 || Hq % Hkv || Hq > 65535)
    return mlxb_fail(MLXB_BAD_ARG, "attention (portions, tcgen05): %d query heads over %d key/value heads", Hq, Hkv);
  if ((ldq & 7) || (ldo & 7) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)tiles & 15) ||
      ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || ldq < Hq * HD)
    return mlxb_fail(MLXB_BAD_ARG, "attention (portions, tcgen05): rows and pools must be 16-byte aligned");
  CUtensorMap mq, mk, mv;
  if (int e = make_map(&mq, q, n_tokens, Hq * HD, ldq, TQ, "q")) return e;
  const long long pool_rows = (long long)n_pages * Hkv * page;
  if (int e = make_map(&mk, k_pool, pool_rows, HD, HD, page, "k pool")) return e;
  if (int e = make_map(&mv, v_pool, pool_rows, HD, HD, page, "v pool")) return e;
  const size_t smem = sizeof(AtSmem) + 1024;
  static bool raised = false;
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess)
      return mlxb_fail((int)e, "attention (portions, tcgen05): %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    raised = true;
  }
  launch_pdl(attention_prefill_tc_kernel, dim3(n_tiles, Hq), dim3(AT_THREADS), smem, stream, mq, mk, mv,
             (const int4*)tiles, block_table, max_pages, n_pages, page, Hq, Hkv, window,
             scale * 1.4426950408889634f, (__nv_bfloat16*)out, ldo, status);
  return mlxb_check_launch("attention (portions, tcgen05)");
}
