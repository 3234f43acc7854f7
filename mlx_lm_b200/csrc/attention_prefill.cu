// Causal attention of prompt portions over the paged key/value cache, on tensor cores.
//
// A portion (the next n > 1 tokens of one request) is cut into tiles of 64 or 128 queries; one CTA of four
// or eight warps handles (tile, query head), 16 queries a warp.  It walks the request's keys in blocks of 64
// positions, from the first block the tile may see (0, or the window's lower edge) to the block of
// the tile's last query; the keys of this very step are already in the pages.  K and V blocks are
// gathered through the block table with 16-byte cp.async into double-buffered shared memory (rows
// padded by 16 bytes, which makes every ldmatrix conflict-free for any head size that is a multiple
// of 16), so the next block loads while the current one is multiplied.
//   S = Q K^T        mma.sync m16n8k16, bf16 inputs, float32 accumulators; Q stays in registers
//   softmax          float32, online (running maximum and sum per query row), exp2 of scores
//                    pre-multiplied by scale*log2(e); masked: key > query position, key below the
//                    window, rows beyond the tile
//   O += P V         P rounded to bf16 as the A operand (the accumulator layout of S is the A layout
//                    of the next product), V through ldmatrix.trans
// Key split: a tile's key blocks form a chain that the CTA walks one after the other, and the tiles with the
// longest chains (the last queries of a long prompt) decide how long the kernel runs.  With KSPLIT = 2 the
// CTA has two groups of warps for the same queries; group g takes the key blocks whose index is g modulo 2,
// each group with shared-memory stages and barriers of its own, and the groups' partial results (maximum,
// sum, output) are merged through shared memory at the end.  The chain a warp walks is half as long.
// The order in which a query's keys are added depends only on its position: blocks of 64 positions
// from block 0 (or the window's first block) upward, even and odd blocks apart, then the two merged.
//
// (Heads of 64 in tiles of 128 queries run on the tcgen05 kernel of attention_prefill_tc.cu instead; this one
// serves every other head size that is a multiple of 16, and tiles of 64.)
//
// Single-token rows (decode steps) have a kernel of their own below (attention_rows_kernel): one query per
// (row, head), the CTA's warps share each key block by keys instead of by queries.
//
// A tile's keys before its first query are older than this step, so the first block of each group is asked for
// before the wait for the previous kernel if it lies wholly before that query; queries, and the blocks that hold
// this step's own keys, are fetched after it.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

constexpr int BKV = 64;   // keys per block; a warp owns 16 queries, a CTA of 4 or 8 warps a tile of 64 or 128

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (ex2.approx: relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}

// tiles: int32 [n_tiles][4] = (row of the tile's first token among the step's tokens, queries in the tile
// (1..16*WARPS), block-table row of the request, position of the tile's first query).
__device__ __forceinline__ void group_barrier(int id, int threads) {
  if (threads == 32) { __syncwarp(); return; }      // a group of one warp
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// QW: warps that share the tile's queries (16 each); KSPLIT: groups of QW warps that share the key blocks.
template <int DH, int QW, int KSPLIT>
__global__ void __launch_bounds__(QW * KSPLIT * 32, (DH <= 64 ? 512 : 256) / (QW * KSPLIT * 32))
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int ldq, const int4* __restrict__ tiles,
                         const int* __restrict__ block_table, int max_pages, int n_pages, int page, int Hq, int Hkv,
                         int window, float scale_log2e, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out, int ldo,
                         int* __restrict__ status) {
  constexpr int THREADS = QW * 32;            // threads of one group: they gather and use the same key blocks
  constexpr int STRIDE = DH + 8;              // elements per shared-memory row (16 bytes of padding)
  constexpr int KS = DH / 16;                 // k steps of Q K^T
  constexpr int NT = DH / 8;                  // n tiles of the output
  constexpr int CHUNKS = DH / 8;              // 16-byte chunks per key row
  constexpr int NIT = (BKV * CHUNKS + THREADS - 1) / THREADS;   // chunks a thread copies per block
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int group = (threadIdx.x >> 5) / QW;            // which share of the key blocks
  const int gtid = threadIdx.x - group * THREADS;       // thread index within the group
  __nv_bfloat16* sk = reinterpret_cast<__nv_bfloat16*>(smem_raw) + group * (4 * BKV * STRIDE);   // [2][BKV][STRIDE]
  __nv_bfloat16* sv = sk + 2 * BKV * STRIDE;                                                     // [2][BKV][STRIDE]

  pdl_trigger();
  const int4 tile = tiles[blockIdx.x];      // the step's inputs: no kernel writes them
  const int row0 = tile.x, n_rows = tile.y, req = tile.z, pos0 = tile.w;
  if (n_rows <= 0) return;                  // a tile without queries pads the list to a size seen before
  const int h = blockIdx.y, hk = h / (Hq / Hkv);
  const int warp = gtid >> 5, lane = threadIdx.x & 31, g = lane >> 2, qd = lane & 3;
  const int* bt = block_table + (size_t)req * max_pages;
  const int shift = __ffs(page) - 1;

  const int last_pos = pos0 + n_rows - 1;
  const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int kb_lo = first_key / BKV, kb_hi = last_pos / BKV;

  // Which chunks of a block this thread copies: fixed for the whole kernel.
  int c_row[NIT], c_soff[NIT], c_goff[NIT];
#pragma unroll
  for (int j = 0; j < NIT; ++j) {
    const int i = gtid + j * THREADS;
    const int kr = i / CHUNKS, ch = i - kr * CHUNKS;
    c_row[j] = i < BKV * CHUNKS ? kr : -1;
    c_soff[j] = kr * STRIDE + ch * 8;
    c_goff[j] = hk * page * DH + ch * 8;
  }
  const size_t page_elems = (size_t)Hkv * page * DH;

  // gather one block of keys and values into stage `st`
  auto load_block = [&](int kb, int st) {
    __nv_bfloat16* dk = sk + st * BKV * STRIDE;
    __nv_bfloat16* dv = sv + st * BKV * STRIDE;
#pragma unroll
    for (int j = 0; j < NIT; ++j) {
      if (c_row[j] < 0) continue;
      const int key = kb * BKV + c_row[j];
      bool ok = key <= last_pos && key >= first_key;
      size_t off = 0;
      if (ok) {
        const int lp = key >> shift;
        const int pg = lp < max_pages ? bt[lp] : -1;
        if (pg < 0 || pg >= n_pages) {
          atomicOr(status, pg < 0 ? MLXB_ST_POSITION_RANGE : MLXB_ST_PAGE_RANGE);
          ok = false;
        } else {
          off = (size_t)pg * page_elems + (size_t)((key & (page - 1)) * DH + c_goff[j]);
        }
      }
      cp_async16(dk + c_soff[j], k_pool + off, ok);
      cp_async16(dv + c_soff[j], v_pool + off, ok);
    }
    cp_async_commit();
  };

  // this group's blocks: kb_first, kb_first + KSPLIT, ... (block indices congruent to `group`)
  const int kb_first = kb_lo + ((group - kb_lo) % KSPLIT + KSPLIT) % KSPLIT;
  // keys before the tile's first query are older than this step: such a block can be on its way before the
  // wait for the kernel that wrote this step's queries, keys and values
  const bool early = kb_first <= kb_hi && (kb_first + 1) * BKV <= pos0;
  if (early) load_block(kb_first, 0);
  pdl_wait();
  q = after_wait(q);
  k_pool = after_wait(k_pool);
  v_pool = after_wait(v_pool);
  if (!early && kb_first <= kb_hi) load_block(kb_first, 0);

  // this warp's 16 queries: rows r_lo = 16*warp + g and r_hi = r_lo + 8 of the tile
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
  const bool v_lo = r_lo < n_rows, v_hi = r_hi < n_rows;
  const int p_lo = v_lo ? pos0 + r_lo : -1, p_hi = v_hi ? pos0 + r_hi : -1;   // -1: nothing is visible
  const int lo_lo = (window > 0 && p_lo - window + 1 > 0) ? p_lo - window + 1 : 0;
  const int lo_hi = (window > 0 && p_hi - window + 1 > 0) ? p_hi - window + 1 : 0;
  unsigned qa[KS][4];
  {
    const __nv_bfloat16* q_lo = q + (size_t)(row0 + (v_lo ? r_lo : 0)) * ldq + h * DH;
    const __nv_bfloat16* q_hi = q + (size_t)(row0 + (v_hi ? r_hi : 0)) * ldq + h * DH;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int d = ks * 16 + 2 * qd;
      qa[ks][0] = v_lo ? *reinterpret_cast<const unsigned*>(q_lo + d) : 0u;
      qa[ks][1] = v_hi ? *reinterpret_cast<const unsigned*>(q_hi + d) : 0u;
      qa[ks][2] = v_lo ? *reinterpret_cast<const unsigned*>(q_lo + d + 8) : 0u;
      qa[ks][3] = v_hi ? *reinterpret_cast<const unsigned*>(q_hi + d + 8) : 0u;
    }
  }
  const int warp_first_pos = pos0 + warp * 16;
  const int warp_last_pos = min(last_pos, warp_first_pos + 15);
  const bool warp_whole = warp * 16 + 15 < n_rows;                       // all 16 rows are real queries
  const int warp_floor = (window > 0 && warp_last_pos - window + 1 > 0) ? warp_last_pos - window + 1 : 0;

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
  // running maximum in units of the exponent (score * scale * log2 e), running sum per lane
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  const int mi = lane >> 3, mr = lane & 7;   // ldmatrix: which 8x8 matrix this lane addresses, and its row

  for (int kb = kb_first; kb <= kb_hi; kb += KSPLIT) {
    const int st = ((kb - kb_first) / KSPLIT) & 1;
    const bool more = kb + KSPLIT <= kb_hi;
    if (more) load_block(kb + KSPLIT, st ^ 1);
    if (more) cp_async_wait<1>(); else cp_async_wait<0>();
    if (KSPLIT == 1) __syncthreads(); else group_barrier(1 + group, THREADS);

    if (kb * BKV <= warp_last_pos) {     // otherwise every key of the block lies after this warp's queries
      const __nv_bfloat16* bk = sk + st * BKV * STRIDE;
      const __nv_bfloat16* bv = sv + st * BKV * STRIDE;
      float s[BKV / 8][4];
#pragma unroll
      for (int i = 0; i < BKV / 8; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[i][c] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < BKV / 16; ++np) {   // pairs of key tiles
          unsigned b[4];
          ldmatrix_x4(b, bk + (np * 16 + (mi >> 1) * 8 + mr) * STRIDE + ks * 16 + (mi & 1) * 8);
          mma_bf16(s[2 * np], qa[ks], b[0], b[1]);
          mma_bf16(s[2 * np + 1], qa[ks], b[2], b[3]);
        }
      }
      // mask (only blocks that touch the diagonal, the window's edge or the tile's end need it) and row maxima
      const bool open = warp_whole && kb * BKV + BKV - 1 <= warp_first_pos && kb * BKV >= warp_floor;
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
      if (open) {
#pragma unroll
        for (int i = 0; i < BKV / 8; ++i) {
          mx_lo = fmaxf(mx_lo, fmaxf(s[i][0], s[i][1]));
          mx_hi = fmaxf(mx_hi, fmaxf(s[i][2], s[i][3]));
        }
      } else {
        const int key0 = kb * BKV + 2 * qd;
#pragma unroll
        for (int i = 0; i < BKV / 8; ++i) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int key = key0 + i * 8 + c;
            if (!(key <= p_lo && key >= lo_lo)) s[i][c] = -INFINITY;
            if (!(key <= p_hi && key >= lo_hi)) s[i][2 + c] = -INFINITY;
            mx_lo = fmaxf(mx_lo, s[i][c]);
            mx_hi = fmaxf(mx_hi, s[i][2 + c]);
          }
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo * scale_log2e), mn_hi = fmaxf(m_hi, mx_hi * scale_log2e);   // scale > 0
      const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo, base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      const float corr_lo = fast_exp2(m_lo - base_lo), corr_hi = fast_exp2(m_hi - base_hi);   // 2^-inf = 0
      m_lo = mn_lo;
      m_hi = mn_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
      unsigned pa[BKV / 16][4];
#pragma unroll
      for (int i = 0; i < BKV / 8; ++i) {   // exponent = score * scale * log2(e) - maximum, one fused multiply-add
        const float e0 = fast_exp2(fmaf(s[i][0], scale_log2e, -base_lo)), e1 = fast_exp2(fmaf(s[i][1], scale_log2e, -base_lo));
        const float e2 = fast_exp2(fmaf(s[i][2], scale_log2e, -base_hi)), e3 = fast_exp2(fmaf(s[i][3], scale_log2e, -base_hi));
        sum_lo += e0 + e1;
        sum_hi += e2 + e3;
        // accumulator tiles 2j and 2j+1 are the A fragment of the j-th 16-key step of P V
        pa[i >> 1][(i & 1) * 2] = pack_bf16(e0, e1);
        pa[i >> 1][(i & 1) * 2 + 1] = pack_bf16(e2, e3);
      }
      l_lo = l_lo * corr_lo + sum_lo;   // per-lane partial sums; the four lanes of a row are added at the end
      l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        o[i][0] *= corr_lo; o[i][1] *= corr_lo;
        o[i][2] *= corr_hi; o[i][3] *= corr_hi;
      }
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk) {
#pragma unroll
        for (int dp = 0; dp < NT / 2; ++dp) {   // pairs of output-dim tiles
          unsigned b[4];
          ldmatrix_x4_trans(b, bv + (kk * 16 + (mi & 1) * 8 + mr) * STRIDE + dp * 16 + (mi >> 1) * 8);
          mma_bf16(o[2 * dp], pa[kk], b[0], b[1]);
          mma_bf16(o[2 * dp + 1], pa[kk], b[2], b[3]);
        }
      }
    }
    // everyone is done with stage st before it is loaded again
    if (KSPLIT == 1) __syncthreads(); else group_barrier(1 + group, THREADS);
  }

  if (KSPLIT > 1) {
    // merge the groups: thread t of every group holds the same elements of the same queries
    float* xch = reinterpret_cast<float*>(smem_raw);   // [KSPLIT - 1][NT * 4 + 4][THREADS]; the stages are free now
    __syncthreads();
    if (group > 0) {
      float* dst = xch + (size_t)(group - 1) * (NT * 4 + 4) * THREADS + gtid;
#pragma unroll
      for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) dst[(i * 4 + c) * THREADS] = o[i][c];
      dst[(NT * 4 + 0) * THREADS] = m_lo;
      dst[(NT * 4 + 1) * THREADS] = m_hi;
      dst[(NT * 4 + 2) * THREADS] = l_lo;
      dst[(NT * 4 + 3) * THREADS] = l_hi;
    }
    __syncthreads();
    if (group > 0) return;
#pragma unroll
    for (int gg = 1; gg < KSPLIT; ++gg) {
      const float* src = xch + (size_t)(gg - 1) * (NT * 4 + 4) * THREADS + gtid;
      const float om_lo = src[(NT * 4 + 0) * THREADS], om_hi = src[(NT * 4 + 1) * THREADS];
      const float ol_lo = src[(NT * 4 + 2) * THREADS], ol_hi = src[(NT * 4 + 3) * THREADS];
      const float mn_lo = fmaxf(m_lo, om_lo), mn_hi = fmaxf(m_hi, om_hi);
      const float b_lo = mn_lo == -INFINITY ? 0.f : mn_lo, b_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      const float wa_lo = fast_exp2(m_lo - b_lo), wb_lo = fast_exp2(om_lo - b_lo);   // 2^-inf = 0
      const float wa_hi = fast_exp2(m_hi - b_hi), wb_hi = fast_exp2(om_hi - b_hi);
      l_lo = l_lo * wa_lo + ol_lo * wb_lo;
      l_hi = l_hi * wa_hi + ol_hi * wb_hi;
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        o[i][0] = o[i][0] * wa_lo + src[(i * 4 + 0) * THREADS] * wb_lo;
        o[i][1] = o[i][1] * wa_lo + src[(i * 4 + 1) * THREADS] * wb_lo;
        o[i][2] = o[i][2] * wa_hi + src[(i * 4 + 2) * THREADS] * wb_hi;
        o[i][3] = o[i][3] * wa_hi + src[(i * 4 + 3) * THREADS] * wb_hi;
      }
      m_lo = mn_lo;
      m_hi = mn_hi;
    }
  }

  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
  __nv_bfloat16* o_lo = out + (size_t)(row0 + r_lo) * ldo + h * DH + 2 * qd;
  __nv_bfloat16* o_hi = out + (size_t)(row0 + r_hi) * ldo + h * DH + 2 * qd;
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    if (v_lo) *reinterpret_cast<unsigned*>(o_lo + i * 8) = pack_bf16(o[i][0] * inv_lo, o[i][1] * inv_lo);
    if (v_hi) *reinterpret_cast<unsigned*>(o_hi + i * 8) = pack_bf16(o[i][2] * inv_hi, o[i][3] * inv_hi);
  }
}

template <int DH, int QW, int KSPLIT>
static int launch(const void* q, int ldq, const int* tiles, int n_tiles, const int* block_table, int max_pages,
                  int n_pages, int page, int Hq, int Hkv, int window, float scale, const void* k_pool,
                  const void* v_pool, void* out, int ldo, int* status, cudaStream_t stream) {
  constexpr int WARPS = QW * KSPLIT;
  size_t smem = (size_t)KSPLIT * 2 * 2 * BKV * (DH + 8) * sizeof(__nv_bfloat16);
  const size_t merge = (size_t)(KSPLIT - 1) * (DH / 8 * 4 + 4) * QW * 32 * sizeof(float);
  if (merge > smem) smem = merge;
  auto kern = attention_prefill_kernel<DH, QW, KSPLIT>;
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    raised = true;
  }
  launch_pdl(kern, dim3(n_tiles, Hq), dim3(WARPS * 32), smem, stream, (const __nv_bfloat16*)q, ldq,
             (const int4*)tiles, block_table, max_pages, n_pages, page, Hq, Hkv, window,
             scale * 1.4426950408889634f, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
             (__nv_bfloat16*)out, ldo, status);
  return mlxb_check_launch("attention (portions)");
}

// bfloat16 only.  q: [*, >= Hq*Dh] at row stride ldq; out: [*, Hq*Dh] at row stride ldo (both strides even,
// bases 4-byte aligned); tiles: int32 [n_tiles][4], see the kernel; pools [n_pages, Hkv, page, Dh].
// Dh: a multiple of 16 up to 128; other sizes are refused (the generic kernel takes them).
// tile_rows: queries per tile, 64 or 128 (the caller cut the portions into tiles of at most that many).
MLXB_EXPORT int mlxb_attention_prefill(const void* q, int ldq, const int* tiles, int n_tiles, int tile_rows,
                                       const int* block_table, int max_pages, int n_pages, int page, int Hq, int Hkv,
                                       int Dh, int window, float scale, const void* k_pool, const void* v_pool,
                                       void* out, int ldo, int* status, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (page <= 0 || (page & (page - 1))) return mlxb_fail(MLXB_BAD_ARG, "attention (portions): page size %d", page);
  if (Hkv <= 0 || Hq <= 0 || Hq % Hkv || Hq > 65535)
    return mlxb_fail(MLXB_BAD_ARG, "attention (portions): %d query heads over %d key/value heads", Hq, Hkv);
  if ((ldq & 1) || (ldo & 1) || ((uintptr_t)q & 3) || ((uintptr_t)out & 3) || ((uintptr_t)tiles & 15))
    return mlxb_fail(MLXB_BAD_ARG, "attention (portions): rows must be 4-byte aligned, the tile list 16-byte aligned");
  if (tile_rows != 64 && tile_rows != 128)
    return mlxb_fail(MLXB_BAD_ARG, "attention (portions): tiles of %d queries (64 or 128)", tile_rows);
#define GO(D)                                                                                                         \
  case D:                                                                                                             \
    if (tile_rows == 128)                                                                                             \
      return launch<D, 8, 1>(q, ldq, tiles, n_tiles, block_table, max_pages, n_pages, page, Hq, Hkv, window, scale,   \
                             k_pool, v_pool, out, ldo, status, stream);                                               \
    return launch<D, 4, 2>(q, ldq, tiles, n_tiles, block_table, max_pages, n_pages, page, Hq, Hkv, window, scale,     \
                           k_pool, v_pool, out, ldo, status, stream)
  switch (Dh) {
    GO(16); GO(32); GO(48); GO(64); GO(80); GO(96); GO(112); GO(128);
    default:
      return mlxb_fail(MLXB_BAD_ARG, "attention (portions): head size %d is not a multiple of 16 up to 128", Dh);
  }
#undef GO
}


// ---------------------------------------------------------------------------------------------------------------
// Single-token rows (decode steps): one query per (row, head).
//
// One CTA of RW warps handles (row, query head) and walks the row's keys in blocks of 64 positions, gathered
// through the block table with 16-byte cp.async into a ring of RS shared-memory stages by all its threads (so the
// page lookups are shared, and RS - 1 blocks are in flight while one is multiplied).  Inside a block the warps
// split the KEYS: warp w takes keys 64/RW * w .. of every block, multiplies them with the query on the tensor cores
// (mma.sync m16n8k16 with the query in row 0 of the 16-row operand; the other rows are zeros and cost nothing that
// matters, the kernel is bound by reading keys and values), keeps a running maximum, sum and output of its own,
// and the warps' results are merged in warp order at the end.  Per key this issues a tenth of the instructions
// of a kernel that multiplies on the CUDA cores: no unpacking of bfloat16, no shuffles and no exponential per
// thread and key.  The order in which a row's keys are added depends only on its position.
// Blocks that lie wholly before the row's position hold keys older than this step and are asked for before the
// wait for the kernel that wrote this step's query, key and value.
// The launcher sends only steps of many rows here ((row, head) pairs several times the number of SMs): with few
// pairs a row's keys would have to be shared among CTAs, and the split-key kernel of attention.cu, which does
// that, is the faster one there (measured; so is a variant of this kernel that shares a row among a thread-block
// cluster and merges through distributed shared memory).
template <int DH, int RW, int RS>
__global__ void __launch_bounds__(RW * 32)
attention_rows_kernel(const __nv_bfloat16* __restrict__ q, int ldq, const int4* __restrict__ tiles,
                      const int* __restrict__ block_table, int max_pages, int n_pages, int page, int Hq, int Hkv,
                      int window, float scale_log2e, const __nv_bfloat16* __restrict__ k_pool,
                      const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out, int ldo,
                      int* __restrict__ status) {
  constexpr int THREADS = RW * 32;
  constexpr int STRIDE = DH + 8;              // elements per shared-memory row (16 bytes of padding)
  constexpr int KS = DH / 16;                 // k steps of q K^T
  constexpr int NT = DH / 8;                  // n tiles of the output
  constexpr int CHUNKS = DH / 8;              // 16-byte chunks per key row
  constexpr int WK = BKV / RW;                // keys of a block a warp takes: 16 (4 warps) or 32 (2 warps)
  constexpr int NIT = (BKV * CHUNKS + THREADS - 1) / THREADS;   // chunks of K (and of V) a thread copies per block
  static_assert(WK % 16 == 0, "a warp takes whole 16-key steps");
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* sk = reinterpret_cast<__nv_bfloat16*>(smem_raw);    // [RS][BKV][STRIDE]
  __nv_bfloat16* sv = sk + RS * BKV * STRIDE;                        // [RS][BKV][STRIDE]

  pdl_trigger();
  const int4 tile = tiles[blockIdx.x];        // the step's inputs: no kernel writes them
  const int row = tile.x, req = tile.z, pos = tile.w;
  if (tile.y <= 0) return;                    // a row that pads the step
  const int h = blockIdx.y, hk = h / (Hq / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, qd = lane & 3;
  const int* bt = block_table + (size_t)req * max_pages;
  const int shift = __ffs(page) - 1;
  const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int kb_lo = first_key / BKV, kb_hi = pos / BKV;
  const int n_blocks = kb_hi - kb_lo + 1;
  const size_t page_elems = (size_t)Hkv * page * DH;

  auto load_block = [&](int kb, int st) {     // gather block kb into stage st; always one commit group
    if (kb <= kb_hi) {
      __nv_bfloat16* dk = sk + st * BKV * STRIDE;
      __nv_bfloat16* dv = sv + st * BKV * STRIDE;
#pragma unroll
      for (int j = 0; j < NIT; ++j) {
        const int i = threadIdx.x + j * THREADS;
        if (i >= BKV * CHUNKS) break;
        const int kr = i / CHUNKS, ch = i - kr * CHUNKS;
        const int key = kb * BKV + kr;
        bool ok = key <= pos && key >= first_key;
        size_t off = 0;
        if (ok) {
          const int lp = key >> shift;
          const int pg = lp < max_pages ? bt[lp] : -1;
          if (pg < 0 || pg >= n_pages) {
            atomicOr(status, pg < 0 ? MLXB_ST_POSITION_RANGE : MLXB_ST_PAGE_RANGE);
            ok = false;
          } else {
            off = (size_t)pg * page_elems + (size_t)((hk * page + (key & (page - 1))) * DH + ch * 8);
          }
        }
        cp_async16(dk + kr * STRIDE + ch * 8, k_pool + off, ok);
        cp_async16(dv + kr * STRIDE + ch * 8, v_pool + off, ok);
      }
    }
    cp_async_commit();
  };

  // the first RS - 1 blocks: those that are older than this step before the wait, the others after it
  int issued = 0;
  while (issued < RS - 1 && issued < n_blocks && (kb_lo + issued + 1) * BKV <= pos) {
    load_block(kb_lo + issued, issued);
    ++issued;
  }
  pdl_wait();
  q = after_wait(q);
  k_pool = after_wait(k_pool);
  v_pool = after_wait(v_pool);
  for (; issued < RS - 1; ++issued) load_block(kb_lo + issued, issued);

  // the query in row 0 of the A operand (lanes g == 0), zeros in the other rows
  unsigned qa[KS][4];
  {
    const __nv_bfloat16* qr = q + (size_t)row * ldq + h * DH;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int d = ks * 16 + 2 * qd;
      qa[ks][0] = g == 0 ? *reinterpret_cast<const unsigned*>(qr + d) : 0u;
      qa[ks][2] = g == 0 ? *reinterpret_cast<const unsigned*>(qr + d + 8) : 0u;
      qa[ks][1] = qa[ks][3] = 0u;
    }
  }
  float o[NT][2];      // row g of the product: only g == 0 is the query's
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = 0.f;
  float m = -INFINITY, l = 0.f;   // running maximum in units of the exponent, this lane's share of the running sum
  const int mi = lane >> 3, mr = lane & 7;   // ldmatrix: which 8x8 matrix this lane addresses, and its row

  for (int i = 0; i < n_blocks; ++i) {
    const int kb = kb_lo + i, st = i % RS;
    cp_async_wait<RS - 2>();      // block i has landed (a group per block, RS - 1 of them issued ahead)
    __syncthreads();              // ... for every thread's copies; and everyone is done with block i - 1
    load_block(kb + RS - 1, (i + RS - 1) % RS);     // into the stage block i - 1 used
    const int key_w = kb * BKV + warp * WK;         // this warp's first key of the block
    if (key_w <= pos && key_w + WK > first_key) {
      const __nv_bfloat16* bk = sk + (st * BKV + warp * WK) * STRIDE;
      const __nv_bfloat16* bv = sv + (st * BKV + warp * WK) * STRIDE;
      float s[WK / 8][4];
#pragma unroll
      for (int t = 0; t < WK / 8; ++t)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[t][c] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < WK / 16; ++np) {   // pairs of 8-key tiles
          unsigned b[4];
          ldmatrix_x4(b, bk + (np * 16 + (mi >> 1) * 8 + mr) * STRIDE + ks * 16 + (mi & 1) * 8);
          mma_bf16(s[2 * np], qa[ks], b[0], b[1]);
          mma_bf16(s[2 * np + 1], qa[ks], b[2], b[3]);
        }
      }
      // mask and maximum of row g (the query's row where g == 0; the other rows are rows of zeros)
      const bool open = key_w + WK - 1 <= pos && key_w >= first_key;
      float mx = -INFINITY;
#pragma unroll
      for (int t = 0; t < WK / 8; ++t)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int key = key_w + t * 8 + 2 * qd + c;
          if (!open && !(key <= pos && key >= first_key)) s[t][c] = -INFINITY;
          mx = fmaxf(mx, s[t][c]);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mn = fmaxf(m, mx * scale_log2e);      // scale > 0
      const float base = mn == -INFINITY ? 0.f : mn;
      const float corr = fast_exp2(m - base);           // 2^-inf = 0
      m = mn;
      float sum = 0.f;
      unsigned pa[WK / 16][4];
#pragma unroll
      for (int t = 0; t < WK / 8; ++t) {
        const float e0 = fast_exp2(fmaf(s[t][0], scale_log2e, -base)), e1 = fast_exp2(fmaf(s[t][1], scale_log2e, -base));
        sum += e0 + e1;
        pa[t >> 1][(t & 1) * 2] = pack_bf16(e0, e1);
        pa[t >> 1][(t & 1) * 2 + 1] = 0u;
      }
      l = l * corr + sum;
#pragma unroll
      for (int t = 0; t < NT; ++t) { o[t][0] *= corr; o[t][1] *= corr; }
#pragma unroll
      for (int kk = 0; kk < WK / 16; ++kk) {
#pragma unroll
        for (int dp = 0; dp < NT / 2; ++dp) {   // pairs of output-dim tiles
          unsigned b[4];
          ldmatrix_x4_trans(b, bv + (kk * 16 + (mi & 1) * 8 + mr) * STRIDE + dp * 16 + (mi >> 1) * 8);
          float acc0[4] = {o[2 * dp][0], o[2 * dp][1], 0.f, 0.f}, acc1[4] = {o[2 * dp + 1][0], o[2 * dp + 1][1], 0.f, 0.f};
          mma_bf16(acc0, pa[kk], b[0], b[1]);
          mma_bf16(acc1, pa[kk], b[2], b[3]);
          o[2 * dp][0] = acc0[0]; o[2 * dp][1] = acc0[1];
          o[2 * dp + 1][0] = acc1[0]; o[2 * dp + 1][1] = acc1[1];
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();      // the stages are free: they carry the warps' results now

  // merge the warps in warp order: lanes g == 0 of warp w hold (m, l share, o) of the query for their dims
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  float* xch = reinterpret_cast<float*>(smem_raw);     // [RW][2 + DH]
  if (g == 0) {
    float* dst = xch + warp * (2 + DH);
    if (qd == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
    for (int t = 0; t < NT; ++t) { dst[2 + t * 8 + 2 * qd] = o[t][0]; dst[2 + t * 8 + 2 * qd + 1] = o[t][1]; }
  }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < RW; ++w) M = fmaxf(M, xch[w * (2 + DH)]);
  const float base = M == -INFINITY ? 0.f : M;
  float L = 0.f;
#pragma unroll
  for (int w = 0; w < RW; ++w) L = fmaf(xch[w * (2 + DH) + 1], fast_exp2(xch[w * (2 + DH)] - base), L);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int d = threadIdx.x; d < DH; d += THREADS) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < RW; ++w) acc = fmaf(xch[w * (2 + DH) + 2 + d], fast_exp2(xch[w * (2 + DH)] - base), acc);
    out[(size_t)row * ldo + h * DH + d] = __float2bfloat16_rn(acc * inv);
  }
}

template <int DH, int RW, int RS>
static int launch_rows(const void* q, int ldq, const int* tiles, int n_tiles, const int* block_table, int max_pages,
                       int n_pages, int page, int Hq, int Hkv, int window, float scale, const void* k_pool,
                       const void* v_pool, void* out, int ldo, int* status, cudaStream_t stream) {
  const size_t smem = (size_t)RS * 2 * BKV * (DH + 8) * sizeof(__nv_bfloat16);    // (the merge needs far less)
  auto kern = attention_rows_kernel<DH, RW, RS>;
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    raised = true;
  }
  launch_pdl(kern, dim3(n_tiles, Hq), dim3(RW * 32), smem, stream, (const __nv_bfloat16*)q, ldq, (const int4*)tiles,
             block_table, max_pages, n_pages, page, Hq, Hkv, window, scale * 1.4426950408889634f,
             (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, ldo, status);
  return mlxb_check_launch("attention (single rows)");
}

// Rows with one query each (decode steps): tiles int32 [n_tiles][4] = (token row, 1, block-table row, position),
// or (token row, 0, 0, 0) for a row that pads the step and is left alone.  bfloat16; Dh a multiple of 16 up to 128.
MLXB_EXPORT int mlxb_attention_rows(const void* q, int ldq, const int* tiles, int n_tiles, const int* block_table,
                                    int max_pages, int n_pages, int page, int Hq, int Hkv, int Dh, int window,
                                    float scale, const void* k_pool, const void* v_pool, void* out, int ldo,
                                    int* status, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (page <= 0 || (page & (page - 1))) return mlxb_fail(MLXB_BAD_ARG, "attention (single rows): page size %d", page);
  if (Hkv <= 0 || Hq <= 0 || Hq % Hkv || Hq > 65535)
    return mlxb_fail(MLXB_BAD_ARG, "attention (single rows): %d query heads over %d key/value heads", Hq, Hkv);
  if ((ldq & 1) || (ldo & 1) || ((uintptr_t)q & 3) || ((uintptr_t)out & 3) || ((uintptr_t)tiles & 15))
    return mlxb_fail(MLXB_BAD_ARG, "attention (single rows): rows must be 4-byte aligned, the tile list 16-byte aligned");
#define GO(D)                                                                                                         \
  case D:                                                                                                             \
    return launch_rows<D, 4, (D <= 64 ? 3 : 2)>(q, ldq, tiles, n_tiles, block_table, max_pages, n_pages, page, Hq,    \
                                                Hkv, window, scale, k_pool, v_pool, out, ldo, status, stream)
  switch (Dh) {
    GO(16); GO(32); GO(48); GO(64); GO(80); GO(96); GO(112); GO(128);
    default:
      return mlxb_fail(MLXB_BAD_ARG, "attention (single rows): head size %d is not a multiple of 16 up to 128", Dh);
  }
#undef GO
}
