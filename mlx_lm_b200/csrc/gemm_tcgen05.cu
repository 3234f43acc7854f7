// Linear layer for many rows (prompt portions) on the 5th-generation tensor cores:
//   C[M,N] = epilogue(A[M,K] . W[N,K]^T + bias[N]) (+ residual[M,N])
// A, W, residual bfloat16 (both operands K-major: the K index is contiguous), C bfloat16 or float32.
//
// One CTA computes a 128 x BN tile.  Warp 0 is the TMA producer: it fills a ring of shared-memory
// stages with 128x64 tiles of A and BNx64 tiles of W (cp.async.bulk.tensor, 128-byte swizzle,
// completion counted on an mbarrier per stage; rows and columns outside the matrices arrive as
// zeros).  Warp 1 allocates tensor memory and issues tcgen05.mma (kind::f16, bf16 inputs, float32
// accumulator of 128 lanes x BN columns in TMEM), four K=16 steps per stage, and releases each
// stage with tcgen05.commit.  Warps 2-5 are the epilogue: when the accumulator is complete they
// read it with tcgen05.ld (each warp its 32 lanes), add the bias, apply gelu_new, add the
// residual and store.  No multicast anywhere: every CTA fetches its own tiles.
//
// Every wait on an mbarrier is bounded: after a limit of polls the waiter raises an abort flag in
// shared memory and a bit in the caller's status word; all roles then fall through to the common
// exit, where the tensor memory is freed.  A timeout therefore ends the kernel with an error code
// instead of a hang.
//
// K and the row strides must be multiples of 8 elements (16 bytes), base addresses 16-byte aligned.
// The accumulation order over K is fixed (stage by stage, four steps per stage), independent of M.
#include <cuda.h>

#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

enum { EPI_NONE = 0, EPI_GELU_NEW = 1 };

constexpr int BM = 128, BK = 64;
constexpr int THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false after SPIN_LIMIT polls or when another role gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
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

template <int BN, int STAGES>
struct Smem {
  alignas(1024) __nv_bfloat16 a[STAGES][BM * BK];
  alignas(1024) __nv_bfloat16 b[STAGES][BN * BK];
  alignas(8) uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN, int STAGES, typename TO, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, const __nv_bfloat16* residual, TO* C, int M, int N, int K,
                    int ldc, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  Smem<BN, STAGES>& sm = *reinterpret_cast<Smem<BN, STAGES>*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int k_tiles = (K + BK - 1) / BK;
  constexpr uint32_t STAGE_BYTES = (BM + BN) * BK * sizeof(__nv_bfloat16);
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;   // a power of two >= 32

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    mbar_init(&sm.acc_full, 1);
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
  }
  if (warp == 1) {   // the MMA warp owns the tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = sm.tmem_base;
  volatile int* abort_flag = &sm.abort_flag;
  pdl_trigger();
  pdl_wait();   // A (and the residual) come from the previous kernel

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;
      for (int kt = 0; kt < k_tiles; ++kt) {
        const int s = kt % STAGES;
        const uint32_t ph = (kt / STAGES) & 1;
        if (!mbar_wait(&sm.empty[s], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&sm.full[s], STAGE_BYTES);
        tma_load_2d(sm.a[s], &map_a, kt * BK, m0, &sm.full[s]);
        tma_load_2d(sm.b[s], &map_w, kt * BK, n0, &sm.full[s]);
        issued = kt + 1;
      }
      if (*abort_flag) {   // gave up: let the copies already issued land before the CTA exits
        for (int kt = issued > STAGES ? issued - STAGES : 0; kt < issued; ++kt) {
          const uint32_t addr = smem_u32(&sm.full[kt % STAGES]);
          for (uint32_t i = 0; i < (1u << 20); ++i) {
            uint32_t done;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                         "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(addr), "r"((uint32_t)((kt / STAGES) & 1))
                         : "memory");
            if (done) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN);
      bool ok = true;
      for (int kt = 0; kt < k_tiles && ok; ++kt) {
        const int s = kt % STAGES;
        const uint32_t ph = (kt / STAGES) & 1;
        ok = mbar_wait(&sm.full[s], ph, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = umma_desc(smem_u32(sm.a[s])), db = umma_desc(smem_u32(sm.b[s]));
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)   // 16 bf16 = 32 bytes = 2 units of the descriptor's start address
          umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
        umma_commit(&sm.empty[s]);   // the stage is free once these MMAs have read it
      }
      umma_commit(&sm.acc_full);     // arrives when every MMA issued above has completed
    }
  } else {
    // epilogue: warps 2..5; warp w may touch TMEM lanes 32*(w%4) .. +31, i.e. rows m0 + 32*(w%4) + lane
    const int q = warp & 3;
    const bool ready = mbar_wait(&sm.acc_full, 0, abort_flag);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int m = m0 + q * 32 + lane;
    if (ready) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);   // every lane takes part
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (m < M) {
          const int n_base = n0 + c0;
          const size_t row = (size_t)m * ldc;
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            const int n8 = n_base + g8 * 8;
            if (n8 >= N) break;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int n = n8 + i;
              float x = __uint_as_float(r[g8 * 8 + i]);
              if (n < N) {
                if (bias) x += bias[n];
                if (EPI == EPI_GELU_NEW) x = gelu_new_f(x);
              }
              v[i] = x;
            }
            const bool whole = n8 + 8 <= N;
            if (residual) {
              if (whole && ((row + n8) & 7) == 0) {
                const uint4 u = *reinterpret_cast<const uint4*>(residual + row + n8);
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
            if (sizeof(TO) == 2) {
              __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(C) + row + n8;
              if (whole && ((row + n8) & 7) == 0) {
                uint4 u;
                uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const __nv_bfloat162 pr = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                  w[i] = *reinterpret_cast<const uint32_t*>(&pr);
                }
                *reinterpret_cast<uint4*>(out) = u;
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (n8 + i < N) out[i] = __float2bfloat16_rn(v[i]);
              }
            } else {
              float* out = reinterpret_cast<float*>(C) + row + n8;
              if (whole && ((row + n8) & 3) == 0) {
                *reinterpret_cast<float4*>(out) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(out + 4) = make_float4(v[4], v[5], v[6], v[7]);
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (n8 + i < N) out[i] = v[i];
              }
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && sm.abort_flag) atomicOr(status, MLXB_ST_WAIT_TIMEOUT);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- host side

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

template <int BN, int STAGES, typename TO>
static int launch(const CUtensorMap& ma, const CUtensorMap& mw, const float* bias, const void* residual, void* C,
                  int M, int N, int K, int ldc, int epi, int* status, cudaStream_t stream) {
  const size_t smem = sizeof(Smem<BN, STAGES>) + 1024;
  auto k0 = gemm_tcgen05_kernel<BN, STAGES, TO, EPI_NONE>;
  auto k1 = gemm_tcgen05_kernel<BN, STAGES, TO, EPI_GELU_NEW>;
  auto kern = epi == EPI_GELU_NEW ? k1 : k0;
  static bool raised[2] = {false, false};
  if (!raised[epi == EPI_GELU_NEW]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return mlxb_fail((int)e, "linear (tensor cores): %zu bytes of shared memory: %s", smem,
                                           cudaGetErrorString(e));
    raised[epi == EPI_GELU_NEW] = true;
  }
  const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  launch_pdl(kern, grid, dim3(THREADS), smem, stream, ma, mw, bias, (const __nv_bfloat16*)residual, (TO*)C, M, N, K,
             ldc, status);
  return mlxb_check_launch("linear (tensor cores)");
}

// A: bfloat16 [M, K] at row stride lda; W: bfloat16 [N, K] contiguous; bias float32[N] or null; residual bfloat16
// [M, N] at row stride ldc or null (may alias C); C bfloat16 or float32 (out_f32) [M, N] at row stride ldc.
// K, lda multiples of 8; A and W 16-byte aligned.  status: int32 word that receives MLXB_ST_WAIT_TIMEOUT if a
// bounded wait inside the kernel gives up.
MLXB_EXPORT int mlxb_linear_tcgen05(int out_f32, const void* A, const void* W, const float* bias, const void* residual,
                                    void* C, int M, int N, int K, int lda, int ldc, int epi, int* status,
                                    cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (lda & 7) || lda < K || ldc < N)
    return mlxb_fail(MLXB_BAD_ARG, "linear (tensor cores): K %d and row stride %d must be multiples of 8 (ldc %d, N %d)",
                     K, lda, ldc, N);
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15))
    return mlxb_fail(MLXB_BAD_ARG, "linear (tensor cores): operands must be 16-byte aligned");
  if (epi != EPI_NONE && epi != EPI_GELU_NEW) return mlxb_fail(MLXB_BAD_ARG, "linear: epilogue code %d", epi);
  if ((M + BM - 1) / BM > 65535) return mlxb_fail(MLXB_BAD_ARG, "linear (tensor cores): %d rows are too many", M);
  constexpr int BN = 128, STAGES = 4;
  CUtensorMap ma, mw;
  if (int e = make_map(&ma, A, M, K, lda, BM)) return e;
  if (int e = make_map(&mw, W, N, K, K, BN)) return e;
  if (out_f32) return launch<BN, STAGES, float>(ma, mw, bias, residual, C, M, N, K, ldc, epi, status, stream);
  return launch<BN, STAGES, __nv_bfloat16>(ma, mw, bias, residual, C, M, N, K, ldc, epi, status, stream);
}
