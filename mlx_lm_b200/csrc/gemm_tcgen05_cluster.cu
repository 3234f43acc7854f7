// The tcgen05 linear kernel (gemm_tcgen05.cuh) with thread-block clusters of 2 x 1 CTAs: the two CTAs of a cluster
// work on two row tiles of A against the same BN rows of W, each fetches half of the W tile and the copy is
// delivered to both (a multicast copy).  That takes a third off what the main loop pulls out of L2, which is
// what bounds it.  The tensor maps cover this GPU's own memory only (weights and activations of this process).
// This file, and the library built from it, are kept out of any run on more than one GPU (.gpurunignore.multi);
// the package then uses the plain library (gemm_tcgen05.cu), which has the same entry points.
#define MLXB_TC_CM 2
#define MLXB_TC_CN 1
#include "gemm_tcgen05.cuh"

MLXB_DEFINE_LAST_ERROR()

__device__ __forceinline__ void tma_load_2d_multicast(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                                      uint16_t mask) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster"
      " [%0], [%1, {%4, %5}], [%2], %3;"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "h"(mask), "r"(x), "r"(y) : "memory");
}
