// The tcgen05 linear kernel (gemm_tcgen05.cuh) without thread-block clusters: every CTA fetches its own tiles.
#include "gemm_tcgen05.cuh"

MLXB_DEFINE_LAST_ERROR()

// never called in this library (no clusters): a copy to one CTA
__device__ __forceinline__ void tma_load_2d_multicast(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                                      uint16_t) {
  tma_load_2d(dst, map, x, y, bar);
}
