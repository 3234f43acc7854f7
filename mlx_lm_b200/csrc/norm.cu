// LayerNorm with gain and optional bias.  Statistics are computed in 32-bit
// in two passes over a copy of the row held in shared memory:
//   mean = sum(x)/D;  var = sum((x-mean)^2)/D  (biased);
//   y = (x-mean) * rsqrt(var+eps) * gain + bias.
// `rows` (optional) gathers input rows: output row r is the norm of input row
// rows[r]; this is how the final norm runs only where logits are wanted.
// One block per row; the order of the additions depends on D and the block
// size only, never on which other rows are in the batch.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

template <typename T>
__global__ void layernorm_kernel(const T* __restrict__ x, const int* __restrict__ rows,
                                 const float* __restrict__ gain, const float* __restrict__ bias,
                                 T* __restrict__ y, int D, float eps) {
  extern __shared__ float srow[];  // D floats + 33 for the reductions
  float* red = srow + D;
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const T* xi = x + (size_t)(rows ? rows[r] : r) * D;
  float s = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = to_f(xi[d]);
    srow[d] = v;
    s += v;
  }
  const float mean = block_sum(s, red) / (float)D;
  float q = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float c = srow[d] - mean;
    q += c * c;
  }
  const float var = block_sum(q, red) / (float)D;
  const float rstd = rsqrtf(var + eps);
  T* yo = y + (size_t)r * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = (srow[d] - mean) * rstd * gain[d];
    if (bias) v += bias[d];
    yo[d] = from_f<T>(v);
  }
}

// x: [*, D] of dtype; rows: int32[R] or null (then R rows of x in order);
// gain, bias: float32[D] (bias may be null); y: [R, D] of dtype.
MLXB_EXPORT int mlxb_layernorm(int dtype, const void* x, const int* rows, const float* gain, const float* bias,
                               void* y, int R, int D, float eps, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (D <= 0 || D > 49152) return mlxb_fail(MLXB_BAD_ARG, "layernorm: width %d is outside 1..49152", D);
  const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : (D >= 128 ? 128 : 64));
  const size_t smem = (size_t)(D + 40) * sizeof(float);
  if (dtype == MLXB_F32) {
    if (smem > 48 * 1024)   // 227 KB is the most a CTA can have; set once to the largest width this file accepts
      cudaFuncSetAttribute(layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (49152 + 40) * 4);
    launch_pdl(layernorm_kernel<float>, dim3(R), dim3(threads), smem, stream, (const float*)x, rows, gain, bias,
               (float*)y, D, eps);
  } else if (dtype == MLXB_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(layernorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (49152 + 40) * 4);
    launch_pdl(layernorm_kernel<__nv_bfloat16>, dim3(R), dim3(threads), smem, stream, (const __nv_bfloat16*)x, rows,
               gain, bias, (__nv_bfloat16*)y, D, eps);
  } else {
    return mlxb_fail(MLXB_BAD_DTYPE, "layernorm: dtype code %d", dtype);
  }
  return mlxb_check_launch("layernorm");
}
