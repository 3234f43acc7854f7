// LayerNorm with gain and optional bias.  Statistics are computed in 32-bit
// in two passes over a copy of the row held in registers (one warp per row, widths up to 2048
// that are multiples of 8) or in shared memory (one block per row, any other width):
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
  const T* xi = after_wait(x) + (size_t)(rows ? rows[r] : r) * D;
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

// Rows up to 2048 wide whose width is a multiple of 8: one warp per row, the row in registers (8-element
// chunks, 16-byte loads), warp shuffles for both sums; no shared memory and no block barrier.  The
// reduction order is fixed by D alone.
template <typename T, int NCH>
__global__ void __launch_bounds__(256)
layernorm_warp_kernel(const T* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ gain,
                      const float* __restrict__ bias, T* __restrict__ y, int R, int D, float eps) {
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + warp;
  if (r >= R) return;
  // gain and bias are weights: their lines are asked for before the wait for the kernel that writes x,
  // so that the loads after the statistics find them in L1
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int d = (c * 32 + lane) * 8;
    if (d < D) {
      asm volatile("prefetch.global.L1 [%0];" ::"l"(gain + d));
      if (bias) asm volatile("prefetch.global.L1 [%0];" ::"l"(bias + d));
    }
  }
  const int src_row = rows ? rows[r] : r;      // a step input, not written by a kernel
  pdl_wait();
  const T* xi = after_wait(x) + (size_t)src_row * D;
  float v[NCH][8];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int d = (c * 32 + lane) * 8;
    if (d < D) {
      if (sizeof(T) == 2) {
        const uint4 u = *reinterpret_cast<const uint4*>(xi + d);
        const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v[c][2 * i] = __uint_as_float(w[i] << 16);
          v[c][2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
      } else {
        const float4 a = *reinterpret_cast<const float4*>(xi + d), b = *reinterpret_cast<const float4*>(xi + d + 4);
        v[c][0] = a.x; v[c][1] = a.y; v[c][2] = a.z; v[c][3] = a.w;
        v[c][4] = b.x; v[c][5] = b.y; v[c][6] = b.z; v[c][7] = b.w;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) s += v[c][i];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[c][i] = 0.f;
    }
  }
  const float mean = warp_sum(s) / (float)D;
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    if ((c * 32 + lane) * 8 < D) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { const float t = v[c][i] - mean; q += t * t; }
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / (float)D + eps);
  T* yo = y + (size_t)r * D;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int d = (c * 32 + lane) * 8;
    if (d < D) {
      float o[8], gn[8], bs[8];
      *reinterpret_cast<float4*>(gn) = *reinterpret_cast<const float4*>(gain + d);
      *reinterpret_cast<float4*>(gn + 4) = *reinterpret_cast<const float4*>(gain + d + 4);
      if (bias) {
        *reinterpret_cast<float4*>(bs) = *reinterpret_cast<const float4*>(bias + d);
        *reinterpret_cast<float4*>(bs + 4) = *reinterpret_cast<const float4*>(bias + d + 4);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        o[i] = (v[c][i] - mean) * rstd * gn[i];
        if (bias) o[i] += bs[i];
      }
      if (sizeof(T) == 2) {
        uint4 u;
        unsigned* w = reinterpret_cast<unsigned*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 pr = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
          w[i] = *reinterpret_cast<const unsigned*>(&pr);
        }
        *reinterpret_cast<uint4*>(yo + d) = u;
      } else {
        *reinterpret_cast<float4*>(yo + d) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4*>(yo + d + 4) = make_float4(o[4], o[5], o[6], o[7]);
      }
    }
  }
}

template <typename T>
static bool launch_warp(const void* x, const int* rows, const float* gain, const float* bias, void* y, int R, int D,
                        float eps, cudaStream_t stream) {
  if ((D & 7) || D > 2048 || ((uintptr_t)x & 15) || ((uintptr_t)y & 15) || ((uintptr_t)gain & 15) ||
      ((uintptr_t)bias & 15))
    return false;
  const int nch = (D + 255) / 256;
  const dim3 grid((R + 7) / 8), block(256);
#define LNW(N_) launch_pdl(layernorm_warp_kernel<T, N_>, grid, block, 0, stream, (const T*)x, rows, gain, bias, (T*)y, R, D, eps)
  switch (nch) {
    case 1: LNW(1); break;
    case 2: LNW(2); break;
    case 3: LNW(3); break;
    case 4: LNW(4); break;
    case 5: LNW(5); break;
    case 6: LNW(6); break;
    case 7: LNW(7); break;
    default: LNW(8); break;
  }
#undef LNW
  return true;
}

// x: [*, D] of dtype; rows: int32[R] or null (then R rows of x in order);
// gain, bias: float32[D] (bias may be null); y: [R, D] of dtype.
MLXB_EXPORT int mlxb_layernorm(int dtype, const void* x, const int* rows, const float* gain, const float* bias,
                               void* y, int R, int D, float eps, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (D <= 0 || D > 49152) return mlxb_fail(MLXB_BAD_ARG, "layernorm: width %d is outside 1..49152", D);
  if (dtype != MLXB_F32 && dtype != MLXB_BF16) return mlxb_fail(MLXB_BAD_DTYPE, "layernorm: dtype code %d", dtype);
  if (dtype == MLXB_F32 ? launch_warp<float>(x, rows, gain, bias, y, R, D, eps, stream)
                        : launch_warp<__nv_bfloat16>(x, rows, gain, bias, y, R, D, eps, stream))
    return mlxb_check_launch("layernorm");
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


// Mean and 1/sqrt(var + eps) of bfloat16 rows (width a multiple of 8): stats[r] = (mean, rstd).  For a
// LayerNorm that has been folded into the weights of the linear layer after it, whose epilogue needs only
// these two numbers per row.  One warp per row, same order of additions as the norm itself.
__global__ void __launch_bounds__(256)
row_stats_kernel(const __nv_bfloat16* __restrict__ x, float2* __restrict__ stats, int R, int D, int ld, float eps) {
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + warp;
  if (r >= R) return;
  pdl_wait();
  const __nv_bfloat16* xr = after_wait(x) + (size_t)r * ld;
  float mean, rstd;
  row_stats_bf16(xr, D, eps, lane, mean, rstd, [](const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); });
  if (lane == 0) stats[r] = make_float2(mean, rstd);
}

// x: bfloat16 [R, D] at row stride ld (elements; multiple of 8, base 16-byte aligned); stats: float32 [R, 2].
MLXB_EXPORT int mlxb_row_stats(const void* x, void* stats, int R, int D, int ld, float eps, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (D <= 0 || (D & 7) || (ld & 7) || ld < D || ((uintptr_t)x & 15) || ((uintptr_t)stats & 7))
    return mlxb_fail(MLXB_BAD_ARG, "row_stats: width %d, row stride %d (multiples of 8, 16-byte aligned rows)", D, ld);
  launch_pdl(row_stats_kernel, dim3((R + 7) / 8), dim3(256), 0, stream, (const __nv_bfloat16*)x, (float2*)stats, R, D,
             ld, eps);
  return mlxb_check_launch("row_stats");
}

// Row gather without a norm: y[r] = x[rows[r]], for a model whose output head reads the residual stream as
// it is.  One block per output row; any width, any element type of 2 or 4 bytes.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ rows, T* __restrict__ y, int D,
                                   int n_in) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows[r];
  T* yo = y + (size_t)r * D;
  if (src < 0 || src >= n_in) {     // never read outside x: a bad index gives a row of zeros
    for (int d = threadIdx.x; d < D; d += blockDim.x) yo[d] = from_f<T>(0.f);
    return;
  }
  const T* xi = after_wait(x) + (size_t)src * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) yo[d] = xi[d];
}

// x: [n_in, D] contiguous; rows: int32 [R]; y: [R, D] contiguous.
MLXB_EXPORT int mlxb_gather_rows(int dtype, const void* x, const int* rows, void* y, int R, int D, int n_in,
                                 cudaStream_t stream) {
  if (R <= 0) return 0;
  if (D <= 0 || n_in <= 0 || rows == nullptr) return mlxb_fail(MLXB_BAD_ARG, "gather_rows: width %d, %d input rows", D, n_in);
  const int threads = D >= 1024 ? 256 : (D >= 256 ? 128 : 64);
  if (dtype == MLXB_F32)
    launch_pdl(gather_rows_kernel<float>, dim3(R), dim3(threads), 0, stream, (const float*)x, rows, (float*)y, D, n_in);
  else if (dtype == MLXB_BF16)
    launch_pdl(gather_rows_kernel<__nv_bfloat16>, dim3(R), dim3(threads), 0, stream, (const __nv_bfloat16*)x, rows,
               (__nv_bfloat16*)y, D, n_in);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "gather_rows: dtype code %d", dtype);
  return mlxb_check_launch("gather_rows");
}
