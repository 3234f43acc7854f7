// Shared helpers of the kernel files: element types, error reporting,
// warp/block reductions.  Every kernel file is built into a shared library
// of its own with plain `extern "C"` launchers (no Python or torch headers),
// which the Python side loads with ctypes.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define MLXB_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with mlx_lm_b200/ops (0 = float32, 1 = bfloat16)
enum { MLXB_F32 = 0, MLXB_BF16 = 1 };

// error codes beyond cudaError_t (returned negative)
enum {
  MLXB_OK = 0,
  MLXB_BAD_ARG = -1,       // a size or option the kernel refuses
  MLXB_BAD_DTYPE = -2,
};

// status word bits that kernels set instead of faulting on bad indices
enum {
  MLXB_ST_TOKEN_RANGE = 1,     // token id outside the vocabulary
  MLXB_ST_POSITION_RANGE = 2,  // position outside the table / block table
  MLXB_ST_PAGE_RANGE = 4,      // page id outside the pool
  MLXB_ST_WAIT_TIMEOUT = 8,    // a bounded spin-wait gave up
};

static thread_local char g_mlxb_err[512];

static inline int mlxb_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_mlxb_err, sizeof(g_mlxb_err), fmt, ap);
  va_end(ap);
  return code;
}

static inline int mlxb_check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_mlxb_err, sizeof(g_mlxb_err), "%s: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

// ---- programmatic dependent launch
// Kernels of a step run one after the other on one stream, each a few microseconds long, so the
// gap between them matters.  A kernel launched with launch_pdl() may start while its predecessor
// is still running: it must call pdl_wait() before it reads anything the predecessor wrote or
// writes anything the predecessor may still read; what it does before that (index arithmetic,
// prefetching weights, which no kernel writes) overlaps the predecessor's tail.  pdl_trigger()
// lets the successor start early in the same way.  MLXB_PDL=0 in the environment turns the
// attribute off (every kernel then starts after its predecessor has finished, as usual).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// A pointer to memory the predecessor writes, as seen after pdl_wait().  A `const __restrict__` parameter
// promises the compiler that nobody writes the memory while the kernel runs, which would allow it to move
// a load through such a pointer up into the code before the wait; passing the pointer through this (empty)
// statement after the wait ties every load through the result to a point after it.
template <typename T>
__device__ __forceinline__ T* after_wait(T* p) {
  asm volatile("" : "+l"(p)::"memory");
  return p;
}

static inline int mlxb_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

static inline bool mlxb_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("MLXB_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = mlxb_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define MLXB_DEFINE_LAST_ERROR()                                   \
  MLXB_EXPORT const char* mlxb_last_error() { return g_mlxb_err; }

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- eight bfloat16 values in one 16-byte register group
__device__ __forceinline__ void unpack8(const uint4& u, float (&v)[8]) {
  const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&o)[8]) {
  uint4 u;
  unsigned* w = reinterpret_cast<unsigned*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 pr = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
    w[i] = *reinterpret_cast<const unsigned*>(&pr);
  }
  return u;
}

// LayerNorm of eight consecutive elements d..d+7 of a row with known statistics, rounded to bfloat16:
// (x - mean) * rstd * gain + bias, the arithmetic of norm.cu.
__device__ __forceinline__ uint4 normalise8(const uint4& raw, float mean, float rstd, const float* gain,
                                            const float* bias, int d) {
  float v[8], o[8], gn[8];
  unpack8(raw, v);
  *reinterpret_cast<float4*>(gn) = __ldg(reinterpret_cast<const float4*>(gain + d));
  *reinterpret_cast<float4*>(gn + 4) = __ldg(reinterpret_cast<const float4*>(gain + d + 4));
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = (v[i] - mean) * rstd * gn[i];
  if (bias) {
    float bs[8];
    *reinterpret_cast<float4*>(bs) = __ldg(reinterpret_cast<const float4*>(bias + d));
    *reinterpret_cast<float4*>(bs + 4) = __ldg(reinterpret_cast<const float4*>(bias + d + 4));
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] += bs[i];
  }
  return pack8(o);
}

// Mean and 1/sqrt(var + eps) of one bfloat16 row of width D (a multiple of 8), by one warp, with the order
// of additions of the one-warp-per-row kernel of norm.cu.  `load` fetches 16 bytes.  Rows up to 2048 wide
// stay in registers between the two passes; wider rows are read twice.
template <typename Load>
__device__ __forceinline__ void row_stats_bf16(const __nv_bfloat16* xr, int D, float eps, int lane, float& mean,
                                               float& rstd, Load load) {
  constexpr int KEEP = 8;
  uint4 keep[KEEP];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < KEEP; ++c) {
    const int d = (c * 32 + lane) * 8;
    keep[c] = d < D ? load(xr + d) : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int c = 0; c < KEEP; ++c) {
    float v[8];
    unpack8(keep[c], v);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
  }
  for (int d = (KEEP * 32 + lane) * 8; d < D; d += 256) {
    float v[8];
    unpack8(load(xr + d), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
  }
  mean = warp_sum(s) / (float)D;
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < KEEP; ++c) {
    if ((c * 32 + lane) * 8 < D) {
      float v[8];
      unpack8(keep[c], v);
#pragma unroll
      for (int i = 0; i < 8; ++i) { const float t = v[i] - mean; q += t * t; }
    }
  }
  for (int d = (KEEP * 32 + lane) * 8; d < D; d += 256) {
    float v[8];
    unpack8(load(xr + d), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) { const float t = v[i] - mean; q += t * t; }
  }
  rstd = rsqrtf(warp_sum(q) / (float)D + eps);
}

// Block-wide sum; every thread gets the result.  `red` is shared memory of at
// least 33 floats.  The order of additions is fixed by the block size alone.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  if (wid == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  if (wid == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// The same function written as x * sigmoid(2u), u = sqrt(2/pi) (x + 0.044715 x^3), which is equal to
// 0.5 x (1 + tanh(u)); with the hardware exponential and reciprocal it costs a handful of
// instructions and is accurate to about 1e-6 relative, far below bfloat16 resolution.  Used in the
// epilogues of the bfloat16 tensor-core kernels.
__device__ __forceinline__ float gelu_new_fast(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u2 = 2.f * k0 * (x + k1 * x * x * x);
  return __fdividef(x, 1.f + __expf(-u2));
}

// gelu_new: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
__device__ __forceinline__ float gelu_new_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}
