// Token embedding gather plus learned absolute position add:
//   h[t, :] = round(float(wte[tok[t], :]) + float(wpe[pos[t], :]))
// The sum is formed in 32-bit and rounded once.  `wpe` may be null (a model
// without a position table): then it is a plain gather.
// Ids outside the tables set a status bit and produce zeros instead of
// reading out of bounds.
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

template <typename T>
__global__ void embed_pos_kernel(const int* __restrict__ tok, const int* __restrict__ pos,
                                 const T* __restrict__ wte, const T* __restrict__ wpe,
                                 T* __restrict__ out, int D, int V, int P, float scale,
                                 int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = tok[t];
  const int p = wpe ? pos[t] : 0;
  bool ok = true;
  if (id < 0 || id >= V) { ok = false; if (threadIdx.x == 0) atomicOr(status, MLXB_ST_TOKEN_RANGE); }
  if (wpe && (p < 0 || p >= P)) { ok = false; if (threadIdx.x == 0) atomicOr(status, MLXB_ST_POSITION_RANGE); }
  T* o = out + (size_t)t * D;
  if (!ok) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = from_f<T>(0.f);
    return;
  }
  const T* e = wte + (size_t)id * D;
  const T* q = wpe ? wpe + (size_t)p * D : nullptr;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = to_f(e[d]) * scale;
    if (q) v += to_f(q[d]);
    o[d] = from_f<T>(v);
  }
}

// dtype: MLXB_F32 / MLXB_BF16 for tables and output alike.
MLXB_EXPORT int mlxb_embed_pos(int dtype, const int* tok, const int* pos, const void* wte, const void* wpe,
                               void* out, int T_, int D, int V, int P, float scale, int* status,
                               cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (D <= 0 || V <= 0) return mlxb_fail(MLXB_BAD_ARG, "embed_pos: width %d, vocabulary %d", D, V);
  const int threads = D >= 1024 ? 256 : (D >= 256 ? 128 : 64);
  if (dtype == MLXB_F32)
    embed_pos_kernel<float><<<T_, threads, 0, stream>>>(tok, pos, (const float*)wte, (const float*)wpe,
                                                        (float*)out, D, V, P, scale, status);
  else if (dtype == MLXB_BF16)
    embed_pos_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(tok, pos, (const __nv_bfloat16*)wte,
                                                                (const __nv_bfloat16*)wpe, (__nv_bfloat16*)out,
                                                                D, V, P, scale, status);
  else
    return mlxb_fail(MLXB_BAD_DTYPE, "embed_pos: dtype code %d", dtype);
  return mlxb_check_launch("embed_pos");
}

// Tokens that are still on the device: dst[i] = src[index[i]] where index[i] >= 0 (dst[i] stays as it is where
// index[i] < 0).  Used to feed the tokens a step has just sampled into the next step without a round trip
// through the host; src has n_src words, an index outside it sets MLXB_ST_TOKEN_RANGE and leaves dst[i] alone.
__global__ void gather_tokens_kernel(const int* __restrict__ src, int n_src, const int* __restrict__ index,
                                     int* __restrict__ dst, int n, int* __restrict__ status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int j = index[i];
  if (j < 0) return;
  if (j >= n_src) { atomicOr(status, MLXB_ST_TOKEN_RANGE); return; }
  dst[i] = src[j];
}

MLXB_EXPORT int mlxb_gather_tokens(const int* src, int n_src, const int* index, int* dst, int n, int* status,
                                   cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_src <= 0) return mlxb_fail(MLXB_BAD_ARG, "gather_tokens: %d source words", n_src);
  gather_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(src, n_src, index, dst, n, status);
  return mlxb_check_launch("gather_tokens");
}
