// Sampling from float32 logits, one thread block per row, and the logits
// processors that run before it.
//
// sample:  logprobs = logits - logsumexp(logits)            (mlx_lm/generate.py:411)
//          temp == 0  -> argmax                              (mlx_lm/sample_utils.py:46-47)
//          else filters in mlx-lm's order top-p -> min-p -> XTC -> top-k
//          (mlx_lm/sample_utils.py:50-60), then a categorical draw from
//          softmax(logprobs / temp) over what is left (:279-281).
//   The draw is Gumbel-max with a counter-based generator (Philox4x32-10) keyed by
//   (seed, request id, position, vocabulary index): a token's draw does not depend on what
//   else is in the batch or on how the request was cut into steps.
//   Filters are thresholds found by bisection over the order-preserving integer image of the
//   float values, each probe a block-wide reduction over the row (no sort, no scratch memory):
//     top-p  keeps i iff the sum of probabilities of all j with logit_j <= logit_i exceeds 1-top_p
//            (ascending cumulative sum > 1-top_p, sample_utils.py:204-237);
//     min-p  keeps logprob >= max logprob + log(min_p), and at least min_tokens_to_keep (:154-201);
//     XTC    with probability xtc_probability removes every token whose renormalised probability is
//            above the smallest probability that exceeds xtc_threshold, special tokens excepted (:240-276);
//            the special tokens are the row's own: words `special_offset`, `special_count` of its record
//            name a range of the list the launcher is given;
//     top-k  keeps the k largest of what is left (:129-151).
//   Tokens of equal logit are kept or dropped together.
//
// process: logit_bias, then repetition, presence and frequency penalties over the last
//          `context` tokens of each row (mlx_lm/sample_utils.py:72-126, 284-369).
#include "common.cuh"

MLXB_DEFINE_LAST_ERROR()

struct SampleParams {   // 16 x 32-bit words per row
  float temp, top_p, min_p, xtc_probability, xtc_threshold;
  int top_k, min_tokens_to_keep;
  unsigned seed_lo, seed_hi, request, position;
  int special_offset, special_count;   // this row's XTC special tokens: xtc_special[offset .. offset + count)
  int pad[3];
};

__device__ __forceinline__ unsigned fkey(float f) {
  unsigned b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ void philox4x32_10(unsigned c0, unsigned c1, unsigned c2, unsigned c3, unsigned k0,
                                              unsigned k1, unsigned out[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const unsigned n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ float uniform01(unsigned x) {  // in (0, 1)
  return ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

// block-wide reductions over unsigned / (value, index) pairs; `red` holds >= 66 words
__device__ __forceinline__ int block_sum_int(int v, int* red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  if (wid == 0) {
    int t = lane < nw ? red[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// argmax with the smallest index among equal values
__device__ __forceinline__ void block_argmax(float& v, int& idx, float* redv, int* redi) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
  if (lane == 0) { redv[wid] = v; redi[wid] = idx; }
  __syncthreads();
  if (wid == 0) {
    float tv = lane < nw ? redv[lane] : -INFINITY;
    int ti = lane < nw ? redi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, tv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, ti, o);
      if (ov > tv || (ov == tv && oi < ti)) { tv = ov; ti = oi; }
    }
    if (lane == 0) { redv[32] = tv; redi[32] = ti; }
  }
  __syncthreads();
  v = redv[32];
  idx = redi[32];
}

struct Keep {          // which vocabulary entries are still candidates
  unsigned lo_key;     // keep fkey(logit) >= lo_key
  bool xtc;            // and, if set, drop q_i > xtc_cut unless special
  float xtc_cut, lse_kept;
  const int* special;
  int n_special;
  __device__ __forceinline__ bool operator()(int i, float l, float lse) const {
    if (fkey(l) < lo_key) return false;
    if (xtc) {
      const float q = expf(l - lse_kept);
      if (q > xtc_cut) {
        for (int s = 0; s < n_special; ++s)
          if (special[s] == i) return true;
        return false;
      }
    }
    return true;
  }
};

__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, int ld, int V, const SampleParams* __restrict__ params,
              const int* __restrict__ xtc_special, int n_special, int* __restrict__ out_token,
              float* __restrict__ out_logprob, float* __restrict__ out_logprobs, int ldo,
              const int* status_in, int* __restrict__ status_out) {
  __shared__ float redf[40];
  __shared__ int redi[40];
  pdl_trigger();
  pdl_wait();
  logits = after_wait(logits);
  const int row = blockIdx.x;
  // The step's status word rides along with the tokens: one copy to the host brings both.
  if (status_out && row == 0 && threadIdx.x == 0) *status_out = __ldcg(after_wait(status_in));
  const float* lg = logits + (size_t)row * ld;
  const SampleParams P = params[row];
  const int tid = threadIdx.x, nt = blockDim.x;

  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < V; i += nt) {
    const float l = lg[i];
    if (l > bv) { bv = l; bi = i; }
  }
  block_argmax(bv, bi, redf, redi);
  const float m = bv;
  const int amax = bi;
  float s = 0.f;
  for (int i = tid; i < V; i += nt) s += expf(lg[i] - m);
  const float lse = m + logf(block_sum(s, redf));
  if (out_logprobs)
    for (int i = tid; i < V; i += nt) out_logprobs[(size_t)row * ldo + i] = lg[i] - lse;

  if (P.temp == 0.f) {
    if (tid == 0) { out_token[row] = amax; out_logprob[row] = m - lse; }
    return;
  }

  const bool has_special = xtc_special && P.special_count > 0 && P.special_offset >= 0 &&
                           P.special_offset + P.special_count <= n_special;
  Keep keep{0u, false, 0.f, lse, has_special ? xtc_special + P.special_offset : nullptr,
            has_special ? P.special_count : 0};

  if (P.top_p > 0.f && P.top_p < 1.f) {
    // smallest key u with  sum_{key_i <= u} p_i  >  1 - top_p
    const float c = 1.f - P.top_p;
    unsigned lo = 0u, hi = fkey(m);
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1);
      float acc = 0.f;
      for (int i = tid; i < V; i += nt) {
        const float l = lg[i];
        if (fkey(l) <= mid) acc += expf(l - lse);
      }
      if (block_sum(acc, redf) > c) hi = mid; else lo = mid + 1;
    }
    keep.lo_key = lo;
  }

  if (P.min_p > 0.f) {
    unsigned thr = fkey(m + logf(P.min_p));
    if (P.min_tokens_to_keep > 1) {
      // largest key u with count(key_i >= u) >= k
      unsigned lo = 0u, hi = fkey(m);
      while (lo < hi) {
        const unsigned mid = lo + ((hi - lo) >> 1) + ((hi - lo) & 1u);
        int cnt = 0;
        for (int i = tid; i < V; i += nt) cnt += fkey(lg[i]) >= mid;
        if (block_sum_int(cnt, redi) >= P.min_tokens_to_keep) lo = mid; else hi = mid - 1;
      }
      thr = min(thr, lo);
    }
    keep.lo_key = max(keep.lo_key, thr);
  }

  if (P.xtc_probability > 0.f) {
    unsigned r[4];
    philox4x32_10(0xffffffffu, P.position, P.request, 1u, P.seed_lo, P.seed_hi, r);
    if (!(uniform01(r[0]) > P.xtc_probability)) {
      float z = 0.f;
      for (int i = tid; i < V; i += nt) {
        const float l = lg[i];
        if (fkey(l) >= keep.lo_key) z += expf(l - lse);
      }
      const float lse_kept = lse + logf(block_sum(z, redf));
      float least = INFINITY;   // smallest renormalised probability above the threshold
      for (int i = tid; i < V; i += nt) {
        const float l = lg[i];
        if (fkey(l) >= keep.lo_key) {
          const float q = expf(l - lse_kept);
          if (q > P.xtc_threshold) least = fminf(least, q);
        }
      }
      least = -block_max(-least, redf);
      keep.xtc = true;
      keep.xtc_cut = least;
      keep.lse_kept = lse_kept;
    }
  }

  if (P.top_k > 0 && P.top_k < V) {
    unsigned lo = keep.lo_key, hi = fkey(m);
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1) + ((hi - lo) & 1u);
      int cnt = 0;
      for (int i = tid; i < V; i += nt) {
        const float l = lg[i];
        cnt += (fkey(l) >= mid) && keep(i, l, lse);
      }
      if (block_sum_int(cnt, redi) >= P.top_k) lo = mid; else hi = mid - 1;
    }
    keep.lo_key = max(keep.lo_key, lo);
  }

  const float inv_t = 1.f / P.temp;
  bv = -INFINITY;
  bi = 0x7fffffff;
  for (int i = tid; i < V; i += nt) {
    const float l = lg[i];
    if (!keep(i, l, lse)) continue;
    unsigned r[4];
    philox4x32_10((unsigned)i, P.position, P.request, 0u, P.seed_lo, P.seed_hi, r);
    const float g = -logf(-logf(uniform01(r[0])));
    const float v = (l - lse) * inv_t + g;
    if (v > bv) { bv = v; bi = i; }
  }
  block_argmax(bv, bi, redf, redi);
  if (tid == 0) {
    const int tok = bi == 0x7fffffff ? amax : bi;   // nothing left (cannot happen with valid options): most likely
    out_token[row] = tok;
    out_logprob[row] = lg[tok] - lse;
  }
}

// logits: float32 [R, V] at row stride ld.  params: R records of 16 words (SampleParams).
// xtc_special: int32 [n_special], the rows' XTC special tokens one list after the other; each record names its range.
// out_logprobs (optional): float32 [R, V] at row stride ldo receives logits - logsumexp.
// status_in / status_out (optional, both or neither): the word at status_in is copied to status_out.
MLXB_EXPORT int mlxb_sample(const float* logits, int ld, int R, int V, const void* params, const int* xtc_special,
                            int n_special, int* out_token, float* out_logprob, float* out_logprobs, int ldo,
                            const int* status_in, int* status_out, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) return mlxb_fail(MLXB_BAD_ARG, "sample: vocabulary %d, row stride %d", V, ld);
  if (n_special < 0 || (n_special > 0 && !xtc_special))
    return mlxb_fail(MLXB_BAD_ARG, "sample: %d special tokens without a list", n_special);
  if ((status_in == nullptr) != (status_out == nullptr))
    return mlxb_fail(MLXB_BAD_ARG, "sample: the status word needs both a source and a destination");
  const int threads = V >= 16384 ? 1024 : (V >= 2048 ? 512 : 256);
  launch_pdl(sample_kernel, dim3(R), dim3(threads), 0, stream, logits, ld, V, (const SampleParams*)params,
             xtc_special, n_special, out_token, out_logprob, out_logprobs, ldo, status_in, status_out);
  return mlxb_check_launch("sample");
}

struct ProcessParams {   // 8 x 32-bit words per row
  float repetition_penalty, presence_penalty, frequency_penalty;
  int repetition_context, presence_context, frequency_context;
  int n_bias, pad;
};

// context: int32 [R, C], each row left-padded with -1, most recent token last.
// bias_index / bias_value: [R, B] (index -1 = unused).
__global__ void process_kernel(float* __restrict__ logits, int ld, int V, const ProcessParams* __restrict__ params,
                               const int* __restrict__ context, int C, const int* __restrict__ bias_index,
                               const float* __restrict__ bias_value, int B) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  float* lg = logits + (size_t)row * ld;
  const ProcessParams P = params[row];
  for (int b = threadIdx.x; b < B && b < P.n_bias; b += blockDim.x) {
    const int i = bias_index[(size_t)row * B + b];
    if (i >= 0 && i < V) lg[i] += bias_value[(size_t)row * B + b];
  }
  __syncthreads();
  const int* ctx = context + (size_t)row * C;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    const int tok = ctx[i];
    if (tok < 0 || tok >= V) continue;
    bool last = true;
    for (int j = i + 1; j < C; ++j)
      if (ctx[j] == tok) { last = false; break; }
    if (!last) continue;                    // the most recent occurrence speaks for the token
    const int d = C - i;                    // 1 = the newest token
    int freq = 0;
    for (int j = 0; j <= i; ++j)
      if (ctx[j] == tok && C - j <= P.frequency_context) ++freq;
    float l = lg[tok];
    if (P.repetition_penalty != 0.f && P.repetition_penalty != 1.f && d <= P.repetition_context)
      l = l < 0.f ? l * P.repetition_penalty : l / P.repetition_penalty;
    if (P.presence_penalty != 0.f && d <= P.presence_context) l -= P.presence_penalty;
    if (P.frequency_penalty != 0.f) l -= P.frequency_penalty * (float)freq;
    lg[tok] = l;
  }
}

MLXB_EXPORT int mlxb_process_logits(float* logits, int ld, int R, int V, const void* params, const int* context,
                                    int C, const int* bias_index, const float* bias_value, int B,
                                    cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V || C < 0 || B < 0) return mlxb_fail(MLXB_BAD_ARG, "process_logits: V %d ld %d C %d B %d", V, ld, C, B);
  process_kernel<<<R, 128, 0, stream>>>(logits, ld, V, (const ProcessParams*)params, context, C, bias_index,
                                        bias_value, B);
  return mlxb_check_launch("process_logits");
}
