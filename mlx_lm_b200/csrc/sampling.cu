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

// What the categorical draw maximises (Gumbel-max): logit / temperature + Gumbel noise from 32 random bits.  The
// row's logsumexp is left out: it is the same for every candidate.
__device__ __forceinline__ float draw_value(float logit, float inv_temp, unsigned bits) {
  return fmaf(logit, inv_temp, -logf(-logf(uniform01(bits))));
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

// One row by one thread block: every pass walks the whole row.
__device__ __forceinline__ void sample_row(const float* __restrict__ lg, int V, const SampleParams& P, int row,
                                           const int* __restrict__ xtc_special, int n_special,
                                           int* __restrict__ out_token, float* __restrict__ out_logprob,
                                           float* __restrict__ out_logprobs, int ldo, float* redf, int* redi) {
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
    const float v = draw_value(l, inv_t, r[0]);
    if (v > bv) { bv = v; bi = i; }
  }
  block_argmax(bv, bi, redf, redi);
  if (tid == 0) {
    const int tok = bi == 0x7fffffff ? amax : bi;   // nothing left (cannot happen with valid options): most likely
    out_token[row] = tok;
    out_logprob[row] = lg[tok] - lse;
  }
}

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
  sample_row(logits + (size_t)row * ld, V, params[row], row, xtc_special, n_special, out_token, out_logprob,
             out_logprobs, ldo, redf, redi);
}

// Wide vocabularies: a row is cut into SAMPLE_SLICES slices, one thread block each.  A block finds its slice's
// maximum (first index among equals), the sum of exponentials relative to it and, for a row that is drawn from
// without filters, the slice's best draw value; it leaves these in scratch memory and takes a ticket.  The block
// that takes a row's last ticket merges the slices in slice order (so the result does not depend on which block
// that is, nor on how many rows the launch has) and writes the token.  Nobody waits for anybody.  A row with
// filters (top-p, min-p, XTC, top-k) is done whole by that last block, as in sample_kernel.
constexpr int SAMPLE_SLICES = 8;
constexpr int SAMPLE_SLICE_WORDS = 8;    // maximum, its index, sum, best draw value, its index, 3 unused
constexpr int SAMPLE_SPLIT_FROM = 8192;  // vocabulary sizes from which rows are cut
constexpr int SAMPLE_SPLIT_THREADS = 256;
constexpr int SAMPLE_KEEP = 8;           // logits a thread keeps in registers between its passes

// (maximum with the first index among equals, sum of exponentials relative to that maximum) of two parts
struct SoftmaxPart { float m; int idx; float s; };
__device__ __forceinline__ SoftmaxPart merge(const SoftmaxPart& a, const SoftmaxPart& b) {   // a: lower indices on ties
  SoftmaxPart o;
  const bool take_b = b.m > a.m || (b.m == a.m && b.idx < a.idx);
  o.m = take_b ? b.m : a.m;
  o.idx = take_b ? b.idx : a.idx;
  const float sa = a.m == -INFINITY ? 0.f : a.s * expf(a.m - o.m), sb = b.m == -INFINITY ? 0.f : b.s * expf(b.m - o.m);
  o.s = sa + sb;
  return o;
}

__global__ void __launch_bounds__(SAMPLE_SPLIT_THREADS)
sample_split_kernel(const float* __restrict__ logits, int ld, int V, const SampleParams* __restrict__ params,
                    const int* __restrict__ xtc_special, int n_special, int* __restrict__ out_token,
                    float* __restrict__ out_logprob, const int* status_in, int* __restrict__ status_out,
                    int* __restrict__ tickets, float* __restrict__ partials) {
  __shared__ float redf[40];
  __shared__ int redi[40];
  __shared__ float w_m[8], w_s[8], w_g[8];
  __shared__ int w_i[8], w_gi[8];
  __shared__ int s_last;
  const int row = blockIdx.y, slice = blockIdx.x;
  const SampleParams P = params[row];      // written by the host before the step, not by the kernel before
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  constexpr int nt = SAMPLE_SPLIT_THREADS;
  const bool filters = P.temp != 0.f && ((P.top_p > 0.f && P.top_p < 1.f) || P.min_p > 0.f ||
                                         P.xtc_probability > 0.f || (P.top_k > 0 && P.top_k < V));
  const bool draws = P.temp != 0.f && !filters;
  const int per = (((V + SAMPLE_SLICES - 1) / SAMPLE_SLICES) + 3) & ~3;
  const int i0 = slice * per, i1 = min(V, i0 + per);
  pdl_trigger();
  pdl_wait();
  logits = after_wait(logits);
  if (status_out && row == 0 && slice == 0 && tid == 0) *status_out = __ldcg(after_wait(status_in));
  const float* lg = logits + (size_t)row * ld;

  // one pass over global memory: the first SAMPLE_KEEP logits of a thread stay in registers
  float keep[SAMPLE_KEEP];
  SoftmaxPart mine = {-INFINITY, 0x7fffffff, 0.f};
#pragma unroll
  for (int k = 0; k < SAMPLE_KEEP; ++k) {
    const int i = i0 + tid + k * nt;
    keep[k] = i < i1 ? lg[i] : -INFINITY;
    if (keep[k] > mine.m) { mine.m = keep[k]; mine.idx = i; }
  }
  for (int i = i0 + tid + SAMPLE_KEEP * nt; i < i1; i += nt) {
    const float l = lg[i];
    if (l > mine.m) { mine.m = l; mine.idx = i; }
  }
  if (mine.m != -INFINITY) {
#pragma unroll
    for (int k = 0; k < SAMPLE_KEEP; ++k) mine.s += expf(keep[k] - mine.m);   // exp(-inf) = 0 for what lies outside
    for (int i = i0 + tid + SAMPLE_KEEP * nt; i < i1; i += nt) mine.s += expf(lg[i] - mine.m);
  }
  float gv = -INFINITY;
  int gi = 0x7fffffff;
  if (draws) {
    const float inv_t = 1.f / P.temp;
#pragma unroll
    for (int k = 0; k < SAMPLE_KEEP; ++k) {
      const int i = i0 + tid + k * nt;
      if (i < i1) {
        unsigned r[4];
        philox4x32_10((unsigned)i, P.position, P.request, 0u, P.seed_lo, P.seed_hi, r);
        const float v = draw_value(keep[k], inv_t, r[0]);
        if (v > gv) { gv = v; gi = i; }
      }
    }
    for (int i = i0 + tid + SAMPLE_KEEP * nt; i < i1; i += nt) {
      unsigned r[4];
      philox4x32_10((unsigned)i, P.position, P.request, 0u, P.seed_lo, P.seed_hi, r);
      const float v = draw_value(lg[i], inv_t, r[0]);
      if (v > gv) { gv = v; gi = i; }
    }
  }
  // one reduction for all of it, in a fixed tree: lanes, then warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    SoftmaxPart other;
    other.m = __shfl_xor_sync(0xffffffffu, mine.m, o);
    other.idx = __shfl_xor_sync(0xffffffffu, mine.idx, o);
    other.s = __shfl_xor_sync(0xffffffffu, mine.s, o);
    mine = merge(mine, other);
    const float ov = __shfl_xor_sync(0xffffffffu, gv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, gi, o);
    if (ov > gv || (ov == gv && oi < gi)) { gv = ov; gi = oi; }
  }
  if (lane == 0) { w_m[wid] = mine.m; w_i[wid] = mine.idx; w_s[wid] = mine.s; w_g[wid] = gv; w_gi[wid] = gi; }
  __syncthreads();
  if (tid == 0) {
    SoftmaxPart all = {w_m[0], w_i[0], w_s[0]};
    float bg = w_g[0];
    int bgi = w_gi[0];
    for (int w = 1; w < nt / 32; ++w) {
      all = merge(all, SoftmaxPart{w_m[w], w_i[w], w_s[w]});
      if (w_g[w] > bg || (w_g[w] == bg && w_gi[w] < bgi)) { bg = w_g[w]; bgi = w_gi[w]; }
    }
    float* rec = partials + ((size_t)row * SAMPLE_SLICES + slice) * SAMPLE_SLICE_WORDS;
    rec[0] = all.m;
    rec[1] = __int_as_float(all.idx);
    rec[2] = all.s;
    rec[3] = bg;
    rec[4] = __int_as_float(bgi);
    __threadfence();
    s_last = atomicAdd(&tickets[row], 1) == SAMPLE_SLICES - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (tid == 0) tickets[row] = 0;             // for the next launch
  if (filters) {   // not what this kernel is launched for, but right: the whole row by this block
    sample_row(lg, V, P, row, xtc_special, n_special, out_token, out_logprob, nullptr, 0, redf, redi);
    return;
  }
  if (tid == 0) {
    const float* recs = partials + (size_t)row * SAMPLE_SLICES * SAMPLE_SLICE_WORDS;
    float rm[SAMPLE_SLICES], rs[SAMPLE_SLICES], rg[SAMPLE_SLICES];
    int ri[SAMPLE_SLICES], rgi[SAMPLE_SLICES];
#pragma unroll
    for (int k = 0; k < SAMPLE_SLICES; ++k) {      // all loads first: they do not depend on one another
      const float* rk = recs + k * SAMPLE_SLICE_WORDS;
      rm[k] = __ldcg(rk);
      ri[k] = __float_as_int(__ldcg(rk + 1));
      rs[k] = __ldcg(rk + 2);
      rg[k] = __ldcg(rk + 3);
      rgi[k] = __float_as_int(__ldcg(rk + 4));
    }
    SoftmaxPart all = {-INFINITY, 0x7fffffff, 0.f};
    float bg = -INFINITY;
    int bgi = 0x7fffffff;
#pragma unroll
    for (int k = 0; k < SAMPLE_SLICES; ++k) {      // slices in index order: the first of equals wins
      all = merge(all, SoftmaxPart{rm[k], ri[k], rs[k]});
      if (rg[k] > bg) { bg = rg[k]; bgi = rgi[k]; }
    }
    const float lse = all.m + logf(all.s);
    const int tok = (draws && bgi != 0x7fffffff) ? bgi : all.idx;
    out_token[row] = tok;
    out_logprob[row] = lg[tok] - lse;
  }
}

// logits: float32 [R, V] at row stride ld.  params: R records of 16 words (SampleParams).
// xtc_special: int32 [n_special], the rows' XTC special tokens one list after the other; each record names its range.
// out_logprobs (optional): float32 [R, V] at row stride ldo receives logits - logsumexp.
// status_in / status_out (optional, both or neither): the word at status_in is copied to status_out.
// scratch (optional): mlxb_sample_scratch_words(R) 32-bit words, zero when first given and left zero by every
// launch; with it (and without out_logprobs) rows of wide vocabularies are cut into slices over several thread blocks.
MLXB_EXPORT int mlxb_sample_scratch_words(int R) { return R * (SAMPLE_SLICES * SAMPLE_SLICE_WORDS + 1); }

MLXB_EXPORT int mlxb_sample(const float* logits, int ld, int R, int V, const void* params, const int* xtc_special,
                            int n_special, int* out_token, float* out_logprob, float* out_logprobs, int ldo,
                            const int* status_in, int* status_out, void* scratch, int scratch_words,
                            cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) return mlxb_fail(MLXB_BAD_ARG, "sample: vocabulary %d, row stride %d", V, ld);
  if (n_special < 0 || (n_special > 0 && !xtc_special))
    return mlxb_fail(MLXB_BAD_ARG, "sample: %d special tokens without a list", n_special);
  if ((status_in == nullptr) != (status_out == nullptr))
    return mlxb_fail(MLXB_BAD_ARG, "sample: the status word needs both a source and a destination");
  const int threads = V >= 16384 ? 1024 : (V >= 2048 ? 512 : 256);
  if (scratch != nullptr && out_logprobs == nullptr && V >= SAMPLE_SPLIT_FROM && R <= 65535) {
    if (scratch_words < mlxb_sample_scratch_words(R) || ((uintptr_t)scratch & 15))
      return mlxb_fail(MLXB_BAD_ARG, "sample: %d words of scratch memory for %d rows, %d needed (16-byte aligned)",
                       scratch_words, R, mlxb_sample_scratch_words(R));
    // tickets first, one word per row the scratch memory has room for (the same words whatever R is, so that they
    // are zero when a launch begins), the slices' records behind them
    const int room = scratch_words / (SAMPLE_SLICES * SAMPLE_SLICE_WORDS + 1);
    int* tickets = (int*)scratch;
    float* partials = (float*)scratch + room;
    launch_pdl(sample_split_kernel, dim3(SAMPLE_SLICES, R), dim3(SAMPLE_SPLIT_THREADS), 0, stream, logits, ld, V,
               (const SampleParams*)params, xtc_special, n_special, out_token, out_logprob, status_in, status_out,
               tickets, partials);
    return mlxb_check_launch("sample");
  }
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
