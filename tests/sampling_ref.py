"""Plain statements of the samplers and logits processors, from the formulas of
mlx_lm/sample_utils.py (sort-based, as written there), plus the counter-based random numbers
(Philox4x32-10, Salmon et al. 2011) that the engine's Gumbel-max draw uses."""
import math

import numpy as np

M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = 0xFFFFFFFF


def philox4x32_10(c, k):
    c0, c1, c2, c3 = c
    k0, k1 = k
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> 32, p0 & MASK, p1 >> 32, p1 & MASK
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0, k1 = (k0 + W0) & MASK, (k1 + W1) & MASK
    return c0, c1, c2, c3


def uniform01(x):
    return np.float32((np.float32(x >> 8) + np.float32(0.5)) * np.float32(1.0 / 16777216.0))


def gumbel(i, position, request, seed):
    u = uniform01(philox4x32_10((i, position, request, 0), (seed & MASK, (seed >> 32) & MASK))[0])
    return -math.log(-math.log(float(u)))


def xtc_uniform(position, request, seed):
    return float(uniform01(philox4x32_10((MASK, position, request, 1), (seed & MASK, (seed >> 32) & MASK))[0]))


def log_softmax(x):
    x = np.asarray(x, dtype=np.float64)
    m = x.max()
    return x - (m + math.log(np.exp(x - m).sum()))


def apply_top_p(logprobs, top_p):
    """mlx_lm/sample_utils.py:204-237: ascending sort, cumulative sum, keep where cumulative > 1 - top_p."""
    order = np.argsort(logprobs, kind="stable")
    cum = np.cumsum(np.exp(logprobs[order]))
    keep = np.zeros(len(logprobs), dtype=bool)
    keep[order] = cum > 1 - top_p
    return np.where(keep, logprobs, -np.inf)


def apply_min_p(logprobs, min_p, min_tokens_to_keep=1):
    """mlx_lm/sample_utils.py:154-201."""
    remove = logprobs < logprobs.max() + math.log(min_p)
    if min_tokens_to_keep > 1:
        top = np.argsort(logprobs, kind="stable")[-min_tokens_to_keep:]
        remove[top] = False
    return np.where(remove, -np.inf, logprobs)


def apply_xtc(logprobs, threshold, special, applies):
    """mlx_lm/sample_utils.py:240-276, with the coin already tossed (``applies``)."""
    if not applies:
        return logprobs
    probs = np.exp(log_softmax(logprobs))
    above = np.where(probs > threshold, probs, np.inf)
    mask = probs > above.min()
    mask[list(special)] = False
    return np.where(mask, -np.inf, logprobs)


def apply_top_k(logprobs, k):
    """mlx_lm/sample_utils.py:129-151."""
    order = np.argsort(-logprobs, kind="stable")
    out = logprobs.copy()
    out[order[k:]] = -np.inf
    return out


def sample(logits, temp=0.0, top_p=0.0, min_p=0.0, min_tokens_to_keep=1, top_k=0, xtc_probability=0.0,
           xtc_threshold=0.1, xtc_special=(), seed=0, request=0, position=0):
    """Token and its log-probability, filters in the order top-p, min-p, XTC, top-k
    (mlx_lm/sample_utils.py:46-67), the categorical draw as Gumbel-max."""
    lp = log_softmax(logits)
    if temp == 0:
        tok = int(np.argmax(lp))
        return tok, float(lp[tok]), lp
    x = lp.copy()
    if 0 < top_p < 1:
        x = apply_top_p(x, top_p)
    if min_p != 0:
        x = apply_min_p(x, min_p, min_tokens_to_keep)
    if xtc_probability > 0:
        x = apply_xtc(x, xtc_threshold, xtc_special, not (xtc_uniform(position, request, seed) > xtc_probability))
    if top_k > 0:
        x = apply_top_k(x, top_k)
    best, tok = -np.inf, -1
    for i in np.nonzero(np.isfinite(x))[0]:
        v = x[i] / temp + gumbel(int(i), position, request, seed)
        if v > best:
            best, tok = v, int(i)
    return tok, float(lp[tok]), x


def process(logits, tokens, logit_bias=None, repetition_penalty=None, repetition_context_size=20,
            presence_penalty=None, presence_context_size=20, frequency_penalty=None, frequency_context_size=20):
    """mlx_lm/sample_utils.py:72-126, 284-369, in that order."""
    x = np.asarray(logits, dtype=np.float64).copy()
    for t, v in (logit_bias or {}).items():
        x[t] += v
    if repetition_penalty:
        for t in set(tokens[-repetition_context_size:]):
            x[t] = x[t] * repetition_penalty if x[t] < 0 else x[t] / repetition_penalty
    if presence_penalty:
        for t in set(tokens[-presence_context_size:]):
            x[t] -= presence_penalty
    if frequency_penalty:
        for t in tokens[-frequency_context_size:]:
            x[t] -= frequency_penalty
    return x
