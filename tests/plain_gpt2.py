"""Plain, slow GPT-2 forward pass used as the oracle of the test-suite.

Whole sequences, no cache, one function per part, float32 (or float64) on the
CPU.  It shares no code with the package: weights come in as a dictionary
``HF tensor name -> torch tensor`` and the configuration as a plain dict with
the keys of ``config.json``.

Every function cites the place in ml-explore/mlx-lm (paths inside that
project) whose behaviour it restates.  The bodies of ``nn.LayerNorm``,
``nn.gelu_approx``, ``nn.Linear`` and ``mx.fast.scaled_dot_product_attention``
live in MLX, not in mlx-lm; for those the formula is written out here and
the citation names the call site.

``tests/golden/make_golden.py`` runs mlx-lm's own ``models/gpt2.py`` on a
tiny random model (over a torch stand-in for the few MLX symbols it uses) and
``tests/test_plain.py`` compares this file with the stored outputs.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def strip_prefix(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Names without a ``transformer.`` / ``model.`` prefix and without the
    causal-mask buffers ``h.N.attn.bias`` / ``h.N.attn.masked_bias``
    (mlx_lm/models/gpt2.py:171-174 deletes ``attn.bias``; :191-196 handles the
    ``model.`` prefix)."""
    out = {}
    for name, t in weights.items():
        for p in ("transformer.", "model."):
            if name.startswith(p):
                name = name[len(p):]
        if name.endswith(".attn.bias") or name.endswith(".attn.masked_bias"):
            continue
        out[name] = t
    return out


def inner_width(cfg: dict) -> int:
    """mlx_lm/models/gpt2.py:76-77 hard-codes ``4 * n_embd``; ``n_inner`` of
    config.json (null means 4 * n_embd) is the generalisation used here."""
    n_inner = cfg.get("n_inner")
    return 4 * cfg["n_embd"] if n_inner is None else int(n_inner)


def embed(tokens: torch.Tensor, wte: torch.Tensor) -> torch.Tensor:
    """``hidden = wte(inputs)`` — mlx_lm/models/gpt2.py:132."""
    return wte[tokens]


def add_positions(h: torch.Tensor, wpe: torch.Tensor, offset: int = 0) -> torch.Tensor:
    """``position_ids = arange(L) + offset; hidden += wpe(position_ids)`` —
    mlx_lm/models/gpt2.py:137-144."""
    L = h.shape[0]
    pos = torch.arange(L) + offset
    return h + wpe[pos]


def layer_norm(x: torch.Tensor, gain: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """``nn.LayerNorm(D, eps)`` with affine gain and bias, biased variance
    over the last axis — call sites mlx_lm/models/gpt2.py:92-96, 123, 151."""
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * gain + bias


def conv1d_linear(x: torch.Tensor, w_in_out: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    """HF Conv1D ``[in, out]`` weight: ``y = x @ W + b``.  mlx-lm transposes
    these to ``[out, in]`` at load and calls ``nn.Linear``
    (mlx_lm/models/gpt2.py:175-190, 41-42, 76-77)."""
    y = x @ w_in_out
    return y if b is None else y + b


def gelu_new(x: torch.Tensor) -> torch.Tensor:
    """``nn.gelu_approx`` (tanh form) — call site mlx_lm/models/gpt2.py:80."""
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def split_heads(qkv: torch.Tensor, n_head: int):
    """``q, k, v = split(qkv, 3, -1)`` then ``reshape(L, H, Dh)`` with head j
    = columns [j*Dh, (j+1)*Dh) — mlx_lm/models/gpt2.py:52-58.  Returns three
    ``[H, L, Dh]`` tensors."""
    L, three_d = qkv.shape
    d = three_d // 3
    q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
    f = lambda t: t.reshape(L, n_head, d // n_head).permute(1, 0, 2)
    return f(q), f(k), f(v)


def causal_attention(q, k, v, window: Optional[int] = None) -> torch.Tensor:
    """``softmax(scale * q k^T + causal mask) v`` with ``scale = Dh**-0.5`` —
    mlx_lm/models/gpt2.py:39, 63-65 and mlx_lm/models/base.py:132-139; the mask
    is ``linds >= rinds`` and, with a window, ``linds < rinds + window``
    (mlx_lm/models/base.py:24-36).  Inputs ``[H, L, Dh]``; output ``[L, H*Dh]``
    (heads concatenated in order, mlx_lm/models/gpt2.py:67)."""
    H, L, Dh = q.shape
    scores = (q @ k.transpose(1, 2)) * (Dh ** -0.5)
    li = torch.arange(L)[:, None]
    ri = torch.arange(L)[None, :]
    mask = li >= ri
    if window is not None:
        mask = mask & (li < ri + window)
    scores = scores.masked_fill(~mask, float("-inf"))
    p = torch.softmax(scores, dim=-1)
    o = p @ v
    return o.permute(1, 0, 2).reshape(L, H * Dh)


def attention_part(x, w, prefix: str, n_head: int) -> torch.Tensor:
    """``c_proj(sdpa(split(c_attn(x))))`` — mlx_lm/models/gpt2.py:52-68."""
    qkv = conv1d_linear(x, w[prefix + "c_attn.weight"], w[prefix + "c_attn.bias"])
    q, k, v = split_heads(qkv, n_head)
    o = causal_attention(q, k, v)
    return conv1d_linear(o, w[prefix + "c_proj.weight"], w[prefix + "c_proj.bias"])


def mlp_part(x, w, prefix: str) -> torch.Tensor:
    """``c_proj(gelu_approx(c_fc(x)))`` — mlx_lm/models/gpt2.py:80."""
    h = conv1d_linear(x, w[prefix + "c_fc.weight"], w[prefix + "c_fc.bias"])
    return conv1d_linear(gelu_new(h), w[prefix + "c_proj.weight"], w[prefix + "c_proj.bias"])


def block(x, w, i: int, cfg: dict) -> torch.Tensor:
    """``h = x + attn(ln_1(x)); out = h + mlp(ln_2(h))`` —
    mlx_lm/models/gpt2.py:104-108."""
    eps = cfg["layer_norm_epsilon"]
    p = f"h.{i}."
    r = attention_part(layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps), w, p + "attn.", cfg["n_head"])
    h = x + r
    r = mlp_part(layer_norm(h, w[p + "ln_2.weight"], w[p + "ln_2.bias"], eps), w, p + "mlp.")
    return h + r


def hidden_states(tokens: List[int], weights: Dict[str, torch.Tensor], cfg: dict,
                  dtype=torch.float32) -> torch.Tensor:
    """All blocks and the final norm — mlx_lm/models/gpt2.py:126-151."""
    w = {k: v.to(dtype) for k, v in strip_prefix(weights).items()}
    t = torch.as_tensor(tokens, dtype=torch.long)
    x = add_positions(embed(t, w["wte.weight"]), w["wpe.weight"])
    for i in range(cfg["n_layer"]):
        x = block(x, w, i, cfg)
    return layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], cfg["layer_norm_epsilon"])


def logits(tokens: List[int], weights: Dict[str, torch.Tensor], cfg: dict,
           dtype=torch.float32) -> torch.Tensor:
    """``wte.as_linear(ln_f(h))``: tied head, no bias, every position —
    mlx_lm/models/gpt2.py:166-167.  Returns ``[L, V]``."""
    w = strip_prefix(weights)
    return hidden_states(tokens, weights, cfg, dtype) @ w["wte.weight"].to(dtype).T


def log_probs(lg: torch.Tensor) -> torch.Tensor:
    """``logits - logsumexp(logits)`` — mlx_lm/generate.py:411, 1434."""
    return lg - torch.logsumexp(lg, dim=-1, keepdim=True)


def greedy_generate(prompt: List[int], n: int, weights, cfg, dtype=torch.float32) -> List[int]:
    """Argmax decoding by re-running the whole sequence for every new token
    (``temp == 0`` sampler, mlx_lm/sample_utils.py:46-47)."""
    seq = list(prompt)
    out = []
    for _ in range(n):
        tok = int(torch.argmax(logits(seq, weights, cfg, dtype)[-1]))
        out.append(tok)
        seq.append(tok)
    return out
