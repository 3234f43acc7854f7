"""Plain torch statements of what each CUDA kernel computes, in float32 (or
float64), used by the kernel tests.  Arguments mirror ``mlx_lm_b200.ops`` so
a test can call both with the same tensors; nothing here is imported by the
package."""
import math

import torch


def embed_pos(tokens, positions, wte, wpe, scale=1.0):
    h = wte.float()[tokens.long()] * scale
    if wpe is not None:
        h = h + wpe.float()[positions.long()]
    return h


def layernorm(x, gain, bias, eps, rows=None):
    x = x.float()
    if rows is not None:
        x = x[rows.long()]
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    y = (x - mean) * torch.rsqrt(var + eps) * gain.float()
    return y if bias is None else y + bias.float()


def gelu_new(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def linear(x, w, bias=None, activation=None, residual=None):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if activation == "gelu_new":
        y = gelu_new(y)
    elif activation == "relu":
        y = torch.relu(y)
    elif activation not in (None, "none"):
        raise ValueError(activation)
    if residual is not None:
        y = y + residual.float()
    return y


def kv_write(k_src, v_src, positions, token_req, block_table, k_pool, v_pool):
    """In place on clones of the pools; returns (k_pool, v_pool)."""
    k_pool, v_pool = k_pool.clone(), v_pool.clone()
    n_pages, H, page, Dh = k_pool.shape
    for t in range(k_src.shape[0]):
        r = int(token_req[t])
        if r < 0:
            continue
        p = int(positions[t])
        pg = int(block_table[r, p // page])
        if pg < 0:
            continue
        k_pool[pg, :, p % page, :] = k_src[t].reshape(H, Dh)
        v_pool[pg, :, p % page, :] = v_src[t].reshape(H, Dh)
    return k_pool, v_pool


def gather_kv(pool, block_table_row, first, last, page):
    """Rows ``first..last`` of one request from a pool ``[n_pages, H, page, Dh]`` -> ``[H, n, Dh]``."""
    rows = []
    for j in range(first, last + 1):
        pg = int(block_table_row[j // page])
        assert pg >= 0, f"position {j} has no page"
        rows.append(pool[pg, :, j % page, :])
    return torch.stack(rows, dim=1)


def attention(q, positions, token_req, block_table, k_pool, v_pool, n_heads, scale, window=0, dtype=torch.float32):
    """Every token attends keys max(0, p-window+1)..p of its request.  q: [T, n_heads*Dh] -> [T, n_heads*Dh]."""
    n_pages, Hkv, page, Dh = k_pool.shape
    T = q.shape[0]
    out = torch.zeros(T, n_heads * Dh, dtype=dtype)
    rep = n_heads // Hkv
    for t in range(T):
        r = int(token_req[t])
        if r < 0:
            continue
        p = int(positions[t])
        lo = max(0, p - window + 1) if window and window > 0 else 0
        k = gather_kv(k_pool, block_table[r], lo, p, page).to(dtype).cpu()   # [Hkv, n, Dh]
        v = gather_kv(v_pool, block_table[r], lo, p, page).to(dtype).cpu()
        qt = q[t].to(dtype).cpu().reshape(n_heads, Dh)
        k = k.repeat_interleave(rep, dim=0)
        v = v.repeat_interleave(rep, dim=0)
        s = torch.einsum("hd,hnd->hn", qt, k) * scale
        out[t] = torch.einsum("hn,hnd->hd", torch.softmax(s, -1), v).reshape(-1)
    return out
