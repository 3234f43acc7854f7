"""Token mixers.  ``Attention``: multi-head (or grouped-query) causal
attention over a paged key/value cache.

One fused projection gives ``[q | k | v]`` per token (q = the first
``n_heads*head_dim`` columns, then k, then v, head j = columns
``[j*head_dim, (j+1)*head_dim)`` of each: mlx_lm/models/gpt2.py:52-58).  This
step's keys and values go into the request's pages first, then every token
attends keys ``max(0, p-window+1) .. p`` of its request through the block
table with scale ``head_dim**-0.5`` (mlx_lm/models/gpt2.py:39, 63-65), and
the output projection adds the residual in its epilogue.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Init, Mixer, Normed, PagedKVSpec, PositionEncoding, register_part
from .linear import Linear


class Attention(Mixer):
    replayable = True
    kernel_libs = ("attention", "attention_prefill", "attention_prefill_tc")

    def __init__(self, name: str, width: int, n_heads: int, head_dim: int, n_kv_heads: Optional[int] = None,
                 window: Optional[int] = None, bias: bool = True, stored: str = "out_in",
                 qkv_name: str = "c_attn", out_name: str = "c_proj", scale: Optional[float] = None,
                 position: Optional[PositionEncoding] = None, init: Init = Init(), bias_init: Init = Init()):
        n_kv_heads = n_heads if n_kv_heads is None else n_kv_heads
        if n_heads % n_kv_heads:
            raise ValueError(f"{name}: {n_heads} query heads are not a multiple of {n_kv_heads} key/value heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"{name}: head size {head_dim} must be a multiple of 16 between 16 and 256")
        self.name, self.width = name, width
        self.n_heads, self.n_kv_heads, self.head_dim, self.window = n_heads, n_kv_heads, head_dim, window
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.position = position
        self.q_width, self.kv_width = n_heads * head_dim, n_kv_heads * head_dim
        self.qkv = Linear(f"{name}.{qkv_name}", width, self.q_width + 2 * self.kv_width, bias, stored,
                          init=init, bias_init=bias_init)
        self.out = Linear(f"{name}.{out_name}", self.q_width, width, bias, stored, init=init, bias_init=bias_init)

    def children(self):
        return (self.qkv, self.out)

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_heads, self.head_dim, self.window)

    def fold_input_norm(self, norm) -> bool:
        return self.qkv.fold_norm(norm)

    def forward(self, ctx, x, residual, cache):
        T = x.shape[0]
        qkv = ctx.ws.get("qkv", T, self.q_width + 2 * self.kv_width, x.dtype)
        q = qkv[:, :self.q_width]
        src = x.source if isinstance(x, Normed) else x      # a Normed: the norm is folded into the projection
        if (cache.write and self.position is None and x.dtype == torch.bfloat16 and self.width % 8 == 0
                and src.stride(0) % 8 == 0 and src.data_ptr() % 16 == 0):
            # nothing to do to q and k before the cache: the projection's epilogue puts keys and values
            # into the pages itself
            fold = self.qkv.fold_of(ctx, x, few=T <= ops.SMALL_M) if isinstance(x, Normed) else None
            n_qkv = self.q_width + 2 * self.kv_width
            ops.label(self.qkv.name, 2.0 * T * self.width * n_qkv,
                      x.dtype.itemsize * (self.width * n_qkv + T * self.width + T * n_qkv))
            ops.linear_qkv_to_cache(src, self.qkv.weight, self.qkv.bias, qkv, ctx.positions, ctx.token_req,
                                    cache.block_table, cache.k, cache.v, self.q_width, ctx.status, ctx.stream,
                                    fold=fold)
        else:
            self.qkv.forward(ctx, x, qkv)
            k = qkv[:, self.q_width:self.q_width + self.kv_width]
            v = qkv[:, self.q_width + self.kv_width:]
            if self.position is not None:
                self.position.rotate(ctx, q, k)
            if cache.write:
                ops.kv_write(k, v, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, ctx.status,
                             ctx.stream)
        o = ctx.ws.get("attn_out", T, self.q_width, x.dtype)
        ops.label(self.name + ".attention")      # its cost depends on the requests' lengths: the caller knows them
        self.attend(ctx, q, cache, o)
        return self.out.forward(ctx, o, residual, residual=residual)

    def attend(self, ctx, q, cache, o) -> None:
        """Rows of requests that bring one token go to a kernel for single queries (on tensor cores in bfloat16
        for head sizes that are multiples of 16 up to 128, else the split-key kernel on the CUDA cores), the
        rest to the kernel for portions; all write their rows of ``o``."""
        window = self.window or 0
        single_tiles = getattr(ctx, "single_tiles", None)
        if (ctx.n_single and single_tiles is not None
                and ops.attention_rows_supported(q.dtype, self.head_dim, ctx.n_single, self.n_heads)):
            ops.attention_rows(q, single_tiles, ctx.n_single, cache.block_table, cache.k, cache.v, o, self.n_heads,
                               self.scale, window, ctx.status, ctx.stream)
        elif ctx.n_single:
            scratch = ctx.ws.flat("attn_partial", ops.attention_decode_scratch(
                ctx.n_single, self.n_heads, self.head_dim, ctx.max_len), torch.float32)
            counters = ctx.ws.flat("attn_tickets", ctx.n_single * self.n_heads, torch.int32)
            ops.attention_decode(q, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, o,
                                 self.n_heads, self.scale, window, scratch, counters, ctx.max_len, ctx.status,
                                 ctx.stream, rows=ctx.single_rows)
        if ctx.n_portion:
            if ops.attention_portions_supported(q.dtype, self.head_dim) and ctx.portion_tiles is not None:
                ops.attention_portions(q, ctx.portion_tiles, ctx.n_portion_tiles, cache.block_table, cache.k,
                                       cache.v, o, self.n_heads, self.scale, window, ctx.status, ctx.stream)
            else:
                ops.attention_generic(q, ctx.positions, ctx.token_req, cache.block_table, cache.k, cache.v, o,
                                      self.n_heads, self.scale, window, ctx.status, ctx.stream,
                                      rows=ctx.portion_rows)


register_part("mixer", "attention", Attention)
