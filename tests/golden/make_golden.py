#!/usr/bin/env python3
"""Anchor of the plain implementation: run mlx-lm's own GPT-2 model code.

MLX cannot be installed on the machines this project is developed on, but
``mlx_lm/models/gpt2.py``, ``base.py`` and ``cache.py`` only touch a handful
of MLX symbols.  This script puts a torch-backed stand-in for exactly those
symbols into ``sys.modules`` (``mlx.core``, ``mlx.nn``, ``mlx.utils``), points
an empty ``mlx_lm`` package stub at a checkout of mlx-lm so that the three
model files are imported *unmodified* from there, builds a tiny random GPT-2,
and stores

* the weights in HF layout (Conv1D ``[in, out]``, with an ``attn.bias``
  buffer that ``Model.sanitize`` has to drop),
* logits of a whole prompt, and
* logits of the same tokens cut into a 9-token portion and single steps
  through mlx-lm's ``KVCache``

in ``tests/golden/gpt2_tiny.safetensors`` / ``gpt2_tiny.json``.

What this anchors is the *composition* in gpt2.py (split order of c_attn,
head layout, position offsets taken from the cache, pre-norm placement,
residual order, 4*n_embd MLP, tied head, sanitize).  LayerNorm, gelu_approx,
Linear and the fused attention are MLX library code; the stand-ins below
restate their documented formulas.

Usage:  python tests/golden/make_golden.py /path/to/mlx-lm
The outputs are committed; tests only read them.
"""

import importlib
import json
import math
import os
import sys
import types

import torch
from safetensors.torch import save_file


class Arr(torch.Tensor):
    """Tensor whose ``transpose(*axes)`` permutes, as an MLX array's does."""

    def transpose(self, *axes):
        if len(axes) == 1 and isinstance(axes[0], (tuple, list)):
            axes = tuple(axes[0])
        if not axes:
            axes = tuple(reversed(range(self.dim())))
        return self.permute(*axes)


def _arr(x):
    return x.as_subclass(Arr) if isinstance(x, torch.Tensor) else torch.as_tensor(x).as_subclass(Arr)


def install_stand_in(ref_root: str):
    mx = types.ModuleType("mlx.core")
    mx.array = lambda x=0, dtype=None: _arr(torch.as_tensor(x))
    mx.arange = lambda *a, **k: _arr(torch.arange(*a))
    mx.zeros = lambda shape, dtype=None: _arr(torch.zeros(tuple(shape), dtype=dtype or torch.float32))
    mx.concatenate = lambda xs, axis=0: _arr(torch.cat(list(xs), dim=axis))
    mx.split = lambda x, n, axis=0: [_arr(t) for t in torch.chunk(x, n, dim=axis)]
    mx.float32 = torch.float32
    mx.bool_ = torch.bool

    def sdpa(q, k, v, scale, mask=None, sinks=None):
        # documented semantics of mx.fast.scaled_dot_product_attention:
        # softmax(scale * q k^T + mask) v, "causal" aligning the last query
        # with the last key.
        s = (q @ k.permute(0, 1, 3, 2)) * scale
        if isinstance(mask, str):
            qL, kL = s.shape[-2:]
            qi = torch.arange(kL - qL, kL)[:, None]
            ki = torch.arange(kL)[None]
            s = s.masked_fill(~(qi >= ki), float("-inf"))
        elif mask is not None:
            s = s.masked_fill(~mask, float("-inf")) if mask.dtype == torch.bool else s + mask
        return _arr(torch.softmax(s, dim=-1) @ v)

    fast = types.ModuleType("mlx.core.fast")
    fast.scaled_dot_product_attention = sdpa
    mx.fast = fast

    nn = types.ModuleType("mlx.nn")

    class Module:
        def __init__(self):
            pass

    class Linear(Module):
        def __init__(self, i, o, bias=True):
            self.weight = _arr(torch.zeros(o, i))
            self.bias = _arr(torch.zeros(o)) if bias else None

        def __call__(self, x):
            y = x @ self.weight.permute(1, 0)
            return _arr(y + self.bias if self.bias is not None else y)

    class Embedding(Module):
        def __init__(self, n, d):
            self.weight = _arr(torch.zeros(n, d))

        def __call__(self, ids):
            return _arr(self.weight[ids])

        def as_linear(self, x):
            return _arr(x @ self.weight.permute(1, 0))

    class LayerNorm(Module):
        def __init__(self, d, eps=1e-5):
            self.weight = _arr(torch.ones(d))
            self.bias = _arr(torch.zeros(d))
            self.eps = eps

        def __call__(self, x):
            m = x.mean(-1, keepdim=True)
            v = ((x - m) ** 2).mean(-1, keepdim=True)
            return _arr((x - m) * torch.rsqrt(v + self.eps) * self.weight + self.bias)

    def gelu_approx(x):
        return _arr(0.5 * x * (1 + torch.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * x ** 3))))

    nn.Module, nn.Linear, nn.Embedding, nn.LayerNorm, nn.gelu_approx = Module, Linear, Embedding, LayerNorm, gelu_approx

    utils = types.ModuleType("mlx.utils")
    for n in ("tree_flatten", "tree_map", "tree_reduce", "tree_unflatten"):
        setattr(utils, n, lambda *a, **k: (_ for _ in ()).throw(NotImplementedError(n)))

    mlx = types.ModuleType("mlx")
    mlx.core, mlx.nn, mlx.utils = mx, nn, utils
    sys.modules.update({"mlx": mlx, "mlx.core": mx, "mlx.core.fast": fast, "mlx.nn": nn, "mlx.utils": utils})

    pkg = types.ModuleType("mlx_lm")
    pkg.__path__ = [os.path.join(ref_root, "mlx_lm")]
    sys.modules["mlx_lm"] = pkg
    models = types.ModuleType("mlx_lm.models")
    models.__path__ = [os.path.join(ref_root, "mlx_lm", "models")]
    sys.modules["mlx_lm.models"] = models


CFG = dict(model_type="gpt2", n_ctx=64, n_embd=48, n_head=3, n_layer=2, n_positions=64,
           layer_norm_epsilon=1e-5, vocab_size=257)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <checkout of ml-explore/mlx-lm>")
    ref_root = sys.argv[1]
    install_stand_in(ref_root)
    gpt2 = importlib.import_module("mlx_lm.models.gpt2")
    cache_mod = importlib.import_module("mlx_lm.models.cache")

    g = torch.Generator().manual_seed(1234)
    D, H, L, V, P = CFG["n_embd"], CFG["n_head"], CFG["n_layer"], CFG["vocab_size"], CFG["n_positions"]
    rnd = lambda *s, std=0.05, mean=0.0: torch.randn(*s, generator=g) * std + mean
    hf = {"wte.weight": rnd(V, D), "wpe.weight": rnd(P, D),
          "ln_f.weight": rnd(D, std=0.1, mean=1.0), "ln_f.bias": rnd(D)}
    for i in range(L):
        p = f"h.{i}."
        hf[p + "ln_1.weight"] = rnd(D, std=0.1, mean=1.0)
        hf[p + "ln_1.bias"] = rnd(D)
        hf[p + "ln_2.weight"] = rnd(D, std=0.1, mean=1.0)
        hf[p + "ln_2.bias"] = rnd(D)
        hf[p + "attn.c_attn.weight"] = rnd(D, 3 * D)
        hf[p + "attn.c_attn.bias"] = rnd(3 * D)
        hf[p + "attn.c_proj.weight"] = rnd(D, D)
        hf[p + "attn.c_proj.bias"] = rnd(D)
        hf[p + "mlp.c_fc.weight"] = rnd(D, 4 * D)
        hf[p + "mlp.c_fc.bias"] = rnd(4 * D)
        hf[p + "mlp.c_proj.weight"] = rnd(4 * D, D)
        hf[p + "mlp.c_proj.bias"] = rnd(D)
        hf[p + "attn.bias"] = torch.tril(torch.ones(P, P)).reshape(1, 1, P, P)

    model = gpt2.Model(gpt2.ModelArgs.from_dict(dict(CFG, unknown_key=1)))
    sane = model.sanitize({k: _arr(v.clone()) for k, v in hf.items()})
    assert not any(k.endswith(".attn.bias") for k in sane), "sanitize must drop the mask buffer"
    assert all(k.startswith("model.") for k in sane)
    for name, t in sane.items():
        obj = model
        parts = name.split(".")
        for a in parts[:-1]:
            obj = obj[int(a)] if a.isdigit() else getattr(obj, a)
        assert tuple(getattr(obj, parts[-1]).shape) == tuple(t.shape), (name, t.shape)
        setattr(obj, parts[-1], _arr(t.contiguous()))

    tokens = torch.randint(0, V, (23,), generator=g)
    whole = model(_arr(tokens[None]))[0]

    cache = [cache_mod.KVCache() for _ in model.layers]
    rows = [model(_arr(tokens[None, :9]), cache=cache)[0]]
    for t in range(9, len(tokens)):
        rows.append(model(_arr(tokens[None, t:t + 1]), cache=cache)[0])
    stepped = torch.cat(rows, dim=0)
    diff = float((whole - stepped).abs().max())
    print(f"logits {tuple(whole.shape)}; whole vs 9 + single steps through KVCache: max abs diff {diff:.3e}")

    here = os.path.dirname(os.path.abspath(__file__))
    out = {k: v.contiguous() for k, v in hf.items()}
    out["golden.logits_whole"] = torch.Tensor(whole).contiguous()
    out["golden.logits_stepped"] = torch.Tensor(stepped).contiguous()
    save_file(out, os.path.join(here, "gpt2_tiny.safetensors"))
    with open(os.path.join(here, "gpt2_tiny.json"), "w") as f:
        json.dump({"config": CFG, "tokens": tokens.tolist(), "whole_vs_stepped_max_abs": diff,
                   "made_by": "tests/golden/make_golden.py over mlx_lm/models/{gpt2,base,cache}.py (v0.32.0)"}, f, indent=1)


if __name__ == "__main__":
    main()
