"""The plain implementation against mlx-lm's own gpt2.py (stored outputs of
tests/golden/make_golden.py) and against itself (whole vs. prefix)."""
import json
import os

import torch
from safetensors.torch import load_file

import plain_gpt2 as plain

HERE = os.path.dirname(os.path.abspath(__file__))


def _golden():
    t = load_file(os.path.join(HERE, "golden", "gpt2_tiny.safetensors"))
    meta = json.load(open(os.path.join(HERE, "golden", "gpt2_tiny.json")))
    weights = {k: v for k, v in t.items() if not k.startswith("golden.")}
    return weights, meta, t["golden.logits_whole"], t["golden.logits_stepped"]


def test_plain_matches_reference_model_code():
    weights, meta, whole, stepped = _golden()
    got = plain.logits(meta["tokens"], weights, meta["config"])
    assert got.shape == whole.shape
    assert float((got - whole).abs().max()) < 2e-5
    assert float((got - stepped).abs().max()) < 2e-5
    # float64 tells rounding from a wrong formula
    got64 = plain.logits(meta["tokens"], weights, meta["config"], dtype=torch.float64)
    assert float((got64 - whole.double()).abs().max()) < 2e-5


def test_plain_is_causal():
    weights, meta, _, _ = _golden()
    toks = meta["tokens"]
    a = plain.logits(toks, weights, meta["config"])
    b = plain.logits(toks[:11], weights, meta["config"])
    assert float((a[:11] - b).abs().max()) < 1e-5


def test_parts():
    x = torch.randn(5, 12)
    g, b = torch.randn(12), torch.randn(12)
    ref = torch.nn.functional.layer_norm(x, (12,), g, b, 1e-6)
    assert torch.allclose(plain.layer_norm(x, g, b, 1e-6), ref, atol=1e-6)
    ref = torch.nn.functional.gelu(x, approximate="tanh")
    assert torch.allclose(plain.gelu_new(x), ref, atol=1e-6)
    q, k, v = (torch.randn(2, 7, 4) for _ in range(3))
    o = plain.causal_attention(q, k, v, window=3)
    # position 6 with window 3 sees keys 4, 5, 6 only
    s = (q[:, 6:7] @ k[:, 4:7].transpose(1, 2)) * 4 ** -0.5
    ref = (torch.softmax(s, -1) @ v[:, 4:7]).permute(1, 0, 2).reshape(1, 8)
    assert torch.allclose(o[6:7], ref, atol=1e-6)
    assert plain.inner_width({"n_embd": 8}) == 32 and plain.inner_width({"n_embd": 8, "n_inner": 20}) == 20
