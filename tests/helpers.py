"""Shared by the tests: the two tiny configurations, model folders with seeded
random weights, and a driver for ``bin/trace_run`` that builds the step
files for the usual ways of cutting requests into steps."""
import json
import os
import subprocess
import sys

import numpy as np
import torch
from safetensors.torch import load_file, save_file

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# Two configurations that differ in every size and option.
CONFIG_A = dict(model_type="gpt2", n_layer=2, n_embd=64, n_head=4, n_inner=None, vocab_size=512, n_positions=128,
                layer_norm_epsilon=1e-5, activation_function="gelu_new")
CONFIG_B = dict(model_type="gpt2", n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000, n_positions=256,
                layer_norm_epsilon=1e-6, activation_function="gelu_new", ln_gain_std=0.1)


# A third configuration: heads of 64 (the head size of the benchmarked models, which alone runs the tcgen05
# attention kernel for portions), two heads, sizes that differ from A and B.
CONFIG_C = dict(model_type="gpt2", n_layer=2, n_embd=128, n_head=2, n_inner=384, vocab_size=640, n_positions=512,
                layer_norm_epsilon=3e-6, activation_function="gelu_new", ln_gain_std=0.2)

# The layer sizes of GPT-2 medium (width 1024, 16 heads of 64, inner width 4096, vocabulary 50257, 1024
# positions) with two of its 24 layers: the shapes of the benchmark's launches at a cost of seconds on the CPU.
MEDIUM_2_LAYERS = dict(model_type="gpt2", n_layer=2, n_embd=1024, n_head=16, n_inner=4096, vocab_size=50257,
                       n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new", ln_gain_std=0.1)


def make_model_dir(path, config, seed, peaky=0.0, dtype="bfloat16"):
    """Write a random model folder; ``peaky`` > 0 multiplies the query and key columns of every
    c_attn weight so that attention is sharp and a wrong or missing key changes the logits visibly."""
    from mlx_lm_b200.weights import write_random_model

    write_random_model(path, dict(config), seed, dtype=dtype)
    file = os.path.join(path, "model.safetensors")
    if peaky:
        w = load_file(file)
        D = config["n_embd"]
        for k in list(w):
            if k.endswith("attn.c_attn.weight"):
                t = w[k].float()
                t[:, :2 * D] *= peaky
                w[k] = t.to(w[k].dtype)
        save_file(w, file)
    return load_file(file)


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class Trace:
    """Collects steps; remembers which (request, position) each written row belongs to."""

    def __init__(self):
        self.steps = []
        self.rows = []   # per step: list of (rid, position)
        self._len = {}

    def step(self, entries, end=()):
        """entries: list of (rid, tokens, want) with want = indices into tokens or 'all' / 'last' / 'none'."""
        rec, rows = [], []
        for rid, tokens, want in entries:
            n = len(tokens)
            if want == "all":
                want = list(range(n))
            elif want == "last":
                want = [n - 1]
            elif want == "none":
                want = []
            start = self._len.get(rid, 0)
            rows.extend((rid, start + w) for w in want)
            self._len[rid] = start + n
            rec.append({"id": rid, "tokens": list(map(int, tokens)), "want": list(want)})
        self.steps.append({"step": len(self.steps), "entries": rec, "end": list(end)})
        self.rows.append(rows)
        for rid in end:
            self._len.pop(rid, None)

    # ---- the usual cuttings -------------------------------------------------
    def whole(self, rid, tokens):
        self.step([(rid, tokens, "all")], end=[rid])

    def bulk_then_single(self, rid, tokens, tail=32):
        n = len(tokens)
        head = max(n - tail, 1)
        self.step([(rid, tokens[:head], "all")])
        for t in range(head, n):
            self.step([(rid, tokens[t:t + 1], "all")], end=[rid] if t == n - 1 else [])
        if head == n:
            self.steps[-1]["end"] = [rid]

    def portions(self, rid, tokens, sizes=(7, 2, 16, 3, 5, 2, 33, 2, 1, 17)):
        t, i, n = 0, 0, len(tokens)
        while t < n:
            m = min(sizes[i % len(sizes)], n - t)
            self.step([(rid, tokens[t:t + m], "all")], end=[rid] if t + m == n else [])
            t += m
            i += 1


def mixed_schedule(trace, requests, seed=0, max_live=4, sizes=(1, 1, 5, 2, 1, 19, 1, 3, 1, 34, 2, 1)):
    """Up to ``max_live`` requests at a time: each step takes a portion of some and single tokens of
    others; requests start staggered and end at different times.  ``requests``: list of (rid, tokens)."""
    rng = np.random.RandomState(seed)
    waiting = list(requests)
    live = {}   # rid -> (tokens, done)
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.rand() < 0.6):
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0]
        entries, end = [], []
        for rid in list(live):
            toks, done = live[rid]
            if len(live) > 1 and rng.rand() < 0.25:
                continue   # this request sits the step out
            m = min(sizes[k % len(sizes)], len(toks) - done)
            k += 1
            entries.append((rid, toks[done:done + m], "all"))
            live[rid][1] = done + m
            if done + m == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            trace.step(entries, end=end)


def max_live_tokens(trace, round_to=64):
    """What --max-tokens must be at least: the most tokens live at once, per request rounded up."""
    live, worst = {}, 0
    for s in trace.steps:
        for e in s["entries"]:
            live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum((v + round_to - 1) // round_to * round_to for v in live.values()))
        for rid in s["end"]:
            live.pop(rid, None)
    return worst


def run_trace(model_dir, trace, dtype, out_dir, max_tokens=None, extra=(), timeout=600, env=None):
    """Run bin/trace_run over the trace; returns {(rid, position): float32 row}."""
    os.makedirs(out_dir, exist_ok=True)
    if max_tokens is None:
        max_tokens = max_live_tokens(trace)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens",
           str(max_tokens), *extra]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True,
                            env=dict(os.environ, **env) if env else None)
    try:
        for s in trace.steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"trace_run answered {line!r} to step {s['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    cfg = json.load(open(os.path.join(model_dir, "config.json")))
    V = cfg["vocab_size"]
    got = {}
    for s, rows in zip(trace.steps, trace.rows):
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if not rows:
            assert not os.path.exists(path)
            continue
        a = np.fromfile(path, dtype="<f4").reshape(len(rows), V)
        for key, row in zip(rows, a):
            assert key not in got, f"{key} written twice"
            got[key] = row
    return got
