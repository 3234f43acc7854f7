#!/usr/bin/env python3
"""Times the plain implementation on the two tiny workloads (CPU seconds): A = prompts of 7 and 13 tokens with
16 greedy tokens each (seed 0); B = prompts of 5, 31 and 64 tokens with 24 tokens each (seed 1; greedy here, the
plain implementation has no sampler).  Every new token re-runs the whole sequence: no cache."""
import os
import sys
import tempfile
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import plain_gpt2 as plain  # noqa: E402
from helpers import CONFIG_A, CONFIG_B, make_model_dir, random_tokens  # noqa: E402

for name, cfg, seed, lens, n_new in (("A", CONFIG_A, 0, (7, 13), 16), ("B", CONFIG_B, 1, (5, 31, 64), 24)):
    with tempfile.TemporaryDirectory() as d:
        w = make_model_dir(d, cfg, seed)
    prompts = [random_tokens(n, cfg["vocab_size"], seed * 10 + i) for i, n in enumerate(lens)]
    t0 = time.perf_counter()
    for p in prompts:
        plain.greedy_generate(p, n_new, w, cfg)
    dt = time.perf_counter() - t0
    print(f"tiny {name}: {len(prompts)} prompts x {n_new} tokens in {dt:.3f} s ({torch.get_num_threads()} threads)")
