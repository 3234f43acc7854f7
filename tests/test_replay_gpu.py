"""bin/trace_run against the plain implementation: each request alone and whole; most of it in
one step and the last 32 tokens one by one; in portions of changing size down to two tokens and
one; and mixed, up to four live requests with portions of some beside single tokens of others,
in a pool so small that pages are used again.  In float32 and in bfloat16, for both tiny
configurations and for a variant with sharp attention."""
import os

import numpy as np
import pytest
import torch

import plain_gpt2 as plain
from helpers import (CONFIG_A, CONFIG_B, CONFIG_C, Trace, make_model_dir, max_live_tokens, mixed_schedule, random_tokens,
                     run_trace)

pytestmark = pytest.mark.gpu

# Largest |difference| allowed, as a fraction of max(1, largest |reference logit| of the row).  float32: the
# worst case measured on a B200 is 1.3e-6.  bfloat16: per case, about twice the worst difference measured there
# (A 3.6e-3, A-sharp 4.4e-3, B 5.6e-3, B-sharp 1.5e-2, C 5.7e-3, C-sharp 1.7e-2; the test prints them): sharp
# attention turns the rounding of the scores into larger differences, so those cases have a limit of their own.
# A request reading one wrong page moves the logits of A by 0.035 or more
# (tests/test_engine_gpu.py::test_a_wrong_page_is_seen).
TOL_F32 = 5e-6

CASES = {   # configuration, seed, sharpness of attention, request lengths, bfloat16 limit
    "A": (CONFIG_A, 0, 0.0, [23, 29, 100, 128, 65], 7.5e-3),
    "A-sharp": (CONFIG_A, 3, 12.0, [128, 61, 97], 9e-3),
    "B": (CONFIG_B, 1, 0.0, [29, 55, 88, 200, 256], 1.2e-2),
    "B-sharp": (CONFIG_B, 2, 12.0, [88, 256, 130], 3e-2),
    # heads of 64: lengths that cross the 128-key blocks and the 128-query tiles of the tcgen05 attention kernel
    "C": (CONFIG_C, 4, 0.0, [130, 257, 300, 512], 1.2e-2),
    "C-sharp": (CONFIG_C, 5, 8.0, [512, 129, 384], 3e-2),
}


def build_trace(lengths, vocab, seed):
    reqs = {f"r{i}": random_tokens(n, vocab, 100 * seed + i) for i, n in enumerate(lengths)}
    tr = Trace()
    for name, toks in reqs.items():
        tr.whole(f"{name}:whole", toks)
    for name, toks in reqs.items():
        tr.bulk_then_single(f"{name}:tail", toks, tail=32)
    long = max(len(t) for t in reqs.values()) > 256
    for name, toks in reqs.items():
        if long:     # also portions of more than one query tile, and one that ends on a tile's edge
            tr.portions(f"{name}:portions", toks, sizes=(7, 2, 16, 3, 5, 2, 130, 33, 2, 1, 17, 200, 39))
        else:
            tr.portions(f"{name}:portions", toks)
    mixed_schedule(tr, [(f"{name}:mixed", toks) for name, toks in reqs.items()], seed=seed)
    mixed_schedule(tr, [(f"{name}:mixed2", toks) for name, toks in reversed(list(reqs.items()))], seed=seed + 7,
                   sizes=(2, 1, 1, 1, 16, 1, 1, 48, 1, 2, 1, 1, 1, 9) if not long else
                   (2, 1, 130, 1, 16, 1, 1, 257, 1, 2, 65, 1, 1, 128, 9))
    return reqs, tr


@pytest.mark.parametrize("case", list(CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_matches_plain(case, dtype, tmp_path):
    replay_and_compare(case, dtype, tmp_path, page_size=16)


@pytest.mark.parametrize("case,page_size", [("C-sharp", 8), ("A-sharp", 32), ("C", 32), ("B", 64)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_with_other_page_sizes(case, page_size, dtype, tmp_path):
    """The same cuttings with pages of 8, 32 and 64 tokens: page edges fall elsewhere in every kernel that
    walks a block table (the cache write in the projections' epilogues, the three attention kernels)."""
    replay_and_compare(case, dtype, tmp_path, page_size=page_size)


@pytest.mark.parametrize("case", ["C-sharp", "A", "B-sharp"])
def test_replay_with_single_token_rows_on_tensor_cores(case, tmp_path):
    """Steps of few rows send their single-token rows to the split-key kernel on the CUDA cores; only steps of
    very many rows use the tensor-core kernel for them.  Here it is made to take every single-token row
    (MLXB_ROWS_MIN_PAIRS=0), so that the cuttings, page reuse included, run through it too."""
    replay_and_compare(case, "bfloat16", tmp_path, page_size=16, env={"MLXB_ROWS_MIN_PAIRS": "0"})


def replay_and_compare(case, dtype, tmp_path, page_size, env=None):
    config, seed, sharp, lengths, tol_bf16 = CASES[case]
    limit = TOL_F32 if dtype == "float32" else tol_bf16
    weights = make_model_dir(str(tmp_path / "model"), config, seed, peaky=sharp)
    reqs, tr = build_trace(lengths, config["vocab_size"], seed)
    # the pool holds exactly what the busiest moment needs, so freed pages are taken again
    got = run_trace(str(tmp_path / "model"), tr, dtype, str(tmp_path / "out"), max_tokens=max_live_tokens(tr),
                    extra=["--page-size", str(page_size)], env=env)
    ref = {name: plain.logits(toks, weights, config).numpy() for name, toks in reqs.items()}
    worst, worst_key = 0.0, None
    n_rows = 0
    for (rid, pos), row in got.items():
        name = rid.split(":")[0]
        r = ref[name][pos]
        err = float(np.abs(row - r).max()) / max(1.0, float(np.abs(r).max()))
        n_rows += 1
        if err > worst:
            worst, worst_key = err, (rid, pos)
    # every position of every request in every cutting was written
    assert n_rows == 5 * sum(lengths)  # whole, tail, portions, mixed, mixed2
    biggest = max(float(np.abs(r).max()) for r in ref.values())
    print(f"{case} {dtype} pages of {page_size}: worst relative difference {worst:.3e} at {worst_key} over {n_rows} rows "
          f"(largest |logit| {biggest:.2f})")
    assert worst <= limit, f"worst at {worst_key}: {worst}"
    # the same position gives the same logits however it was cut (tighter than against the reference)
    cut_tol = limit * 0.5
    for name, toks in reqs.items():
        for pos in range(len(toks)):
            base = got[(f"{name}:whole", pos)]
            scale = max(1.0, float(np.abs(base).max()))
            for cut in ("tail", "portions", "mixed", "mixed2"):
                d = float(np.abs(got[(f"{name}:{cut}", pos)] - base).max()) / scale
                assert d <= cut_tol, f"{name} position {pos}: {cut} differs from whole by {d}"
