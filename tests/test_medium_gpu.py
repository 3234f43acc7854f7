"""The engine at the layer sizes the benchmark runs (GPT-2 medium: width 1024, 16 heads of 64, inner width 4096,
vocabulary 50257) with two layers instead of 24, against the plain implementation on the CPU: a mixed schedule
of six requests of 100 to 600 tokens in a pool so small that pages are used again, and decoding as CUDA graphs
at batch 8 and batch 64 over page edges.  These are the launches whose time the benchmark reports (the few-rows
linear kernels at 8 and 64 rows, single-token attention with 256- and 512-thread CTAs, the tcgen05 linear and
attention kernels for portions, the output head at 33 to 64 rows), none of which the tiny configurations reach.
mlx-lm holds batched generation to its single-request results in the same way
(tests/test_generate.py:182-265)."""
import numpy as np
import pytest
import torch

import plain_gpt2 as plain
from helpers import MEDIUM_2_LAYERS, Trace, make_model_dir, max_live_tokens, mixed_schedule, random_tokens

pytestmark = pytest.mark.gpu

CFG = MEDIUM_2_LAYERS
V = CFG["vocab_size"]
# Largest |difference| allowed as a fraction of max(1, largest |reference logit| of the row): about twice the
# worst measured on a B200 (float32 1.1e-5, bfloat16 1.3e-2; the tests print them).  Attention is sharpened by
# a factor of 2: enough that a wrong page shows (the last test), and the rounding of the scores is not yet
# amplified (at a factor of 4 bfloat16 differs by 4e-2).
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}
PEAKY = 2.0


@pytest.fixture(scope="module")
def medium(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("medium2"))
    weights = make_model_dir(d, CFG, 17, peaky=PEAKY)
    w32 = {k: v.float() for k, v in weights.items()}
    return d, w32


def reference_rows(w32, tokens, positions):
    """Plain logits of one sequence at the given positions only (the head is the expensive part)."""
    h = plain.hidden_states(tokens, w32, CFG)
    return h[torch.tensor(positions)] @ w32["wte.weight"].T


def rel_rows(got, ref):
    got, ref = got.float().cpu(), ref.float()
    return float(((got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1).clamp(min=1.0)).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_schedule_at_the_benchmarked_layer_sizes(dtype, medium):
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.weights import load_model
    d, w32 = medium
    lens = [100, 600, 257, 385, 130, 512]
    reqs = [(f"r{i}", random_tokens(n, V, 40 + i)) for i, n in enumerate(lens)]
    tr = Trace()
    mixed_schedule(tr, reqs, seed=3, sizes=(1, 1, 130, 2, 1, 257, 1, 64, 1, 300, 17, 1, 128, 1, 40))
    n_pages = max_live_tokens(tr, round_to=16) // 16         # what the busiest moment needs, so pages are used again
    model, _ = load_model(d, dtype=dtype)
    eng = Engine(model, page_size=16, n_pages=n_pages, max_requests=4)
    done = {rid: 0 for rid, _ in reqs}
    wanted = {rid: [] for rid, _ in reqs}        # (position, row of logits)
    for s in tr.steps:
        entries, where = [], []
        for e in s["entries"]:
            rid, n = e["id"], len(e["tokens"])
            if not eng.has_request(rid):
                eng.add_request(rid)
            start = done[rid]
            # the first and the last token of the entry, and the rows on either side of a 128-position edge
            want = sorted({0, n - 1} | {i for i in range(n) if (start + i) % 128 in (0, 127)})
            entries.append(StepEntry(rid, e["tokens"], want))
            where.extend((rid, start + i) for i in want)
            done[rid] = start + n
        lg = eng.step(entries).float().cpu()
        for (rid, pos), row in zip(where, lg):
            wanted[rid].append((pos, row))
        for rid in s["end"]:
            eng.finish(rid)
    eng.check_status()
    assert eng.cache.pages_in_use() == [0] and eng.cache.high_water() == [n_pages]
    worst = 0.0
    for rid, toks in reqs:
        pos = [p for p, _ in wanted[rid]]
        assert pos[-1] == len(toks) - 1 and pos[0] == 0
        worst = max(worst, rel_rows(torch.stack([r for _, r in wanted[rid]]), reference_rows(w32, toks, pos)))
    print(f"medium widths, mixed schedule, {dtype}: worst relative difference {worst:.3e}")
    assert worst <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("batch", [8, 64])
def test_decoding_as_cuda_graphs_at_the_benchmarked_layer_sizes(dtype, batch, medium):
    """40 decode steps of `batch` requests through ``Engine.decode_sampled`` (one CUDA graph per bucket of batch
    sizes), the given sequences fed token by token; the graph's logits against the plain implementation."""
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.engine.scheduler import Request
    from mlx_lm_b200.sampling import GREEDY
    from mlx_lm_b200.sampling.device import DeviceSampler
    from mlx_lm_b200.weights import load_model
    d, w32 = medium
    n_steps = 40
    rng = np.random.RandomState(batch)
    # prompts whose decoding crosses page edges, the 128-position edge and, for a few, position 256
    lens = [int(x) for x in rng.randint(20, 150, size=batch)]
    lens[0], lens[1], lens[2] = 100, 127, 230
    seqs = [random_tokens(n + n_steps, V, 900 + i) for i, n in enumerate(lens)]
    model, _ = load_model(d, dtype=dtype)
    eng = Engine(model, page_size=16, n_pages=sum((len(t) + 15) // 16 for t in seqs), max_requests=batch)
    sampler = DeviceSampler(model.device, seed=0, engine=eng)
    reqs = []
    for i, (n, t) in enumerate(zip(lens, seqs)):
        eng.add_request(i)
        reqs.append(Request(i, list(t[:n + 1]), n + 1, 10 ** 6, GREEDY))
    for i in range(0, batch, 8):       # prompts, eight requests a step
        eng.step([StepEntry(r.uid, seqs[r.uid][:lens[r.uid]], []) for r in reqs[i:i + 8]])
    got = [[] for _ in reqs]
    for s in range(n_steps):
        eng.decode_sampled([StepEntry(r.uid, [r.tokens[-1]], [0]) for r in reqs], reqs, sampler)
        graph = eng._graphs[(batch, False)]
        lg = graph.logits[:batch].float().cpu()
        for i, r in enumerate(reqs):
            got[i].append(lg[i])
            if s + 1 < n_steps:
                r.tokens.append(seqs[i][lens[i] + s + 1])        # the given sequence, not the sampled token
    assert eng.host_status == 0
    eng.check_status()
    if batch == 8:
        # one more step with the first entry of request 0's host block table pointed at its second page: its row
        # must be off by more than the limit (so the limit sees a wrong page at these sizes), the other rows
        # must not move
        pages = eng.cache.requests[0].pages[0]
        first, pages[0] = pages[0], pages[1]
        seqs = [t + random_tokens(1, V, 7) for t in seqs]
        for i, r in enumerate(reqs):
            r.tokens.append(seqs[i][-1])
        eng.decode_sampled([StepEntry(r.uid, [r.tokens[-1]], [0]) for r in reqs], reqs, sampler)
        off = eng._graphs[(batch, False)].logits[:batch].float().cpu()
        ref_last = torch.stack([plain.hidden_states(t, w32, CFG)[-1] for t in seqs]) @ w32["wte.weight"].T
        assert rel_rows(off[:1], ref_last[:1]) > 1.5 * TOL[dtype], "a wrong page is not seen"
        assert rel_rows(off[1:], ref_last[1:]) <= TOL[dtype]
        seqs = [t[:-1] for t in seqs]
        pages[0] = first
    hidden = [plain.hidden_states(t, w32, CFG)[n:n + n_steps] for n, t in zip(lens, seqs)]
    ref = torch.cat(hidden) @ w32["wte.weight"].T
    worst = rel_rows(torch.cat([torch.stack(g) for g in got]), ref)
    print(f"medium widths, decode graphs at batch {batch}, {dtype}: worst relative difference {worst:.3e} largest |logit| {float(ref.abs().max()):.2f}")
    assert worst <= TOL[dtype]
