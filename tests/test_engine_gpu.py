"""The engine in-process on the GPU: parts alone, long decoding, the first tokens of a sequence,
generation through the entry points, and a toy mixer with state of its own that is registered,
built and stepped from this file alone."""
import math
import os
from dataclasses import dataclass
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import kernel_refs as R
import plain_gpt2 as plain
from helpers import CONFIG_A, CONFIG_B, CONFIG_C, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
# Largest |difference| allowed as a fraction of max(1, largest |reference logit|): about twice the worst measured
# on a B200 with the tiny configurations (float32 5e-7, bfloat16 5.6e-3; run with -s to see them) ...
TOL = {"float32": 5e-6, "bfloat16": 1.2e-2}
# ... and at the widths of the larger models (float32 7.5e-6, bfloat16 1.3e-2: more terms per sum)
TOL_WIDE = {"float32": 2e-5, "bfloat16": 2.5e-2}


SEEN = []      # every relative difference a test computed; its largest is printed after the test (pytest -s)


def rel(got, ref):
    ref = torch.as_tensor(ref).float().cpu()
    r = float((torch.as_tensor(got).float().cpu() - ref).abs().max()) / max(1.0, float(ref.abs().max()))
    SEEN.append(r)
    return r


@pytest.fixture(autouse=True)
def report_largest_difference(request):
    SEEN.clear()
    yield
    if SEEN:
        print(f"\n{request.node.name}: largest relative difference {max(SEEN):.3e}")


def part_ctx(T=0, positions=None, token_req=None):
    from mlx_lm_b200 import ops
    from mlx_lm_b200.engine import Workspace
    return SimpleNamespace(ws=Workspace("cuda"), stream=ops.current_stream(), n_tokens=T,
                           status=torch.zeros(1, dtype=torch.int32, device="cuda"),
                           positions=positions, token_req=token_req, tokens=None, max_len=64,
                           n_single=T if T == 1 else 0, n_portion=0 if T == 1 else T, single_rows=None,
                           portion_rows=None, portion_tiles=None, n_portion_tiles=0)


def bind(part, dtype, seed=0):
    """Random tensors for a part's own specs, placed as the loader places them."""
    from mlx_lm_b200.weights.loader import place
    g = torch.Generator().manual_seed(seed)
    host, dev = {}, {}
    for s in part.all_param_specs():
        t = (torch.randn(s.shape, generator=g) * 0.3 + (1.0 if s.name.endswith("ln.weight") else 0.0))
        t = t.to(torch.bfloat16).float()       # representable in both dtypes
        host[s.name] = t
        dev[s.name] = place(s, t, dtype, "cuda")
    part.bind_all(dev, dtype, "cuda")
    return host


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parts_alone(dtype):
    from mlx_lm_b200.engine import LayerCacheView
    from mlx_lm_b200.parts import MLP, Attention, LayerNorm, Linear, PreNormBlock
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    g = torch.Generator().manual_seed(1)
    T, D = 37, 80
    x = torch.randn(T, D, generator=g).to(torch.bfloat16).float()
    xd = x.to(dtype).cuda()
    ctx = part_ctx(T)

    lin = Linear("p", D, 56, bias=True, stored="in_out")
    w = bind(lin, dtype)
    out = torch.empty(T, 56, dtype=dtype, device="cuda")
    lin.forward(ctx, xd, out, activation="gelu_new")
    assert rel(out, plain.gelu_new(plain.conv1d_linear(x, w["p.weight"], w["p.bias"]))) <= tol

    ln = LayerNorm("ln", D, 1e-3)
    w = bind(ln, dtype)
    assert rel(ln.forward(ctx, xd), plain.layer_norm(x, w["ln.weight"], w["ln.bias"], 1e-3)) <= tol

    mlp = MLP("m", D, 136, stored="in_out")
    w = bind(mlp, dtype)
    res = xd.clone()
    y = mlp.forward(ctx, xd, res)
    assert rel(y, x + plain.mlp_part(x, {"c_fc.weight": w["m.c_fc.weight"], "c_fc.bias": w["m.c_fc.bias"],
                                         "c_proj.weight": w["m.c_proj.weight"], "c_proj.bias": w["m.c_proj.bias"]},
                                     "")) <= tol

    # attention over pages: two requests, the second continuing at position 21 of a longer one
    H, Dh, page = 5, 16, 16
    att = Attention("a", D, H, Dh, stored="in_out")
    w = bind(att, dtype, seed=3)
    wd = {k[2:]: v for k, v in w.items()}
    positions = torch.arange(T, dtype=torch.int32).cuda()
    token_req = torch.zeros(T, dtype=torch.int32).cuda()
    bt = torch.tensor([[3, 0, 2, 1]], dtype=torch.int32).cuda()
    cache = LayerCacheView("kv", True, k=torch.zeros(4, H, page, Dh, dtype=dtype, device="cuda"),
                           v=torch.zeros(4, H, page, Dh, dtype=dtype, device="cuda"), block_table=bt, page_size=page)
    ctx = part_ctx(T, positions, token_req)
    res = xd.clone()
    y = att.forward(ctx, xd, res, cache)
    assert rel(y, x + plain.attention_part(x, wd, "", H)) <= tol
    # the same tokens in two steps give the same rows
    cache.k.zero_(); cache.v.zero_()
    ya = att.forward(part_ctx(21, positions[:21], token_req[:21]), xd[:21], xd[:21].clone(), cache).clone()
    yb = att.forward(part_ctx(T - 21, positions[21:], token_req[21:]), xd[21:], xd[21:].clone(), cache)
    assert rel(torch.cat([ya, yb]), y) <= tol
    # and one more token alone takes the single-token path
    x1 = torch.randn(1, D, generator=g).to(torch.bfloat16).float()
    p1 = torch.tensor([T], dtype=torch.int32).cuda()
    y1 = att.forward(part_ctx(1, p1, token_req[:1]), x1.to(dtype).cuda(), x1.to(dtype).cuda().clone(), cache)
    xx = torch.cat([x, x1])
    assert rel(y1, (xx + plain.attention_part(xx, wd, "", H))[T:]) <= tol

    blk = PreNormBlock(LayerNorm("b.ln_1", D, 1e-5), Attention("b.attn", D, H, Dh, stored="in_out"),
                       LayerNorm("b.ln_2", D, 1e-5), MLP("b.mlp", D, 100, stored="in_out"))
    w = bind(blk, dtype, seed=4)
    cache.k.zero_(); cache.v.zero_()
    y = blk.forward(ctx, xd.clone(), cache)
    wd = {"h.0." + k[2:]: v for k, v in w.items()}
    assert rel(y, plain.block(x, wd, 0, {"layer_norm_epsilon": 1e-5, "n_head": H})) <= tol


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("config,seed", [(CONFIG_A, 3), (CONFIG_B, 4)])
def test_long_decoding_and_first_tokens(dtype, config, seed, tmp_path):
    """Every position of the longest sequence the model allows, one token per step."""
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.weights import load_model
    weights = make_model_dir(str(tmp_path), config, seed, peaky=6.0)
    model, _ = load_model(str(tmp_path), dtype=dtype)
    n = config["n_positions"]
    toks = random_tokens(n, config["vocab_size"], seed)
    ref = plain.logits(toks, weights, config)
    eng = Engine(model, page_size=16, n_pages=n // 16, max_requests=1)
    eng.add_request("r")
    worst = 0.0
    for t in range(n):
        lg = eng.step([StepEntry("r", toks[t:t + 1], [0])])
        worst = max(worst, rel(lg[0], ref[t]))
        if t < 3:
            assert rel(lg[0], ref[t]) <= TOL[dtype], f"position {t}"
    eng.check_status()
    assert worst <= TOL[dtype]
    assert eng.n_replayed >= n - 2        # steps of a shape seen before re-issue their recorded launches
    with pytest.raises(ValueError):
        eng.step([StepEntry("r", [0], [0])])          # position n is beyond the table
    eng.finish("r")
    assert eng.cache.pages_in_use() == [0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,heads", [(1600, 25), (1280, 20)])
def test_layer_sizes_of_the_larger_models(dtype, width, heads, tmp_path):
    """One layer at the widths of GPT-2 XL and large (heads of 64, a width that is no multiple of 256, an inner
    width of four times that), small vocabulary: a prompt in one step (the tcgen05 linear and attention kernels,
    row statistics for the folded norms), then portions and single tokens (the few-rows kernels with norms folded
    over 50 or 40 blocks of 32), against the plain implementation."""
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.weights import load_model
    config = dict(CONFIG_A, n_embd=width, n_head=heads, n_layer=1, n_inner=4 * width, vocab_size=777, n_positions=512,
                  ln_gain_std=0.2)
    weights = make_model_dir(str(tmp_path), config, 31, peaky=2.0)
    model, _ = load_model(str(tmp_path), dtype=dtype)
    toks = random_tokens(300, 777, 5)
    ref = plain.logits(toks, weights, config)
    eng = Engine(model, page_size=16, n_pages=64, max_requests=2)
    eng.add_request("a")
    lg = eng.step([StepEntry("a", toks[:200], [0, 127, 128, 199])])
    for row, pos in enumerate([0, 127, 128, 199]):
        assert rel(lg[row], ref[pos]) <= TOL_WIDE[dtype], pos
    lg = eng.step([StepEntry("a", toks[200:260], [59])])          # a portion of 60: few rows
    assert rel(lg[0], ref[259]) <= TOL_WIDE[dtype]
    worst = 0.0
    for t in range(260, 300):                                     # single tokens
        lg = eng.step([StepEntry("a", toks[t:t + 1], [0])])
        worst = max(worst, rel(lg[0], ref[t]))
    assert worst <= TOL_WIDE[dtype], worst
    eng.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_wrong_page_is_seen(dtype, tmp_path):
    """The comparison with the plain implementation must fail when a request reads one wrong page: after a
    prompt is in the cache, the request's first entry in the host block table is pointed at its second page
    (positions 0-15 then read the keys and values of positions 16-31; nothing else changes) and the next tokens
    are decoded.  At configuration A, without sharpened attention, in both precisions: the limits of these
    tests are tight enough to see it.  (Exchanging two pages of one request would show nothing: a decoded
    token attends the same set of keys in another order.)"""
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.weights import load_model
    weights = make_model_dir(str(tmp_path), CONFIG_A, 0)
    model, _ = load_model(str(tmp_path), dtype=dtype)
    toks = random_tokens(80, 512, 7)
    ref = plain.logits(toks, weights, CONFIG_A)
    eng = Engine(model, page_size=16, n_pages=8, max_requests=1)
    eng.add_request("r")
    right = eng.step([StepEntry("r", toks[:64], [40, 63])])
    assert rel(right, ref[[40, 63]]) <= TOL[dtype]
    pages = eng.cache.requests["r"].pages[0]
    first, pages[0] = pages[0], pages[1]
    worst = 0.0
    for t in range(64, 80):
        worst = max(worst, rel(eng.step([StepEntry("r", toks[t:t + 1], [0])])[0], ref[t]))
    assert worst > 1.5 * TOL[dtype], f"a wrong page moved the logits by only {worst}"     # measured: 2.5e-2
    eng.check_status()                                  # every id is a page of the pool: no kernel can tell
    pages[0] = first


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("config", [CONFIG_A, CONFIG_C], ids=["heads of 16", "heads of 64"])
def test_pages_nobody_was_given_keep_their_canaries(dtype, config, tmp_path):
    """Every page of the pools is filled with a canary (NaN) before the first step; pages that are handed out are
    then cleared by the test, as the manager's zero-filled pool would have them.  Requests come and go through
    portions, single tokens, mixed steps and decode graphs, with pages given back and used again.  At the end
    the pages that were never handed out still hold the canary bit for bit (no kernel wrote outside its block
    table), and every logit along the way is finite and right (no kernel read outside it: a NaN would have
    spread, masked or not)."""
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.sampling import GREEDY
    from mlx_lm_b200.sampling.device import DeviceSampler
    from mlx_lm_b200.weights import load_model
    weights = make_model_dir(str(tmp_path), config, 9)
    model, _ = load_model(str(tmp_path), dtype=dtype)
    eng = Engine(model, page_size=16, n_pages=40, max_requests=4)
    group = eng.cache.kv_groups[0]
    for pool in (group.k, group.v):
        pool.fill_(float("nan"))
    cleared = set()

    def clear_new_pages():
        for req in eng.cache.requests.values():
            for pg in req.pages[0]:
                if pg not in cleared:
                    cleared.add(pg)
                    group.k[:, pg].zero_()
                    group.v[:, pg].zero_()

    class Req:
        def __init__(self, uid, tokens):
            self.uid, self.tokens, self.sampler, self.processors = uid, list(tokens), GREEDY, ()

    def step(entries):
        # pages a step will take are handed out inside it: reserve by hand first, so that they can be cleared
        for e in entries:
            eng.cache.reserve(e.rid, len(e.tokens))
        clear_new_pages()
        for e in entries:
            eng.cache.rollback(e.rid)
        return eng.step(entries)

    V = config["vocab_size"]
    seqs = {r: random_tokens(n, V, 40 + i) for i, (r, n) in enumerate([("a", 128), ("b", 37), ("c", 70), ("d", 33)])}
    refs = {r: plain.logits(t, weights, config) for r, t in seqs.items()}
    done = {r: 0 for r in seqs}

    def entry(r, n, want="last"):
        toks = seqs[r][done[r]:done[r] + n]
        done[r] += len(toks)
        return StepEntry(r, toks, [len(toks) - 1] if want == "last" else list(range(len(toks))))

    def check(entries, logits):
        assert bool(torch.isfinite(logits).all())
        row = 0
        for e in entries:
            end = done[e.rid]
            for w in e.want:
                assert rel(logits[row], refs[e.rid][end - len(e.tokens) + w]) <= TOL[dtype]
                row += 1

    for r in ("a", "b"):
        eng.add_request(r)
    es = [entry("a", 100), entry("b", 30, "all")]
    check(es, step(es))
    eng.add_request("c")
    es = [entry("a", 1), entry("b", 7, "all"), entry("c", 40)]      # mixed: a decodes, b ends, c starts
    check(es, step(es))
    eng.finish("b")                                                  # its pages go back ...
    eng.add_request("d")
    es = [entry("d", 33, "all"), entry("a", 2), entry("c", 30)]      # ... and d takes them
    check(es, step(es))
    eng.finish("d")
    eng.finish("c")
    sampler = DeviceSampler(model.device, seed=0, engine=eng)
    req = Req(0, seqs["a"][:done["a"]])                               # (the uid only keys the random draws)
    for _ in range(20):                                              # decode graphs (the tokens are the sequence's own)
        e = StepEntry("a", [seqs["a"][done["a"]]], [0])
        eng.cache.reserve("a", 1)
        clear_new_pages()
        eng.cache.rollback("a")
        eng.decode_sampled([e], [req], sampler)
        done["a"] += 1
        req.tokens.append(seqs["a"][done["a"] - 1])
    es = [entry("a", 5, "all")]
    check(es, step(es))
    eng.finish("a")
    eng.check_status()
    used = eng.cache.kv_groups[0].pool.high_water
    assert used < 40 and cleared == set(range(used))               # page ids are handed out from 0 up, freed ones first
    for pool in (group.k, group.v):
        rest = pool[:, used:]
        assert bool(torch.isnan(rest).all()), "a page that no request was given has been written"
    assert eng.cache.pages_in_use() == [0]


def test_status_bits_become_errors_and_are_cleared(tmp_path):
    """What a kernel reports in the status word (here written by the test: a bounded wait that gave up, a page
    id outside the pool) is raised by ``check_status`` in words and cleared, and the engine goes on."""
    from mlx_lm_b200 import ops
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.weights import load_model
    make_model_dir(str(tmp_path), CONFIG_A, 0)
    model, _ = load_model(str(tmp_path), dtype="bfloat16")
    eng = Engine(model, page_size=16, n_pages=4, max_requests=1)
    eng.status.fill_(ops.ST_WAIT_TIMEOUT | ops.ST_PAGE_RANGE)
    with pytest.raises(ops.KernelError) as err:
        eng.check_status()
    assert "bounded wait" in str(err.value) and "page id outside the pool" in str(err.value)
    assert eng.read_status() == 0 and eng.host_status == 0
    eng.add_request(0)
    assert eng.step([StepEntry(0, [1, 2, 3], [2])]).shape == (1, 512)
    eng.check_status()


def test_step_refuses_bad_input(tmp_path):
    from mlx_lm_b200.cache import OutOfPages
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.weights import load_model
    make_model_dir(str(tmp_path), CONFIG_A, 0)
    model, _ = load_model(str(tmp_path), dtype="float32")
    eng = Engine(model, page_size=16, n_pages=2, max_requests=2)
    eng.add_request(1)
    with pytest.raises(ValueError):
        eng.step([StepEntry(1, [512], [0])])
    with pytest.raises(ValueError):
        eng.step([StepEntry(1, [1, 2], [2])])
    with pytest.raises(KeyError):
        eng.step([StepEntry(2, [1], [0])])
    with pytest.raises(ValueError):
        eng.step([StepEntry(1, [1], [0]), StepEntry(1, [2], [0])])
    with pytest.raises(OutOfPages):
        eng.step([StepEntry(1, list(range(33)), [0])])
    assert eng.cache.pages_in_use() == [0]
    assert eng.step([StepEntry(1, [1, 2, 3], [])]) is None


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_points(dtype, tmp_path):
    from mlx_lm_b200 import batch_generate, generate, load, stream_generate
    config = dict(CONFIG_A, ln_gain_std=0.3)
    weights = make_model_dir(str(tmp_path), config, 5, peaky=10.0)
    model, tokenizer = load(str(tmp_path), dtype=dtype)
    prompts = [random_tokens(7, 512, 0), random_tokens(13, 512, 1)]
    want = [plain.greedy_generate(p, 16, weights, config) for p in prompts]

    def agrees(got, ref, prompt):
        """Equal, or different first where the plain model's two best logits are closer than the dtype resolves."""
        for i, (a, b) in enumerate(zip(got, ref)):
            if a != b:
                lg = plain.logits(prompt + ref[:i], weights, config)[-1]
                top = torch.topk(lg, 2).values
                return dtype == "bfloat16" and float(top[0] - top[1]) < 0.05 * float(lg.abs().max())
        return len(got) == len(ref)

    for p, w in zip(prompts, want):
        text = generate(model, tokenizer, p, max_tokens=16)
        got = [int(t) for t in text.split()]
        assert agrees(got, w, p), (got, w)
        streamed = list(stream_generate(model, tokenizer, " ".join(map(str, p)), max_tokens=16))
        assert [r.token for r in streamed] == got and streamed[-1].finish_reason == "length"
        assert streamed[-1].generation_tokens == 16 and streamed[0].prompt_tokens == len(p)
    out = batch_generate(model, tokenizer, prompts, max_tokens=16, return_token_ids=True, return_logprobs=True)
    for got, w, p in zip(out.token_ids, want, prompts):
        assert agrees(got, w, p)
    assert out.stats.generation_tokens == 32 and out.stats.prompt_tokens == 20
    assert all(len(l) == 16 and all(x <= 0 for x in l) for l in out.logprobs)
    # an end-of-sequence token stops a request and is not part of its output
    tokenizer.add_eos_token(want[0][5])
    text = generate(model, tokenizer, prompts[0], max_tokens=16)
    first = want[0].index(want[0][5])
    assert [int(t) for t in text.split()] == want[0][:first]


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_as_a_cuda_graph_equals_the_eager_step(dtype, tmp_path):
    """Pure decode steps are replayed as CUDA graphs per batch-size bucket; tokens and log-probabilities
    must be those of the eager step, also for a batch smaller than its bucket and after requests left."""
    from mlx_lm_b200 import load
    from mlx_lm_b200.generate import BatchGenerator, get_engine
    from mlx_lm_b200.sampling import make_sampler
    make_model_dir(str(tmp_path), dict(CONFIG_B, ln_gain_std=0.3), 8, peaky=8.0)
    model, _ = load(str(tmp_path), dtype=dtype)
    prompts = [random_tokens(n, 1000, 50 + n) for n in (3, 17, 40, 33, 9)]       # 5 requests: bucket of 8
    max_tokens = [30, 12, 25, 5, 18]

    def run(use_graphs, lookahead=True, sampler=make_sampler(0.7, top_k=20)):
        engine = get_engine(model, page_size=16, num_pages=64, max_requests=8)
        engine.use_graphs = use_graphs
        gen = BatchGenerator(model, engine=engine, sampler=sampler, seed=3,
                             completion_batch_size=8, prefill_batch_size=8)
        gen.scheduler.lookahead = lookahead
        uids = gen.insert(prompts, max_tokens)
        out = {u: [] for u in uids}
        while gen.scheduler.has_work():
            for r in gen.next_generated():
                out[r.uid].append((r.token, round(r.logprobs, 4 if dtype == "float32" else 1)))
        assert engine.cache.pages_in_use() == [0]
        return [out[u] for u in uids], engine

    eager, _ = run(False)
    graphed, engine = run(True)
    assert {b for b, _ in engine._graphs} >= {8, 4, 2, 1}           # the batch shrank through the buckets
    assert [[t for t, _ in o] for o in eager] == [[t for t, _ in o] for o in graphed]
    assert eager == graphed
    engine.check_status()
    # the step launched ahead of the tokens (the default above) changes nothing, with filters and without
    assert run(True, lookahead=False)[0] == graphed
    plain = make_sampler(0.9)
    assert run(True, True, plain)[0] == run(True, False, plain)[0] == run(False, True, plain)[0]


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_failed_step_leaves_the_cache_as_it_was(dtype, tmp_path, monkeypatch):
    """If the model raises in the middle of a step, the step's positions are not part of the requests: lengths
    and pages are what they were, and the same tokens run again give the logits of an undisturbed run."""
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.weights import load_model
    weights = make_model_dir(str(tmp_path), CONFIG_A, 2, peaky=6.0)
    model, _ = load_model(str(tmp_path), dtype=dtype)
    toks, other = random_tokens(60, 512, 1), random_tokens(20, 512, 2)
    ref = plain.logits(toks, weights, CONFIG_A)
    eng = Engine(model, page_size=16, n_pages=8, max_requests=2)
    eng.add_request("a"); eng.add_request("b")
    eng.step([StepEntry("a", toks[:30], []), StepEntry("b", other[:5], [])])
    before = (eng.cache.length("a"), eng.cache.length("b"), eng.cache.pages_in_use())
    real_run = model.run
    blocks = model.description.blocks

    def failing(ctx):          # the first block runs (and writes keys for the new positions), then the step dies
        blocks[0].forward(ctx, model.description.embedding.forward(ctx, model.description.position),
                          ctx.cache_view(model.description.order[0]))
        raise RuntimeError("fault injected on the host")

    monkeypatch.setattr(model, "run", failing)
    with pytest.raises(RuntimeError, match="injected"):
        eng.step([StepEntry("a", toks[30:50], [19]), StepEntry("b", other[5:6], [0])])     # crosses a page edge
    eng.cache.check()
    assert (eng.cache.length("a"), eng.cache.length("b"), eng.cache.pages_in_use()) == before
    monkeypatch.setattr(model, "run", real_run)
    lg = eng.step([StepEntry("a", toks[30:60], list(range(30))), StepEntry("b", other[5:6], [])])
    assert rel(lg, ref[30:60]) <= TOL[dtype]
    eng.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_trim_and_run_again(dtype, tmp_path):
    """mlx-lm trims a prompt cache and generates again (tests/test_prompt_cache.py:266-294, ``KVCache.trim``,
    mlx_lm/models/cache.py:378-381): here 70 tokens are run, the cache is cut back to 37 (across a page edge),
    another request takes the freed pages, and the tail run again gives the rows of an uninterrupted run."""
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.weights import load_model
    weights = make_model_dir(str(tmp_path), CONFIG_B, 9, peaky=8.0)
    model, _ = load_model(str(tmp_path), dtype=dtype)
    toks, other = random_tokens(70, 1000, 3), random_tokens(40, 1000, 4)
    ref, ref_other = plain.logits(toks, weights, CONFIG_B), plain.logits(other, weights, CONFIG_B)
    eng = Engine(model, page_size=16, n_pages=6, max_requests=2)        # 70 tokens hold 5 of the 6 pages
    eng.add_request("a")
    first = eng.step([StepEntry("a", toks, list(range(70)))]).clone()
    assert rel(first, ref) <= TOL[dtype]
    held = list(eng.cache.requests["a"].pages[0])
    eng.cache.truncate("a", 37)
    assert eng.cache.length("a") == 37 and eng.cache.pages_in_use() == [3]
    eng.add_request("b")                                                 # takes the two pages just freed, and one more
    lg = eng.step([StepEntry("b", other, [39])])
    assert set(eng.cache.requests["b"].pages[0]) >= set(held[3:]) and rel(lg[0], ref_other[39]) <= TOL[dtype]
    eng.finish("b")
    again = [eng.step([StepEntry("a", toks[37:39], [0, 1])]).clone(),      # two tokens, then one, then the rest
             eng.step([StepEntry("a", toks[39:40], [0])]).clone(),
             eng.step([StepEntry("a", toks[40:70], list(range(30)))]).clone()]
    assert rel(torch.cat(again), ref[37:]) <= TOL[dtype]
    assert rel(torch.cat(again), first[37:]) <= TOL[dtype] * 0.5
    eng.check_status()
    eng.cache.check()


def test_a_folded_norm_before_a_very_wide_layer(tmp_path):
    """33 to 64 rows into a layer of 16384 or more outputs run on the tcgen05 kernel; with the norm before it
    folded into its weights that kernel needs the rows' statistics, not the few-rows kernel's epsilon."""
    from mlx_lm_b200.parts import LayerNorm, Linear
    D, N = 64, 16384
    ln, lin = LayerNorm("ln", D, 1e-5), Linear("wide", D, N, bias=True)
    w = bind(ln, torch.bfloat16, seed=1)
    w.update(bind(lin, torch.bfloat16, seed=2))
    ref_w, ref_b = w["wide.weight"], w["wide.bias"]
    assert lin.fold_norm(ln)
    g = torch.Generator().manual_seed(5)
    for rows in (40, 20, 130):
        x = (torch.randn(rows, D, generator=g) * 2 + 0.5).to(torch.bfloat16)
        ctx = part_ctx(rows)
        out = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
        assert lin.few_rows(rows) == (rows <= 32)
        lin.forward(ctx, ln.deferred(ctx, x.cuda()), out)
        want = plain.layer_norm(x.float(), w["ln.weight"], w["ln.bias"], 1e-5) @ ref_w.T + ref_b
        assert rel(out, want) <= 2e-2, rows


def test_a_model_without_a_final_norm(tmp_path):
    """``ModelDescription.final_norm`` may be None: the rows whose logits are wanted are then gathered as they
    are and go to the output head (a toy model defined here)."""
    from mlx_lm_b200.config import BaseModelArgs, register_architecture
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.parts import (MLP, Attention, Init, LayerNorm, ModelDescription, NoPosition, OutputHead,
                                   PreNormBlock, TokenEmbedding)
    from mlx_lm_b200.weights import load_model, write_random_model
    from safetensors.torch import load_file
    W, V = 48, 83

    @dataclass
    class Args(BaseModelArgs):
        model_type: str
        activation: str

    def build(a):
        emb = TokenEmbedding("emb", V, W, init=Init(0.0, 0.5))
        blk = PreNormBlock(LayerNorm("n1", W, 1e-5), Attention("mix", W, 3, 16, qkv_name="qkv", out_name="out",
                                                               init=Init(0.0, 0.3)),
                           LayerNorm("n2", W, 1e-5), MLP("ff", W, 72, activation=a.activation, up_name="up",
                                                         down_name="down", init=Init(0.0, 0.3)))
        return ModelDescription("toy_no_final_norm", W, V, emb, NoPosition(), [blk], None,
                                OutputHead(V, W, tied_to=None, name="head"), args=a)

    register_architecture("toy_no_final_norm", Args, build, replace=True)
    for dtype, tolerance in (("float32", 5e-5), ("bfloat16", 3e-2)):
        write_random_model(str(tmp_path), dict(model_type="toy_no_final_norm", activation="relu"), seed=8)
        w = {k: v.float() for k, v in load_file(str(tmp_path / "model.safetensors")).items()}
        toks = random_tokens(30, V, 1)
        x = w["emb.weight"][torch.tensor(toks)]
        h = plain.layer_norm(x, w["n1.weight"], w["n1.bias"], 1e-5)
        q, k, v = plain.split_heads(h @ w["mix.qkv.weight"].T + w["mix.qkv.bias"], 3)
        x = x + plain.causal_attention(q, k, v) @ w["mix.out.weight"].T + w["mix.out.bias"]
        h = plain.layer_norm(x, w["n2.weight"], w["n2.bias"], 1e-5)
        x = x + torch.relu(h @ w["ff.up.weight"].T + w["ff.up.bias"]) @ w["ff.down.weight"].T + w["ff.down.bias"]
        ref = x @ w["head.weight"].T
        model, _ = load_model(str(tmp_path), dtype=dtype)
        eng = Engine(model, page_size=16, n_pages=4, max_requests=1, max_len=64)
        eng.add_request(0)
        got = [eng.step([StepEntry(0, toks[:17], [3, 16, 0])]).clone(), eng.step([StepEntry(0, toks[17:18], [0])]).clone(),
               eng.step([StepEntry(0, toks[18:], list(range(12)))]).clone()]
        assert rel(torch.cat(got), ref[[3, 16, 0, 17] + list(range(18, 30))]) <= tolerance, dtype
        eng.check_status()


def test_benchmark_and_random_weights_sub_commands(tmp_path):
    """``python -m mlx_lm_b200 random_weights`` writes a model folder and ``... benchmark`` times it with the
    report lines of mlx-lm's benchmark (mlx_lm/benchmark.py:117-176), for a batch of one and of three."""
    import json
    import subprocess
    import sys
    from helpers import ROOT
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(dict(CONFIG_A, ln_gain_std=0.2)))
    run = lambda *a: subprocess.run([sys.executable, "-m", "mlx_lm_b200", *a], cwd=ROOT, capture_output=True,
                                    text=True, timeout=600)
    r = run("random_weights", "--config", str(cfg), "--seed", "3", "--out", str(tmp_path / "m"))
    assert r.returncode == 0, r.stderr
    assert (tmp_path / "m" / "config.json").exists() and (tmp_path / "m" / "model.safetensors").exists()
    for batch in (1, 3):
        r = run("benchmark", "--model", str(tmp_path / "m"), "-p", "16", "-g", "8", "-n", "1", "-b", str(batch))
        assert r.returncode == 0, r.stderr
        lines = r.stdout.strip().splitlines()
        assert lines[0] == "Running warmup.."
        assert lines[1] == f"Timing with prompt_tokens=16, generation_tokens=8, batch_size={batch}."
        assert lines[2].startswith("Trial 1:  prompt_tps=") and "generation_tps=" in lines[2] and "total_time=" in lines[2]
        assert lines[3].startswith("Averages: prompt_tps=") and "peak_memory=" in lines[3]


def test_command_line(tmp_path):
    """`python -m mlx_lm_b200 generate` with a model folder and with --random-weights/--config gives the tokens
    the Python entry point gives."""
    import json
    import subprocess
    import sys
    from helpers import ROOT
    from mlx_lm_b200 import generate, load
    config = dict(CONFIG_A, ln_gain_std=0.3)
    make_model_dir(str(tmp_path / "m"), config, 11)
    model, tokenizer = load(str(tmp_path / "m"), dtype="float32")
    want = generate(model, tokenizer, [5, 17, 3], max_tokens=12)
    run = lambda *a: subprocess.run([sys.executable, "-m", "mlx_lm_b200", "generate", *a], cwd=ROOT, capture_output=True,
                                    text=True, timeout=300)
    r = run("--model", str(tmp_path / "m"), "--prompt", "5 17 3", "-m", "12", "--dtype", "float32", "--verbose", "F")
    assert r.returncode == 0, r.stderr
    assert r.stdout.split() == want.split()
    r = run("--model", str(tmp_path / "m"), "--prompt-tokens", "5,17,3", "--max-tokens", "12", "--fp32")
    assert r.returncode == 0 and "Prompt: 3 tokens" in r.stdout and "Generation: 12 tokens" in r.stdout
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(config))
    r = run("--random-weights", "11", "--config", str(cfg), "--prompt", "5 17 3", "-m", "12", "--temp", "0.7",
            "--top-p", "0.9", "--seed", "4", "--verbose", "F")
    assert r.returncode == 0 and len(r.stdout.split()) == 12


def test_temperature_sampling_does_not_depend_on_batching(tmp_path):
    from mlx_lm_b200 import load
    from mlx_lm_b200.generate import BatchGenerator
    from mlx_lm_b200.sampling import make_logits_processors, make_sampler
    make_model_dir(str(tmp_path), CONFIG_B, 1)
    model, _ = load(str(tmp_path), dtype="float32")
    prompts = [random_tokens(n, 1000, n) for n in (5, 31, 64)]

    def run(**kw):
        gen = BatchGenerator(model, max_tokens=24, sampler=make_sampler(0.8, top_p=0.95), seed=1,
                             logits_processors=make_logits_processors(repetition_penalty=1.1), **kw)
        uids = gen.insert(prompts)
        out = {u: [] for u in uids}
        while gen.scheduler.has_work():
            for r in gen.next_generated():
                out[r.uid].append(r.token)
        return [out[u] for u in uids]

    together = run(completion_batch_size=8, prefill_batch_size=8)
    one_by_one = run(completion_batch_size=1, prefill_batch_size=1)
    small_steps = run(completion_batch_size=2, prefill_batch_size=1, prefill_step_size=7, max_tokens_per_step=9)
    assert together == one_by_one == small_steps
    assert all(len(t) == 24 for t in together) and len({tuple(t) for t in together}) == 3


def test_two_generators_taking_turns_on_one_engine(tmp_path):
    """Two generators on the engine of one model, each with decode steps launched ahead of their tokens, called in
    turns: the steps of one go through the same CUDA graph between a step of the other and the step after it, so the
    tokens must come from the host then (the graph's output buffer holds the other's by that time).  Each gets the
    tokens it gets alone."""
    from mlx_lm_b200 import load
    from mlx_lm_b200.generate import BatchGenerator, get_engine
    from mlx_lm_b200.sampling import make_sampler
    make_model_dir(str(tmp_path), dict(CONFIG_B, ln_gain_std=0.3), 5, peaky=6.0)
    model, _ = load(str(tmp_path), dtype="bfloat16")
    engine = get_engine(model, page_size=16, num_pages=96, max_requests=8)
    jobs = [([random_tokens(n, 1000, 7 + n) for n in (9, 30)], 20, make_sampler(0.8)),
            ([random_tokens(n, 1000, 90 + n) for n in (14, 5)], 26, make_sampler(0.0))]

    def start(job):
        prompts, max_tokens, sampler = job
        gen = BatchGenerator(model, engine=engine, sampler=sampler, seed=11, max_tokens=max_tokens,
                             completion_batch_size=4, prefill_batch_size=4)
        return gen, gen.insert(prompts), {}

    def drain(gen, out, steps):
        for _ in range(steps):
            if not gen.scheduler.has_work():
                return
            for r in gen.next_generated():
                out.setdefault(r.uid, []).append(r.token)

    alone = []
    for job in jobs:
        gen, uids, out = start(job)
        drain(gen, out, 10 ** 6)
        alone.append([out[u] for u in uids])
    a, b = start(jobs[0]), start(jobs[1])
    while a[0].scheduler.has_work() or b[0].scheduler.has_work():
        drain(a[0], a[2], 1)
        drain(b[0], b[2], 2)
    assert [a[2][u] for u in a[1]] == alone[0] and [b[2][u] for u in b[1]] == alone[1]
    assert engine.cache.pages_in_use() == [0]
    engine.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_scheduler_preempts_and_recomputes_on_the_gpu(dtype, tmp_path):
    """A pool too small for all requests at once: some are preempted and recomputed, and every
    request still gets the tokens it gets when it runs alone (in bfloat16: up to a choice between two logits
    that the plain model has closer together than bfloat16 resolves).  The decode graphs are left and entered
    again at other batch sizes on the way, with a step launched ahead whenever nobody waits."""
    from mlx_lm_b200 import load
    from mlx_lm_b200.generate import BatchGenerator, get_engine
    config = dict(CONFIG_A, ln_gain_std=0.3)
    weights = make_model_dir(str(tmp_path), config, 6, peaky=10.0)
    model, _ = load(str(tmp_path), dtype=dtype)
    prompts = [random_tokens(30, 512, 10 + i) for i in range(3)]
    want = [plain.greedy_generate(p, 20, weights, config) for p in prompts]
    engine = get_engine(model, page_size=16, num_pages=6, max_requests=4)
    gen = BatchGenerator(model, max_tokens=20, engine=engine, completion_batch_size=3, prefill_batch_size=3)
    uids = gen.insert(prompts)
    out = {u: [] for u in uids}
    while gen.scheduler.has_work():
        for r in gen.next_generated():
            out[r.uid].append(r.token)
    assert gen.scheduler.stats.preemptions > 0
    for u, w, p in zip(uids, want, prompts):
        got = out[u]
        assert len(got) == len(w)
        for i, (a, b) in enumerate(zip(got, w)):
            if a != b:
                lg = plain.logits(p + w[:i], weights, config)[-1]
                top = torch.topk(lg, 2).values
                assert dtype == "bfloat16" and float(top[0] - top[1]) < 0.05 * float(lg.abs().max()), (got, w)
                break
    assert engine.cache.pages_in_use() == [0]
    engine.check_status()


# ----------------------------------------------------------------------------------------------
# A mixer with state of its own, defined here: y_t = mean of x_0..x_t of the request, projected.

def test_a_toy_mixer_with_state_can_be_registered_built_and_stepped(tmp_path):
    from mlx_lm_b200.config import BaseModelArgs, register_architecture
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.parts import (MLP, Attention, Init, LayerNorm, Linear, Mixer, ModelDescription, NoPosition,
                                   OutputHead, PreNormBlock, RunEntry, StateSpec, TokenEmbedding, register_part)
    from mlx_lm_b200.weights import load_model, write_random_model
    from safetensors.torch import load_file

    class RunningMean(Mixer):
        """State per request: [sum of inputs (width) | count]."""

        def __init__(self, name, width):
            self.name, self.width = name, width
            self.proj = Linear(f"{name}.proj", width, width, bias=False, init=Init(0.0, 0.2))

        def children(self):
            return (self.proj,)

        def cache_spec(self):
            return StateSpec((self.width + 1,))

        def forward(self, ctx, x, residual, cache):
            y = torch.empty_like(x)
            for s in ctx.spans:       # a request's tokens in order; the state carries over between steps
                st = cache.state[s.slot]
                xs = x[s.first_token:s.first_token + s.n_tokens].float()
                sums = st[:self.width] + torch.cumsum(xs, 0)
                counts = st[self.width] + torch.arange(1, s.n_tokens + 1, device=x.device)
                y[s.first_token:s.first_token + s.n_tokens] = (sums / counts[:, None]).to(x.dtype)
                if cache.write:
                    st[:self.width] = sums[-1]
                    st[self.width] = counts[-1]
            return self.proj.forward(ctx, y, residual, residual=residual)

    register_part("mixer", "running_mean", RunningMean, replace=True)

    @dataclass
    class ToyArgs(BaseModelArgs):
        model_type: str
        width: int
        vocab_size: int
        mixers: list

    def build(a):
        emb = TokenEmbedding("emb", a.vocab_size, a.width, init=Init(0.0, 0.5))
        blocks = []
        for i, kind in enumerate(a.mixers):       # the configuration chooses the mixer layer by layer
            mixer = (RunningMean(f"l{i}.mix", a.width) if kind == "running_mean" else
                     Attention(f"l{i}.mix", a.width, 2, a.width // 2, qkv_name="qkv", out_name="out",
                               init=Init(0.0, 0.2)))
            blocks.append(PreNormBlock(LayerNorm(f"l{i}.n1", a.width, 1e-5), mixer, LayerNorm(f"l{i}.n2", a.width, 1e-5),
                                       MLP(f"l{i}.ff", a.width, 3 * a.width, up_name="up", down_name="down",
                                           init=Init(0.0, 0.2))))
        # block 0 runs twice; its second run reads and extends the same state
        order = [RunEntry(0)] + [RunEntry(i) for i in range(1, len(blocks))] + [RunEntry(0)]
        return ModelDescription("toy_state", a.width, a.vocab_size, emb, NoPosition(), blocks,
                                LayerNorm("nf", a.width, 1e-5), OutputHead(a.vocab_size, a.width, tied_to=emb),
                                order=order, args=a)

    register_architecture("toy_state", ToyArgs, build, replace=True)
    cfg = dict(model_type="toy_state", width=32, vocab_size=97, mixers=["running_mean", "attention", "running_mean"])
    write_random_model(str(tmp_path), cfg, seed=3)
    w = {k: v.float() for k, v in load_file(str(tmp_path / "model.safetensors")).items()}

    def plain_toy(tokens):
        def ln(x, n):
            return plain.layer_norm(x, w[n + ".weight"], w[n + ".bias"], 1e-5)

        def ff(x, n):
            return plain.gelu_new(x @ w[n + ".up.weight"].T + w[n + ".up.bias"]) @ w[n + ".down.weight"].T \
                + w[n + ".down.bias"]

        def mean_mix(x, n, state):
            sums = state[0] + torch.cumsum(x, 0)
            counts = state[1] + torch.arange(1, len(x) + 1)
            state[0], state[1] = sums[-1], counts[-1]
            return (sums / counts[:, None]) @ w[n + ".proj.weight"].T

        def attn(x, n):
            qkv = x @ w[n + ".qkv.weight"].T + w[n + ".qkv.bias"]
            q, k, v = plain.split_heads(qkv, 2)
            return plain.causal_attention(q, k, v) @ w[n + ".out.weight"].T + w[n + ".out.bias"]

        x = w["emb.weight"][torch.tensor(tokens)]
        states = {0: [torch.zeros(32), torch.zeros(())], 2: [torch.zeros(32), torch.zeros(())]}
        for i in (0, 1, 2, 0):
            h = ln(x, f"l{i}.n1")
            x = x + (attn(h, f"l{i}.mix") if i == 1 else mean_mix(h, f"l{i}.mix", states[i]))
            x = x + ff(ln(x, f"l{i}.n2"), f"l{i}.ff")
        return ln(x, "nf") @ w["emb.weight"].T

    # block 0 runs twice per step on a running state, so whole-sequence and stepped runs differ by
    # construction; the plain model is therefore run with the same cutting as the engine
    model, _ = load_model(str(tmp_path), dtype="float32")
    eng = Engine(model, page_size=16, n_pages=8, max_requests=3, max_len=64)
    assert [g.cache_ids for g in eng.cache.state_groups] == [[0, 2]] and [g.cache_ids for g in eng.cache.kv_groups] == [[1]]
    toks = random_tokens(40, 97, 0)
    eng.add_request("a")
    got = eng.step([StepEntry("a", toks, list(range(40)))]).clone()
    assert rel(got, plain_toy(toks)) <= 5e-5
    eng.finish("a")
    # a second request re-uses the slot: its state must start from zero again
    eng.add_request("b")
    assert rel(eng.step([StepEntry("b", toks[:9], list(range(9)))]), plain_toy(toks[:9])) <= 5e-5
    eng.finish("b")
    # layers 1 and 2 alone (single runs) are cut-invariant: a model without the repeated block
    cfg2 = dict(cfg, mixers=["attention", "running_mean"])

    def build2(a):
        d = build(a)
        d.order = [RunEntry(i) for i in range(len(d.blocks))]
        return d

    register_architecture("toy_state2", ToyArgs, build2, replace=True)
    d2 = tmp_path / "m2"
    write_random_model(str(d2), dict(cfg2, model_type="toy_state2"), seed=4)
    model2, _ = load_model(str(d2), dtype="float32")
    eng2 = Engine(model2, page_size=16, n_pages=8, max_requests=3, max_len=64)
    eng2.add_request("w"); eng2.add_request("c"); eng2.add_request("o")
    whole = eng2.step([StepEntry("w", toks, list(range(40)))]).clone()
    other = random_tokens(12, 97, 9)
    rows = []
    rows.append(eng2.step([StepEntry("c", toks[:7], list(range(7))), StepEntry("o", other[:5], [])]).clone())
    rows.append(eng2.step([StepEntry("o", other[5:6], []), StepEntry("c", toks[7:9], [0, 1])]).clone())
    rows.append(eng2.step([StepEntry("c", toks[9:40], list(range(31)))]).clone())
    assert rel(torch.cat(rows), whole) <= 5e-5


# ----------------------------------------------------------------------------------------------
# Two more toy parts, defined here: a rotary position encoding (rotates q and k before keys enter the
# cache) and a feed-forward that routes each token to one of two experts.  Neither becomes a model of
# anyone's; they show that the interfaces of positions and feed-forwards carry such parts.

def test_toy_rotary_positions_and_routed_feed_forward(tmp_path):
    from mlx_lm_b200.config import BaseModelArgs, register_architecture
    from mlx_lm_b200.engine import Engine, StepEntry
    from mlx_lm_b200.parts import (MLP, Attention, FeedForward, Init, LayerNorm, Linear, ModelDescription, OutputHead,
                                   PositionEncoding, PreNormBlock, TokenEmbedding)
    from mlx_lm_b200.weights import load_model, write_random_model
    from safetensors.torch import load_file

    W, H, Dh, V = 32, 2, 16, 61

    def rotate_rows(t, positions, n_heads):
        """Rotate pairs (d, d + Dh/2) of every head by angle position * 10000^(-2d/Dh), in float32."""
        T = t.shape[0]
        x = t.float().reshape(T, n_heads, 2, Dh // 2)
        inv = 10000.0 ** (-torch.arange(Dh // 2, device=t.device, dtype=torch.float32) * 2 / Dh)
        ang = positions.float()[:, None, None] * inv
        c, s = torch.cos(ang), torch.sin(ang)
        a, b = x[:, :, 0], x[:, :, 1]
        return torch.stack([a * c - b * s, a * s + b * c], dim=2).reshape(T, n_heads * Dh)

    class Rotary(PositionEncoding):
        max_positions = None

        def rotate(self, ctx, q, k):          # in place on this step's queries and keys (views of one buffer)
            q.copy_(rotate_rows(q, ctx.positions, H).to(q.dtype))
            k.copy_(rotate_rows(k, ctx.positions, H).to(k.dtype))

    class Routed(FeedForward):
        """Each token goes to the expert whose router logit is larger (float32 router)."""

        def __init__(self, name, width, inner):
            self.router = Linear(f"{name}.router", width, 2, bias=False, init=Init(0.0, 0.5))
            self.experts = [MLP(f"{name}.e{i}", width, inner, up_name="up", down_name="down", init=Init(0.0, 0.2))
                            for i in range(2)]

        def children(self):
            return (self.router, *self.experts)

        def forward(self, ctx, x, residual):
            logits = ctx.ws.get("router", x.shape[0], 2, torch.float32)
            self.router.forward(ctx, x, logits)
            choice = logits.argmax(dim=-1)
            for i, e in enumerate(self.experts):
                idx = (choice == i).nonzero().flatten()
                if idx.numel():
                    residual[idx] = e.forward(ctx, x[idx].contiguous(), residual[idx].contiguous())
            return residual

    from dataclasses import dataclass

    @dataclass
    class Args(BaseModelArgs):
        model_type: str
        n_layer: int

    def build(a):
        emb = TokenEmbedding("emb", V, W, init=Init(0.0, 0.5))
        rot = Rotary()
        blocks = [PreNormBlock(LayerNorm(f"l{i}.n1", W, 1e-5), Attention(f"l{i}.mix", W, H, Dh, qkv_name="qkv", out_name="out",
                                                                         position=rot, init=Init(0.0, 0.3)),
                               LayerNorm(f"l{i}.n2", W, 1e-5), Routed(f"l{i}.ff", W, 48)) for i in range(a.n_layer)]
        return ModelDescription("toy_rotary_routed", W, V, emb, None, blocks, LayerNorm("nf", W, 1e-5),
                                OutputHead(V, W, tied_to=emb), args=a)

    register_architecture("toy_rotary_routed", Args, build, replace=True)
    write_random_model(str(tmp_path), dict(model_type="toy_rotary_routed", n_layer=2), seed=5)
    w = {k: v.float() for k, v in load_file(str(tmp_path / "model.safetensors")).items()}

    def plain_toy(tokens):
        T = len(tokens)
        pos = torch.arange(T)
        x = w["emb.weight"][torch.tensor(tokens)]
        for i in range(2):
            h = plain.layer_norm(x, w[f"l{i}.n1.weight"], w[f"l{i}.n1.bias"], 1e-5)
            qkv = h @ w[f"l{i}.mix.qkv.weight"].T + w[f"l{i}.mix.qkv.bias"]
            q, k, v = qkv[:, :W], qkv[:, W:2 * W], qkv[:, 2 * W:]
            q, k = rotate_rows(q, pos, H), rotate_rows(k, pos, H)
            hs = lambda t: t.reshape(T, H, Dh).permute(1, 0, 2)
            x = x + plain.causal_attention(hs(q), hs(k), hs(v)) @ w[f"l{i}.mix.out.weight"].T + w[f"l{i}.mix.out.bias"]
            h = plain.layer_norm(x, w[f"l{i}.n2.weight"], w[f"l{i}.n2.bias"], 1e-5)
            choice = (h @ w[f"l{i}.ff.router.weight"].T).argmax(-1)
            y = torch.zeros_like(x)
            for e in range(2):
                p = f"l{i}.ff.e{e}."
                ye = plain.gelu_new(h @ w[p + "up.weight"].T + w[p + "up.bias"]) @ w[p + "down.weight"].T + w[p + "down.bias"]
                y = torch.where((choice == e)[:, None], ye, y)
            x = x + y
        return plain.layer_norm(x, w["nf.weight"], w["nf.bias"], 1e-5) @ w["emb.weight"].T

    model, _ = load_model(str(tmp_path), dtype="float32")
    assert model.description.max_positions is None
    eng = Engine(model, page_size=16, n_pages=8, max_requests=2, max_len=64)
    assert not eng.use_replay                  # these parts do host-side work: their steps are never re-issued from a recording
    toks = random_tokens(50, V, 3)
    ref = plain_toy(toks)
    eng.add_request("a")
    rows = [eng.step([StepEntry("a", toks[:19], list(range(19)))]).clone(),
            eng.step([StepEntry("a", toks[19:21], [0, 1])]).clone(),
            eng.step([StepEntry("a", toks[21:50], list(range(29)))]).clone()]
    assert rel(torch.cat(rows), ref) <= 1e-4
    # both experts were used by this sequence (else the routing is not exercised)
    h0 = plain.layer_norm(w["emb.weight"][torch.tensor(toks)], w["l0.n1.weight"], w["l0.n1.bias"], 1e-5)
    assert ref.shape == (50, V) and h0.shape == (50, W)
