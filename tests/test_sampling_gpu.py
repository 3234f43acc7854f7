"""The sampling and logits-processor kernels against tests/sampling_ref.py."""
import numpy as np
import pytest
import torch

import sampling_ref as S

pytestmark = pytest.mark.gpu


def run_sampler(logits, sampler, seed=0, request=0, position=0, full=False):
    from mlx_lm_b200 import ops
    x = torch.tensor(np.asarray(logits, dtype=np.float32)).cuda().reshape(1, -1)
    params = torch.tensor(np.frombuffer(sampler.words(seed, request, position), dtype=np.int32).copy()).cuda()
    tok = torch.empty(1, dtype=torch.int32, device="cuda")
    lp = torch.empty(1, dtype=torch.float32, device="cuda")
    out = torch.empty_like(x) if full else None
    sp = torch.tensor(list(sampler.xtc_special_tokens), dtype=torch.int32).cuda() if sampler.xtc_special_tokens else None
    # without full log-probabilities the row of a wide vocabulary is cut into slices over several thread blocks
    ops.sample(x, params, tok, lp, ops.current_stream(), xtc_special=sp, out_logprobs=out,
               scratch=None if full else ops.sample_scratch(1, "cuda"))
    return int(tok.item()), float(lp.item()), (out[0].cpu().numpy() if full else None)


def test_greedy_and_logprobs():
    from mlx_lm_b200.sampling import make_sampler
    rng = np.random.RandomState(0)
    for V in (33, 512, 1000, 50257):
        x = rng.randn(V).astype(np.float32) * 3
        x[V // 3] = x.max()          # a tie: the smaller index wins, as argmax does
        tok, lp, full = run_sampler(x, make_sampler(0.0), full=True)
        rt, rlp, rfull = S.sample(x)
        assert tok == rt == int(np.argmax(x)) and abs(lp - rlp) < 1e-4
        assert np.abs(full - rfull).max() < 1e-4


def test_hand_made_distributions():
    """The 4-entry cases mlx-lm checks its filters with (tests/test_sample_utils.py:19-105)."""
    from mlx_lm_b200.sampling import make_sampler
    logits = np.log(np.array([0.9, 0.0, 0.0, 0.1]) + 1e-30)
    assert run_sampler(logits, make_sampler(1.0, top_p=0.8))[0] == 0
    probs = np.array([0.0, 0.5, 0.4, 0.1])
    seen = {run_sampler(np.log(probs + 1e-30), make_sampler(1.0, top_p=0.4), position=p)[0] for p in range(40)}
    assert seen == {1}
    seen = {run_sampler(np.log(probs + 1e-30), make_sampler(1.0, top_p=0.6), position=p)[0] for p in range(60)}
    assert seen == {1, 2}
    seen = {run_sampler(np.log(probs + 1e-30), make_sampler(1.0, top_k=1), position=p)[0] for p in range(20)}
    assert seen == {1}
    seen = {run_sampler(np.log(probs + 1e-30), make_sampler(1.0, min_p=0.75), position=p)[0] for p in range(40)}
    assert seen == {1, 2}
    seen = {run_sampler(np.log(probs + 1e-30), make_sampler(1.0, min_p=0.95), position=p)[0] for p in range(20)}
    assert seen == {1}
    # XTC removes the tokens above the least probable one that exceeds the threshold
    probs = np.array([0.4, 0.3, 0.15, 0.15])
    seen = {run_sampler(np.log(probs), make_sampler(1.0, xtc_probability=1.0, xtc_threshold=0.2), position=p)[0]
            for p in range(60)}
    assert seen == {1, 2, 3}
    seen = {run_sampler(np.log(probs), make_sampler(1.0, xtc_probability=1.0, xtc_threshold=0.2,
                                                    xtc_special_tokens=(0,)), position=p)[0] for p in range(60)}
    assert seen == {0, 1, 2, 3}


@pytest.mark.parametrize("V", [257, 1000, 50257])
def test_filters_and_draw_match_the_plain_sampler(V):
    from mlx_lm_b200.sampling import make_sampler
    rng = np.random.RandomState(V)
    settings = [dict(temp=0.8), dict(temp=1.3, top_p=0.9), dict(temp=0.7, min_p=0.05, min_tokens_to_keep=3),
                dict(temp=1.0, top_k=7), dict(temp=0.9, top_p=0.95, min_p=0.01, top_k=40),
                dict(temp=1.1, xtc_probability=0.5, xtc_threshold=0.05, top_k=30),
                dict(temp=1.0, top_p=0.5, xtc_probability=1.0, xtc_threshold=0.1, xtc_special_tokens=(3, 5))]
    n_checked = 0
    for si, kw in enumerate(settings):
        for trial in range(4 if V > 10000 else 10):
            x = (rng.randn(V) * 2.5).astype(np.float32)
            seed, request, position = 1234 + si, trial, 17 * trial + 3
            tok, lp, _ = run_sampler(x, make_sampler(**kw), seed, request, position)
            ref_kw = dict(kw)
            special = ref_kw.pop("xtc_special_tokens", ())
            rt, rlp, kept = S.sample(x, xtc_special=special, seed=seed, request=request, position=position, **ref_kw)
            assert np.isfinite(kept[tok]), f"{kw}: token {tok} was filtered out by the plain sampler"
            assert tok == rt, (kw, trial)
            assert abs(lp - rlp) < 2e-4
            n_checked += 1
    assert n_checked


def test_draw_follows_the_distribution_and_the_key():
    from mlx_lm_b200.sampling import make_sampler
    probs = np.array([0.5, 0.25, 0.125, 0.125])
    s = make_sampler(1.0)
    counts = np.zeros(4)
    for p in range(2000):
        counts[run_sampler(np.log(probs), s, seed=5, request=1, position=p)[0]] += 1
    assert np.abs(counts / 2000 - probs).max() < 0.04
    # temperature sharpens
    counts = np.zeros(4)
    for p in range(1000):
        counts[run_sampler(np.log(probs), make_sampler(0.25), seed=5, request=1, position=p)[0]] += 1
    assert counts[0] / 1000 > 0.85
    a = [run_sampler(np.log(probs), s, seed=5, request=1, position=p)[0] for p in range(64)]
    assert a == [run_sampler(np.log(probs), s, seed=5, request=1, position=p)[0] for p in range(64)]
    assert a != [run_sampler(np.log(probs), s, seed=6, request=1, position=p)[0] for p in range(64)]
    assert a != [run_sampler(np.log(probs), s, seed=5, request=2, position=p)[0] for p in range(64)]


def test_rows_are_independent():
    """A row's token does not depend on the other rows of the batch."""
    from mlx_lm_b200 import ops
    from mlx_lm_b200.sampling import make_sampler
    rng = np.random.RandomState(1)
    x = torch.tensor(rng.randn(5, 1000).astype(np.float32) * 2).cuda()
    samplers = [make_sampler(0.9, top_p=0.8), make_sampler(0.0), make_sampler(1.2, top_k=5), make_sampler(0.7),
                make_sampler(1.0, min_p=0.1)]
    rec = b"".join(s.words(9, r, 40 + r) for r, s in enumerate(samplers))
    params = torch.tensor(np.frombuffer(rec, dtype=np.int32).copy()).cuda()
    tok = torch.empty(5, dtype=torch.int32, device="cuda")
    lp = torch.empty(5, dtype=torch.float32, device="cuda")
    ops.sample(x, params, tok, lp, ops.current_stream())
    alone = [run_sampler(x[r].cpu().numpy(), s, 9, r, 40 + r)[0] for r, s in enumerate(samplers)]
    assert tok.tolist() == alone


def test_rows_cut_into_slices_give_the_same_tokens():
    """Wide vocabularies: with scratch memory a row is cut into slices over several thread blocks and merged by
    the block that finishes last.  Tokens are those of the one-block kernel, whatever the options, with ties
    across slices, rows of -inf, and launches of changing numbers of rows on the same scratch memory."""
    from mlx_lm_b200 import ops
    from mlx_lm_b200.sampling import make_sampler
    V = 50257
    rng = np.random.RandomState(7)
    samplers = [make_sampler(0.0), make_sampler(0.8), make_sampler(1.3, top_p=0.9), make_sampler(0.0),
                make_sampler(1.0, top_k=7), make_sampler(0.6), make_sampler(0.9, min_p=0.02), make_sampler(0.0)]
    x = rng.randn(len(samplers), V).astype(np.float32) * 3
    x[0, 40000] = x[0, 123] = x[0].max() + 1.0        # equal maxima in different slices: the first wins
    x[3, :] = -np.inf
    x[3, 50000] = 0.5                                  # all but one entry masked out
    x[5, 6283:2 * 6283] = -np.inf                      # a slice that is empty of candidates
    scratch = ops.sample_scratch(len(samplers), "cuda")
    for n in (8, 3, 5, 8, 1):
        rows = list(range(n))
        rec = b"".join(samplers[r].words(11, r, 70 + r) for r in rows)
        params = torch.tensor(np.frombuffer(rec, dtype=np.int32).copy()).cuda()
        xs = torch.tensor(x[:n]).cuda()
        tok, lp = (torch.empty(n, dtype=t, device="cuda") for t in (torch.int32, torch.float32))
        tok1, lp1 = (torch.empty(n, dtype=t, device="cuda") for t in (torch.int32, torch.float32))
        ops.sample(xs, params, tok, lp, ops.current_stream(), scratch=scratch)
        ops.sample(xs, params, tok1, lp1, ops.current_stream())
        assert tok.tolist() == tok1.tolist(), n
        assert torch.allclose(lp, lp1, atol=2e-5), n
        assert int(scratch[:len(samplers)].abs().sum().item()) == 0   # tickets back at zero
    first = torch.empty(1, dtype=torch.int32, device="cuda")
    ops.sample(torch.tensor(x[:1]).cuda(), torch.tensor(np.frombuffer(samplers[0].words(11, 0, 70), dtype=np.int32).copy()).cuda(),
               first, torch.empty(1, dtype=torch.float32, device="cuda"), ops.current_stream(), scratch=scratch)
    assert first.item() == 123
    with pytest.raises(ops.KernelError):
        ops.sample(torch.tensor(x[:8]).cuda(), params.repeat(8), torch.empty(8, dtype=torch.int32, device="cuda"),
                   torch.empty(8, dtype=torch.float32, device="cuda"), ops.current_stream(),
                   scratch=ops.sample_scratch(2, "cuda"))


def test_logits_processors():
    from mlx_lm_b200 import ops
    from mlx_lm_b200.sampling import make_logits_processors
    rng = np.random.RandomState(2)
    V = 300
    x = rng.randn(3, V).astype(np.float32)
    histories = [[5, 7, 5, 9, 5, 200, 7] + list(range(30, 60)), [1, 2, 3], list(range(100, 130)) + [4, 4, 4, 299]]
    settings = [dict(logit_bias={5: 2.0, 11: -3.0}, repetition_penalty=1.3, repetition_context_size=10),
                dict(presence_penalty=0.7, frequency_penalty=0.2, frequency_context_size=2),
                dict(repetition_penalty=0.8, presence_penalty=0.5, presence_context_size=3, frequency_penalty=0.25,
                     frequency_context_size=25, logit_bias={299: 1.0})]
    procs = [make_logits_processors(**kw)[0] for kw in settings]
    C = max(p.context_size for p in procs)
    B = max(len(p.logit_bias) for p in procs)
    params = np.stack([np.frombuffer(p.words(), dtype=np.int32) for p in procs])
    ctx = np.full((3, C), -1, dtype=np.int32)
    bidx = np.full((3, B), -1, dtype=np.int32)
    bval = np.zeros((3, B), dtype=np.float32)
    for i, (p, h) in enumerate(zip(procs, histories)):
        tail = h[-p.context_size:]
        ctx[i, C - len(tail):] = tail
        for j, (t, v) in enumerate(p.logit_bias):
            bidx[i, j], bval[i, j] = t, v
    dev = torch.tensor(x).cuda()
    ops.process_logits(dev, torch.tensor(params.reshape(-1)).cuda(), torch.tensor(ctx).cuda(),
                       torch.tensor(bidx).cuda(), torch.tensor(bval).cuda(), ops.current_stream())
    for i, (kw, h) in enumerate(zip(settings, histories)):
        assert np.abs(dev[i].cpu().numpy() - S.process(x[i], h, **kw)).max() < 1e-5, i
    assert make_logits_processors() == []


def test_device_sampler_rows_keep_their_own_options():
    """Through ``DeviceSampler``, as the scheduler calls it: every row has its own XTC special tokens (one
    request's exemptions protect nothing in another's row), processors run in the order of each request's list,
    the engine's status word comes back with the tokens, and an unseeded sampler draws a seed of its own."""
    from types import SimpleNamespace

    from mlx_lm_b200.sampling import make_logits_processors, make_sampler
    from mlx_lm_b200.sampling.device import DeviceSampler
    probs = np.array([0.4, 0.3, 0.15, 0.15])
    plain_xtc = make_sampler(1.0, xtc_probability=1.0, xtc_threshold=0.2)
    keeps_0 = make_sampler(1.0, xtc_probability=1.0, xtc_threshold=0.2, xtc_special_tokens=(0,))
    engine = SimpleNamespace(status=torch.zeros(1, dtype=torch.int32, device="cuda"), host_status=-1, h2d_bytes=0,
                             d2h_bytes=0)
    ds = DeviceSampler("cuda", seed=4, engine=engine)
    seen = [set(), set(), set()]
    for p in range(60):
        reqs = [SimpleNamespace(uid=u, tokens=[0] * p, sampler=s, processors=())
                for u, s in enumerate((keeps_0, plain_xtc, keeps_0))]
        logits = torch.tensor(np.log(np.stack([probs] * 3)), dtype=torch.float32).cuda()
        toks, _ = ds(logits, reqs)
        for u, t in enumerate(toks):
            seen[u].add(t)
        assert engine.host_status == 0
    assert seen[0] == seen[2] == {0, 1, 2, 3} and seen[1] == {1, 2, 3}
    engine.status.fill_(6)
    ds(logits, reqs)
    assert engine.host_status == 6
    # order of processors: a callable that doubles the logits and a bias of +1 on token 2 do not commute
    (bias,) = make_logits_processors(logit_bias={2: 1.0})
    double = lambda tokens, lg: lg * 2.0
    base = torch.tensor([[0.0, 1.0, 1.2, -1.0]], dtype=torch.float32)
    greedy = make_sampler(0.0)
    out = []
    for procs in ((double, bias), (bias, double)):
        lg = base.clone().cuda()
        ds([lg][0], [SimpleNamespace(uid=0, tokens=[1], sampler=greedy, processors=procs)])
        out.append(lg[0].cpu().tolist())
    assert out[0] == pytest.approx([0.0, 2.0, 3.4, -2.0]) and out[1] == pytest.approx([0.0, 2.0, 4.4, -2.0])
    assert DeviceSampler("cuda", seed=None).seed != DeviceSampler("cuda", seed=None).seed
