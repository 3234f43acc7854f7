"""The scheduler's decisions, driven without a device: a fake engine with the real cache manager
and a fake sampler whose token is a function of (request, position) only, so that any way of
batching, cutting and preempting must produce the same tokens."""
import pytest

from mlx_lm_b200.cache import CacheManager, OutOfPages
from mlx_lm_b200.engine.scheduler import Scheduler, StopSequenceMatcher
from mlx_lm_b200.parts import PagedKVSpec


class FakeEngine:
    def __init__(self, n_pages, page_size=16, max_requests=8, max_len=256):
        self.cache = CacheManager({0: PagedKVSpec(2, 16, None)}, page_size=page_size, n_pages=n_pages,
                                  max_requests=max_requests, max_len=max_len)
        self.max_len = max_len
        self.steps = []          # per step: list of (rid, start position, n tokens, wants)
        self.fed = {}            # rid -> tokens fed since its last admission

    def add_request(self, rid):
        self.cache.add_request(rid)
        self.fed[rid] = []

    def finish(self, rid):
        self.cache.release(rid)

    def step(self, entries):
        rec, rows = [], []
        for e in entries:
            start = self.cache.reserve(e.rid, len(e.tokens))
            assert start == len(self.fed[e.rid]), "tokens must continue where the cache ends"
            self.fed[e.rid].extend(e.tokens)
            rec.append((e.rid, start, len(e.tokens), list(e.want)))
            rows.extend((e.rid, start + w) for w in e.want)
        for e in entries:
            self.cache.commit(e.rid)
        self.cache.check()
        self.steps.append(rec)
        return rows


def token_fn(uid, position):
    return (uid * 7919 + position * 104729) % 1000


def fake_sample(rows, requests):
    assert [r.uid for r in requests] == [rid for rid, _ in rows]
    return [token_fn(rid, pos + 1) for rid, pos in rows], [0.0] * len(rows)


def run(sched, limit=10000):
    out, reasons = {}, {}
    n = 0
    while sched.has_work():
        _, gens = sched.next()
        for r in gens:
            out.setdefault(r.uid, []).append(r.token)
            if r.finish_reason:
                reasons[r.uid] = r.finish_reason
        n += 1
        assert n < limit, "the scheduler does not finish"
    return out, reasons


def expected(uid, prompt_len, n):
    return [token_fn(uid, prompt_len + i) for i in range(n)]


def test_single_request_is_cut_under_the_budget():
    eng = FakeEngine(n_pages=16)
    s = Scheduler(eng, fake_sample, prefill_step_size=40, max_tokens_per_step=64)
    uid = s.insert(list(range(100)), max_tokens=5)
    out, reasons = run(s)
    assert out[uid] == expected(uid, 100, 5) and reasons[uid] == "length"
    sizes = [e[2] for step in eng.steps for e in step]
    assert sizes == [40, 40, 20, 1, 1, 1, 1]
    wants = [e[3] for step in eng.steps for e in step]
    assert wants[:3] == [[], [], [19]]         # logits only where the prompt ends
    assert eng.cache.pages_in_use() == [0]


def test_decode_first_then_prompts_fill_the_budget():
    eng = FakeEngine(n_pages=64)
    s = Scheduler(eng, fake_sample, max_requests=4, max_prefilling=2, prefill_step_size=32, max_tokens_per_step=40)
    a = s.insert(list(range(10)), max_tokens=30)
    s.next()                                   # a is decoding from now on
    b = s.insert(list(range(70)), max_tokens=3)
    c = s.insert(list(range(50)), max_tokens=3)
    s.next()
    step = eng.steps[-1]
    assert step[0][:3] == (a, 10, 1)           # the decoding request first, one token
    assert step[1][:3] == (b, 0, 32)           # then a portion of the oldest prompt
    assert step[2][:3] == (c, 0, 7)            # and what is left of the budget: 40 - 1 - 32
    out, reasons = run(s)
    assert out[b] == expected(b, 70, 3) and out[c] == expected(c, 50, 3)
    assert len(out[a]) + 2 == 30 or len(out[a]) == 28
    assert all(sum(e[2] for e in st) <= 40 for st in eng.steps)


def test_admission_limits():
    eng = FakeEngine(n_pages=64, max_requests=8)
    s = Scheduler(eng, fake_sample, max_requests=3, max_prefilling=1, prefill_step_size=16, max_tokens_per_step=64)
    uids = [s.insert(list(range(40)), max_tokens=4) for _ in range(5)]
    s.next()
    assert len(s.running) == 1                 # one request in its prompt at a time
    out, reasons = run(s)
    assert max(len(st) for st in eng.steps) <= 3
    for u in uids:
        assert out[u] == expected(u, 40, 4)


def test_batch_equals_single_and_per_request_max_tokens():
    prompts = [list(range(5 + 9 * i)) for i in range(6)]
    max_tokens = [3, 9, 1, 12, 5, 7]
    eng = FakeEngine(n_pages=64)
    s = Scheduler(eng, fake_sample, max_requests=3, max_prefilling=2, prefill_step_size=8, max_tokens_per_step=20)
    uids = [s.insert(p, m) for p, m in zip(prompts, max_tokens)]
    out, reasons = run(s)
    for u, p, m in zip(uids, prompts, max_tokens):
        assert out[u] == expected(u, len(p), m) and reasons[u] == "length"
    assert eng.cache.pages_in_use() == [0] and not eng.cache.requests


def test_stop_sequence_and_remove():
    eng = FakeEngine(n_pages=32)
    s = Scheduler(eng, fake_sample)
    want = expected(0, 6, 10)
    stop = StopSequenceMatcher([[want[3], want[4]], [99999]])
    a = s.insert(list(range(6)), 10, stop=stop)
    b = s.insert(list(range(9)), 50)
    out = {}
    for _ in range(3):
        for r in s.next()[1]:
            out.setdefault(r.uid, []).append(r)
    s.remove([b])
    assert eng.cache.pages_in_use()[0] > 0 and b not in eng.cache.requests
    while s.has_work():
        for r in s.next()[1]:
            out.setdefault(r.uid, []).append(r)
    assert [r.token for r in out[a]] == want[:5] and out[a][-1].finish_reason == "stop"
    assert out[a][-1].all_tokens == list(range(6)) + want[:5]
    # three tokens, then the one response that says it was taken out
    assert [r.finish_reason for r in out[b]] == [None, None, None, "cancelled"] and eng.cache.pages_in_use() == [0]


def test_pages_run_out_newest_request_is_recomputed():
    # 6 pages of 16: three requests of 30 prompt tokens take 2 pages each; decoding past 32 needs a third
    eng = FakeEngine(n_pages=6)
    s = Scheduler(eng, fake_sample, max_requests=3, max_prefilling=3, prefill_step_size=64, max_tokens_per_step=128)
    uids = [s.insert(list(range(100 * i, 100 * i + 30)), max_tokens=20) for i in range(3)]
    out, reasons = run(s)
    assert s.stats.preemptions > 0
    for i, u in enumerate(uids):
        assert out[u] == expected(u, 30, 20), "a recomputed request must continue with the same tokens"
        assert reasons[u] == "length"
    # a preempted request came back with prompt + generated tokens in one or more portions from position 0
    restarts = [e for st in eng.steps for e in st if e[1] == 0]
    assert len(restarts) > 3
    assert eng.cache.pages_in_use() == [0]
    # the oldest request is never the victim: it starts from position 0 exactly once
    assert sum(1 for e in restarts if e[0] == uids[0]) == 1


def test_request_that_can_never_fit_is_refused():
    eng = FakeEngine(n_pages=4)
    s = Scheduler(eng, fake_sample)
    with pytest.raises(ValueError):
        s.insert(list(range(60)), max_tokens=10)      # 69 positions = 5 pages > 4
    with pytest.raises(ValueError):
        s.insert(list(range(250)), max_tokens=10)     # beyond the model's positions
    with pytest.raises(ValueError):
        s.insert([], max_tokens=1)
    u = s.insert(list(range(60)), max_tokens=5)       # 64 positions = 4 pages: fits alone
    out, _ = run(s)
    assert out[u] == expected(u, 60, 5)


@pytest.mark.parametrize("seed", range(12))
def test_random_workloads_give_every_request_its_own_tokens(seed):
    """Random prompt lengths, budgets, pool sizes and arrival times: whatever the scheduler decides (portions,
    admissions, preemptions), every request gets the tokens it would get alone, no step exceeds its budgets, no
    page is left behind, and the oldest running request is never the one that starts over."""
    import random

    rng = random.Random(seed)
    page = rng.choice([8, 16])
    n_pages = rng.randint(6, 24)
    max_requests = rng.randint(2, 5)
    step_size = rng.choice([8, 16, 48, 200])
    budget = rng.choice([16, 64, 256])
    eng = FakeEngine(n_pages=n_pages, page_size=page, max_requests=8, max_len=256)
    s = Scheduler(eng, fake_sample, max_requests=max_requests, max_prefilling=rng.randint(1, max_requests),
                  prefill_step_size=step_size, max_tokens_per_step=budget)
    capacity = min(n_pages * page, 256)
    todo = []
    for _ in range(rng.randint(3, 9)):
        plen = rng.randint(1, max(1, min(120, capacity - 2)))
        new = rng.randint(1, max(1, min(40, capacity - plen)))
        todo.append((plen, new))
    info, out, reasons = {}, {}, {}
    n = 0
    while todo or s.has_work():
        while todo and (not s.has_work() or rng.random() < 0.3):
            plen, new = todo.pop()
            u = s.insert([rng.randrange(1000) for _ in range(plen)], max_tokens=new)
            info[u] = (plen, new)
        before = len(eng.steps)
        _, gens = s.next()
        for r in gens:
            out.setdefault(r.uid, []).append(r.token)
            if r.finish_reason:
                reasons[r.uid] = r.finish_reason
        for st in eng.steps[before:]:
            assert sum(cnt for _, _, cnt, _ in st) <= max(budget, 1)
            assert len(st) <= max_requests
            assert all(cnt <= step_size for _, start, cnt, _ in st if cnt > 1)
        assert sum(eng.cache.pages_in_use()) <= n_pages
        n += 1
        assert n < 20000, "the scheduler does not finish"
    for u, (plen, new) in info.items():
        assert out[u] == expected(u, plen, new), (seed, u)
        assert reasons[u] == "length"
    assert eng.cache.pages_in_use() == [0]
    eng.cache.check()


def test_stop_matcher():
    m = StopSequenceMatcher([[1, 2, 3], [7]])
    assert not m.matches([1, 2]) and m.matches([0, 1, 2, 3]) and m.matches([7]) and not m.matches([7, 1])
    assert not StopSequenceMatcher().matches([1])


def test_generate_step_drives_the_scheduler_for_one_request(monkeypatch):
    """The host side of ``generate_step`` with the fake engine and a stand-in for the device sampler: one pair
    per generated token, the vector that belongs to it, progress for every portion of the prompt, no
    end-of-sequence stop, and the request is gone afterwards."""
    import importlib
    from types import SimpleNamespace

    G = importlib.import_module("mlx_lm_b200.generate")
    eng = FakeEngine(n_pages=8)

    class Vector:
        def __init__(self, token):
            self.token = token

        def clone(self):
            return ("log-probabilities of", self.token)

    class StandInSampler:
        def __init__(self, device, seed=0, return_logprobs=False, engine=None):
            assert return_logprobs and engine is eng
            self.last_logprobs = None

        def __call__(self, rows, requests):
            tokens, logprobs = fake_sample(rows, requests)
            self.last_logprobs = [Vector(t) for t in tokens]
            return tokens, logprobs

    monkeypatch.setattr(G, "DeviceSampler", StandInSampler)
    monkeypatch.setattr(G, "get_engine", lambda model: eng)
    seen = []
    pairs = list(G.generate_step(list(range(11)), SimpleNamespace(device="cpu"), max_tokens=5, prefill_step_size=4,
                                 prompt_progress_callback=lambda done, total: seen.append((done, total))))
    want = expected(0, 11, 5)
    assert [t for t, _ in pairs] == want
    assert [v for _, v in pairs] == [("log-probabilities of", t) for t in want]
    assert seen == [(4, 11), (8, 11), (11, 11)]
    assert [sum(cnt for _, _, cnt, _ in st) for st in eng.steps] == [4, 4, 3, 1, 1, 1, 1]
    assert eng.cache.pages_in_use() == [0]
    # a generator that is dropped half way gives its pages back as well
    gen = G.generate_step(list(range(20)), SimpleNamespace(device="cpu"), max_tokens=50)
    next(gen), next(gen)
    gen.close()
    assert eng.cache.pages_in_use() == [0]


def test_a_status_word_from_the_kernels_stops_the_tokens():
    """The sampler brings the kernels' status word back with the tokens; if it is not zero the scheduler raises
    instead of handing the step's tokens out, and clears the word."""
    from mlx_lm_b200.ops import ST_PAGE_RANGE, ST_WAIT_TIMEOUT, KernelError

    class Reporting(FakeEngine):
        host_status = 0
        cleared = 0

        def clear_status(self):
            self.host_status = 0
            self.cleared += 1

    eng = Reporting(n_pages=8)
    s = Scheduler(eng, fake_sample)
    uid = s.insert(list(range(10)), max_tokens=4)
    _, gens = s.next()
    assert [r.uid for r in gens] == [uid]
    eng.host_status = ST_PAGE_RANGE | ST_WAIT_TIMEOUT
    with pytest.raises(KernelError) as err:
        s.next()
    assert "page id outside the pool" in str(err.value) and "bounded wait" in str(err.value)
    assert eng.host_status == 0 and eng.cleared == 1


def test_removed_requests_are_reported_as_cancelled_once():
    eng = FakeEngine(n_pages=16)
    s = Scheduler(eng, fake_sample, max_requests=1)
    a = s.insert(list(range(20)), max_tokens=50)
    b = s.insert(list(range(5)), max_tokens=50)          # still waiting: only one request runs
    s.next()
    gone = s.remove([a, b])
    assert sorted(r.uid for r in gone) == [a, b] and all(r.finish_reason == "cancelled" and r.token == -1 for r in gone)
    assert eng.cache.pages_in_use() == [0] and s.has_work()
    _, gens = s.next()
    assert sorted((r.uid, r.finish_reason) for r in gens) == [(a, "cancelled"), (b, "cancelled")]
    assert not s.has_work() and s.next() == ([], [])


def test_two_schedulers_on_one_engine_do_not_collide():
    """Uids start at 0 in every scheduler (they key the random draws); in the engine a request is named with
    the scheduler's namespace as well."""
    class Spaces(FakeEngine):
        n = 0

        def new_namespace(self):
            self.n += 1
            return self.n

    eng = Spaces(n_pages=16)
    s1, s2 = Scheduler(eng, fake_rid_sample), Scheduler(eng, fake_rid_sample)
    u1, u2 = s1.insert(list(range(9)), max_tokens=3), s2.insert(list(range(4)), max_tokens=3)
    assert u1 == u2 == 0
    s1.next(); s2.next(); s1.next(); s2.next()
    assert set(eng.cache.requests) == {(1, 0), (2, 0)}
    run(s1); run(s2)
    assert eng.cache.pages_in_use() == [0]


def fake_rid_sample(rows, requests):
    assert [r.rid for r in requests] == [rid for rid, _ in rows]
    return [token_fn(r.uid, pos + 1) for r, (_, pos) in zip(requests, rows)], [0.0] * len(rows)


# ---------------------------------------------------------------------------------------------- one step ahead

class Handle:
    def __init__(self, rids, tokens):
        self.rids, self.tokens, self.collected = rids, tokens, False


class AheadEngine(FakeEngine):
    """A fake of the engine's launch/collect pair: a launched step books its pages at once; its tokens (a function
    of request and position, as in ``fake_sample``) become known to the caller only at ``decode_collect``."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.launched, self.ahead_rows, self.in_flight = 0, 0, []

    def decode_sampled(self, entries, requests, sample):
        return self.decode_collect(self.decode_launch(entries, requests, sample))

    def decode_launch(self, entries, requests, sample, source=None):
        assert len(self.in_flight) < 2, "at most two steps in flight"
        rec, toks = [], []
        for i, e in enumerate(entries):
            assert len(e.tokens) == 1
            start = self.cache.reserve(e.rid, 1)
            assert start == len(self.fed[e.rid])
            if source is not None and source[1][i] >= 0:
                assert not source[0].collected
                tok = source[0].tokens[source[1][i]]          # handed over "on the device"
                assert source[0].rids[source[1][i]] == e.rid
                self.ahead_rows += 1
            else:
                tok = e.tokens[0]
            self.fed[e.rid].append(tok)
            rec.append((e.rid, start, 1, [0]))
            uid = e.rid[1] if isinstance(e.rid, tuple) else e.rid
            toks.append(token_fn(uid, start + 1))
        for e in entries:
            self.cache.commit(e.rid)
        self.cache.check()
        self.steps.append(rec)
        self.launched += 1
        h = Handle([e.rid for e in entries], toks)
        self.in_flight.append(h)
        return h

    def decode_collect(self, h):
        assert self.in_flight and self.in_flight[0] is h, "steps are collected in the order they were launched"
        self.in_flight.pop(0)
        h.collected = True
        return list(h.tokens), [0.0] * len(h.tokens)


def both_ways(n_pages, inserts, **kw):
    """The same requests with and without the step ahead: (tokens, reasons, engine) of each."""
    res = []
    for ahead in (False, True):
        eng = AheadEngine(n_pages=n_pages)
        s = Scheduler(eng, fake_sample, **kw)
        s.lookahead = ahead
        for prompt, max_tokens, stop in inserts:
            s.insert(prompt, max_tokens, stop=StopSequenceMatcher(stop) if stop else None)
        out, reasons = run(s)
        assert eng.cache.pages_in_use() == [0] and not eng.in_flight
        eng.cache.check()
        res.append((out, reasons, eng))
    return res


def test_a_step_ahead_gives_the_same_tokens():
    inserts = [(list(range(20)), 9, None), (list(range(33)), 30, None), (list(range(5)), 1, None),
               (list(range(47)), 17, None), (list(range(8)), 30, None)]
    (out0, why0, e0), (out1, why1, e1) = both_ways(64, inserts, max_requests=3, prefill_step_size=16,
                                                  max_tokens_per_step=32)
    assert out0 == out1 and why0 == why1
    for uid, (prompt, n, _) in enumerate(inserts):
        assert out1[uid] == expected(uid, len(prompt), n)
    assert e1.ahead_rows > 20 and e0.ahead_rows == 0
    # a request at its last token is not in the step ahead: nobody computes a token past max_tokens
    assert sum(len(st) for st in e1.steps) == sum(len(st) for st in e0.steps)


def test_a_stop_found_one_step_late_drops_the_row_computed_in_vain():
    # request 0 stops when its fourth token comes; the step ahead has computed its fifth by then
    stop_tok = expected(0, 12, 4)[3]
    inserts = [(list(range(12)), 20, [[stop_tok]]), (list(range(7)), 10, None)]
    (out0, why0, e0), (out1, why1, e1) = both_ways(32, inserts, max_requests=4)
    assert out0 == out1 and why0 == why1 == {0: "stop", 1: "length"}
    assert len(out1[0]) == 4
    assert sum(len(st) for st in e1.steps) == sum(len(st) for st in e0.steps) + 1     # the one row in vain


def test_pages_that_run_out_end_the_run_ahead_and_preemption_still_works():
    inserts = [(list(range(30)), 40, None), (list(range(30)), 40, None), (list(range(30)), 40, None)]
    (out0, why0, e0), (out1, why1, e1) = both_ways(11, inserts, max_requests=3)      # 11 pages of 16: not enough for all
    assert out0 == out1 and why0 == why1
    for uid in range(3):
        assert out1[uid] == expected(uid, 30, 40)


def test_cancelling_while_a_step_is_in_flight():
    eng = AheadEngine(n_pages=32)
    s = Scheduler(eng, fake_sample, max_requests=4)
    a = s.insert(list(range(10)), 50)
    b = s.insert(list(range(6)), 50)
    seen = {a: [], b: []}
    for _ in range(6):
        for r in s.next()[1]:
            seen[r.uid].append(r.token)
    assert s._inflight is not None
    s.remove([a])                                   # its row of the step in flight is dropped when that step is read
    for _ in range(5):
        for r in s.next()[1]:
            if r.finish_reason != "cancelled":
                assert r.uid == b
                seen[b].append(r.token)
    assert seen[b] == expected(b, 6, len(seen[b])) and len(seen[a]) <= 6
    s.remove([b])                                   # nobody left: the step in flight is waited for and dropped
    assert s._inflight is None and not eng.in_flight
    assert eng.cache.pages_in_use() == [0]
    eng.cache.check()
