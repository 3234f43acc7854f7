"""Continuous batching above the step function.

mlx-lm's ``BatchGenerator`` (mlx_lm/generate.py:1565-1945) keeps a queue of
unprocessed sequences, one rectangular prompt batch and one decode batch, and
runs them as separate model calls.  Here every iteration is ONE step of the
engine: each running request contributes the tokens it has not run yet — one
for a decoding request, a portion of the prompt for a prefilling one — under
a budget of tokens per step, decoding requests first.

Decisions, all made in ``plan`` (plain Python, no device):

* admit     from the front of ``waiting`` while fewer than ``max_requests`` run, fewer than
            ``max_prefilling`` of them are still in their prompt, a state slot is free and pages for
            the request's first portion are free;
* portions  a prompt is cut under ``prefill_step_size`` per request and ``max_tokens_per_step`` for
            the whole step, and further down to what the free pages can hold;
* pages run out
            if a decoding request cannot get the page its next token needs, or nothing at all can
            run, the most recently admitted running request is preempted: it gives back all its
            pages and goes to the FRONT of ``waiting`` with prompt := prompt + tokens generated so
            far (recompute); tokens already handed out stay handed out.  A request that could never
            fit the pool alone is refused at ``insert``;
* finishing ``"length"`` at ``max_tokens`` generated tokens, ``"stop"`` when a stop sequence matches
            (mlx_lm/generate.py:1504-1514), ``"cancelled"`` for a request taken out with ``remove``
            (reported once, by the next ``next``); pages and slot are given back at once.

One step ahead: while the device runs a pure decode step, the host cannot know its tokens, but it knows nearly
everything else about the step after it (who goes on, positions, pages, sampling records), and the tokens can stay on
the device.  So before ``next`` waits for a decode step it launches the following one (``lookahead``; the engine's
``decode_launch`` with the step in flight as the source of the tokens) whenever nothing else is due: nobody waits to be
admitted, nobody is in its prompt, pages are there.  Requests that reach ``max_tokens`` with the step in flight are
left out; a request that turns out to have stopped (a stop sequence) or was cancelled has one row computed in vain,
which is dropped when that step is read.  The tokens are the same with and without (mlx-lm overlaps the same way:
``mx.async_eval`` of the next step before the current token is read, mlx_lm/generate.py:434-451).

After every step that hands out tokens the scheduler looks at the status word the kernels set instead of
faulting (a token, position or page id out of range, a bounded wait that gave up), which the sampler brought
back with the tokens, and raises ``KernelError`` rather than hand out tokens of a step that went wrong.

The scheduler talks to an engine through five calls (``add_request``, ``finish``, ``step``,
``cache`` for page arithmetic, ``max_len``), and to a ``sample`` callable; tests drive it with fakes.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

from ..cache import OutOfPages
from ..sampling import GREEDY, LogitsProcessors, Sampler
from .step import StepEntry


class StopSequenceMatcher:
    """Match any of several token sequences at the end of a stream (mlx_lm/generate.py:887-956 does
    this with an Aho-Corasick trie; the sequences here are few and short, so the tail is compared)."""

    def __init__(self, stop_sequences: Optional[Sequence[Sequence[int]]] = None):
        self.sequences = [tuple(s) for s in (stop_sequences or []) if len(s)]
        self.longest = max((len(s) for s in self.sequences), default=0)

    def matches(self, generated: Sequence[int]) -> bool:
        n = len(generated)
        for s in self.sequences:
            k = len(s)
            if k <= n and tuple(generated[n - k:]) == s:
                return True
        return False


@dataclass
class Request:
    uid: int
    tokens: List[int]                 # prompt, then generated tokens as they come
    n_prompt: int
    max_tokens: int
    sampler: Sampler = GREEDY
    processors: Sequence = ()
    stop: StopSequenceMatcher = field(default_factory=StopSequenceMatcher)
    n_cached: int = 0                 # tokens whose keys/values are in the cache
    n_generated: int = 0
    admitted_at: int = -1             # admission counter; -1 while waiting
    preemptions: int = 0
    rid: object = None                # the request's name in the engine (None: its uid)

    def __post_init__(self):
        if self.rid is None:
            self.rid = self.uid

    @property
    def remaining(self) -> int:
        return len(self.tokens) - self.n_cached

    @property
    def generated(self) -> List[int]:
        return self.tokens[self.n_prompt:]


@dataclass
class Response:
    """One generated token (the shape of ``GenerationBatch.Response``, mlx_lm/generate.py:1321-1328)."""
    uid: int
    token: int
    logprobs: float                   # log-probability of ``token``; a [V] tensor if full log-probs were asked for
    finish_reason: Optional[str]
    prompt_cache: Optional[object] = None
    all_tokens: Optional[List[int]] = None


@dataclass
class PromptProgress:
    """Progress of a prompt (``PromptProcessingBatch.Response``, mlx_lm/generate.py:1096-1101)."""
    uid: int
    progress: Tuple[int, int]
    end_of_segment: bool
    end_of_prompt: bool


@dataclass
class PlannedEntry:
    request: Request
    n_tokens: int
    wants_logits: bool


@dataclass
class SchedulerStats:
    steps: int = 0
    tokens: int = 0
    prompt_tokens: int = 0
    generation_tokens: int = 0
    preemptions: int = 0
    most_running: int = 0


class Scheduler:
    def __init__(self, engine, sample: Callable, max_requests: int = 32, max_prefilling: int = 8,
                 prefill_step_size: int = 2048, max_tokens_per_step: int = 2048):
        self.engine, self.sample = engine, sample
        self.max_requests = max_requests
        self.max_prefilling = max(1, max_prefilling)
        self.prefill_step_size = max(1, prefill_step_size)
        self.max_tokens_per_step = max(1, max_tokens_per_step)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._uid = 0
        # uids start at 0 in every scheduler (and key the random draws, so that a seed gives the same tokens
        # again); in the engine a request is named by (scheduler, uid), so that two schedulers on one engine
        # never collide
        self._namespace = engine.new_namespace() if hasattr(engine, "new_namespace") else None
        self._cancelled: List[Response] = []
        self._inflight = None          # (handle, planned entries) of a decode step launched but not read yet
        self.lookahead = True
        self._admissions = 0
        self.stats = SchedulerStats()
        self.last_step_tokens = self.last_step_prompt_tokens = 0

    # ------------------------------------------------------------------ requests in and out
    def insert(self, prompt: Sequence[int], max_tokens: int, sampler: Optional[Sampler] = None,
               processors: Sequence = (), stop: Optional[StopSequenceMatcher] = None) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("a prompt needs at least one token")
        cache = self.engine.cache
        total = len(prompt) + max_tokens
        if total - 1 > self.engine.max_len:
            raise ValueError(f"prompt of {len(prompt)} tokens plus {max_tokens} new tokens needs {total - 1} "
                             f"positions; the model has {self.engine.max_len}")
        need = (total - 1 + cache.page_size - 1) // cache.page_size
        for g in cache.kv_groups:
            held = need if g.spec.window is None else min(
                need, (g.spec.window + self.prefill_step_size) // cache.page_size + 2)
            if held > g.pool.n_pages:
                raise ValueError(f"the request may hold {held} pages; the pool has {g.pool.n_pages} in all")
        uid = self._uid
        self._uid += 1
        self.waiting.append(Request(uid, prompt, len(prompt), max_tokens, sampler or GREEDY, tuple(processors),
                                    stop or StopSequenceMatcher(),
                                    rid=uid if self._namespace is None else (self._namespace, uid)))
        return uid

    def remove(self, uids: Sequence[int]) -> List[Response]:
        """Take requests out at any stage (mlx_lm/generate.py:1777-1802).  Each gets one last response with
        ``finish_reason="cancelled"`` and no token (-1), returned here and once more by the next ``next``."""
        uids = set(uids)
        gone = [r for r in self.running if r.uid in uids]
        for r in gone:
            self.engine.finish(r.rid)
            self.running.remove(r)
        gone += [r for r in self.waiting if r.uid in uids]
        self.waiting = deque(r for r in self.waiting if r.uid not in uids)
        out = [Response(r.uid, -1, 0.0, "cancelled", all_tokens=list(r.tokens)) for r in gone]
        self._cancelled.extend(out)
        if self._inflight is not None and not any(p.request in self.running for p in self._inflight[1]):
            self.engine.decode_collect(self._inflight[0])      # nobody is left to read that step: wait and drop it
            self._inflight = None
        return out

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self._cancelled or self._inflight)

    # ------------------------------------------------------------------ decisions
    def _preempt(self, victim: Request) -> None:
        self.engine.finish(victim.rid)
        self.running.remove(victim)
        victim.n_cached = 0
        victim.admitted_at = -1
        victim.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(victim)

    def _fits(self, taken: List[int], r: Request, n: int) -> Optional[List[int]]:
        """The pages per group that n more tokens of r take, if the pools still have them beside the ``taken``
        pages of the entries planned so far; else None."""
        cache = self.engine.cache
        need = cache.pages_needed(r.rid, n)
        for t, c, g in zip(taken, need, cache.kv_groups):
            if t + c > g.pool.n_free:
                return None
        return need

    def _largest_portion(self, taken: List[int], r: Request, n: int) -> int:
        """The longest portion <= n of r's tokens whose pages are free (0 if not even one token fits)."""
        if self._fits(taken, r, n) is not None:
            return n
        lo, hi = 0, n - 1
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self._fits(taken, r, mid) is not None:
                lo = mid
            else:
                hi = mid - 1
        return lo

    def _take(self, taken: List[int], r: Request, n: int) -> None:
        for g, c in enumerate(self.engine.cache.pages_needed(r.rid, n)):
            taken[g] += c

    def plan(self) -> List[PlannedEntry]:
        """Decide this step's entries; admits and preempts as a side effect."""
        while True:
            planned: List[PlannedEntry] = []
            taken = [0] * len(self.engine.cache.kv_groups)      # pages the planned entries will take, per group
            budget = self.max_tokens_per_step
            starved: Optional[Request] = None
            # decoding requests first, oldest first
            for r in sorted(self.running, key=lambda r: r.admitted_at):
                if r.remaining != 1 or budget <= 0:
                    continue
                need = self._fits(taken, r, 1)
                if need is not None:
                    planned.append(PlannedEntry(r, 1, True))
                    taken = [t + c for t, c in zip(taken, need)]
                    budget -= 1
                else:
                    starved = r
                    break
            if starved is not None:
                victim = max(self.running, key=lambda r: r.admitted_at)
                self._preempt(victim)
                continue
            # portions of prompts that are under way
            for r in sorted(self.running, key=lambda r: r.admitted_at):
                if r.remaining <= 1 or budget <= 0:
                    continue
                n = self._largest_portion(taken, r, min(r.remaining, self.prefill_step_size, budget))
                if n > 0:
                    planned.append(PlannedEntry(r, n, n == r.remaining))
                    self._take(taken, r, n)
                    budget -= n
            # admissions
            while (self.waiting and budget > 0 and len(self.running) < self.max_requests
                   and sum(1 for r in self.running if r.remaining > 1) < self.max_prefilling
                   and self.engine.cache.has_free_slot()):
                r = self.waiting[0]
                self.engine.add_request(r.rid)
                n = self._largest_portion(taken, r, min(r.remaining, self.prefill_step_size, budget))
                if n == 0:
                    self.engine.finish(r.rid)
                    break
                self._take(taken, r, n)
                self.waiting.popleft()
                r.admitted_at = self._admissions
                self._admissions += 1
                self.running.append(r)
                planned.append(PlannedEntry(r, n, n == r.remaining))
                budget -= n
            if planned or not self.running:
                if not planned and self.waiting:
                    raise OutOfPages("a waiting request cannot start although nothing is running")
                return planned
            # nothing can move: free the newest request's pages and try again
            self._preempt(max(self.running, key=lambda r: r.admitted_at))

    # ------------------------------------------------------------------ one iteration
    def next(self) -> Tuple[List[PromptProgress], List[Response]]:
        cancelled, self._cancelled = self._cancelled, []
        if self._inflight is not None:
            return [], cancelled + self._read_inflight()
        planned = self.plan()
        self.last_step_tokens = self.last_step_prompt_tokens = 0
        if not planned:
            return [], cancelled
        entries = [StepEntry(p.request.rid, p.request.tokens[p.request.n_cached:p.request.n_cached + p.n_tokens],
                             [p.n_tokens - 1] if p.wants_logits else []) for p in planned]
        sampled = [p.request for p in planned if p.wants_logits]
        fused = (len(sampled) == len(planned) and hasattr(self.engine, "decode_sampled")
                 and all(p.n_tokens == 1 for p in planned))
        if fused and self.lookahead and hasattr(self.engine, "decode_launch"):
            handle = self.engine.decode_launch(entries, sampled, self.sample)
            if handle is not None:      # a CUDA graph took it: on its way; the step after it may follow before we wait
                self._inflight = (handle, planned)
                return [], cancelled + self._read_inflight()
        if fused:     # a pure decode step: model and sampler in one call (a CUDA graph where it fits)
            tokens, logprobs = self.engine.decode_sampled(entries, sampled, self.sample)
        else:
            logits = self.engine.step(entries)
            tokens, logprobs = self.sample(logits, sampled) if sampled else ([], [])
        if sampled:
            self._check_status()
        prompts, responses = self._account(planned, tokens, logprobs)
        return prompts, cancelled + responses

    def _read_inflight(self) -> List[Response]:
        """The tokens of the decode step in flight; before waiting for them, the step after it is launched if it
        can be laid out without them."""
        handle, planned = self._inflight
        self._inflight = None
        ahead = self._launch_ahead(handle, planned)
        tokens, logprobs = self.engine.decode_collect(handle)
        self._check_status()
        self.last_step_tokens = self.last_step_prompt_tokens = 0
        _, responses = self._account(planned, tokens, logprobs)
        self._inflight = ahead
        return responses

    def _launch_ahead(self, handle, planned: List[PlannedEntry]):
        """Launch the decode step that follows the one in flight, or None if that step cannot be decided yet:
        somebody waits for admission or was cancelled, somebody is still in its prompt, nobody goes on, or pages
        are short (``plan`` then decides, with the tokens in hand)."""
        if self.waiting or self._cancelled:
            return None
        live = {id(r) for r in self.running}
        flying = {id(p.request) for p in planned}
        if any(id(r) not in flying for r in self.running):
            return None
        rows, goes_on = [], []
        for i, p in enumerate(planned):
            r = p.request
            if id(r) in live and r.n_generated + 1 < r.max_tokens:      # not cancelled, not at its last token
                rows.append(i)
                goes_on.append(r)
        if not goes_on:
            return None
        taken = [0] * len(self.engine.cache.kv_groups)
        for r in goes_on:
            need = self._fits(taken, r, 1)
            if need is None:
                return None
            taken = [t + c for t, c in zip(taken, need)]
        entries = [StepEntry(r.rid, [0], [0]) for r in goes_on]     # the tokens are on the device
        try:
            ahead = self.engine.decode_launch(entries, goes_on, self.sample, source=(handle, rows))
        except OutOfPages:       # (the check above should have seen it) nothing was booked: decide with the tokens in hand
            return None
        if ahead is None:
            return None
        return ahead, [PlannedEntry(r, 1, True) for r in goes_on]

    def _account(self, planned: List[PlannedEntry], tokens, logprobs) -> Tuple[List[PromptProgress], List[Response]]:
        """Book a finished step: progress of prompts, the new tokens, who is done.  Rows of requests that have left
        meanwhile (stopped or cancelled while the step was in flight) are dropped."""
        self.stats.steps += 1
        self.stats.most_running = max(self.stats.most_running, len(self.running))
        live = {id(r) for r in self.running}
        prompts: List[PromptProgress] = []
        for p in planned:
            r = p.request
            if id(r) not in live:
                continue
            if r.n_cached < r.n_prompt:
                done = min(r.n_cached + p.n_tokens, r.n_prompt)
                self.stats.prompt_tokens += done - r.n_cached
                self.last_step_prompt_tokens += done - r.n_cached
                prompts.append(PromptProgress(r.uid, (done, r.n_prompt), done == r.n_prompt, done == r.n_prompt))
            r.n_cached += p.n_tokens
            self.stats.tokens += p.n_tokens
            self.last_step_tokens += p.n_tokens
        responses: List[Response] = []
        sampled = [p.request for p in planned if p.wants_logits]
        for r, tok, lp in zip(sampled, tokens, logprobs):
            if id(r) not in live:
                continue
            r.tokens.append(int(tok))
            r.n_generated += 1
            self.stats.generation_tokens += 1
            reason = None
            if r.stop.matches(r.generated):
                reason = "stop"
            elif r.n_generated >= r.max_tokens:
                reason = "length"
            if reason is not None:
                self.engine.finish(r.rid)
                self.running.remove(r)
            responses.append(Response(r.uid, int(tok), lp, reason,
                                      all_tokens=list(r.tokens) if reason is not None else None))
        return prompts, responses

    def _check_status(self) -> None:
        """Raise if a kernel of the steps since the last look reported something (``Engine.host_status``: the
        status word as the sampler's copy of the tokens brought it to the host; no synchronisation here)."""
        word = getattr(self.engine, "host_status", 0)
        if word:
            from ..ops import KernelError, describe_status
            self.engine.clear_status()
            raise KernelError("a kernel reported: " + describe_status(word) + "; the tokens of this step are not "
                              "handed out")
