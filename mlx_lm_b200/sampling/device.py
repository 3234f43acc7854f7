"""Runs the logits processors and the sampling kernel for the rows of one step and brings the
chosen tokens back to the host in one copy."""

from __future__ import annotations

import os
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from . import LogitsProcessors


class DeviceSampler:
    """``sampler(logits[R, V], requests) -> (tokens, logprobs)`` for the scheduler.

    Row ``i`` of ``logits`` belongs to ``requests[i]``, which carries its ``Sampler``, its
    processors, its token history and its uid; the position of the token being drawn is the
    length of that history, so the random draw is a function of (seed, uid, position) alone.

    ``seed=None`` draws a seed from the operating system, so that two unseeded runs differ, as they do in
    mlx-lm, whose generator is seeded only by ``--seed`` (mlx_lm/generate.py:2067-2068).  With an ``engine``
    the kernel brings the engine's status word back together with the tokens (``engine.host_status``)."""

    def __init__(self, device, seed: Optional[int] = 0, return_logprobs: bool = False, engine=None):
        if seed is None:
            seed = int.from_bytes(os.urandom(8), "little")
        self.device, self.seed, self.return_logprobs, self.engine = device, int(seed), return_logprobs, engine
        self._cap = 0
        self._host = self._dev_params = self._out = self._out_host = self._scratch = None
        self.last_logprobs = None

    def _ensure(self, R: int) -> None:
        if R <= self._cap:
            return
        cap = max(64, 2 * R)
        self._host = torch.empty(cap * ops.SAMPLE_WORDS, dtype=torch.int32).pin_memory()
        self._dev_params = torch.empty(cap * ops.SAMPLE_WORDS, dtype=torch.int32, device=self.device)
        self._out = torch.zeros(2 * cap + 1, dtype=torch.int32, device=self.device)   # tokens | logprob bits | status
        self._scratch = ops.sample_scratch(cap, self.device)
        self._out_host = torch.zeros(2 * cap + 1, dtype=torch.int32).pin_memory()
        self._cap = cap

    def __call__(self, logits: torch.Tensor, requests: Sequence) -> Tuple[List[int], List[float]]:
        R = len(requests)
        stream = ops.current_stream()
        self._ensure(R)
        self._process(logits, requests, stream)
        special: List[int] = []          # every row's own XTC special tokens, one list after the other
        recs = []
        for r in requests:
            recs.append(r.sampler.words(self.seed, r.uid, len(r.tokens), special_offset=len(special)))
            special.extend(r.sampler.xtc_special_tokens)
        self._host.numpy()[:R * ops.SAMPLE_WORDS] = np.frombuffer(b"".join(recs), dtype=np.int32)
        self._dev_params[:R * ops.SAMPLE_WORDS].copy_(self._host[:R * ops.SAMPLE_WORDS], non_blocking=True)
        xs = torch.tensor(special, dtype=torch.int32, device=self.device) if special else None
        cap = self._cap
        tok = self._out[:R]
        lp = self._out[cap:cap + R].view(torch.float32)
        full = None
        if self.return_logprobs:
            full = torch.empty_like(logits)
        status = self.engine.status if self.engine is not None else None
        ops.sample(logits, self._dev_params, tok, lp, stream, xtc_special=xs, out_logprobs=full, status=status,
                   status_out=self._out[2 * cap:] if status is not None else None,
                   scratch=None if any(r.sampler.filters for r in requests) else self._scratch)
        self.last_logprobs = full
        self._out_host.copy_(self._out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        h = self._out_host.numpy()
        if self.engine is not None:
            self.engine.host_status = int(h[2 * cap])
            self.engine.h2d_bytes += 4 * (R * ops.SAMPLE_WORDS + len(special))
            self.engine.d2h_bytes += 4 * self._out.numel()
        return h[:R].tolist(), h[cap:cap + R].view(np.float32).tolist()

    def _process(self, logits, requests, stream) -> None:
        """Each request's processors in the order of its list.  The lists are walked in rounds: in round j the
        rows whose j-th processor is a ``LogitsProcessors`` record go through the kernel together (the other
        rows get a record that does nothing), and a row whose j-th processor is a callable is given to it as
        mlx-lm does: ``f(tokens, logits[1, V]) -> logits`` (mlx_lm/generate.py:402-404)."""
        rounds = max((len(r.processors) for r in requests), default=0)
        for j in range(rounds):
            procs = []
            for i, r in enumerate(requests):
                p = r.processors[j] if j < len(r.processors) else None
                if p is not None and not isinstance(p, LogitsProcessors):
                    row = logits[i:i + 1]
                    new = p(torch.tensor(r.tokens, device=logits.device), row)
                    if new is not row:
                        row.copy_(new)
                    p = None
                procs.append(p)
            if any(procs):
                self._run_records(logits, requests, procs, stream)

    def _run_records(self, logits, requests, procs, stream) -> None:
        R = len(requests)
        C = max(max((p.context_size for p in procs if p), default=0), 1)
        B = max(max((len(p.logit_bias) for p in procs if p), default=0), 1)
        params = np.zeros((R, ops.PROCESS_WORDS), dtype=np.int32)
        ctx = np.full((R, C), -1, dtype=np.int32)
        bidx = np.full((R, B), -1, dtype=np.int32)
        bval = np.zeros((R, B), dtype=np.float32)
        for i, (r, p) in enumerate(zip(requests, procs)):
            if p is None:
                continue
            params[i] = np.frombuffer(p.words(), dtype=np.int32)
            tail = r.tokens[-p.context_size:] if p.context_size else []
            if tail:
                ctx[i, C - len(tail):] = tail
            for j, (t, v) in enumerate(p.logit_bias):
                bidx[i, j], bval[i, j] = t, v
        dev = lambda a: torch.from_numpy(a).to(self.device)
        ops.process_logits(logits, dev(params.reshape(-1)), dev(ctx), dev(bidx), dev(bval), stream)
