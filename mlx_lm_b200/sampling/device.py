"""Runs the logits processors and the sampling kernel for the rows of one step and brings the
chosen tokens back to the host in one copy."""

from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from . import LogitsProcessors


class DeviceSampler:
    """``sampler(logits[R, V], requests) -> (tokens, logprobs)`` for the scheduler.

    Row ``i`` of ``logits`` belongs to ``requests[i]``, which carries its ``Sampler``, its
    processors, its token history and its uid; the position of the token being drawn is the
    length of that history, so the random draw is a function of (seed, uid, position) alone."""

    def __init__(self, device, seed: int = 0, return_logprobs: bool = False):
        self.device, self.seed, self.return_logprobs = device, int(seed), return_logprobs
        self._cap = 0
        self._host = self._dev_params = self._out = self._out_host = None
        self.last_logprobs = None

    def _ensure(self, R: int) -> None:
        if R <= self._cap:
            return
        cap = max(64, 2 * R)
        self._host = torch.empty(cap * ops.SAMPLE_WORDS, dtype=torch.int32).pin_memory()
        self._dev_params = torch.empty(cap * ops.SAMPLE_WORDS, dtype=torch.int32, device=self.device)
        self._out = torch.empty(2 * cap, dtype=torch.int32, device=self.device)   # tokens | logprob bits
        self._out_host = torch.empty(2 * cap, dtype=torch.int32).pin_memory()
        self._cap = cap

    def __call__(self, logits: torch.Tensor, requests: Sequence) -> Tuple[List[int], List[float]]:
        R = len(requests)
        stream = ops.current_stream()
        self._ensure(R)
        self._process(logits, requests, stream)
        rec = b"".join(r.sampler.words(self.seed, r.uid, len(r.tokens)) for r in requests)
        self._host.numpy()[:R * ops.SAMPLE_WORDS] = np.frombuffer(rec, dtype=np.int32)
        self._dev_params[:R * ops.SAMPLE_WORDS].copy_(self._host[:R * ops.SAMPLE_WORDS], non_blocking=True)
        special = {t for r in requests for t in r.sampler.xtc_special_tokens}
        xs = torch.tensor(sorted(special), dtype=torch.int32, device=self.device) if special else None
        cap = self._cap
        tok = self._out[:R]
        lp = self._out[cap:cap + R].view(torch.float32)
        full = None
        if self.return_logprobs:
            full = torch.empty_like(logits)
        ops.sample(logits, self._dev_params, tok, lp, stream, xtc_special=xs, out_logprobs=full)
        self.last_logprobs = full
        self._out_host[:cap + R].copy_(self._out[:cap + R], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        h = self._out_host.numpy()
        return h[:R].tolist(), h[cap:cap + R].view(np.float32).tolist()

    def _process(self, logits, requests, stream) -> None:
        procs = []
        for r in requests:
            mine = [p for p in r.processors if isinstance(p, LogitsProcessors)]
            if len(mine) > 1:
                raise ValueError("give one LogitsProcessors record per request (make_logits_processors returns one)")
            procs.append(mine[0] if mine else None)
        for i, r in enumerate(requests):   # user callables, as mlx-lm runs them: f(tokens, logits) -> logits
            for p in r.processors:
                if not isinstance(p, LogitsProcessors):
                    row = logits[i:i + 1]
                    new = p(torch.tensor(r.tokens, device=logits.device), row)
                    if new is not row:
                        row.copy_(new)
        if not any(procs):
            return
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
