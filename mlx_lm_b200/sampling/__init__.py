"""Samplers and logits processors with mlx-lm's names and meanings
(``make_sampler`` / ``make_logits_processors``, mlx_lm/sample_utils.py:10-126).

In mlx-lm a sampler is a function on an array of log-probabilities.  Here the
work is one CUDA kernel per step for all rows, so ``make_sampler`` returns a
``Sampler`` record of options that the scheduler packs, row by row, into the
kernel's parameter table; the record is also callable on a float32 CUDA tensor
of logits or log-probabilities ``[R, V]`` and returns token ids, for use
outside the scheduler.  ``make_logits_processors`` returns one
``LogitsProcessors`` record in a list (mlx-lm returns a list of closures); a
plain callable ``f(tokens, logits) -> logits`` in that list is run as is, on a
``[1, V]`` float32 CUDA tensor.
"""

from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np


@dataclass(frozen=True)
class Sampler:
    temp: float = 0.0
    top_p: float = 0.0
    min_p: float = 0.0
    min_tokens_to_keep: int = 1
    top_k: int = 0
    xtc_probability: float = 0.0
    xtc_threshold: float = 0.1
    xtc_special_tokens: tuple = ()
    seed: Optional[int] = None     # None: the scheduler's seed

    @property
    def filters(self) -> bool:
        """Whether the draw is restricted (top-p, min-p, XTC, top-k): such rows take many passes over the
        vocabulary in the kernel, greedy and plain temperature rows one."""
        return self.temp != 0 and (0 < self.top_p < 1 or self.min_p > 0 or self.xtc_probability > 0 or self.top_k > 0)

    def words(self, seed: int, request: int, position: int, special_offset: int = 0) -> bytes:
        """The 16 words of csrc/sampling.cu's SampleParams for one row.  ``special_offset``: where this
        row's XTC special tokens begin in the list the kernel is given."""
        s = self.seed if self.seed is not None else seed
        return struct.pack("<5f2i4I5i", self.temp, self.top_p, self.min_p, self.xtc_probability, self.xtc_threshold,
                           self.top_k, self.min_tokens_to_keep, s & 0xFFFFFFFF, (s >> 32) & 0xFFFFFFFF,
                           request & 0xFFFFFFFF, position & 0xFFFFFFFF, special_offset,
                           len(self.xtc_special_tokens), 0, 0, 0)

    def __call__(self, logprobs, seed: int = 0, request: int = 0, position: int = 0):
        import torch

        from .. import ops

        R = logprobs.shape[0]
        rec = np.frombuffer(b"".join(self.words(seed, request + r, position) for r in range(R)), dtype=np.int32)
        params = torch.from_numpy(rec.copy()).to(logprobs.device)
        tok = torch.empty(R, dtype=torch.int32, device=logprobs.device)
        lp = torch.empty(R, dtype=torch.float32, device=logprobs.device)
        special = None
        if self.xtc_special_tokens:
            special = torch.tensor(list(self.xtc_special_tokens), dtype=torch.int32, device=logprobs.device)
        ops.sample(logprobs.contiguous(), params, tok, lp, ops.current_stream(), xtc_special=special)
        return tok


def make_sampler(temp: float = 0.0, top_p: float = 0.0, min_p: float = 0.0, min_tokens_to_keep: int = 1,
                 top_k: int = 0, xtc_probability: float = 0.0, xtc_threshold: float = 0.1,
                 xtc_special_tokens: Sequence[int] = (), seed: Optional[int] = None) -> Sampler:
    """Options as in mlx_lm/sample_utils.py:10-69; the same values are refused
    (:142-146, 175-182, 256-263)."""
    if temp < 0:
        raise ValueError(f"`temp` has to be non-negative, but is {temp}")
    if not 0 <= min_p <= 1.0:
        raise ValueError(f"`min_p` has to be a float in the [0, 1] interval, but is {min_p}")
    if not isinstance(min_tokens_to_keep, int) or min_tokens_to_keep < 1:
        raise ValueError(f"`min_tokens_to_keep` has to be a positive integer, but is {min_tokens_to_keep}")
    if not isinstance(top_k, int) or top_k < 0:
        raise ValueError(f"`top_k` has to be a non-negative integer, but is {top_k}")
    if not 0 <= xtc_threshold <= 0.5:
        raise ValueError(f"`threshold` has to be a float in the [0, 0.5] interval, but is {xtc_threshold}")
    if not 0 <= xtc_probability <= 1.0:
        raise ValueError(f"`probability` has to be a float in the [0, 1] interval, but is {xtc_probability}")
    if len(xtc_special_tokens) > 64:
        raise ValueError("at most 64 xtc_special_tokens")
    if temp == 0:
        return Sampler(seed=seed)
    return Sampler(float(temp), float(top_p), float(min_p), min_tokens_to_keep, top_k, float(xtc_probability),
                   float(xtc_threshold), tuple(int(t) for t in xtc_special_tokens), seed)


@dataclass(frozen=True)
class LogitsProcessors:
    logit_bias: tuple = ()                 # ((token, value), ...)
    repetition_penalty: float = 0.0
    repetition_context_size: int = 20
    presence_penalty: float = 0.0
    presence_context_size: int = 20
    frequency_penalty: float = 0.0
    frequency_context_size: int = 20

    @property
    def context_size(self) -> int:
        sizes = [0]
        if self.repetition_penalty:
            sizes.append(self.repetition_context_size)
        if self.presence_penalty:
            sizes.append(self.presence_context_size)
        if self.frequency_penalty:
            sizes.append(self.frequency_context_size)
        return max(sizes)

    def words(self) -> bytes:
        """The 8 words of csrc/sampling.cu's ProcessParams for one row."""
        return struct.pack("<3f5i", self.repetition_penalty, self.presence_penalty, self.frequency_penalty,
                           self.repetition_context_size, self.presence_context_size, self.frequency_context_size,
                           len(self.logit_bias), 0)


def make_logits_processors(logit_bias: Optional[Dict[int, float]] = None, repetition_penalty: Optional[float] = None,
                           repetition_context_size: Optional[int] = 20, presence_penalty: Optional[float] = None,
                           presence_context_size: Optional[int] = 20, frequency_penalty: Optional[float] = None,
                           frequency_context_size: Optional[int] = 20) -> List[LogitsProcessors]:
    """Options as in mlx_lm/sample_utils.py:72-126.  Returns a list (empty if nothing is set)."""
    if repetition_penalty is not None and (not isinstance(repetition_penalty, (int, float)) or repetition_penalty < 0):
        raise ValueError(f"penalty must be a non-negative float, got {repetition_penalty}")
    p = LogitsProcessors(tuple((int(k), float(v)) for k, v in (logit_bias or {}).items()),
                         float(repetition_penalty or 0.0), int(repetition_context_size or 20),
                         float(presence_penalty or 0.0), int(presence_context_size or 20),
                         float(frequency_penalty or 0.0), int(frequency_context_size or 20))
    if not p.logit_bias and not p.repetition_penalty and not p.presence_penalty and not p.frequency_penalty:
        return []
    return [p]


GREEDY = Sampler()

__all__ = ["Sampler", "LogitsProcessors", "make_sampler", "make_logits_processors", "GREEDY"]
