"""What every part of a model is made of: named tensors it expects from the
weight files, a ``bind`` step that receives them in the run's dtype on the
device, and a ``forward`` that launches kernels.  No part knows which model
it is in: sizes, constants and tensor names are constructor parameters.

Kinds of parts and the interface each must have
-----------------------------------------------
``Norm``            ``forward(ctx, x, rows=None) -> y``  (``rows``: int32
                    device tensor selecting input rows)
``PositionEncoding`` ``embedding_table()`` (table added to the token embedding
                    by position, or None), ``rotate(ctx, q, k)`` (in place, on
                    this step's queries and keys, before keys enter the cache)
                    and ``max_positions`` (None = unbounded)
``Mixer``           ``cache_spec()`` (what it keeps per request: a
                    ``PagedKVSpec``, a ``StateSpec`` or None) and
                    ``forward(ctx, x, residual, cache) -> residual + mix(x)``
``FeedForward``     ``forward(ctx, x, residual) -> residual + f(x)``
``Block``           ``forward(ctx, x, cache) -> x'``: the arrangement of two
                    norms, a mixer and a feed-forward

A new kind is added by subclassing and registering under a name
(``register_part``); architectures refer to parts by those names or hand over
instances directly.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

MATRIX = "matrix"    # cast to the run's dtype (bfloat16 or float32)
VECTOR = "vector"    # gains and biases: always held in float32
INT_TABLE = "int"    # integer tables: held as int32


@dataclass(frozen=True)
class Init:
    """How the random-weights mode fills a tensor: normal(mean, std) or a constant."""
    mean: float = 0.0
    std: float = 0.02


@dataclass(frozen=True)
class ParamSpec:
    name: str                  # tensor name in the weight files (no "transformer."/"model." prefix)
    shape: Tuple[int, ...]     # shape as stored in the files
    kind: str = MATRIX
    init: Init = Init()


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every position (``window=None``) or of the last ``window`` positions."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, one row of ``shape`` per request, float32."""
    shape: Tuple[int, ...]


class Part:
    kernel_libs: Tuple[str, ...] = ()   # names under csrc/ this part launches kernels from
    # True if forward() does nothing but launch kernels through mlx_lm_b200.ops, with arguments that are
    # fixed by the step's shape (token, request, wanted-row, single-token and tile counts).  The engine
    # then re-issues a recorded step of the same shape without calling forward() again.  Leave it False
    # for a part that does anything else (host-side loops over requests, torch operators, ...).
    replayable: bool = False

    def param_specs(self) -> List[ParamSpec]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """Take the loaded tensors (already cast and on the device) this part named."""

    def children(self) -> Sequence["Part"]:
        return ()

    def all_param_specs(self) -> List[ParamSpec]:
        out = list(self.param_specs())
        for c in self.children():
            out.extend(c.all_param_specs())
        return out

    def all_replayable(self) -> bool:
        return self.replayable and all(c.all_replayable() for c in self.children())

    def all_kernel_libs(self) -> List[str]:
        out = list(self.kernel_libs)
        for c in self.children():
            out.extend(c.all_kernel_libs())
        return out

    def bind_all(self, tensors, dtype, device) -> None:
        self.bind(tensors, dtype, device)
        for c in self.children():
            c.bind_all(tensors, dtype, device)


class Norm(Part):
    def forward(self, ctx, x, rows=None):
        raise NotImplementedError

    def fold_args(self):
        """``(gain, bias, eps)`` if this is a LayerNorm (mean and variance over the row, gain, optional bias)
        that a linear layer can fold into its weights, else None."""
        return None

    def deferred(self, ctx, x, rows=None, tag: str = "normed") -> "Normed":
        """This norm of ``x`` as a value that is computed when (and if) somebody asks for the tensor."""
        return Normed(ctx, self, x, rows, tag)


class Normed:
    """The output of a norm that has not run yet.  A consumer that has folded the norm into its own weights
    (``Linear.fold_norm``) takes ``source``, the rows before the norm, and saves the norm's kernel; any other
    consumer calls ``tensor()``, which runs the norm once.  A block hands a ``Normed`` only to a mixer or
    feed-forward whose ``fold_input_norm`` said yes when the weights were bound; parts that do not know this
    class never see it."""

    def __init__(self, ctx, norm: Norm, source: torch.Tensor, rows, tag: str):
        self.ctx, self.norm, self.source, self.rows, self.tag = ctx, norm, source, rows, tag
        n = source.shape[0] if rows is None else rows.numel()
        self.shape = (n, source.shape[1])
        self.dtype = source.dtype
        self._tensor: Optional[torch.Tensor] = None

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = self.norm.forward(self.ctx, self.source, rows=self.rows, tag=self.tag)
        return self._tensor


class PositionEncoding(Part):
    max_positions: Optional[int] = None

    def embedding_table(self) -> Optional[torch.Tensor]:
        return None

    def rotate(self, ctx, q, k) -> None:
        return None


class Mixer(Part):
    def fold_input_norm(self, norm: Norm) -> bool:
        """Called once the weights are bound: may this part be given the rows before ``norm`` (as a ``Normed``)
        instead of the normed tensor?  True only if it applies the norm itself."""
        return False

    def cache_spec(self):
        return None

    def forward(self, ctx, x, residual, cache):
        raise NotImplementedError


class FeedForward(Part):
    def fold_input_norm(self, norm: Norm) -> bool:
        return False

    def forward(self, ctx, x, residual):
        raise NotImplementedError


class Block(Part):
    def cache_spec(self):
        return None

    def forward(self, ctx, x, cache):
        raise NotImplementedError


KINDS = ("norm", "position", "mixer", "feed_forward", "block")
_REGISTRY: Dict[str, Dict[str, Callable[..., Part]]] = {k: {} for k in KINDS}


def register_part(kind: str, name: str, factory: Callable[..., Part], replace: bool = False) -> None:
    if kind not in _REGISTRY:
        raise ValueError(f"unknown kind of part {kind!r}; kinds are {KINDS}")
    if name in _REGISTRY[kind] and not replace:
        raise ValueError(f"{kind} {name!r} is already registered")
    _REGISTRY[kind][name] = factory


def make_part(kind: str, name: str, **params) -> Part:
    try:
        factory = _REGISTRY[kind][name]
    except KeyError:
        raise ValueError(f"no {kind} named {name!r}; registered: {sorted(_REGISTRY.get(kind, {}))}") from None
    return factory(**params)


def registered_parts(kind: str) -> List[str]:
    return sorted(_REGISTRY[kind])
