"""A model as data: an embedding, a position encoding, a list of blocks, the
order in which they run, a final norm and an output head.

``ModelDescription`` is what an architecture's builder returns.  Its
``order`` is a list of ``RunEntry``: which block runs, which cache it uses and
whether it writes to it.  A block may appear twice in the order, and a block
may read the cache another block wrote (``cache`` = that block's index,
``write=False``).  ``Model`` binds loaded tensors to the parts and runs a
step: it is the only place that walks the order.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from .base import MATRIX, Block, Init, Norm, ParamSpec, Part, PositionEncoding
from .linear import Linear


@dataclass(frozen=True)
class RunEntry:
    block: int                   # index into ModelDescription.blocks
    cache: Optional[int] = None  # index of the block whose cache is used (None: this block's own)
    write: bool = True           # whether this run appends its keys/values or state to that cache

    @property
    def cache_id(self) -> int:
        return self.block if self.cache is None else self.cache


class TokenEmbedding(Part):
    """``h = table[token] * scale (+ position table[position])`` (mlx_lm/models/gpt2.py:132, 144)."""
    replayable = True
    kernel_libs = ("embed",)

    def __init__(self, name: str, vocab_size: int, width: int, scale: float = 1.0, init: Init = Init()):
        self.name, self.vocab_size, self.width, self.scale, self.init = name, vocab_size, width, scale, init
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.name + ".weight", (self.vocab_size, self.width), MATRIX, self.init)]

    def bind(self, tensors, dtype, device) -> None:
        self.table = tensors[self.name + ".weight"]

    def forward(self, ctx, position: Optional[PositionEncoding]):
        x = ctx.ws.get("residual", ctx.n_tokens, self.width, self.table.dtype)
        table = position.embedding_table() if position is not None else None
        ops.label(self.name, ctx.n_tokens * self.width, (3 if table is not None else 2) * x.element_size() * ctx.n_tokens * self.width)
        ops.embed_pos(ctx.tokens, ctx.positions, self.table, table, x, ctx.status, ctx.stream, scale=self.scale)
        return x


class OutputHead(Part):
    """Logits in float32.  Tied: the embedding table is the weight and there is no bias
    (``wte.as_linear``, mlx_lm/models/gpt2.py:166-167); untied: a linear layer of its own."""
    replayable = True

    def __init__(self, vocab_size: int, width: int, tied_to: Optional[TokenEmbedding] = None,
                 name: str = "lm_head", bias: bool = False):
        self.vocab_size, self.width, self.tied_to = vocab_size, width, tied_to
        self.linear = Linear(name, width, vocab_size, bias=bias and tied_to is None)

    def children(self):
        return () if self.tied_to is not None else (self.linear,)

    def all_kernel_libs(self):
        return list(self.linear.kernel_libs)

    def bind(self, tensors, dtype, device) -> None:
        if self.tied_to is not None:
            self.linear.use_weight(self.tied_to.table)

    def forward(self, ctx, x):
        out = ctx.ws.get("logits", x.shape[0], self.vocab_size, torch.float32)
        out = self.linear.forward(ctx, x, out)
        ops.label("after the output head")
        return out


@dataclass
class ModelDescription:
    model_type: str
    width: int
    vocab_size: int
    embedding: TokenEmbedding
    position: Optional[PositionEncoding]
    blocks: List[Block]
    final_norm: Optional[Norm]
    head: OutputHead
    order: List[RunEntry] = field(default_factory=list)
    ignored_tensors: Sequence[str] = ()   # regular expressions of tensor names a file may hold and the model drops
    args: object = None

    def __post_init__(self):
        if not self.order:
            self.order = [RunEntry(i) for i in range(len(self.blocks))]
        for e in self.order:
            if not 0 <= e.block < len(self.blocks) or not 0 <= e.cache_id < len(self.blocks):
                raise ValueError(f"run order names block {e.block} / cache {e.cache_id} of {len(self.blocks)} blocks")
        used = {e.cache_id for e in self.order}
        written = {e.cache_id for e in self.order if e.write}
        for c in used:
            if self.blocks[c].cache_spec() is not None and c not in written:
                raise ValueError(f"cache of block {c} is read but no run writes it")

    def parts(self) -> List[Part]:
        ps: List[Part] = [self.embedding]
        if self.position is not None:
            ps.append(self.position)
        ps.extend(self.blocks)
        if self.final_norm is not None:
            ps.append(self.final_norm)
        ps.append(self.head)
        return ps

    def param_specs(self) -> List[ParamSpec]:
        """Every tensor the model expects, in the order the random-weights mode draws them."""
        out: List[ParamSpec] = []
        for p in self.parts():
            out.extend(p.all_param_specs())
        names = [s.name for s in out]
        if len(set(names)) != len(names):
            dup = sorted({n for n in names if names.count(n) > 1})
            raise ValueError(f"two parts name the same tensor: {dup}")
        return out

    def kernel_libs(self) -> List[str]:
        libs: List[str] = []
        for p in self.parts():
            libs.extend(p.all_kernel_libs())
        return list(dict.fromkeys(libs))

    def cache_specs(self) -> Dict[int, object]:
        """``cache id -> spec`` for every cache the run order uses."""
        out = {}
        for e in self.order:
            spec = self.blocks[e.cache_id].cache_spec()
            if spec is not None:
                out[e.cache_id] = spec
        return out

    @property
    def max_positions(self) -> Optional[int]:
        return self.position.max_positions if self.position is not None else None


class Model:
    """A description bound to tensors on a device in one dtype."""

    def __init__(self, description: ModelDescription, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
                 device):
        self.description = description
        self.args = description.args
        self.model_type = description.model_type
        self.dtype, self.device = dtype, torch.device(device)
        for p in description.parts():
            p.bind_all(tensors, dtype, self.device)

    @property
    def layers(self):
        return self.description.blocks

    @property
    def vocab_size(self) -> int:
        return self.description.vocab_size

    def n_parameters(self) -> int:
        n = 0
        for s in self.description.param_specs():
            c = 1
            for d in s.shape:
                c *= d
            n += c
        return n

    def run(self, ctx) -> Optional[torch.Tensor]:
        """All of this step's tokens through the blocks in run order; float32 logits
        ``[len(ctx.logit_rows), vocab]`` at the wanted rows, or None if none is wanted."""
        d = self.description
        x = d.embedding.forward(ctx, d.position)
        for entry in d.order:
            x = d.blocks[entry.block].forward(ctx, x, ctx.cache_view(entry))
        if ctx.n_logit_rows == 0:
            return None
        if d.final_norm is not None:
            h = d.final_norm.forward(ctx, x, rows=ctx.logit_rows, tag="final_normed")
        else:
            h = ctx.gather_rows(x)
        return d.head.forward(ctx, h)
