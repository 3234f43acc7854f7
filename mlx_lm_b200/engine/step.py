"""The step function: one batch of (request, its next tokens) through the
model, from the cache, returning logits at the wanted places.

mlx-lm runs prompt processing and decoding as two rectangular model calls
(``PromptProcessingBatch.prompt`` on right-padded ``[B, L]`` slices and
``GenerationBatch._step`` on ``[B, 1]``: mlx_lm/generate.py:1208-1254,
1402-1460).  Here a step is one flat list of tokens: every entry brings the
next ``n >= 1`` tokens of one request — a portion of a prompt cut anywhere,
or a single decoded token — and they all run as one batch.  Each token knows
its request and its position; keys and values are appended to the request's
pages and attention reads them back through the block table, so a step runs
only the tokens it is given.

All integer inputs of a step (tokens, positions, request of each token, rows
whose logits are wanted, block tables, slots, per-request offsets) are packed
into one pinned host buffer and reach the device in one copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache import CacheManager
from ..ops import build as kernel_build
from ..parts.model import Model, RunEntry


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()      # indices into ``tokens`` whose logits are asked for


class Workspace:
    """Activation buffers by name, kept between steps and grown on demand."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[tuple, torch.Tensor] = {}
        self.generation = 0      # goes up whenever a buffer is made or replaced (its address changes)

    def get(self, tag: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        key = (tag, cols, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.shape[0] < rows:
            cap = max(rows, 16)
            if buf is not None:
                cap = max(cap, 2 * buf.shape[0])
            buf = torch.zeros((cap, cols), dtype=dtype, device=self.device)   # rows a step never writes stay finite
            self._bufs[key] = buf
            self.generation += 1
        return buf[:rows]

    def flat(self, tag: str, n: int, dtype: torch.dtype) -> torch.Tensor:
        """Scratch memory of at least ``n`` elements whose size varies from step to step."""
        key = (tag, 0, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.zeros(max(n, 1024, 2 * (buf.numel() if buf is not None else 0)), dtype=dtype,
                              device=self.device)   # zero: ticket counters of kernels start from zero
            self._bufs[key] = buf
            self.generation += 1
        return buf

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


@dataclass
class LayerCacheView:
    """What one run of a block sees of its cache in this step."""
    kind: str                      # "kv", "state" or "none"
    write: bool = True
    k: Optional[torch.Tensor] = None             # [n_pages, heads, page, head_dim]
    v: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None   # int32 [R, table_width] on the device
    page_size: int = 0
    state: Optional[torch.Tensor] = None         # [n_slots, *shape] float32
    slots: Optional[torch.Tensor] = None         # int32 [R] on the device


@dataclass
class RequestSpan:
    """One entry of the step as parts with sequential state need it (host side)."""
    rid: Hashable
    slot: int
    first_token: int     # row of the entry's first token among the step's tokens
    n_tokens: int
    first_position: int


class StepContext:
    """Everything a part may read while a step runs."""

    def __init__(self, engine: "Engine"):
        self.engine = engine
        self.ws = engine.ws
        self.dtype, self.device = engine.model.dtype, engine.model.device
        self.status = engine.status
        self.stream = 0
        self.n_tokens = 0
        self.n_requests = 0
        self.n_logit_rows = 0
        self.tokens = self.positions = self.token_req = self.logit_rows = None
        self.req_first_token = self.req_first_position = None
        self.spans: List[RequestSpan] = []
        self.max_q_len = 0
        self.max_len = engine.max_len
        # tokens of requests that bring a single token (decode) and of those that bring a portion:
        # int32 device lists of token rows, None meaning "all tokens of the step"
        self.n_single = self.n_portion = 0
        self.single_rows = self.portion_rows = None
        # portions cut into tiles of ops.PREFILL_TILE queries: int32 [n, 4] = (first token row, queries,
        # block-table row, first position), longest context first
        self.portion_tiles = None
        self.n_portion_tiles = 0
        # the single-token rows as tiles of one query: int32 [n_single, 4] = (token row, 1, block-table row,
        # position), or (token row, 0, 0, 0) for a row that pads the step
        self.single_tiles = None
        self._tables: List[torch.Tensor] = []
        self._slots: Optional[torch.Tensor] = None

    def cache_view(self, entry: RunEntry) -> LayerCacheView:
        mgr = self.engine.cache
        if entry.cache_id not in mgr._where:
            return LayerCacheView("none", write=False)
        kind, gi = mgr.where(entry.cache_id)
        if kind == "kv":
            g = mgr.kv_groups[gi]
            i = g.index_of(entry.cache_id)
            return LayerCacheView("kv", entry.write, k=g.k[i], v=g.v[i], block_table=self._tables[gi],
                                  page_size=mgr.page_size)
        g = mgr.state_groups[gi]
        return LayerCacheView("state", entry.write, state=g.data[g.index_of(entry.cache_id)], slots=self._slots)

    def gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        """The rows of ``x`` whose logits are wanted, as a tensor of their own (what a final norm does on the
        way for a model that has one)."""
        out = self.ws.get("wanted_rows", self.n_logit_rows, x.shape[1], x.dtype)
        ops.gather_rows(x, self.logit_rows, out, self.stream)
        return out


class Engine:
    """A model, its cache and the step function."""

    def __init__(self, model: Model, page_size: int = 16, max_tokens: Optional[int] = None,
                 n_pages: Optional[int] = None, max_requests: int = 64, max_len: Optional[int] = None):
        ops.require_cuda()
        self.model = model
        d = model.description
        limit = d.max_positions
        self.max_len = min(x for x in (max_len, limit, 1 << 20) if x is not None)
        if n_pages is None:
            if max_tokens is None:
                max_tokens = max_requests * self.max_len
            n_pages = (max_tokens + page_size - 1) // page_size
        libs = [n for n in d.kernel_libs() if model.dtype == torch.bfloat16 or n not in ops.BF16_ONLY_LIBS]
        kernel_build.ensure_built(libs)      # compiled now, in parallel, if this is their first use
        self.cache = CacheManager(d.cache_specs(), page_size=page_size, n_pages=n_pages, max_requests=max_requests,
                                  max_len=self.max_len, dtype=model.dtype, device=model.device)
        self.ws = Workspace(model.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=model.device)
        self.h2d_bytes = self.d2h_bytes = 0     # bytes the steps copied to and from the device (counted at the copies)
        self.last_calls = None    # the recorded launches of the last step that went through a launch plan
        self.host_status = 0      # the status word as a sampler's copy of a step's tokens last brought it to the host
        self._namespaces = 0
        self._host = [None, None]
        self._host_events = [None, None]
        self._dev: Optional[torch.Tensor] = None
        self._flip = 0
        self.n_steps = 0
        self.use_graphs = True
        self._graphs = {}
        # Steps of a shape seen before are re-issued from a recording of their kernel launches (raw
        # arguments), which skips the Python of the parts and of the kernel wrappers: possible when every
        # part only launches kernels whose arguments are fixed by the shape (Part.replayable).
        self.use_replay = all(p.all_replayable() for p in d.parts())
        self._plans: Dict[tuple, tuple] = {}
        self.n_replayed = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, rid: Hashable) -> None:
        self.cache.add_request(rid)

    def finish(self, rid: Hashable) -> None:
        self.cache.release(rid)

    def has_request(self, rid: Hashable) -> bool:
        return rid in self.cache.requests

    def new_namespace(self) -> int:
        """A number no earlier caller got: schedulers that share this engine name their requests
        ``(namespace, uid)`` and so never collide."""
        self._namespaces += 1
        return self._namespaces

    # ------------------------------------------------------------------ the step
    def _int_buffers(self, n: int):
        i = self._flip
        self._flip ^= 1
        if self._host[i] is None or self._host[i].numel() < n:
            cap = max(4096, 2 * n)
            self._host[i] = torch.empty(cap, dtype=torch.int32).pin_memory()
            self._host_events[i] = None
        if self._dev is None or self._dev.numel() < n:
            self._dev = torch.empty(max(4096, 2 * n), dtype=torch.int32, device=self.model.device)
        if self._host_events[i] is not None:
            self._host_events[i].synchronize()
        return i, self._host[i], self._dev

    def _upload(self, i: int, n: int) -> None:
        self._dev[:n].copy_(self._host[i][:n], non_blocking=True)
        self.h2d_bytes += 4 * n
        ev = torch.cuda.Event()
        ev.record()
        self._host_events[i] = ev   # the pinned buffer may be rewritten once this has passed

    def _validate(self, entries: Sequence[StepEntry]) -> None:
        mgr = self.cache
        vocab = self.model.vocab_size
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if e.rid not in mgr.requests:
                raise KeyError(f"request {e.rid!r} is not live")
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.rid!r}: an entry needs at least one token")
            if min(e.tokens) < 0 or max(e.tokens) >= vocab:
                raise ValueError(f"request {e.rid!r}: token id outside 0..{vocab - 1}")
            if any(not 0 <= w < n for w in e.want):
                raise ValueError(f"request {e.rid!r}: wanted place outside its {n} tokens")
            if mgr.length(e.rid) + n > self.max_len:
                raise ValueError(f"request {e.rid!r}: position {mgr.length(e.rid) + n - 1} is beyond the model's "
                                 f"{self.max_len} positions")
        if not mgr.can_reserve([(e.rid, len(e.tokens)) for e in entries]):
            from ..cache import OutOfPages
            raise OutOfPages(f"this step needs more pages than are free {mgr.pages_free()}")

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries' tokens as one batch.  Returns float32 logits ``[n_wanted, vocab]`` on the
        device in the order of the entries and of their ``want`` lists (None if nothing is wanted)."""
        if not entries:
            return None
        mgr = self.cache
        self._validate(entries)

        ctx = StepContext(self)
        TQ = ops.PREFILL_TILE
        W = mgr.table_width
        pad = lambda n: (n + 3) & ~3
        n_real = len(entries)
        L = sum(len(e.want) for e in entries)
        n_single = sum(1 for e in entries if len(e.tokens) == 1)
        n_portions = n_real - n_single
        # Shapes are rounded up so that few distinct step shapes occur (each shape's launches are recorded once
        # and re-issued): every portion gets a span of rows that is a multiple of the attention tile (of 16 rows
        # for a portion of up to 64 tokens, so that a short tail beside decoding requests stays a step of few
        # rows), and the number of single-token entries goes up to the next power of two (multiples of 64 above
        # 64).  The extra rows carry request index -1: the cache write and the attention kernels skip them, the
        # other kernels compute rows nobody reads.  Models with parts that loop over the step's entries on the
        # host keep exact shapes.
        rounding = self.use_replay

        def rows_of(n: int) -> int:
            if n == 1 or not rounding:
                return n
            return (n + 15) // 16 * 16 if n <= 64 else (n + TQ - 1) // TQ * TQ

        span = [rows_of(len(e.tokens)) for e in entries]
        n_fake = 0
        if rounding and n_single:
            bucket = 1
            while bucket < n_single and bucket < 64:
                bucket *= 2
            if n_single > 64:
                bucket = (n_single + 63) // 64 * 64
            n_fake = bucket - n_single
        n_single_rows = n_single + n_fake
        n_tiles = sum((len(e.tokens) + TQ - 1) // TQ for e in entries if len(e.tokens) > 1)
        T_portions = sum(sp for sp, e in zip(span, entries) if len(e.tokens) > 1)
        L_rows = max(L, n_single_rows + n_portions) if rounding and L else L   # wanted rows first, then filler
        R = n_real + n_fake
        n_pad_rows = 0              # rows without a request behind the last portion
        if rounding and n_portions:
            # The same for the step as a whole, so that steps of a scheduler that cuts prompts under a budget
            # repeat their shapes: the portions' rows together go up to a multiple of 256 (of 64 below that), the
            # list of tiles to an even length (a multiple of 4 above 8; tiles of 0 queries are skipped by the
            # kernels), the requests to a multiple of 4 and the wanted rows to a multiple of 8.
            grid = 256 if T_portions > 256 else 64
            n_pad_rows = (T_portions + grid - 1) // grid * grid - T_portions
            step_t = 2 if n_tiles <= 8 else 4
            n_tiles = (n_tiles + step_t - 1) // step_t * step_t
            R = (R + 3) // 4 * 4
            if L_rows:
                L_rows = (L_rows + 7) // 8 * 8
        T = sum(span) + n_fake + n_pad_rows
        mixed = 0 < n_single_rows < n_real + n_fake
        off, sizes = {}, [("tokens", T), ("positions", T), ("token_req", T), ("logit_rows", L_rows), ("slots", R),
                          ("req_first_token", R + 1), ("req_first_position", R),
                          ("single_rows", n_single_rows if mixed else 0),
                          ("portion_rows", T - n_single_rows if mixed else 0), ("tiles", 4 * n_tiles),
                          ("single_tiles", 4 * n_single_rows)]
        sizes += [(f"table{g}", R * W) for g in range(len(mgr.kv_groups))]
        total = 0
        for name, n in sizes:
            off[name] = total
            total += pad(max(n, 1))
        hi, host, dev = self._int_buffers(total)
        h = host.numpy()
        h[off["tokens"]: off["tokens"] + T] = 0
        h[off["positions"]: off["positions"] + T] = 0
        h[off["token_req"]: off["token_req"] + T] = -1
        try:
            t0 = 0
            rows: List[int] = []
            single_rows: List[int] = []
            portion_rows: List[int] = []
            tiles: List[tuple] = []
            single_tiles: List[tuple] = []
            for r, e in enumerate(entries):
                n = len(e.tokens)
                start = mgr.reserve(e.rid, n)
                slot = mgr.requests[e.rid].slot
                h[off["tokens"] + t0: off["tokens"] + t0 + n] = e.tokens
                h[off["positions"] + t0: off["positions"] + t0 + n] = np.arange(start, start + n, dtype=np.int32)
                h[off["token_req"] + t0: off["token_req"] + t0 + n] = r
                h[off["slots"] + r] = slot
                h[off["req_first_token"] + r] = t0
                h[off["req_first_position"] + r] = start
                rows.extend(t0 + w for w in e.want)
                if mixed:
                    (single_rows if n == 1 else portion_rows).extend(range(t0, t0 + span[r]))
                if n > 1:
                    tiles.extend((t0 + a, min(TQ, n - a), r, start + a) for a in range(0, n, TQ))
                else:
                    single_tiles.append((t0, 1, r, start))
                ctx.spans.append(RequestSpan(e.rid, slot, t0, n, start))
                ctx.max_q_len = max(ctx.max_q_len, n)
                t0 += span[r]
            for f in range(n_fake):                      # filler single-token entries
                r = n_real + f
                h[off["slots"] + r] = 0
                h[off["req_first_token"] + r] = t0
                h[off["req_first_position"] + r] = 0
                if mixed:
                    single_rows.append(t0)
                single_tiles.append((t0, 0, 0, 0))
                t0 += 1
            if mixed and n_pad_rows:
                portion_rows.extend(range(t0, t0 + n_pad_rows))        # rows without a request: every kernel skips them
            for r in range(n_real + n_fake, R):                        # requests that only fill the tables up
                h[off["slots"] + r] = 0
                h[off["req_first_token"] + r] = T
                h[off["req_first_position"] + r] = 0
            h[off["req_first_token"] + R] = T
            if L_rows:
                rows.extend([rows[0]] * (L_rows - L))
                h[off["logit_rows"]: off["logit_rows"] + L_rows] = rows
            if mixed:
                h[off["single_rows"]: off["single_rows"] + n_single_rows] = single_rows
                h[off["portion_rows"]: off["portion_rows"] + T - n_single_rows] = portion_rows
            if n_tiles:
                tiles.sort(key=lambda t: -(t[3] + t[1]))     # tiles with the most keys start first
                tiles.extend([(0, 0, 0, 0)] * (n_tiles - len(tiles)))      # tiles of 0 queries: skipped
                h[off["tiles"]: off["tiles"] + 4 * n_tiles] = np.asarray(tiles, dtype=np.int32).reshape(-1)
            if n_single_rows:
                h[off["single_tiles"]: off["single_tiles"] + 4 * n_single_rows] = \
                    np.asarray(single_tiles, dtype=np.int32).reshape(-1)
            rids = [e.rid for e in entries]
            for g in range(len(mgr.kv_groups)):
                o = off[f"table{g}"]
                h[o: o + R * W] = -1
                mgr.block_table(g, rids, out=h[o: o + n_real * W].reshape(n_real, W))
            self._upload(hi, total)

            view = lambda name, n: dev[off[name]: off[name] + n]
            ctx.stream = ops.current_stream()
            ctx.n_tokens, ctx.n_requests, ctx.n_logit_rows = T, R, L_rows
            ctx.tokens, ctx.positions, ctx.token_req = view("tokens", T), view("positions", T), view("token_req", T)
            ctx.logit_rows = view("logit_rows", L_rows)
            ctx.req_first_token, ctx.req_first_position = view("req_first_token", R + 1), view("req_first_position", R)
            ctx._slots = view("slots", R)
            ctx.n_single, ctx.n_portion = n_single_rows, T - n_single_rows
            if mixed:
                ctx.single_rows = view("single_rows", n_single_rows)
                ctx.portion_rows = view("portion_rows", T - n_single_rows)
            if n_tiles:
                ctx.portion_tiles, ctx.n_portion_tiles = view("tiles", 4 * n_tiles), n_tiles
            if n_single_rows:
                ctx.single_tiles = view("single_tiles", 4 * n_single_rows)
            ctx._tables = [view(f"table{g}", R * W).view(R, W) for g in range(len(mgr.kv_groups))]
            logits = self._run(ctx, (T, R, L_rows, n_single_rows, n_tiles, ctx.stream, dev.data_ptr()))
        except BaseException:
            # The step did not run to its end: its positions are not part of the requests.  The pages taken for
            # them go back, and the requests continue from where they were.
            for e in entries:
                mgr.rollback(e.rid)
            raise
        for e in entries:
            mgr.commit(e.rid)
        self.n_steps += 1
        return logits if logits is None or L_rows == L else logits[:L]

    def _run(self, ctx: "StepContext", shape: tuple) -> Optional[torch.Tensor]:
        if not self.use_replay:
            return self.model.run(ctx)
        plan = self._plans.get(shape)
        if plan is not None and plan[0] == self.ws.generation:
            ops.replay(plan[1])
            self.n_replayed += 1
            self.last_calls = plan[1]
            return plan[2]
        ops.start_recording()
        try:
            logits = self.model.run(ctx)
        finally:
            calls = ops.stop_recording()
        if len(self._plans) >= 256:
            self._plans.clear()
        self._plans[shape] = (self.ws.generation, calls, logits)
        self.last_calls = calls
        return logits

    # ------------------------------------------------------------------ decode steps as CUDA graphs
    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64)

    def decode_sampled(self, entries: Sequence[StepEntry], requests: Sequence, sampler):
        """One token for each of the requests, sampled on the device: ``(tokens, logprobs)`` as lists.

        When every entry brings a single token and the samplers need nothing beyond the sampling
        kernel, the whole step (model and sampler) is replayed as a CUDA graph captured for the next
        batch size in ``GRAPH_BUCKETS``; otherwise it is ``step`` followed by ``sampler``."""
        step = self.decode_launch(entries, requests, sampler)
        if step is None:
            return sampler(self.step(entries), requests)
        return self.decode_collect(step)

    def decode_launch(self, entries: Sequence[StepEntry], requests: Sequence, sampler, source=None):
        """Enqueue such a step as a CUDA graph and return at once with a handle for ``decode_collect``; None if the
        step does not fit a graph (more rows than the largest bucket, an entry of several tokens, samplers that
        need more than the sampling kernel).  ``source = (handle, rows)``: the entries' tokens are rows ``rows`` of
        what the step behind ``handle`` samples (still on its way), see ``DecodeGraph.launch``.  At most two steps
        are in flight; they are collected in the order they were launched."""
        from .decode_graph import DecodeGraph, StaleSource

        n = len(entries)
        ok = (self.use_graphs and n <= self.GRAPH_BUCKETS[-1] and all(len(e.tokens) == 1 for e in entries)
              and DecodeGraph.samplers_fit(requests, sampler))
        if not ok:
            return None
        bucket = next(b for b in self.GRAPH_BUCKETS if b >= n)
        filters = any(r.sampler.filters for r in requests)
        graph = self._graphs.get((bucket, filters))
        if graph is None:
            graph = self._graphs[(bucket, filters)] = DecodeGraph(self, bucket, filters)
        try:
            return graph.launch(entries, requests, sampler.seed, source)
        except StaleSource:
            return None      # somebody else's step went through that graph meanwhile: the caller reads its tokens first

    def decode_collect(self, step):
        """Wait for a step launched by ``decode_launch``: ``(tokens, logprobs)`` as lists."""
        return self._graphs[step.key].collect(step)

    def read_status(self) -> int:
        """Bits kernels set instead of faulting (token, position or page id out of range, a bounded wait that
        gave up).  Reading synchronises with the device and clears the word."""
        s = int(self.status.item())
        if s:
            self.clear_status()
        return s

    def clear_status(self) -> None:
        self.status.zero_()
        self.host_status = 0

    def check_status(self) -> None:
        s = self.read_status()
        if s:
            raise ops.KernelError("a kernel reported: " + ops.describe_status(s))
