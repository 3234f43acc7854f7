"""A decode step as a CUDA graph.

A step in which every request brings one token launches some two hundred small kernels; issued
one by one from Python they cost more host time than device time.  For each batch size in
``Engine.GRAPH_BUCKETS`` the whole step — embedding, every block, final norm, output head and
the sampling kernel — is captured once into a CUDA graph over buffers of fixed address; a step
then writes its integers (tokens, positions, block tables, sampler records) into one pinned
buffer, copies it, replays the graph and reads the chosen tokens back.

A batch smaller than its bucket is padded with rows whose request index is -1: the cache write
and the attention kernels skip them, the other kernels compute rows nobody reads.  The graph has
a workspace of its own, so that a later, larger step cannot move the buffers it was captured on.

A step is ``launch`` (everything enqueued, nothing waited for) and ``collect`` (wait, read the
tokens).  Between the two the caller may launch the step after it: a request's token for that
step is then taken on the device from the output of the step before (``source``), so the device
runs step after step while the host reads the tokens one step behind (mlx-lm overlaps the same
way with ``mx.async_eval``, mlx_lm/generate.py:434-451).  Two pinned staging buffers alternate,
so that a launch never writes what an earlier copy may still read.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..sampling import LogitsProcessors
from .step import StepContext, StepEntry, Workspace


class StaleSource(RuntimeError):
    """The step named as the source of tokens is no longer what its graph's output buffer holds."""


@dataclass
class PendingStep:
    """A launched decode step whose tokens have not been read yet.  It names its graph by the engine's key, not by
    reference: graph and step would keep one another alive until the cycle collector runs, and a CUDA graph must
    not be destroyed at a moment of the collector's choosing (while another one is being captured, for one)."""
    key: tuple                 # (bucket, filters) of its graph in Engine._graphs
    slot: int                  # which staging buffer its results arrive in
    n: int                     # live rows
    event: object
    collected: bool = False


class DecodeGraph:
    @staticmethod
    def samplers_fit(requests: Sequence, sampler) -> bool:
        """Whether the sampling kernel alone covers what these requests ask for."""
        if getattr(sampler, "return_logprobs", False) or not hasattr(sampler, "seed"):
            return False
        return all(not r.processors and not r.sampler.xtc_special_tokens for r in requests)

    def __init__(self, engine, bucket: int, filters: bool = False):
        # filters: whether rows with top-p, min-p, XTC or top-k may come.  Without them the sampling kernel is the
        # one that cuts every row into slices over several thread blocks; a step is replayed on the graph of its kind.
        self.engine, self.B, self.filters = engine, bucket, filters
        mgr = engine.cache
        dev = engine.model.device
        B, W = bucket, mgr.table_width
        pad = lambda n: (n + 3) & ~3
        sizes = [("tokens", B), ("positions", B), ("token_req", B), ("logit_rows", B), ("slots", B),
                 ("req_first_token", B + 1), ("req_first_position", B), ("sample", B * ops.SAMPLE_WORDS),
                 ("single_tiles", 4 * B), ("source_rows", B)]
        sizes += [(f"table{g}", B * W) for g in range(len(mgr.kv_groups))]
        self.off, total = {}, 0
        for name, n in sizes:
            self.off[name] = total
            total += pad(n)
        self.total = total
        self.hosts = []          # pinned staging buffers, one per step that may be in flight (see _staging)
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)
        self.out = torch.zeros(2 * B + 1, dtype=torch.int32, device=dev)  # tokens | log-probability bits | status word
        self.sample_scratch = ops.sample_scratch(B, dev)
        self.out_hosts, self.events = [], []
        self.pending: List[Optional[PendingStep]] = []     # the last step launched from each staging buffer
        self.last: Optional[PendingStep] = None            # the step launched last: what ``out`` holds (or will)
        self.n_launched = 0
        self._staging()
        self._staging()

        view = lambda name, n: self.dev[self.off[name]: self.off[name] + n]
        ctx = StepContext(engine)
        ctx.ws = Workspace(dev)
        ctx.n_tokens = ctx.n_requests = ctx.n_logit_rows = B
        ctx.tokens, ctx.positions, ctx.token_req = view("tokens", B), view("positions", B), view("token_req", B)
        ctx.logit_rows = view("logit_rows", B)
        ctx.req_first_token, ctx.req_first_position = view("req_first_token", B + 1), view("req_first_position", B)
        ctx._slots = view("slots", B)
        ctx._tables = [view(f"table{g}", B * W).view(B, W) for g in range(len(mgr.kv_groups))]
        ctx.n_single, ctx.n_portion, ctx.max_q_len = B, 0, 1
        ctx.single_tiles = view("single_tiles", 4 * B)
        self.ctx = ctx
        self.params = view("sample", B * ops.SAMPLE_WORDS)
        self.tok = self.out[:B]
        self.lp = self.out[B:2 * B].view(torch.float32)

        # once eagerly on a side stream (loads libraries, sizes the workspace), then capture
        self.dev.copy_(self.hosts[0])
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self._launch()
        side.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        # Nothing may be destroyed by the cycle collector while the capture runs (a CUDA graph or a pinned buffer of
        # an engine that is gone would invalidate it): torch collects before the capture begins, and the collector
        # rests until it has ended.
        import gc
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, stream=side):
                self._launch()
        finally:
            if was_enabled:
                gc.enable()
        torch.cuda.current_stream(dev).wait_stream(side)
        self.n_kernels = self._count

    def _staging(self) -> int:
        """One more pair of pinned staging buffers (integers in, tokens out) with its event; its index."""
        B, W, mgr = self.B, self.engine.cache.table_width, self.engine.cache
        host = torch.zeros(self.total, dtype=torch.int32).pin_memory()
        h = host.numpy()
        h[self.off["logit_rows"]: self.off["logit_rows"] + B] = np.arange(B)
        h[self.off["req_first_token"]: self.off["req_first_token"] + B + 1] = np.arange(B + 1)
        h[self.off["token_req"]: self.off["token_req"] + B] = -1
        h[self.off["source_rows"]: self.off["source_rows"] + B] = -1
        tiles = h[self.off["single_tiles"]: self.off["single_tiles"] + 4 * B].reshape(B, 4)
        tiles[:] = 0
        tiles[:, 0] = np.arange(B)          # (token row, 0 queries, ...): a padding row until a request takes it
        for g in range(len(mgr.kv_groups)):
            h[self.off[f"table{g}"]: self.off[f"table{g}"] + B * W] = -1
        self.hosts.append(host)
        self.out_hosts.append(torch.zeros(2 * B + 1, dtype=torch.int32).pin_memory())
        self.events.append(torch.cuda.Event())
        self.pending.append(None)
        return len(self.hosts) - 1

    def _launch(self) -> None:
        ctx = self.ctx
        ctx.stream = ops.current_stream()
        before = ops.launch_count
        self.logits = self.engine.model.run(ctx)
        ops.label("sampler", 0.0, 4.0 * self.logits.numel())
        ops.sample(self.logits, self.params, self.tok, self.lp, ctx.stream, status=self.engine.status,
                   status_out=self.out[2 * self.B:], scratch=None if self.filters else self.sample_scratch)
        self._count = ops.launch_count - before

    def launch(self, entries: Sequence[StepEntry], requests: Sequence, seed: int,
               source: Optional[Tuple[PendingStep, Sequence[int]]] = None) -> PendingStep:
        """Enqueue the step and return without waiting.  ``source = (step, rows)``: entry i's token is not known to
        the host yet; it is row ``rows[i]`` of what ``step`` (launched, not yet collected) samples (``rows[i] < 0``:
        the token of the entry, as without a source), and the request's sampling position is one further than its
        host-side token count says."""
        eng, mgr, B = self.engine, self.engine.cache, self.B
        eng._validate(entries)
        n = len(entries)
        source_graph = eng._graphs.get(source[0].key) if source is not None else None
        if source is not None and (source_graph is None or source_graph.last is not source[0]):
            # another caller's step went through that graph since: its output is no longer the source's
            raise StaleSource("the step to take the tokens from is not the last one launched on its graph")
        # a staging buffer whose last step has been read (two alternate for one caller; a second caller with a
        # step of its own in flight gets a third)
        slot = next((i for i, p in enumerate(self.pending) if p is None or p.collected), -1)
        if slot < 0:
            slot = self._staging() if len(self.hosts) < 8 else 0
            if self.pending[slot] is not None and not self.pending[slot].collected:
                self.pending[slot].event.synchronize()      # eight steps nobody has read: their callers are gone
                self.pending[slot].collected = True
        h, off, W = self.hosts[slot].numpy(), self.off, mgr.table_width
        h[off["token_req"] + n: off["token_req"] + B] = -1
        h[off["source_rows"]: off["source_rows"] + B] = -1
        tiles = h[off["single_tiles"]: off["single_tiles"] + 4 * B].reshape(B, 4)
        tiles[n:, 1:] = 0
        words = []
        rows = source[1] if source is not None else None
        try:
            for i, e in enumerate(entries):
                start = mgr.reserve(e.rid, 1)
                ahead = rows is not None and rows[i] >= 0
                h[off["tokens"] + i] = 0 if ahead else e.tokens[0]
                if ahead:
                    h[off["source_rows"] + i] = rows[i]
                h[off["positions"] + i] = start
                h[off["token_req"] + i] = i
                h[off["slots"] + i] = mgr.requests[e.rid].slot
                h[off["req_first_position"] + i] = start
                tiles[i, 1], tiles[i, 2], tiles[i, 3] = 1, i, start
                r = requests[i]
                words.append(r.sampler.words(seed, r.uid, len(r.tokens) + (1 if ahead else 0)))
            h[off["sample"]: off["sample"] + n * ops.SAMPLE_WORDS] = np.frombuffer(b"".join(words), dtype=np.int32)
            h[off["sample"] + n * ops.SAMPLE_WORDS: off["sample"] + B * ops.SAMPLE_WORDS] = 0
            rids = [e.rid for e in entries]
            for g in range(len(mgr.kv_groups)):
                o = off[f"table{g}"]
                mgr.block_table(g, rids, out=h[o: o + n * W].reshape(n, W))
                h[o + n * W: o + B * W] = -1
            self.dev.copy_(self.hosts[slot], non_blocking=True)
            if source is not None:
                src = source_graph.out[:source_graph.B]
                ops.gather_tokens(src, self.dev[off["source_rows"]: off["source_rows"] + n],
                                  self.dev[off["tokens"]: off["tokens"] + n], eng.status, ops.current_stream())
            self.graph.replay()
            ops.launch_count += self.n_kernels
            self.out_hosts[slot].copy_(self.out, non_blocking=True)
            event = self.events[slot]
            event.record()
            eng.h2d_bytes += 4 * self.total
            eng.d2h_bytes += 4 * self.out.numel()
        except BaseException:
            for e in entries:          # the step was not enqueued whole: undo the reservations
                mgr.rollback(e.rid)
            raise
        # Enqueued: what later steps read of the cache comes after this step in stream order, so the lengths move
        # on now and the next step can be laid out before this one has run.
        for e in entries:
            mgr.commit(e.rid)
        eng.n_steps += 1
        self.n_launched += 1
        step = self.pending[slot] = self.last = PendingStep((self.B, self.filters), slot, n, event)
        return step

    def collect(self, step: PendingStep) -> Tuple[List[int], List[float]]:
        """Wait for a launched step; its tokens and their log-probabilities."""
        step.event.synchronize()
        step.collected = True
        o = self.out_hosts[step.slot].numpy()
        self.engine.host_status = int(o[2 * self.B])
        n, B = step.n, self.B
        return o[:n].tolist(), o[B:B + n].view(np.float32).tolist()

    def run(self, entries: Sequence[StepEntry], requests: Sequence, seed: int) -> Tuple[List[int], List[float]]:
        return self.collect(self.launch(entries, requests, seed))
