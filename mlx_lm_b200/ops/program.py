"""A decode step as a table of phases for the persistent kernel of csrc/decode_program.cu.

The table is made from the launches that a step of single tokens issues (``ops.start_recording``):
each launch of a known kernel becomes one phase with the same pointers and sizes, and a LayerNorm
whose output only the next linear layer reads is folded into that layer.  A step that launches
anything else has no program (``compile_program`` returns None) and runs as the chain of kernels
it is.  No part knows about this: whatever model is put together from parts whose single-token
kernels are the ones below gets the program.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import List, Optional, Sequence, Tuple

import torch

from . import build

OP_EMBED, OP_NORM, OP_LINEAR, OP_ATTENTION = 1, 2, 3, 4
F_LN, F_GELU, F_OUT_F32, F_SCATTER = 1, 2, 4, 8
MAX_ROWS = 64


class Phase(ctypes.Structure):
    """Mirror of ``struct Phase`` in csrc/decode_program.cu."""
    _fields_ = [
        ("A", c_void_p), ("W", c_void_p), ("bias", c_void_p), ("ln_gain", c_void_p), ("ln_bias", c_void_p),
        ("rows", c_void_p), ("residual", c_void_p), ("C", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p),
        ("block_table", c_void_p), ("tokens", c_void_p), ("positions", c_void_p), ("token_req", c_void_p),
        ("partial", c_void_p), ("counters", c_void_p), ("next_w", c_void_p), ("next_bytes", c_longlong),
        ("op", c_int), ("flags", c_int), ("M", c_int), ("N", c_int), ("K", c_int), ("lda", c_int), ("ldc", c_int),
        ("max_pages", c_int), ("n_pages", c_int), ("page", c_int), ("Hq", c_int), ("Hkv", c_int), ("Dh", c_int),
        ("window", c_int), ("q_width", c_int), ("n_chunks_max", c_int), ("chunk", c_int), ("vocab", c_int),
        ("n_pos", c_int), ("eps", c_float), ("scale", c_float), ("embed_scale", c_float), ("pad_", c_int),
    ]


def _span(ptr, n_bytes) -> Tuple[int, int]:
    return (int(ptr or 0), int(ptr or 0) + int(n_bytes))


class _Node:
    """A phase with the memory it reads and writes (activations only; weights are never written)."""

    def __init__(self, phase: Phase, reads: List[Tuple[int, int]], writes: List[Tuple[int, int]]):
        self.phase, self.reads, self.writes = phase, reads, writes


def _overlaps(a: Tuple[int, int], spans: Sequence[Tuple[int, int]]) -> bool:
    return any(a[0] < s[1] and s[0] < a[1] for s in spans)


def _translate(fname: str, a: tuple) -> Optional[_Node]:
    """One recorded launch (launcher name, raw arguments) as a phase, or None if it has no phase."""
    p = Phase()
    if fname == "mlxb_embed_pos":
        dtype, tokens, positions, wte, wpe, out, T, D, V, P, scale, _status, _stream = a
        if dtype != 1 or D % 8:
            return None
        p.op, p.A, p.W, p.C, p.tokens, p.positions = OP_EMBED, wte, wpe, out, tokens, positions
        p.M, p.N, p.vocab, p.n_pos, p.embed_scale = T, D, V, P, scale
        return _Node(p, [], [_span(out, T * D * 2)])
    if fname == "mlxb_layernorm":
        dtype, x, rows, gain, bias, out, R, D, eps, _stream = a
        if dtype != 1 or D % 8:
            return None
        p.op, p.A, p.rows, p.ln_gain, p.ln_bias, p.C, p.M, p.K, p.eps = OP_NORM, x, rows, gain, bias, out, R, D, eps
        # with a row gather the rows read are not known here: any row of x up to the end of its buffer
        reads = [_span(x, R * D * 2)] if rows is None else [(int(x), int(x) + (1 << 62))]
        return _Node(p, reads, [_span(out, R * D * 2)])
    if fname == "mlxb_linear_smallm":
        out_f32, A, W, bias, residual, C, M, N, K, lda, ldc, epi, _stream = a
        if epi not in (0, 1):
            return None
        p.op, p.A, p.W, p.bias, p.residual, p.C = OP_LINEAR, A, W, bias, residual, C
        p.M, p.N, p.K, p.lda, p.ldc = M, N, K, lda, ldc
        p.flags = (F_GELU if epi == 1 else 0) | (F_OUT_F32 if out_f32 else 0)
        esz = 4 if out_f32 else 2
        reads = [_span(A, ((M - 1) * lda + K) * 2)]
        if residual:
            reads.append(_span(residual, ((M - 1) * ldc + N) * 2))
        return _Node(p, reads, [_span(C, ((M - 1) * ldc + N) * esz)])
    if fname == "mlxb_linear_smallm_qkv":
        (A, W, bias, C, M, N, K, lda, ldc, positions, token_req, block_table, max_pages, n_pages, page, Hkv, Dh,
         q_width, k_pool, v_pool, _status, _stream) = a
        p.op, p.A, p.W, p.bias, p.C, p.flags = OP_LINEAR, A, W, bias, C, F_SCATTER
        p.M, p.N, p.K, p.lda, p.ldc = M, N, K, lda, ldc
        p.positions, p.token_req, p.block_table = positions, token_req, block_table
        p.max_pages, p.n_pages, p.page, p.Hkv, p.Dh, p.q_width = max_pages, n_pages, page, Hkv, Dh, q_width
        p.k_pool, p.v_pool = k_pool, v_pool
        return _Node(p, [_span(A, ((M - 1) * lda + K) * 2)], [_span(C, ((M - 1) * ldc + q_width) * 2)])
    if fname == "mlxb_attention_decode":
        (dtype, q, ldq, rows, positions, token_req, block_table, max_pages, n_pages, page, Hq, Hkv, Dh, window, scale,
         k_pool, v_pool, partial, counters, n_chunks, chunk, out, ldo, n_rows, _status, _stream) = a
        if dtype != 1 or Dh % 8 or page & (page - 1):
            return None
        p.op, p.A, p.lda, p.rows, p.positions, p.token_req = OP_ATTENTION, q, ldq, rows, positions, token_req
        p.block_table, p.max_pages, p.n_pages, p.page = block_table, max_pages, n_pages, page
        p.Hq, p.Hkv, p.Dh, p.window, p.scale = Hq, Hkv, Dh, window, scale
        p.k_pool, p.v_pool, p.partial, p.counters = k_pool, v_pool, partial, counters
        p.n_chunks_max, p.chunk, p.C, p.ldc, p.M = n_chunks, chunk, out, ldo, n_rows
        far = 1 << 62
        reads = [_span(q, ((n_rows - 1) * ldq + Hq * Dh) * 2)] if rows is None else [(int(q), int(q) + far)]
        writes = [_span(out, ((n_rows - 1) * ldo + Hq * Dh) * 2)] if rows is None else [(int(out), int(out) + far)]
        return _Node(p, reads, writes)
    return None


def _dead_after(nodes: List[_Node], i: int, span: Tuple[int, int]) -> bool:
    """Whether what phase i wrote to ``span`` is read by nobody but phase i + 1 (the table repeats step after
    step, so the search wraps around)."""
    n = len(nodes)
    for k in range(2, n + 1):
        nd = nodes[(i + k) % n]
        if _overlaps(span, nd.reads):
            return False
        if any(w[0] <= span[0] and span[1] <= w[1] for w in nd.writes):
            return True
    return True


class DecodeProgram:
    """The phases of one step shape on the device, and the three words its barrier lives in."""

    def __init__(self, phases: List[Phase], device):
        self.n = len(phases)
        self.max_rows = max(p.M for p in phases)
        dims = {p.Dh for p in phases if p.op == OP_ATTENTION}
        self.head_dim = dims.pop() if dims else 0
        raw = b"".join(bytes(p) for p in phases)
        self.table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
        self.sync = torch.zeros(4, dtype=torch.int32, device=device)
        tpk = 2
        while tpk * 8 < self.head_dim:
            tpk *= 2
        self.libname = f"decode_program:MLXB_DP_TPK={tpk}"
        lib = build.load(self.libname)
        lib.mlxb_decode_program_phase_bytes.restype = c_int
        if lib.mlxb_decode_program_phase_bytes() != ctypes.sizeof(Phase):
            raise RuntimeError(f"decode program: the kernel's phase record has {lib.mlxb_decode_program_phase_bytes()} "
                               f"bytes, the host's {ctypes.sizeof(Phase)}")

    def reset(self) -> None:
        """After a launch that gave up waiting: the barrier starts from zero again."""
        self.sync.zero_()


def compile_program(calls, device) -> Optional[DecodeProgram]:
    """The recorded launches of one single-token step as a program, or None when some launch has no phase,
    a size is out of the kernel's range, or the heads of the attention layers differ in size."""
    nodes: List[_Node] = []
    for _f, _lib, fname, args in calls:
        nd = _translate(fname, args)
        if nd is None:
            return None
        nodes.append(nd)
    if not nodes or any(nd.phase.M > MAX_ROWS or nd.phase.M <= 0 for nd in nodes):
        return None
    if len({nd.phase.Dh for nd in nodes if nd.phase.op == OP_ATTENTION}) > 1:
        return None
    for nd in nodes:
        p = nd.phase
        if p.op == OP_LINEAR and (p.K % 8 or p.lda % 8):
            return None
    # fold a norm into the linear layer that follows it when nobody else reads the norm's output
    fused: List[_Node] = []
    i = 0
    while i < len(nodes):
        nd = nodes[i]
        nxt = nodes[i + 1] if i + 1 < len(nodes) else None
        if (nd.phase.op == OP_NORM and nxt is not None and nxt.phase.op == OP_LINEAR
                and nxt.phase.A == nd.phase.C and nxt.phase.K == nd.phase.K and nxt.phase.lda == nd.phase.K
                and nxt.phase.M == nd.phase.M and _dead_after(nodes, i, nd.writes[0])):
            p = nxt.phase
            p.A, p.rows = nd.phase.A, nd.phase.rows
            p.ln_gain, p.ln_bias, p.eps = nd.phase.ln_gain, nd.phase.ln_bias, nd.phase.eps
            p.flags |= F_LN
            fused.append(_Node(p, nd.reads + nxt.reads[1:], nxt.writes))
            i += 2
        else:
            fused.append(nd)
            i += 1
    phases = [nd.phase for nd in fused]
    # every phase asks L2 for the weights of the phase after it
    for k, p in enumerate(phases[:-1]):
        q = phases[k + 1]
        if q.op == OP_LINEAR:
            p.next_w, p.next_bytes = q.W, q.N * q.K * 2
    return DecodeProgram(phases, device)


_ARGS = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]


def launch(program: DecodeProgram, status, stream) -> None:
    from . import _call
    _call(program.libname, "mlxb_decode_program", _ARGS, program.table.data_ptr(), program.n, program.max_rows,
          program.head_dim, program.sync.data_ptr(), status.data_ptr(), stream)
