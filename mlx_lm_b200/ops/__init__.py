"""Python face of the CUDA kernels.

Each function checks what the kernel cannot check for itself (device, dtype,
contiguity, matching sizes), passes raw pointers and the CUDA stream to the
``extern "C"`` launcher of the kernel's library and raises on a non-zero
return code with the launcher's own message.  There is no fallback: without
a CUDA device, or if a library cannot be built, these functions raise.

Tensors are torch tensors used as typed device buffers; no torch operator
runs in here.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from . import build

import os as _os

F32, BF16 = 0, 1


def _read_activations():
    """``{name: code}`` from the one list of epilogue activations, csrc/activations.cuh, which every linear
    kernel includes: lines ``X(IDENTIFIER, code, name)``."""
    import os
    import re

    with open(os.path.join(build.CSRC, "activations.cuh")) as f:
        text = f.read()
    body = text[text.index("#define MLXB_ACTIVATION_LIST"):]
    body = body[:body.index("\n\n")]
    found = {m.group(3): int(m.group(2)) for m in re.finditer(r"X\((\w+),\s*(\d+),\s*(\w+)\)", body)}
    if "none" not in found or sorted(found.values()) != list(range(len(found))):
        raise RuntimeError(f"csrc/activations.cuh: cannot read the list of activations ({found})")
    return found


ACTIVATION_CODES = _read_activations()
EPI_NONE = ACTIVATION_CODES["none"]
EPI_GELU_NEW = ACTIVATION_CODES["gelu_new"]

_DT = {torch.float32: F32, torch.bfloat16: BF16}

# kernel sources that only a bfloat16 run launches from: a float32 run neither compiles nor loads them
BF16_ONLY_LIBS = frozenset({"gemm_smallm", "gemm_smallm_fold", "gemm_tcgen05", "attention_prefill",
                            "attention_prefill_tc"})

# status word bits set by kernels (csrc/common.cuh)
ST_TOKEN_RANGE, ST_POSITION_RANGE, ST_PAGE_RANGE, ST_WAIT_TIMEOUT = 1, 2, 4, 8


class KernelError(RuntimeError):
    pass


def describe_status(word: int) -> str:
    """The bits of a status word in words."""
    names = [n for b, n in ((ST_TOKEN_RANGE, "token id out of range"),
                            (ST_POSITION_RANGE, "position without a page or out of range"),
                            (ST_PAGE_RANGE, "page id outside the pool"),
                            (ST_WAIT_TIMEOUT, "a bounded wait in a kernel gave up")) if word & b]
    return "; ".join(names) or f"status {word}"


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError(
            "mlx_lm_b200 runs on a CUDA device (NVIDIA B200, sm_100a) only: no device is visible and "
            "there is no CPU path")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise KernelError(f"unsupported dtype {dt}: the engine runs in float32 or bfloat16") from None


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dt, what: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}, not on a CUDA device")
    if dt is not None and t.dtype != dt:
        raise KernelError(f"{what}: dtype {t.dtype}, expected {dt}")


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what}: expected a 2-D tensor with contiguous rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")
    return t.stride(0)


_fn_cache = {}


def _fn(libname: str, fname: str, argtypes):
    key = (libname, fname)
    hit = _fn_cache.get(key)
    if hit is None:
        lib = build.load(libname)
        f = getattr(lib, fname)
        f.argtypes = argtypes
        f.restype = c_int
        hit = _fn_cache[key] = (f, lib)
    return hit


launch_count = 0   # kernel launches issued through this module (bench.py reads and resets it)
_recording = None  # while a list: every launch is appended as (launcher, library, name, arguments, label)
_label = None      # what the launches that follow are part of: (name, flops, bytes), set by the parts


def label(name: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
    """Name the work the following launches belong to (a part's tensor name, say) with the floating-point
    operations and the bytes it has to move, where the caller knows them.  Recorded launches carry the label;
    the measuring tools group and rate kernels by it.  Costs nothing when nothing is recorded."""
    global _label
    if _recording is not None:
        _label = (name, float(flops), float(nbytes))


def start_recording() -> None:
    """Begin to note every launch with its raw arguments, so that a step of the same shape can be
    re-issued later without going through the checks and the parts again (``replay``)."""
    global _recording, _label
    _recording = []
    _label = None


def stop_recording():
    global _recording
    calls, _recording = _recording, None
    return calls


def replay(calls) -> None:
    """Re-issue recorded launches.  The caller guarantees that every buffer they name is still where it was."""
    global launch_count
    for f, lib, fname, args, _ in calls:
        rc = f(*args)
        if rc != 0:
            msg = lib.mlxb_last_error()
            raise KernelError(f"{fname} failed ({rc}): {msg.decode() if msg else ''}")
    launch_count += len(calls)


def _call(libname: str, fname: str, argtypes, *args) -> None:
    global launch_count
    f, lib = _fn(libname, fname, argtypes)
    launch_count += 1
    rc = f(*args)
    if rc != 0:
        msg = lib.mlxb_last_error()
        raise KernelError(f"{fname} failed ({rc}): {msg.decode() if msg else ''}")
    if _recording is not None:
        _recording.append((f, lib, fname, args, _label))


# --------------------------------------------------------------------------
# embedding + position add

_EMBED_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
               c_void_p, c_void_p]


def embed_pos(tokens, positions, wte, wpe, out, status, stream, scale: float = 1.0) -> None:
    """``out[t] = wte[tokens[t]] * scale + wpe[positions[t]]`` (``wpe`` may be None)."""
    _need(tokens, torch.int32, "embed_pos tokens")
    _need(wte, out.dtype, "embed_pos wte")
    T, D = out.shape
    if wte.shape[1] != D or not wte.is_contiguous() or not out.is_contiguous():
        raise KernelError(f"embed_pos: table {tuple(wte.shape)} against output {tuple(out.shape)}")
    if wpe is not None:
        _need(positions, torch.int32, "embed_pos positions")
        _need(wpe, out.dtype, "embed_pos wpe")
        if wpe.shape[1] != D or not wpe.is_contiguous():
            raise KernelError(f"embed_pos: position table {tuple(wpe.shape)} against width {D}")
    _call("embed", "mlxb_embed_pos", _EMBED_ARGS, dtype_code(out.dtype), _p(tokens), _p(positions), _p(wte),
          _p(wpe), _p(out), T, D, wte.shape[0], 0 if wpe is None else wpe.shape[0], scale, _p(status), stream)


def gather_tokens(src, index, dst, status, stream) -> None:
    """``dst[i] = src[index[i]]`` where ``index[i] >= 0`` (int32 all): tokens a step has just sampled, handed
    to the next step on the device."""
    for t, what in ((src, "src"), (index, "index"), (dst, "dst")):
        _need(t, torch.int32, f"gather_tokens {what}")
    if index.numel() < dst.numel():
        raise KernelError(f"gather_tokens: {index.numel()} indices for {dst.numel()} tokens")
    _call("embed", "mlxb_gather_tokens", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
          _p(src), src.numel(), _p(index), _p(dst), dst.numel(), _p(status), stream)


# --------------------------------------------------------------------------
# norms

_LN_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]


def layernorm(x, gain, bias, out, eps: float, stream, rows=None) -> None:
    """``out[r] = LayerNorm(x[rows[r]] if rows is given else x[r])``; statistics in float32."""
    _need(x, out.dtype, "layernorm x")
    _need(gain, torch.float32, "layernorm gain")
    if bias is not None:
        _need(bias, torch.float32, "layernorm bias")
    R, D = out.shape
    if x.shape[1] != D or gain.numel() != D or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError(f"layernorm: x {tuple(x.shape)}, gain {tuple(gain.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _need(rows, torch.int32, "layernorm rows")
        if rows.numel() != R:
            raise KernelError(f"layernorm: {rows.numel()} row indices for {R} output rows")
    elif x.shape[0] != R:
        raise KernelError(f"layernorm: {x.shape[0]} input rows for {R} output rows")
    _call("norm", "mlxb_layernorm", _LN_ARGS, dtype_code(out.dtype), _p(x), _p(rows), _p(gain), _p(bias), _p(out),
          R, D, eps, stream)


_STATS_ARGS = [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]


def row_stats(x, stats, eps: float, stream) -> None:
    """``stats[r] = (mean, 1/sqrt(var + eps))`` of the bfloat16 rows of ``x`` (float32 ``[R, 2]``): what the
    epilogue of a linear layer with a folded LayerNorm needs of the rows."""
    _need(x, torch.bfloat16, "row_stats x")
    _need(stats, torch.float32, "row_stats stats")
    R, D = x.shape
    if stats.shape != (R, 2) or not stats.is_contiguous():
        raise KernelError(f"row_stats: statistics {tuple(stats.shape)} for {R} rows")
    _call("norm", "mlxb_row_stats", _STATS_ARGS, _p(x), _p(stats), R, D, _rows(x, "row_stats x"), eps, stream)


_GATHER_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]


def gather_rows(x, rows, out, stream) -> None:
    """``out[r] = x[rows[r]]`` (a row index outside ``x`` gives a row of zeros)."""
    _need(x, out.dtype, "gather_rows x")
    _need(rows, torch.int32, "gather_rows rows")
    R, D = out.shape
    if x.dim() != 2 or x.shape[1] != D or rows.numel() != R or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError(f"gather_rows: x {tuple(x.shape)}, {rows.numel()} indices, out {tuple(out.shape)}")
    _call("norm", "mlxb_gather_rows", _GATHER_ARGS, dtype_code(out.dtype), _p(x), _p(rows), _p(out), R, D, x.shape[0],
          stream)


# --------------------------------------------------------------------------
# linear layers

_SIMT_ARGS = [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
              c_int, c_void_p]


def linear_generic(x, w, bias, out, stream, epilogue: int = EPI_NONE, residual=None) -> None:
    """``out = epilogue(x @ w.T + bias) + residual`` on the CUDA cores in float32 arithmetic.

    ``x [M,K]``, ``w [N,K]`` (rows are output features) and ``residual [M,N]`` share a dtype;
    ``out [M,N]`` has that dtype or float32; ``bias`` is float32."""
    _need(x, None, "linear x")
    _need(w, x.dtype, "linear w")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lda, ldc = _rows(x, "linear x"), _rows(out, "linear out")
    out_f32 = 0
    if out.dtype != x.dtype:
        if out.dtype != torch.float32:
            raise KernelError(f"linear: output dtype {out.dtype} for input dtype {x.dtype}")
        out_f32 = 1
    if bias is not None:
        _need(bias, torch.float32, "linear bias")
        if bias.numel() != N:
            raise KernelError(f"linear: bias of {bias.numel()} for {N} outputs")
    if residual is not None:
        _need(residual, x.dtype, "linear residual")
        if residual.shape != out.shape or _rows(residual, "linear residual") != ldc:
            raise KernelError("linear: residual must have the output's shape and row stride")
    _call("gemm_simt", "mlxb_linear_simt", _SIMT_ARGS, dtype_code(x.dtype), out_f32, _p(x), _p(w), _p(bias),
          _p(residual), _p(out), M, N, K, lda, ldc, epilogue, stream)


_SMALLM_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                c_void_p]

SMALL_M = 64

_SMALLM_FOLD_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                     c_void_p, c_float, c_void_p]


def _fold_args(fold, N: int, what: str):
    colsum, eps = fold
    _need(colsum, torch.float32, what + " column sums")
    if colsum.numel() != N or not colsum.is_contiguous():
        raise KernelError(f"{what}: {colsum.numel()} column sums for {N} outputs")
    return colsum, float(eps)


def linear_few_rows(x, w, bias, out, stream, epilogue: int = EPI_NONE, residual=None, fold=None) -> None:
    """``linear_generic``'s contract for bfloat16 and at most 64 rows: the weight is streamed from HBM once
    with 16-byte loads and multiplied on the tensor cores (csrc/gemm_smallm.cuh).  ``K`` and the row stride of
    ``x`` must be multiples of 8.

    ``fold = (colsum, eps)``: ``x`` holds the rows before a LayerNorm that has been folded into ``w`` and ``bias``
    (``parts.linear.Linear.fold_norm``); the kernel computes ``rstd (x w^T - mean colsum) + bias`` with the
    rows' mean and 1/std found on the way."""
    _need(x, torch.bfloat16, "linear x")
    _need(w, torch.bfloat16, "linear w")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lda, ldc = _rows(x, "linear x"), _rows(out, "linear out")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"linear: output dtype {out.dtype}")
    if bias is not None:
        _need(bias, torch.float32, "linear bias")
        if bias.numel() != N:
            raise KernelError(f"linear: bias of {bias.numel()} for {N} outputs")
    if residual is not None:
        _need(residual, torch.bfloat16, "linear residual")
        if residual.shape != out.shape or _rows(residual, "linear residual") != ldc:
            raise KernelError("linear: residual must have the output's shape and row stride")
    if fold is not None:
        colsum, eps = _fold_args(fold, N, "linear")
        _call("gemm_smallm_fold", "mlxb_linear_smallm_fold", _SMALLM_FOLD_ARGS, int(out.dtype == torch.float32), _p(x),
              _p(w), _p(bias), _p(residual), _p(out), M, N, K, lda, ldc, epilogue, _p(colsum), eps, stream)
        return
    _call("gemm_smallm", "mlxb_linear_smallm", _SMALLM_ARGS, int(out.dtype == torch.float32), _p(x), _p(w), _p(bias),
          _p(residual), _p(out), M, N, K, lda, ldc, epilogue, stream)


_TC_ARGS = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
            c_void_p, c_void_p]


_TC_FOLD_ARGS = _TC_ARGS[:-1] + [c_void_p, c_void_p, c_void_p]


def linear_tensor_cores(x, w, bias, out, status, stream, epilogue: int = EPI_NONE, residual=None, fold=None) -> None:
    """``linear_generic``'s contract for bfloat16 and many rows, on tcgen05 tensor cores with TMA-fed
    shared-memory stages and the accumulator in tensor memory (csrc/gemm_tcgen05.cu).  ``K`` and the row
    stride of ``x`` must be multiples of 8.  ``status`` receives ``ST_WAIT_TIMEOUT`` if a bounded wait gives up.

    ``fold = (colsum, stats)``: a LayerNorm folded into ``w`` and ``bias``; ``x`` holds the rows before the norm
    and ``stats`` their ``(mean, rstd)`` from ``row_stats``."""
    _need(x, torch.bfloat16, "linear x")
    _need(w, torch.bfloat16, "linear w")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lda, ldc = _rows(x, "linear x"), _rows(out, "linear out")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"linear: output dtype {out.dtype}")
    if bias is not None:
        _need(bias, torch.float32, "linear bias")
        if bias.numel() != N:
            raise KernelError(f"linear: bias of {bias.numel()} for {N} outputs")
    if residual is not None:
        _need(residual, torch.bfloat16, "linear residual")
        if residual.shape != out.shape or _rows(residual, "linear residual") != ldc:
            raise KernelError("linear: residual must have the output's shape and row stride")
    if fold is not None:
        colsum, stats = fold
        _need(colsum, torch.float32, "linear column sums")
        _need(stats, torch.float32, "linear row statistics")
        if colsum.numel() != N or stats.shape != (M, 2) or not stats.is_contiguous():
            raise KernelError(f"linear: {colsum.numel()} column sums, statistics {tuple(stats.shape)} for {M} x {N}")
        _call("gemm_tcgen05", "mlxb_linear_tcgen05_fold", _TC_FOLD_ARGS, int(out.dtype == torch.float32), _p(x), _p(w),
              _p(bias), _p(residual), _p(out), M, N, K, lda, ldc, epilogue, _p(status), _p(colsum), _p(stats), stream)
        return
    _call("gemm_tcgen05", "mlxb_linear_tcgen05", _TC_ARGS, int(out.dtype == torch.float32), _p(x), _p(w), _p(bias),
          _p(residual), _p(out), M, N, K, lda, ldc, epilogue, _p(status), stream)


_QKV_ARGS = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]


_QKV_FOLD_ARGS = _QKV_ARGS[:-1] + [c_void_p, c_float, c_void_p]
_QKV_TC_FOLD_ARGS = _QKV_ARGS[:-1] + [c_void_p, c_void_p, c_void_p]


def linear_qkv_to_cache(x, w, bias, out, positions, token_req, block_table, k_pool, v_pool, q_width: int, status,
                        stream, fold=None) -> None:
    """The fused ``[q | k | v]`` projection of bfloat16 rows with the cache write in its epilogue: query columns
    go to ``out[:, :q_width]``, key and value columns straight into the pages ``[n_pages, Hkv, page, Dh]`` (the
    other columns of ``out`` are not written).  Up to 64 rows run in the weight-streaming kernel, more in the
    tcgen05 kernel.  ``fold``: ``(colsum, eps)`` as in ``linear_few_rows`` for up to 64 rows, ``(colsum, stats)`` as
    in ``linear_tensor_cores`` for more."""
    _need(x, torch.bfloat16, "linear x")
    _need(w, torch.bfloat16, "linear w")
    _need(out, torch.bfloat16, "linear out")
    _need(k_pool, torch.bfloat16, "linear k_pool")
    M, K = x.shape
    N = w.shape[0]
    n_pages, Hkv, page, Dh = k_pool.shape
    if w.shape[1] != K or not w.is_contiguous() or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if N != q_width + 2 * Hkv * Dh or not (k_pool.is_contiguous() and v_pool.is_contiguous()):
        raise KernelError(f"linear (q|k|v): {N} outputs for {q_width} query columns and pools {tuple(k_pool.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "linear bias")
    if fold is not None and M > SMALL_M:
        colsum, stats = fold
        _need(colsum, torch.float32, "linear column sums")
        if not torch.is_tensor(stats) or stats.dtype != torch.float32 or stats.shape != (M, 2) or not stats.is_contiguous():
            raise KernelError(f"linear (q|k|v): more than {SMALL_M} rows need float32 row statistics [{M}, 2]")
        _call("gemm_tcgen05", "mlxb_linear_tcgen05_qkv_fold", _QKV_TC_FOLD_ARGS, _p(x), _p(w), _p(bias), _p(out), M, N, K,
              _rows(x, "linear x"), _rows(out, "linear out"), _p(positions), _p(token_req), _p(block_table),
              block_table.shape[1], n_pages, page, Hkv, Dh, q_width, _p(k_pool), _p(v_pool), _p(status), _p(colsum),
              _p(stats), stream)
        return
    if fold is not None:
        colsum, eps = _fold_args(fold, N, "linear (q|k|v)")
        _call("gemm_smallm_fold", "mlxb_linear_smallm_qkv_fold", _QKV_FOLD_ARGS, _p(x), _p(w), _p(bias), _p(out), M, N, K,
              _rows(x, "linear x"), _rows(out, "linear out"), _p(positions), _p(token_req), _p(block_table),
              block_table.shape[1], n_pages, page, Hkv, Dh, q_width, _p(k_pool), _p(v_pool), _p(status), _p(colsum), eps,
              stream)
        return
    lib, fn = ("gemm_smallm", "mlxb_linear_smallm_qkv") if M <= SMALL_M else ("gemm_tcgen05", "mlxb_linear_tcgen05_qkv")
    _call(lib, fn, _QKV_ARGS, _p(x), _p(w), _p(bias), _p(out), M, N, K,
          _rows(x, "linear x"), _rows(out, "linear out"), _p(positions), _p(token_req), _p(block_table),
          block_table.shape[1], n_pages, page, Hkv, Dh, q_width, _p(k_pool), _p(v_pool), _p(status), stream)


# --------------------------------------------------------------------------
# paged key/value cache and attention

_KVW_ARGS = [c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_void_p, c_void_p, c_int, c_void_p, c_void_p]


def kv_write(k_src, v_src, positions, token_req, block_table, k_pool, v_pool, status, stream) -> None:
    """Store this step's key and value rows into the pages of one layer.

    ``k_src``/``v_src``: ``[T, Hkv*Dh]`` views (same row stride); pools ``[n_pages, Hkv, page, Dh]``."""
    n_pages, Hkv, page, Dh = k_pool.shape
    _need(k_src, k_pool.dtype, "kv_write k")
    _need(v_src, k_pool.dtype, "kv_write v")
    ld = _rows(k_src, "kv_write k")
    if _rows(v_src, "kv_write v") != ld or k_src.shape[1] != Hkv * Dh or v_src.shape != k_src.shape:
        raise KernelError(f"kv_write: k {tuple(k_src.shape)} v {tuple(v_src.shape)} for pool {tuple(k_pool.shape)}")
    if not (k_pool.is_contiguous() and v_pool.is_contiguous() and block_table.is_contiguous()):
        raise KernelError("kv_write: pools and block table must be contiguous")
    _call("attention", "mlxb_kv_write", _KVW_ARGS, dtype_code(k_pool.dtype), _p(k_src), _p(v_src), ld,
          _p(positions), _p(token_req), _p(block_table), block_table.shape[1], n_pages, page, Hkv, Dh,
          _p(k_pool), _p(v_pool), k_src.shape[0], _p(status), stream)


_ATTN_ARGS = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
              c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p]


def _attn_shapes(q, out, k_pool, n_heads, what):
    n_pages, Hkv, page, Dh = k_pool.shape
    _need(q, k_pool.dtype, what + " q")
    _need(out, k_pool.dtype, what + " out")
    if q.shape[1] != n_heads * Dh or out.shape[0] != q.shape[0] or out.shape[1] != n_heads * Dh:
        raise KernelError(f"{what}: q {tuple(q.shape)} out {tuple(out.shape)} for {n_heads} heads of {Dh}")
    return n_pages, Hkv, page, Dh


def attention_generic(q, positions, token_req, block_table, k_pool, v_pool, out, n_heads: int, scale: float,
                      window: int, status, stream, rows=None) -> None:
    """Causal attention of tokens over their requests' pages (float32 math, one warp per token and head).

    ``q``: ``[T, n_heads*Dh]`` view; ``out``: ``[T, n_heads*Dh]``; ``rows``: int32 token indices to run
    (default all ``T``); ``window <= 0`` means all keys."""
    n_pages, Hkv, page, Dh = _attn_shapes(q, out, k_pool, n_heads, "attention")
    n = q.shape[0] if rows is None else rows.numel()
    _call("attention", "mlxb_attention_generic", _ATTN_ARGS, dtype_code(k_pool.dtype), _p(q), _rows(q, "attention q"),
          _p(positions), _p(token_req), _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv, Dh,
          window, scale, _p(k_pool), _p(v_pool), _p(out), _rows(out, "attention out"), _p(rows), n, _p(status),
          stream)


_PRE_ARGS = [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
             c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]

PREFILL_TILE = int(_os.environ.get("MLXB_PREFILL_TILE", "128"))   # queries per CTA of the attention kernels for portions
PREFILL_TC = _os.environ.get("MLXB_PREFILL_TC", "1") != "0"         # heads of 64 in tiles of 128 on the tcgen05 kernel

_PRE_TC_ARGS = [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]


def attention_portions_supported(dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128


def attention_portions(q, tiles, n_tiles: int, block_table, k_pool, v_pool, out, n_heads: int, scale: float,
                       window: int, status, stream, tile_rows: int = 0) -> None:
    """Causal attention of prompt portions on tensor cores (bfloat16, csrc/attention_prefill.cu).

    ``tiles``: int32 device tensor ``[n_tiles, 4]``: first token row of the tile, queries in it (1..64),
    block-table row of its request, position of its first query."""
    n_pages, Hkv, page, Dh = _attn_shapes(q, out, k_pool, n_heads, "attention_portions")
    _need(tiles, torch.int32, "attention_portions tiles")
    if tiles.numel() < 4 * n_tiles:
        raise KernelError(f"attention_portions: {tiles.numel()} integers for {n_tiles} tiles")
    tile_rows = tile_rows or PREFILL_TILE
    ldq, ldo = _rows(q, "attention q"), _rows(out, "attention out")
    if (PREFILL_TC and Dh == 64 and tile_rows == 128 and 8 <= page <= 128 and page & (page - 1) == 0
            and ldq % 8 == 0 and ldo % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0):
        _call("attention_prefill_tc", "mlxb_attention_prefill_tc", _PRE_TC_ARGS, _p(q), ldq, q.shape[0], _p(tiles),
              n_tiles, _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv, Dh, window, scale,
              _p(k_pool), _p(v_pool), _p(out), ldo, _p(status), stream)
        return
    _call("attention_prefill", "mlxb_attention_prefill", _PRE_ARGS, _p(q), _rows(q, "attention q"), _p(tiles), n_tiles,
          tile_rows, _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv, Dh, window, scale, _p(k_pool),
          _p(v_pool), _p(out), _rows(out, "attention out"), _p(status), stream)


_ROWS_ARGS = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
              c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]


# (row, head) pairs from which single-token rows run on the tensor-core kernel: about seven times the number
# of SMs.  Below that the split-key kernel on the CUDA cores is as fast or faster inside a step (GPT-2 medium
# on a B200, 512-token contexts: 16 rows 0.88 against 0.96 ms a step, 32 rows 1.37 both, 64 rows 2.24 against 2.07).
ROWS_MIN_PAIRS = int(_os.environ.get("MLXB_ROWS_MIN_PAIRS", "1024"))


def attention_rows_supported(dtype, head_dim: int, n_rows: int = 1 << 30, n_heads: int = 1) -> bool:
    """Whether these single-token rows run on the tensor-core kernel (else: ``attention_decode``)."""
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128
            and n_rows * n_heads >= ROWS_MIN_PAIRS)


_sm_count = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def attention_rows(q, tiles, n_rows: int, block_table, k_pool, v_pool, out, n_heads: int, scale: float, window: int,
                   status, stream) -> None:
    """Attention of rows with a single query each (decode steps) on tensor cores (bfloat16,
    csrc/attention_prefill.cu): ``tiles`` is an int32 device tensor ``[n_rows, 4]`` = (token row, 1, block-table
    row, position), or (token row, 0, 0, 0) for a padding row."""
    n_pages, Hkv, page, Dh = _attn_shapes(q, out, k_pool, n_heads, "attention_rows")
    _need(tiles, torch.int32, "attention_rows tiles")
    if tiles.numel() < 4 * n_rows:
        raise KernelError(f"attention_rows: {tiles.numel()} integers for {n_rows} rows")
    _call("attention_prefill", "mlxb_attention_rows", _ROWS_ARGS, _p(q), _rows(q, "attention q"), _p(tiles), n_rows,
          _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv, Dh, window, scale, _p(k_pool),
          _p(v_pool), _p(out), _rows(out, "attention out"), _p(status), stream)


_DEC_ARGS = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
             c_void_p]

DECODE_CHUNK = 1024   # key positions per CTA of the single-token attention kernel: a constant, never a function of the batch


def attention_decode_scratch(n_rows: int, n_heads: int, head_dim: int, max_len: int, chunk: int = DECODE_CHUNK) -> int:
    """Float32 elements of scratch memory ``attention_decode`` needs for ``n_rows`` rows."""
    return n_rows * n_heads * ((max_len + chunk - 1) // chunk) * (head_dim + 2)


def attention_decode(q, positions, token_req, block_table, k_pool, v_pool, out, n_heads: int, scale: float,
                     window: int, scratch, counters, max_len: int, status, stream, rows=None,
                     chunk: int = DECODE_CHUNK) -> None:
    """Attention for rows with a single query each (decode steps): keys are cut into chunks of ``chunk``
    positions, one CTA per (chunk, head, row) writes a partial result to ``scratch`` (float32, at least
    ``attention_decode_scratch(...)`` elements) and the CTA that finishes last for a (row, head) combines
    them.  ``counters``: int32, at least rows x heads, zero before the first call (every call leaves it zero)."""
    n_pages, Hkv, page, Dh = _attn_shapes(q, out, k_pool, n_heads, "attention_decode")
    n = q.shape[0] if rows is None else rows.numel()
    n_chunks = (max_len + chunk - 1) // chunk
    _need(scratch, torch.float32, "attention_decode scratch")
    _need(counters, torch.int32, "attention_decode counters")
    if scratch.numel() < n * n_heads * n_chunks * (Dh + 2) or counters.numel() < n * n_heads:
        raise KernelError(f"attention_decode: scratch of {scratch.numel()} floats, {counters.numel()} counters "
                          f"for {n} rows")
    _call("attention", "mlxb_attention_decode", _DEC_ARGS, dtype_code(k_pool.dtype), _p(q), _rows(q, "attention q"),
          _p(rows), _p(positions), _p(token_req), _p(block_table), block_table.shape[1], n_pages, page, n_heads, Hkv,
          Dh, window, scale, _p(k_pool), _p(v_pool), _p(scratch), _p(counters), n_chunks, chunk, _p(out),
          _rows(out, "attention out"), n, _p(status), stream)


# --------------------------------------------------------------------------
# sampling and logits processors

SAMPLE_WORDS, PROCESS_WORDS = 16, 8

_SAMPLE_ARGS = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                c_void_p, c_void_p, c_void_p, c_int, c_void_p]
SAMPLE_SCRATCH_WORDS_PER_ROW = 65      # csrc/sampling.cu: mlxb_sample_scratch_words


def sample_scratch(n_rows: int, device) -> torch.Tensor:
    """Scratch memory for ``sample`` over up to ``n_rows`` rows: zero, and left zero by every launch.  One per
    stream on which launches may overlap."""
    return torch.zeros(max(1, n_rows) * SAMPLE_SCRATCH_WORDS_PER_ROW, dtype=torch.int32, device=device)


def sample(logits, params, out_token, out_logprob, stream, xtc_special=None, out_logprobs=None, status=None,
           status_out=None, scratch=None) -> None:
    """One token per row of float32 ``logits [R, V]``.

    ``params``: int32 ``[R, 16]`` holding the bit patterns of csrc/sampling.cu's ``SampleParams``;
    ``out_token`` int32 ``[R]``, ``out_logprob`` float32 ``[R]`` (log-probability of the chosen token
    under the unfiltered distribution); ``out_logprobs`` (optional) float32 ``[R, V]`` receives
    ``logits - logsumexp(logits)``.  ``xtc_special``: int32 list of the rows' XTC special tokens, each
    row's record naming its range.  ``status`` / ``status_out`` (int32, one word each): the kernel copies
    the step's status word next to its results, so that the host reads both with one copy.  ``scratch``
    (from ``sample_scratch``, for at least this many rows): with it the rows of a wide vocabulary are cut into
    slices over several thread blocks; the tokens are the same with and without it."""
    _need(logits, torch.float32, "sample logits")
    _need(params, torch.int32, "sample params")
    _need(out_token, torch.int32, "sample out_token")
    _need(out_logprob, torch.float32, "sample out_logprob")
    R, V = logits.shape
    if params.numel() < R * SAMPLE_WORDS or out_token.numel() < R or out_logprob.numel() < R:
        raise KernelError(f"sample: {R} rows need {R * SAMPLE_WORDS} parameter words and {R} outputs")
    ldo = 0
    if out_logprobs is not None:
        _need(out_logprobs, torch.float32, "sample out_logprobs")
        if out_logprobs.shape != logits.shape:
            raise KernelError("sample: out_logprobs must have the shape of logits")
        ldo = _rows(out_logprobs, "sample out_logprobs")
    n_special = 0
    if xtc_special is not None:
        _need(xtc_special, torch.int32, "sample xtc_special")
        n_special = xtc_special.numel()
    if (status is None) != (status_out is None):
        raise KernelError("sample: status and status_out go together")
    if status is not None:
        _need(status, torch.int32, "sample status")
        _need(status_out, torch.int32, "sample status_out")
    _call("sampling", "mlxb_sample", _SAMPLE_ARGS, _p(logits), _rows(logits, "sample logits"), R, V, _p(params),
          _p(xtc_special), n_special, _p(out_token), _p(out_logprob), _p(out_logprobs), ldo, _p(status),
          _p(status_out), _p(scratch), 0 if scratch is None else scratch.numel(), stream)


_PROCESS_ARGS = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p]


def process_logits(logits, params, context, bias_index, bias_value, stream) -> None:
    """In place on float32 ``logits [R, V]``: additive bias, then repetition, presence and frequency
    penalties over each row's recent tokens.  ``params`` int32 ``[R, 8]`` (``ProcessParams`` bit
    patterns); ``context`` int32 ``[R, C]`` left-padded with -1; ``bias_index`` int32 / ``bias_value``
    float32 ``[R, B]``."""
    _need(logits, torch.float32, "process_logits logits")
    _need(params, torch.int32, "process_logits params")
    _need(context, torch.int32, "process_logits context")
    R, V = logits.shape
    C = context.shape[1] if context.dim() == 2 else 0
    B = bias_index.shape[1] if bias_index is not None and bias_index.dim() == 2 else 0
    if B:
        _need(bias_index, torch.int32, "process_logits bias_index")
        _need(bias_value, torch.float32, "process_logits bias_value")
    _call("sampling", "mlxb_process_logits", _PROCESS_ARGS, _p(logits), _rows(logits, "process_logits logits"), R, V,
          _p(params), _p(context), C, _p(bias_index) if B else None, _p(bias_value) if B else None, B, stream)
