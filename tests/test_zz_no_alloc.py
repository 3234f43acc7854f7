"""The attention entry point for callers that cannot allocate (csrc/attention_noalloc.h).

Some users of the kernel library have no way to hand it scratch memory: they run where the CUDA
allocator must not be entered, or they are thin bindings without an allocator.  For them the
library carries its own fixed scratch array.  This test calls that entry point through its
exported C symbol, exactly as such a caller would, and checks that it gives what the ordinary
entry point gives with caller-owned scratch: twice in a row with different inputs, because the
array keeps the previous call's contents and the second result must not depend on them.  It also
checks that a request larger than the array is refused, not truncated.

The file sorts last so that a run that stops at the first failure has already run everything else.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_FLOATS = 1 << 20


def _case(seed, n_rows, Hq, Hkv, Dh, page, ctx_lens, dtype):
    g = torch.Generator().manual_seed(seed)
    n_pages_needed = sum((l + page) // page for l in ctx_lens)
    n_pages = n_pages_needed + 5
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max((l + page) // page for l in ctx_lens) + 1
    bt = torch.full((n_rows, width), -1, dtype=torch.int32)
    for r, l in enumerate(ctx_lens):
        for lp in range((l + page) // page):      # positions 0..l, the query sits at position l
            bt[r, lp] = perm.pop()
    mk = lambda *s: torch.randn(*s, generator=g).to(dtype).cuda()
    return dict(q=mk(n_rows, Hq * Dh), k=mk(n_pages, Hkv, page, Dh), v=mk(n_pages, Hkv, page, Dh), bt=bt.cuda(),
                positions=torch.tensor(ctx_lens, dtype=torch.int32).cuda(),
                token_req=torch.arange(n_rows, dtype=torch.int32).cuda(), n_pages=n_pages, width=width)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_point_matches_the_ordinary_one(dtype):
    from mlx_lm_b200 import ops
    from mlx_lm_b200.ops import build

    lib = build.load("attention")
    fn = lib.mlxb_attention_decode_noalloc
    fn.restype = c_int
    fn.argtypes = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                   c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                   c_void_p]
    Hq, Hkv, Dh, page, chunk, max_len = 6, 3, 64, 16, 128, 512
    n_chunks = max_len // chunk
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    for seed, lens in ((1, [300, 0, 127, 128, 511]), (2, [17, 450, 64])):      # two calls in a row
        c = _case(seed, len(lens), Hq, Hkv, Dh, page, lens, dtype)
        n = len(lens)
        want = torch.zeros(n, Hq * Dh, dtype=dtype, device="cuda")
        scratch = torch.empty(ops.attention_decode_scratch(n, Hq, Dh, max_len, chunk), device="cuda")
        counters = torch.zeros(n * Hq, dtype=torch.int32, device="cuda")
        ops.attention_decode(c["q"], c["positions"], c["token_req"], c["bt"], c["k"], c["v"], want, Hq, Dh ** -0.5, 0,
                             scratch, counters, max_len, status, stream, chunk=chunk)
        got = torch.zeros_like(want)
        rc = fn(ops.dtype_code(dtype), c["q"].data_ptr(), Hq * Dh, None, c["positions"].data_ptr(),
                c["token_req"].data_ptr(), c["bt"].data_ptr(), c["width"], c["n_pages"], page, Hq, Hkv, Dh, 0,
                Dh ** -0.5, c["k"].data_ptr(), c["v"].data_ptr(), n_chunks, chunk, got.data_ptr(), Hq * Dh, n,
                status.data_ptr(), stream)
        assert rc == 0, lib.mlxb_last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        scale = max(1e-6, float(want.float().abs().max()))
        assert float((got.float() - want.float()).abs().max()) / scale <= tol
        assert float(got.float().abs().max()) > 0
    # A position the chunks do not cover: that row is skipped and reported in the status word, it takes no
    # ticket from the library's counters, and the next, valid call is as right as before.
    c = _case(3, 3, Hq, Hkv, Dh, page, [40, 200, 90], dtype)
    bad = c["positions"].clone()
    bad[1] = n_chunks * chunk           # first position beyond the covered range
    got = torch.zeros(3, Hq * Dh, dtype=dtype, device="cuda")
    call = lambda positions: fn(ops.dtype_code(dtype), c["q"].data_ptr(), Hq * Dh, None, positions.data_ptr(),
                                c["token_req"].data_ptr(), c["bt"].data_ptr(), c["width"], c["n_pages"], page, Hq, Hkv,
                                Dh, 0, Dh ** -0.5, c["k"].data_ptr(), c["v"].data_ptr(), n_chunks, chunk,
                                got.data_ptr(), Hq * Dh, 3, status.data_ptr(), stream)
    assert call(bad) == 0, lib.mlxb_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == ops.ST_POSITION_RANGE
    assert float(got[1].float().abs().max()) == 0.0 and float(got[0].float().abs().max()) > 0
    status.zero_()
    want = torch.zeros_like(got)
    scratch = torch.empty(ops.attention_decode_scratch(3, Hq, Dh, max_len, chunk), device="cuda")
    counters = torch.zeros(3 * Hq, dtype=torch.int32, device="cuda")
    ops.attention_decode(c["q"], c["positions"], c["token_req"], c["bt"], c["k"], c["v"], want, Hq, Dh ** -0.5, 0,
                         scratch, counters, max_len, status, stream, chunk=chunk)
    assert call(c["positions"]) == 0, lib.mlxb_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert float((got.float() - want.float()).abs().max()) / max(1e-6, float(want.float().abs().max())) <= tol
    # beyond the built-in array: refused with a message, nothing launched
    rows_too_many = MAX_FLOATS // (Hq * n_chunks * (Dh + 2)) + 1
    rc = fn(ops.dtype_code(dtype), c["q"].data_ptr(), Hq * Dh, None, c["positions"].data_ptr(),
            c["token_req"].data_ptr(), c["bt"].data_ptr(), c["width"], c["n_pages"], page, Hq, Hkv, Dh, 0, Dh ** -0.5,
            c["k"].data_ptr(), c["v"].data_ptr(), n_chunks, chunk, got.data_ptr(), Hq * Dh, rows_too_many,
            status.data_ptr(), stream)
    assert rc < 0 and b"built-in array holds" in lib.mlxb_last_error()
