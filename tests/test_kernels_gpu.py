"""Each CUDA kernel alone against its plain statement in kernel_refs.py, at sizes other than the
engine's tiny configurations: widths and vocabularies that are no power of two, head sizes in
steps of 16, grouped heads, windows, pages of several sizes, block tables in scrambled order."""
import math

import numpy as np
import pytest
import torch

import kernel_refs as R

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, f32=1e-5, bf16=1.6e-2):
    return f32 if dtype == torch.float32 else bf16


def rel_err(got, ref):
    ref = ref.float().cpu()
    return float((got.float().cpu() - ref).abs().max()) / max(1e-6, float(ref.abs().max()))


@pytest.fixture(scope="module")
def ops():
    from mlx_lm_b200 import ops as o
    o.require_cuda()
    return o


def stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,D,V,P", [(1, 64, 512, 128), (37, 96, 1000, 256), (300, 1600, 50257, 1024), (5, 40, 33, 7)])
def test_embed_pos(ops, dtype, T, D, V, P):
    g = torch.Generator().manual_seed(T)
    wte = torch.randn(V, D, generator=g).to(dtype).cuda()
    wpe = torch.randn(P, D, generator=g).to(dtype).cuda()
    tok = torch.randint(0, V, (T,), generator=g, dtype=torch.int32).cuda()
    pos = torch.randint(0, P, (T,), generator=g, dtype=torch.int32).cuda()
    tok[0], pos[0] = V - 1, P - 1
    out = torch.empty(T, D, dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.embed_pos(tok, pos, wte, wpe, out, status, stream())
    assert rel_err(out, R.embed_pos(tok.cpu(), pos.cpu(), wte.cpu(), wpe.cpu())) <= tol(dtype, 1e-7, 4e-3)
    ops.embed_pos(tok, pos, wte, None, out, status, stream(), scale=3.0)
    assert rel_err(out, R.embed_pos(tok.cpu(), pos.cpu(), wte.cpu(), None, 3.0)) <= tol(dtype, 1e-7, 4e-3)
    assert int(status.item()) == 0
    # ids outside the tables are reported, not read
    tok[0] = V
    ops.embed_pos(tok, pos, wte, wpe, out, status, stream())
    assert int(status.item()) & ops.ST_TOKEN_RANGE
    assert float(out[0].float().abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("R_,D,eps", [(1, 64, 1e-5), (33, 96, 1e-6), (130, 1600, 1e-5), (7, 1024, 1e-5), (3, 5000, 1e-3),
                                      (2, 13000, 1e-5)])
def test_layernorm(ops, dtype, R_, D, eps):
    g = torch.Generator().manual_seed(D)
    x = (torch.randn(R_, D, generator=g) * 3 + 1.5).to(dtype).cuda()
    gain = (torch.randn(D, generator=g) * 0.1 + 1).cuda()
    bias = (torch.randn(D, generator=g) * 0.1).cuda()
    out = torch.empty_like(x)
    ops.layernorm(x, gain, bias, out, eps, stream())
    assert rel_err(out, R.layernorm(x.cpu(), gain.cpu(), bias.cpu(), eps)) <= tol(dtype, 2e-6, 4e-3)
    ops.layernorm(x, gain, None, out, eps, stream())
    assert rel_err(out, R.layernorm(x.cpu(), gain.cpu(), None, eps)) <= tol(dtype, 2e-6, 4e-3)
    rows = torch.tensor([R_ - 1, 0, R_ // 2], dtype=torch.int32).cuda()
    out3 = torch.empty(3, D, dtype=dtype, device="cuda")
    ops.layernorm(x, gain, bias, out3, eps, stream(), rows=rows)
    assert rel_err(out3, R.layernorm(x.cpu(), gain.cpu(), bias.cpu(), eps, rows.cpu())) <= tol(dtype, 2e-6, 4e-3)


@pytest.mark.parametrize("R_,D,shift", [(1, 64, 0.0), (33, 96, 1.5), (130, 1600, 40.0), (5, 4096, -3.0)])
def test_row_stats(ops, R_, D, shift):
    g = torch.Generator().manual_seed(D + 1)
    x = (torch.randn(R_, D, generator=g) * 3 + shift).to(torch.bfloat16).cuda()
    stats = torch.empty(R_, 2, device="cuda")
    ops.row_stats(x, stats, 1e-5, stream())
    xd = x.cpu().double()
    mean = xd.mean(dim=1)
    rstd = (xd.var(dim=1, unbiased=False) + 1e-5).rsqrt()
    assert float((stats[:, 0].cpu().double() - mean).abs().max()) <= 1e-5 * max(1.0, abs(shift))
    assert float((stats[:, 1].cpu().double() / rstd - 1).abs().max()) <= 1e-5


@pytest.mark.parametrize("M,N,K,shift", [(1, 200, 96, 0.0), (7, 1000, 320, 1.5), (16, 72, 1600, 40.0), (33, 200, 96, -2.0),
                                         (8, 8400, 1024, 1.5), (13, 9000, 2056, -3.0),      # very wide outputs
                                         (64, 1000, 320, 0.5), (200, 264, 96, 1.5), (130, 1000, 1600, 40.0), (2048, 3072, 1024, 2.0),
                                         (300, 520, 1608, -1.0)])
def test_linear_with_folded_norm(ops, M, N, K, shift):
    """LayerNorm folded into the weights (parts.linear.Linear.fold_norm): the few-rows kernel (statistics from its
    own fragments) and the tcgen05 kernel (statistics from row_stats) against LayerNorm followed by the linear
    layer, with gelu and a residual, for rows whose mean is far from zero too."""
    from types import SimpleNamespace
    from mlx_lm_b200.parts.linear import Linear
    from mlx_lm_b200.parts.norms import LayerNorm
    g = torch.Generator().manual_seed(M + N + K)
    x = (torch.randn(M, K, generator=g) * 3 + shift).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    gain = torch.randn(K, generator=g) * 0.3 + 1
    nbias = torch.randn(K, generator=g) * 0.2
    res = torch.randn(M, N, generator=g).to(torch.bfloat16)
    eps = 1e-5
    norm = LayerNorm("ln", K, eps)
    norm.bind({"ln.weight": gain.cuda(), "ln.bias": nbias.cuda()}, torch.bfloat16, "cuda")
    lin = Linear("fc", K, N)
    lin.bind({"fc.weight": w.cuda(), "fc.bias": b.cuda()}, torch.bfloat16, "cuda")
    assert lin.fold_norm(norm)
    ws = {}
    def get(tag, rows, cols, dtype):
        return ws.setdefault(tag, torch.zeros(rows, cols, dtype=dtype, device="cuda"))
    ctx = SimpleNamespace(stream=stream(), status=torch.zeros(1, dtype=torch.int32, device="cuda"),
                          ws=SimpleNamespace(get=get))
    normed = R.layernorm(x, gain, nbias, eps)
    for act, residual in ((None, None), ("gelu_new", None), (None, res)):
        out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        r_dev = None
        if residual is not None:
            out.copy_(residual)          # in place, as the blocks use it
            r_dev = out
        lin.forward(ctx, norm.deferred(ctx, x.cuda()), out, activation=act, residual=r_dev)
        ref = R.linear(normed, w, b, act, residual)
        assert rel_err(out, ref) <= 8e-3, (act, residual is not None)
    assert int(ctx.status.item()) == 0
    with pytest.raises(ops.KernelError):     # the folded layer no longer takes the normed tensor itself
        lin.forward(ctx, normed.to(torch.bfloat16).cuda(), torch.zeros(M, N, dtype=torch.bfloat16, device="cuda"))


def test_layernorm_constant_row_and_large_mean(ops):
    # a row with a large mean and tiny spread: a one-pass variance (E[x^2]-E[x]^2) would lose it
    x = (1000.0 + torch.arange(256).float().remainder(2) * 0.5).repeat(2, 1).cuda()
    gain, bias = torch.ones(256).cuda(), torch.zeros(256).cuda()
    out = torch.empty_like(x)
    ops.layernorm(x, gain, bias, out, 1e-5, stream())
    assert rel_err(out, R.layernorm(x.cpu().double(), gain.cpu().double(), bias.cpu().double(), 1e-5)) <= 1e-4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 192, 64), (7, 320, 96), (64, 1000, 96), (130, 50, 321), (257, 1600, 200),
                                   (3, 7, 5)])
def test_linear_generic(ops, dtype, M, N, K):
    g = torch.Generator().manual_seed(M * N + K)
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(dtype).cuda()
    b = torch.randn(N, generator=g).cuda()
    res = torch.randn(M, N, generator=g).to(dtype).cuda()
    out = torch.empty(M, N, dtype=dtype, device="cuda")
    t = tol(dtype, 2e-6, 6e-3)
    ops.linear_generic(x, w, b, out, stream())
    assert rel_err(out, R.linear(x.cpu(), w.cpu(), b.cpu())) <= t
    ops.linear_generic(x, w, None, out, stream(), epilogue=ops.EPI_GELU_NEW)
    assert rel_err(out, R.linear(x.cpu(), w.cpu(), None, "gelu_new")) <= t
    ops.linear_generic(x, w, b, out, stream(), epilogue=ops.EPI_GELU_NEW, residual=res)
    assert rel_err(out, R.linear(x.cpu(), w.cpu(), b.cpu(), "gelu_new", res.cpu())) <= t
    # in place on the residual, float32 output from bfloat16 inputs, strided input rows
    r2 = res.clone()
    ops.linear_generic(x, w, b, r2, stream(), residual=r2)
    assert rel_err(r2, R.linear(x.cpu(), w.cpu(), b.cpu(), None, res.cpu())) <= t
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.linear_generic(x, w, None, out32, stream())
    assert rel_err(out32, R.linear(x.cpu(), w.cpu())) <= 2e-6
    wide = torch.randn(M, K + 24, generator=g).to(dtype).cuda()
    ops.linear_generic(wide[:, 8:8 + K], w, b, out, stream())
    assert rel_err(out, R.linear(wide[:, 8:8 + K].cpu(), w.cpu(), b.cpu())) <= t


@pytest.mark.parametrize("M,N,K", [(1, 192, 64), (1, 1000, 96), (8, 320, 96), (16, 96, 320), (17, 3072, 1024),
                                   (33, 50257, 64), (64, 1600, 6400), (64, 50257, 1024), (5, 7, 8), (40, 1000, 1608),
                                   # up to 16 rows against a very wide output, inner sizes with a ragged last block
                                   (8, 50257, 1024), (1, 50257, 64), (16, 9000, 1608), (3, 8200, 4096)])
def test_linear_few_rows(ops, M, N, K):
    g = torch.Generator().manual_seed(M * N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=g).cuda()
    res = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.linear_few_rows(x, w, b, out, stream())
    assert rel_err(out, R.linear(x.cpu(), w.cpu(), b.cpu())) <= 6e-3
    ops.linear_few_rows(x, w, b, out, stream(), epilogue=ops.EPI_GELU_NEW, residual=res)
    assert rel_err(out, R.linear(x.cpu(), w.cpu(), b.cpu(), "gelu_new", res.cpu())) <= 6e-3
    r2 = res.clone()
    ops.linear_few_rows(x, w, None, r2, stream(), residual=r2)       # in place on the residual
    assert rel_err(r2, R.linear(x.cpu(), w.cpu(), None, None, res.cpu())) <= 6e-3
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.linear_few_rows(x, w, None, out32, stream())
    assert rel_err(out32, R.linear(x.cpu(), w.cpu())) <= 1e-5       # float32 accumulation of bfloat16 products
    # a row's result does not depend on the other rows of the call: bit for bit among calls of the same size
    # class (up to 16, 32, 64 rows), and up to float32 rounding across classes (their K partitions differ)
    one = torch.empty(1, N, dtype=torch.float32, device="cuda")
    ops.linear_few_rows(x[M - 1:M], w, None, one, stream())
    assert rel_err(one[0], out32[M - 1]) <= 2e-6
    lo = max(0, M - 1 - (M - 1) % 16)                # the rows of the last size class that contain row M-1
    few = torch.empty(M - lo, N, dtype=torch.float32, device="cuda")
    ops.linear_few_rows(x[lo:M], w, None, few, stream())
    if M - lo <= 16:
        assert torch.equal(one[0], few[-1])
    wide = torch.randn(M, K + 24, generator=g).to(torch.bfloat16).cuda()
    ops.linear_few_rows(wide[:, 8:8 + K], w, b, out, stream())
    assert rel_err(out, R.linear(wide[:, 8:8 + K].cpu(), w.cpu(), b.cpu())) <= 6e-3
    with pytest.raises(ops.KernelError):
        ops.linear_few_rows(torch.zeros(65, K, dtype=torch.bfloat16, device="cuda"), w, None,
                            torch.empty(65, N, dtype=torch.bfloat16, device="cuda"), stream())


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (65, 192, 64), (200, 320, 96), (130, 1000, 96), (257, 96, 320),
                                   (2048, 3072, 1024), (300, 1600, 6400), (1000, 50257, 64), (129, 7, 8),
                                   (512, 1024, 4096)])
@pytest.mark.parametrize("pairs", ["single CTAs", "pairs of CTAs"])
def test_linear_tensor_cores(ops, M, N, K, pairs, monkeypatch):
    """The tcgen05 kernel against the plain statement: tiles with ragged edges in M, N and K, many K stages,
    both output dtypes, every epilogue, in place on the residual; once with every tile on one CTA and once with
    every bfloat16 product of more than 128 rows on pairs of CTAs (the launcher otherwise picks by cost)."""
    monkeypatch.setenv("MLXB_TC_PAIR", "1" if pairs == "pairs of CTAs" else "0")
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=g).cuda()
    res = torch.randn(M, N, generator=g).to(torch.bfloat16).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = R.linear(x.cpu(), w.cpu(), b.cpu()) if M * N * K < 2e9 else (x.float() @ w.float().t() + b).cpu()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.linear_tensor_cores(x, w, b, out, status, stream())
    assert int(status.item()) == 0
    assert rel_err(out, ref) <= 6e-3
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.linear_tensor_cores(x, w, b, out32, status, stream())
    assert rel_err(out32, ref) <= 2e-5          # float32 accumulation of exact bfloat16 products
    ops.linear_tensor_cores(x, w, b, out, status, stream(), epilogue=ops.EPI_GELU_NEW, residual=res)
    assert rel_err(out, R.gelu_new(ref) + res.float().cpu()) <= 6e-3
    r2 = res.clone()
    ops.linear_tensor_cores(x, w, None, r2, status, stream(), residual=r2)
    assert rel_err(r2, ref - b.cpu() + res.float().cpu()) <= 6e-3
    # a row's result does not depend on the other rows of the call
    n_sub = min(70, M - 1)
    sub = torch.empty(n_sub, N, dtype=torch.float32, device="cuda")
    ops.linear_tensor_cores(x[M - n_sub:], w, b, sub, status, stream())
    assert torch.equal(sub, out32[M - n_sub:])
    assert int(status.item()) == 0
    # pairs and single CTAs add the same products in the same order
    ops.linear_tensor_cores(x, w, b, out, status, stream())
    monkeypatch.setenv("MLXB_TC_PAIR", "0")
    single = torch.empty_like(out)
    ops.linear_tensor_cores(x, w, b, single, status, stream())
    assert torch.equal(out, single)
    for width in ("128", "192", "256"):          # every tile width, whatever the launcher would pick
        monkeypatch.setenv("MLXB_TC_BN", width)
        monkeypatch.setenv("MLXB_TC_PAIR", "1" if pairs == "pairs of CTAs" else "0")
        forced = torch.empty_like(out)
        ops.linear_tensor_cores(x, w, b, forced, status, stream())
        assert torch.equal(forced, single), width
    assert int(status.item()) == 0


@pytest.mark.parametrize("M,N,K", [(3, 200, 96), (40, 1000, 320), (200, 320, 96)])
def test_every_activation_of_the_list_in_every_linear_kernel(ops, M, N, K):
    """The epilogue activations are one list (csrc/activations.cuh) that every linear kernel is compiled from
    and the Python side reads: each name of the list runs in the generic (both dtypes), the few-rows and the
    tcgen05 kernel and gives what the plain statement gives; a code outside the list is refused."""
    from mlx_lm_b200.parts.linear import ACTIVATIONS
    assert set(ops.ACTIVATION_CODES) == {"none", "gelu_new", "relu"} and ACTIVATIONS[None] == ops.EPI_NONE
    g = torch.Generator().manual_seed(M + N)
    x32 = torch.randn(M, K, generator=g).to(torch.bfloat16).float()
    w32 = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).float()
    b = torch.randn(N, generator=g).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for name, code in ops.ACTIVATION_CODES.items():
        ref = R.linear(x32, w32, b.cpu(), name)
        if name == "relu":
            assert float((ref == 0).float().mean()) > 0.2          # the clamp is exercised
        for dtype in DTYPES:
            x, w = x32.to(dtype).cuda(), w32.to(dtype).cuda()
            out = torch.empty(M, N, dtype=dtype, device="cuda")
            ops.linear_generic(x, w, b, out, stream(), epilogue=code)
            assert rel_err(out, ref) <= tol(dtype, 2e-6, 6e-3), (name, dtype)
        x, w = x32.to(torch.bfloat16).cuda(), w32.to(torch.bfloat16).cuda()
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        if M <= 64:
            ops.linear_few_rows(x, w, b, out, stream(), epilogue=code)
        else:
            ops.linear_tensor_cores(x, w, b, out, status, stream(), epilogue=code)
        assert rel_err(out, ref) <= 6e-3, name
    with pytest.raises(ops.KernelError):
        ops.linear_generic(x, w, b, out, stream(), epilogue=len(ops.ACTIVATION_CODES))
    assert int(status.item()) == 0


def test_gather_rows(ops):
    for dtype in DTYPES:
        x = torch.randn(37, 50).to(dtype).cuda()
        rows = torch.tensor([5, 0, 36, 5, 99, -1], dtype=torch.int32).cuda()     # the last two lie outside
        out = torch.full((6, 50), 7.0, dtype=dtype, device="cuda")
        ops.gather_rows(x, rows, out, stream())
        assert torch.equal(out[:4], x[[5, 0, 36, 5]]) and float(out[4:].abs().max()) == 0.0


def test_linear_tensor_cores_finds_one_hot_entries(ops):
    """One-hot rows and columns: the output must be exactly the picked weight entry, which pins down the
    operand layouts (swizzle, K steps inside a stage, tile edges) far better than random data."""
    M, N, K = 256, 256, 256
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    w = torch.arange(N * K, dtype=torch.float32).reshape(N, K).remainder(251).to(torch.bfloat16).cuda()
    for k_hot in (0, 7, 8, 15, 16, 63, 64, 65, 127, 128, 255):
        x = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda")
        x[:, k_hot] = 1.0
        x[5, k_hot] = 2.0
        out = torch.empty(M, N, dtype=torch.float32, device="cuda")
        ops.linear_tensor_cores(x, w, None, out, status, stream())
        want = w[:, k_hot].float().unsqueeze(0).repeat(M, 1)
        want[5] *= 2
        assert torch.equal(out, want), k_hot
    assert int(status.item()) == 0


@pytest.mark.parametrize("Hq,Hkv,Dh,page,K", [(4, 4, 16, 16, 64), (3, 3, 32, 16, 96), (6, 2, 48, 32, 288), (16, 16, 64, 16, 1024),
                                              (48, 48, 64, 16, 256)])      # 9216 outputs
def test_linear_qkv_to_cache(ops, Hq, Hkv, Dh, page, K):
    """The fused projection writes queries to its output and keys/values into the right page rows, as the
    plain projection followed by kv_write does; padding rows (request -1) write nothing."""
    lens, new = [0, 37, 130, 64, 15], [1, 1, 1, 1, 1]
    c = paged_case(torch.bfloat16, lens=lens, new=new, Hq=Hq, Hkv=Hkv, Dh=Dh, page=page, seed=K)
    g = torch.Generator().manual_seed(K)
    M, N = 6, (Hq + 2 * Hkv) * Dh                                  # 5 live rows and one padding row
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    positions = torch.cat([c["positions"], torch.tensor([0], dtype=torch.int32)])
    token_req = torch.cat([c["token_req"], torch.tensor([-1], dtype=torch.int32)])
    ref = R.linear(x, w, b).to(torch.bfloat16)
    qw, kw = Hq * Dh, Hkv * Dh
    rk, rv = R.kv_write(ref[:, qw:qw + kw], ref[:, qw + kw:], positions, token_req, c["bt"], c["k_pool"], c["v_pool"])
    kp, vp = c["k_pool"].cuda(), c["v_pool"].cuda()
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.linear_qkv_to_cache(x.cuda(), w.cuda(), b.cuda(), out, positions.cuda(), token_req.cuda(), c["bt"].cuda(), kp, vp,
                            qw, status, stream())
    assert int(status.item()) == 0
    assert rel_err(out[:, :qw], ref[:, :qw].float()) <= 8e-3
    assert rel_err(kp, rk.float()) <= 8e-3 and rel_err(vp, rv.float()) <= 8e-3
    changed = (kp.cpu() != c["k_pool"]).any(dim=-1)               # [page, head, row]: only the five written rows
    assert int(changed.sum()) <= 5 * Hkv


@pytest.mark.parametrize("Hq,Hkv,Dh,page,K", [(3, 3, 32, 16, 96), (6, 2, 48, 32, 288), (16, 16, 64, 16, 1024),
                                              (5, 1, 80, 16, 200)])
@pytest.mark.parametrize("pairs", ["single CTAs", "pairs of CTAs"])
def test_linear_qkv_to_cache_many_rows(ops, Hq, Hkv, Dh, page, K, pairs, monkeypatch):
    """More than 64 rows (portions of prompts): the tcgen05 kernel's epilogue does the same cache write.  Rows of
    several requests, starting in the middle of a page, with padding rows between them."""
    monkeypatch.setenv("MLXB_TC_PAIR", "1" if pairs == "pairs of CTAs" else "0")
    lens, new = [0, 37, 130, 5], [150, 75, 1, 91]
    c = paged_case(torch.bfloat16, lens=lens, new=new, Hq=Hq, Hkv=Hkv, Dh=Dh, page=page, seed=K + 1)
    g = torch.Generator().manual_seed(K)
    n_pad = 7
    M, N = c["T"] + n_pad, (Hq + 2 * Hkv) * Dh
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = torch.randn(N, generator=g)
    cut = 150                                                      # padding rows after the first request's rows
    positions = torch.cat([c["positions"][:cut], torch.zeros(n_pad, dtype=torch.int32), c["positions"][cut:]])
    token_req = torch.cat([c["token_req"][:cut], torch.full((n_pad,), -1, dtype=torch.int32), c["token_req"][cut:]])
    ref = R.linear(x, w, b).to(torch.bfloat16)
    qw, kw = Hq * Dh, Hkv * Dh
    rk, rv = R.kv_write(ref[:, qw:qw + kw], ref[:, qw + kw:], positions, token_req, c["bt"], c["k_pool"], c["v_pool"])
    kp, vp = c["k_pool"].cuda(), c["v_pool"].cuda()
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.linear_qkv_to_cache(x.cuda(), w.cuda(), b.cuda(), out, positions.cuda(), token_req.cuda(), c["bt"].cuda(), kp, vp,
                            qw, status, stream())
    assert int(status.item()) == 0
    assert rel_err(out[:, :qw], ref[:, :qw].float()) <= 8e-3
    assert rel_err(kp, rk.float()) <= 8e-3 and rel_err(vp, rv.float()) <= 8e-3
    changed = (kp.cpu() != c["k_pool"]).any(dim=-1)
    assert int(changed.sum()) <= c["T"] * Hkv
    assert float(out[:, qw:].abs().max()) == 0.0                   # key and value columns of the output stay untouched


def test_linear_few_rows_refuses_odd_inner_size(ops):
    x = torch.zeros(2, 12, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(5, 12, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError):
        ops.linear_few_rows(x, w, None, torch.empty(2, 5, dtype=torch.bfloat16, device="cuda"), stream())


def test_linear_row_does_not_depend_on_batch(ops):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(70, 96, generator=g).cuda()
    w = torch.randn(320, 96, generator=g).cuda()
    a = torch.empty(70, 320, device="cuda")
    b = torch.empty(1, 320, device="cuda")
    ops.linear_generic(x, w, None, a, stream())
    ops.linear_generic(x[69:70], w, None, b, stream())
    assert torch.equal(a[69:70], b)


def paged_case(dtype, lens, new, Hq, Hkv, Dh, page, seed, n_pages=None):
    """Requests with ``lens[i]`` cached tokens plus ``new[i]`` tokens in this step, pages handed out in a
    scrambled order.  Returns everything the attention wrappers need, on the GPU, plus host copies."""
    g = torch.Generator().manual_seed(seed)
    Rn = len(lens)
    total = [l + n for l, n in zip(lens, new)]
    need = sum((t + page - 1) // page for t in total)
    n_pages = n_pages or need + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max((t + page - 1) // page for t in total) + 1
    bt = torch.full((Rn, width), -1, dtype=torch.int32)
    for r, t in enumerate(total):
        for lp in range((t + page - 1) // page):
            bt[r, lp] = perm.pop()
    k_pool = torch.randn(n_pages, Hkv, page, Dh, generator=g).to(dtype)
    v_pool = torch.randn(n_pages, Hkv, page, Dh, generator=g).to(dtype)
    T = sum(new)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * Dh, generator=g).to(dtype)
    positions = torch.cat([torch.arange(l, l + n) for l, n in zip(lens, new)]).int()
    token_req = torch.cat([torch.full((n,), r) for r, n in enumerate(new)]).int()
    return dict(bt=bt, k_pool=k_pool, v_pool=v_pool, qkv=qkv, positions=positions, token_req=token_req, T=T,
                Hq=Hq, Hkv=Hkv, Dh=Dh, page=page)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,Dh,page,window", [(4, 4, 16, 16, 0), (3, 3, 32, 16, 0), (6, 2, 48, 32, 0),
                                                    (5, 1, 80, 64, 0), (2, 2, 128, 16, 40), (8, 4, 64, 16, 17)])
def test_kv_write_and_attention(ops, dtype, Hq, Hkv, Dh, page, window):
    c = paged_case(dtype, lens=[0, 37, 130, 64], new=[21, 1, 35, 2], Hq=Hq, Hkv=Hkv, Dh=Dh, page=page, seed=Dh + page)
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    qw, kw = Hq * Dh, Hkv * Dh
    q, k, v = dev["qkv"][:, :qw], dev["qkv"][:, qw:qw + kw], dev["qkv"][:, qw + kw:]
    ops.kv_write(k, v, dev["positions"], dev["token_req"], dev["bt"], dev["k_pool"], dev["v_pool"], status, stream())
    rk, rv = R.kv_write(c["qkv"][:, qw:qw + kw], c["qkv"][:, qw + kw:], c["positions"], c["token_req"], c["bt"],
                        c["k_pool"], c["v_pool"])
    assert torch.equal(dev["k_pool"].cpu(), rk) and torch.equal(dev["v_pool"].cpu(), rv)
    out = torch.empty(c["T"], qw, dtype=dtype, device="cuda")
    scale = Dh ** -0.5
    ops.attention_generic(q, dev["positions"], dev["token_req"], dev["bt"], dev["k_pool"], dev["v_pool"], out, Hq,
                          scale, window, status, stream())
    ref = R.attention(c["qkv"][:, :qw], c["positions"], c["token_req"], c["bt"], rk, rv, Hq, scale, window)
    assert int(status.item()) == 0
    assert rel_err(out, ref) <= tol(dtype, 3e-6, 8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,Dh,page,window,chunk", [(4, 4, 16, 16, 0, 128), (3, 3, 32, 16, 0, 128),
                                                          (6, 2, 48, 32, 0, 64), (5, 1, 80, 64, 0, 128),
                                                          (2, 2, 128, 16, 40, 32), (8, 4, 64, 16, 17, 128),
                                                          (16, 16, 64, 16, 0, 128), (2, 1, 256, 16, 0, 128)])
def test_attention_single_token_rows(ops, dtype, Hq, Hkv, Dh, page, window, chunk):
    """The split-key kernel on the single-token requests of a mixed step, selected by row list, and on a
    step of single tokens only (no row list), against the plain statement."""
    lens, new = [0, 37, 130, 64, 511, 255], [1, 1, 35, 1, 1, 1]
    c = paged_case(dtype, lens=lens, new=new, Hq=Hq, Hkv=Hkv, Dh=Dh, page=page, seed=Dh + page + 1)
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    qw = Hq * Dh
    q = dev["qkv"][:, :qw]
    scale = Dh ** -0.5
    ref = R.attention(c["qkv"][:, :qw], c["positions"], c["token_req"], c["bt"], c["k_pool"], c["v_pool"], Hq, scale,
                      window)
    first = np.cumsum([0] + new)
    single = [int(first[i]) for i, n in enumerate(new) if n == 1]
    rows = torch.tensor(single, dtype=torch.int32).cuda()
    max_len = 640
    scratch = torch.full((ops.attention_decode_scratch(len(single), Hq, Dh, max_len, chunk),), float("nan"),
                         device="cuda")
    counters = torch.zeros(8 * Hq, dtype=torch.int32, device="cuda")
    out = torch.zeros(c["T"], qw, dtype=dtype, device="cuda")
    ops.attention_decode(q, dev["positions"], dev["token_req"], dev["bt"], dev["k_pool"], dev["v_pool"], out, Hq,
                         scale, window, scratch, counters, max_len, status, stream(), rows=rows, chunk=chunk)
    assert int(status.item()) == 0
    assert rel_err(out[single], ref[single]) <= tol(dtype, 3e-6, 8e-3)
    untouched = [t for t in range(c["T"]) if t not in single]
    assert float(out[untouched].float().abs().max()) == 0.0
    # all rows single: tokens 0..n-1 without a row list
    c2 = paged_case(dtype, lens=[5, 300, 129, 0], new=[1, 1, 1, 1], Hq=Hq, Hkv=Hkv, Dh=Dh, page=page, seed=3)
    d2 = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c2.items()}
    out2 = torch.zeros(4, qw, dtype=dtype, device="cuda")
    ops.attention_decode(d2["qkv"][:, :qw], d2["positions"], d2["token_req"], d2["bt"], d2["k_pool"], d2["v_pool"],
                         out2, Hq, scale, window, scratch, counters, max_len, status, stream(), chunk=chunk)
    ref2 = R.attention(c2["qkv"][:, :qw], c2["positions"], c2["token_req"], c2["bt"], c2["k_pool"], c2["v_pool"], Hq,
                       scale, window)
    assert int(status.item()) == 0 and rel_err(out2, ref2) <= tol(dtype, 3e-6, 8e-3)
    assert int(counters.abs().max().item()) == 0        # the ticket counters are left at zero


@pytest.mark.parametrize("Hq,Hkv,Dh,page,window", [(4, 4, 16, 16, 0), (3, 3, 32, 16, 0), (6, 2, 48, 32, 0),
                                                    (5, 1, 80, 64, 0), (2, 2, 128, 16, 40), (8, 4, 64, 16, 17),
                                                    (16, 16, 64, 16, 0), (25, 25, 64, 8, 0)])
def test_attention_single_token_rows_on_tensor_cores(ops, Hq, Hkv, Dh, page, window):
    """Single-token rows as tiles of one query on the tensor-core kernel: the single-token requests of a mixed
    step (contexts that end inside a block, on a block's edge and in its first key), padding rows that must
    write nothing, against the plain statement."""
    lens, new = [0, 37, 130, 64, 511, 255, 63, 127, 128], [1, 1, 35, 1, 1, 1, 1, 1, 1]
    c = paged_case(torch.bfloat16, lens=lens, new=new, Hq=Hq, Hkv=Hkv, Dh=Dh, page=page, seed=Dh + page + 2)
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    qw = Hq * Dh
    q = dev["qkv"][:, :qw]
    scale = Dh ** -0.5
    ref = R.attention(c["qkv"][:, :qw], c["positions"], c["token_req"], c["bt"], c["k_pool"], c["v_pool"], Hq, scale,
                      window)
    first = np.cumsum([0] + new)
    single = [(int(first[i]), 1, i, lens[i]) for i, n in enumerate(new) if n == 1]
    padding = [(int(first[2]) + 3, 0, 0, 0), (int(first[2]) + 4, 0, 0, 0)]       # rows of the portion: untouched
    tiles = torch.tensor(single[:3] + padding[:1] + single[3:] + padding[1:], dtype=torch.int32).cuda()
    out = torch.zeros(c["T"], qw, dtype=torch.bfloat16, device="cuda")
    ops.attention_rows(q, tiles, tiles.shape[0], dev["bt"], dev["k_pool"], dev["v_pool"], out, Hq, scale, window,
                       status, stream())
    assert int(status.item()) == 0
    rows = [t[0] for t in single]
    assert rel_err(out[rows], ref[rows]) <= 8e-3
    untouched = [t for t in range(c["T"]) if t not in rows]
    assert float(out[untouched].float().abs().max()) == 0.0


def make_tiles(lens, new, tile=64):
    tiles, t0 = [], 0
    for r, (l, n) in enumerate(zip(lens, new)):
        if n > 1:
            tiles.extend((t0 + a, min(tile, n - a), r, l + a) for a in range(0, n, tile))
        t0 += n
    return torch.tensor(tiles, dtype=torch.int32).reshape(-1)


@pytest.mark.parametrize("tile", [64, 128])
@pytest.mark.parametrize("Hq,Hkv,Dh,page,window", [(4, 4, 16, 16, 0), (3, 3, 32, 16, 0), (6, 2, 48, 32, 0),
                                                    (5, 1, 80, 64, 0), (2, 2, 128, 16, 40), (8, 4, 64, 16, 17),
                                                    (16, 16, 64, 16, 0), (2, 1, 96, 16, 100), (1, 1, 112, 32, 0),
                                                    (4, 2, 64, 32, 0), (2, 2, 64, 128, 50), (3, 1, 64, 8, 0)])
def test_attention_portions(ops, Hq, Hkv, Dh, page, window, tile):
    """The tensor-core kernel on the portions of a mixed step (single-token requests are left to the other
    kernel): portions that start at position 0, that continue long contexts, that end inside a tile, of two tokens."""
    lens, new = [0, 37, 130, 64, 3, 200, 0], [21, 1, 135, 2, 64, 65, 300]
    c = paged_case(torch.bfloat16, lens=lens, new=new, Hq=Hq, Hkv=Hkv, Dh=Dh, page=page, seed=Dh + page + 2)
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    qw = Hq * Dh
    scale = Dh ** -0.5
    tiles = make_tiles(lens, new, tile).cuda()
    out = torch.zeros(c["T"], qw, dtype=torch.bfloat16, device="cuda")
    ops.attention_portions(dev["qkv"][:, :qw], tiles, tiles.numel() // 4, dev["bt"], dev["k_pool"], dev["v_pool"], out,
                           Hq, scale, window, status, stream(), tile_rows=tile)
    ref = R.attention(c["qkv"][:, :qw], c["positions"], c["token_req"], c["bt"], c["k_pool"], c["v_pool"], Hq, scale,
                      window)
    assert int(status.item()) == 0
    first = np.cumsum([0] + new)
    portion = [t for i, n in enumerate(new) if n > 1 for t in range(first[i], first[i + 1])]
    single = [int(first[i]) for i, n in enumerate(new) if n == 1]
    assert rel_err(out[portion], ref[portion]) <= 8e-3
    assert float(out[single].float().abs().max()) == 0.0


@pytest.mark.parametrize("tile", [64, 128])
def test_attention_portions_sees_each_key_once(ops, tile):
    """Values that encode their own position and sharp queries: query i picks key (i * 7) % (i + 1) exactly, at
    every offset inside tiles, blocks and pages; a key counted twice, skipped or taken from the wrong page shows.
    (Tiles of 64: the mma.sync kernel; tiles of 128 with heads of 64: the tcgen05 kernel.)"""
    Hq = Hkv = 1
    Dh, page, n = 64, 16, 333
    c = paged_case(torch.bfloat16, lens=[0], new=[n], Hq=Hq, Hkv=Hkv, Dh=Dh, page=page, seed=0)
    code = torch.randn(n, Dh, generator=torch.Generator().manual_seed(9)).sign()      # +-1 codes, one per position
    for j in range(n):
        pg = int(c["bt"][0, j // page])
        c["k_pool"][pg, 0, j % page] = (code[j] * 2.0).to(torch.bfloat16)
        c["v_pool"][pg, 0, j % page] = 0
        c["v_pool"][pg, 0, j % page, j % Dh] = 1.0 + j // Dh          # says which key it is
    target = [(i * 7) % (i + 1) for i in range(n)]
    c["qkv"][:, :Dh] = (code[target] * 2.0).to(torch.bfloat16)        # score 4*64*scale=32 on the target, ~0 elsewhere
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tiles = make_tiles([0], [n], tile).cuda()
    out = torch.zeros(n, Dh, dtype=torch.bfloat16, device="cuda")
    ops.attention_portions(dev["qkv"][:, :Dh], tiles, tiles.numel() // 4, dev["bt"], dev["k_pool"], dev["v_pool"], out,
                           Hq, Dh ** -0.5, 0, status, stream(), tile_rows=tile)
    got = out.float().cpu()
    for i in range(n):
        j = target[i]
        assert abs(float(got[i, j % Dh]) - (1.0 + j // Dh)) < 0.05, (i, j)
        assert float(got[i].abs().sum()) < (1.0 + j // Dh) + 0.1, (i, j)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(ops, dtype):
    """One key among hundreds matches the query strongly: the output must be that key's value row,
    wherever its page lies.  Random inputs would hide a key that is skipped or read from the wrong page."""
    Hq = Hkv = 2
    Dh, page = 64, 16
    for target in (0, 15, 16, 17, 255, 256, 300, 399):
        c = paged_case(dtype, lens=[399], new=[1], Hq=Hq, Hkv=Hkv, Dh=Dh, page=page, seed=target)
        qw = Hq * Dh
        c["qkv"][:, :qw] = 0
        c["qkv"][0, :Dh] = 6.0          # head 0 looks for ...
        pg = int(c["bt"][0, target // page])
        c["k_pool"][:, 0] *= 0.05
        c["k_pool"][pg, 0, target % page, :] = 6.0   # ... this key
        dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = torch.empty(1, qw, dtype=dtype, device="cuda")
        want = c["v_pool"][pg, 0, target % page, :].float()
        ops.attention_generic(dev["qkv"][:, :qw], dev["positions"], dev["token_req"], dev["bt"], dev["k_pool"],
                              dev["v_pool"], out, Hq, Dh ** -0.5, 0, status, stream())
        assert float((out[0, :Dh].float().cpu() - want).abs().max()) <= (1e-4 if dtype == torch.float32 else 2e-2), target
        out.zero_()
        scratch = torch.empty(ops.attention_decode_scratch(1, Hq, Dh, 512), device="cuda")
        counters = torch.zeros(Hq, dtype=torch.int32, device="cuda")
        ops.attention_decode(dev["qkv"][:, :qw], dev["positions"], dev["token_req"], dev["bt"], dev["k_pool"],
                             dev["v_pool"], out, Hq, Dh ** -0.5, 0, scratch, counters, 512, status, stream())
        assert float((out[0, :Dh].float().cpu() - want).abs().max()) <= (1e-4 if dtype == torch.float32 else 2e-2), target


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(ops, dtype):
    """With a window of W the key at p-W+1 counts and the key at p-W does not."""
    Hq = Hkv = 1
    Dh, page, W = 32, 16, 40
    for hot, expect_hit in ((200 - W + 1, True), (200 - W, False)):
        c = paged_case(dtype, lens=[200], new=[1], Hq=Hq, Hkv=Hkv, Dh=Dh, page=page, seed=5)
        c["qkv"][0, :Dh] = 8.0
        c["k_pool"] *= 0.02
        pg = int(c["bt"][0, hot // page])
        c["k_pool"][pg, 0, hot % page, :] = 8.0
        dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in c.items()}
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = torch.empty(1, Dh, dtype=dtype, device="cuda")
        ops.attention_generic(dev["qkv"][:, :Dh], dev["positions"], dev["token_req"], dev["bt"], dev["k_pool"],
                              dev["v_pool"], out, Hq, Dh ** -0.5, W, status, stream())
        want = c["v_pool"][pg, 0, hot % page, :].float()
        close = float((out[0].float().cpu() - want).abs().max()) <= 3e-2
        assert close == expect_hit
        out.zero_()
        scratch = torch.empty(ops.attention_decode_scratch(1, Hq, Dh, 256), device="cuda")
        counters = torch.zeros(Hq, dtype=torch.int32, device="cuda")
        ops.attention_decode(dev["qkv"][:, :Dh], dev["positions"], dev["token_req"], dev["bt"], dev["k_pool"],
                             dev["v_pool"], out, Hq, Dh ** -0.5, W, scratch, counters, 256, status, stream())
        close = float((out[0].float().cpu() - want).abs().max()) <= 3e-2
        assert close == expect_hit


def test_a_bounded_wait_that_runs_out(ops):
    """Failure detection without a fault: the tcgen05 linear kernel is built once more with a short limit on
    its barrier waits and a switch that leaves out one arrival (the MMA thread never tells the epilogue warps
    that the first accumulator is complete).  Their wait then runs out: the kernel must come back by itself with
    MLXB_ST_WAIT_TIMEOUT in the status word (no trap, no hang, its tensor memory freed), and the next launch of
    the same library, with the switch off, must be right.  The engine turns that status bit into a KernelError."""
    from ctypes import c_int
    from mlx_lm_b200.ops import build
    name = "gemm_tcgen05:MLXB_TEST_WAIT_TIMEOUT=1"
    lib = build.load(name)
    lib.mlxb_test_withhold_arrival.argtypes, lib.mlxb_test_withhold_arrival.restype = [c_int], c_int
    g = torch.Generator().manual_seed(3)
    M, N, K = 256, 128, 128
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).cuda()
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def launch():
        ops._call(name, "mlxb_linear_tcgen05", ops._TC_ARGS, 0, x.data_ptr(), w.data_ptr(), None, None, out.data_ptr(),
                  M, N, K, K, N, ops.EPI_NONE, status.data_ptr(), stream())
        torch.cuda.synchronize()

    assert lib.mlxb_test_withhold_arrival(1) == 0
    try:
        launch()
        assert int(status.item()) == ops.ST_WAIT_TIMEOUT
        assert float(out.float().abs().max()) == 0.0          # the epilogue never ran
    finally:
        assert lib.mlxb_test_withhold_arrival(0) == 0
    status.zero_()
    launch()
    assert int(status.item()) == 0
    assert rel_err(out, R.linear(x.cpu(), w.cpu())) <= 6e-3
    # and the ordinary library is untouched by all this
    ops.linear_tensor_cores(x, w, None, out, status, stream())
    assert int(status.item()) == 0 and rel_err(out, R.linear(x.cpu(), w.cpu())) <= 6e-3
