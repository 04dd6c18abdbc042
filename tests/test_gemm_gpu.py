"""tcgen05 GEMM against a plain PyTorch fp32 reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from ghassan_b200.ops import gemm as G, _lib
    return G, _lib


def _close(got, ref):
    """(worst error / allowance, ok) under the rule for the output's type (tests/tolerances.py); every product here
    is one fp32 accumulation over exactly representable operands, rounded at most once."""
    from tolerances import kind_of, worst
    ok, w, _ = worst(got, ref, kind_of(got.dtype))
    return w, ok


def _rand(*shape, dtype=torch.float16, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * 0.5).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (300, 200, 320), (128, 64, 64), (1024, 768, 512)])
@pytest.mark.parametrize("bn", [64, 128, 256])
def test_dense_kmajor(dtype, M, N, K, bn):
    G, L = _ops()
    a = _rand(M, K, dtype=dtype, seed=1)
    b = _rand(N, K, dtype=dtype, seed=2)
    out = G.gemm(a, b, block_n=bn)
    L.check_status(what="gemm")
    rel, ok = _close(out, a.float() @ b.float().t())
    assert ok, rel


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("bn", [64, 128])
def test_operand_majors(a_mn, b_mn, bn):
    G, L = _ops()
    M, N, K = 384, 320, 448
    A = _rand(M, K, seed=3)
    B = _rand(N, K, seed=4)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=bn, out_dtype=torch.float32)
    L.check_status(what="gemm")
    rel, ok = _close(out, A.float() @ B.float().t())
    assert ok, rel


def test_fp32_accumulate_and_residual():
    G, L = _ops()
    M, N, K = 256, 192, 128
    a, b = _rand(M, K, seed=5), _rand(N, K, seed=6)
    acc = torch.randn(M, N, device="cuda")
    ref = acc + a.float() @ b.float().t()
    G.gemm(a, b, out=acc, addend=acc)
    L.check_status(what="gemm")
    rel, ok = _close(acc, ref)
    assert ok, rel
    res = torch.randn(M, N, device="cuda")
    out = G.gemm(a, b, out_dtype=torch.float32, addend=res)
    rel, ok = _close(out, res + a.float() @ b.float().t())
    assert ok, rel


@pytest.mark.parametrize("M,d,E", [(200, 256, 192), (4136, 256, 512)])     # the second takes the 256-wide tiles
def test_swiglu_forward_backward_epilogues(M, d, E):
    G, L = _ops()
    x = _rand(M, d, seed=7)
    wg, wu = _rand(E, d, seed=8) * 0.2, _rand(E, d, seed=9) * 0.2
    wgu = G.interleave_gate_up(wg, wu).contiguous()
    gu = torch.zeros(M, 2 * E, dtype=torch.float16, device="cuda")
    act = G.gemm_swiglu(x, wgu, gu_out=gu)
    L.check_status(what="swiglu fwd")
    g_ref = x.float() @ wg.float().t()
    u_ref = x.float() @ wu.float().t()
    a_ref = torch.nn.functional.silu(g_ref) * u_ref
    g_got, u_got = G.deinterleave_cols(gu)
    assert _close(g_got, g_ref)[1] and _close(u_got, u_ref)[1]
    rel, ok = _close(act, a_ref)
    assert ok, rel
    # backward: d_act = dy @ W_down ; (dg, du) from saved (g, u)
    wd = _rand(d, E, seed=10) * 0.2
    dy = _rand(M, d, seed=11)
    dgu = G.gemm_swiglu_bwd(dy, wd, gu)
    L.check_status(what="swiglu bwd")
    dact = dy.float() @ wd.float()
    gf, uf = g_got.float(), u_got.float()
    sg = torch.sigmoid(gf)
    dg_ref = dact * uf * (sg * (1 + gf * (1 - sg)))
    du_ref = dact * gf * sg
    dg, du = G.deinterleave_cols(dgu)
    assert _close(dg, dg_ref)[1], _close(dg, dg_ref)[0]
    assert _close(du, du_ref)[1], _close(du, du_ref)[0]


def _make_groups(counts, pad_to=128):
    """Padded segment offsets, tile->expert map (per 128 rows) and live tile count for the given row counts."""
    offs = [0]
    tiles = []
    for e, c in enumerate(counts):
        pad = (c + pad_to - 1) // pad_to * pad_to
        tiles += [e] * (pad // 128)
        offs.append(offs[-1] + pad)
    return offs, tiles


def test_grouped_rows_and_grouped_reduce():
    G, L = _ops()
    counts = [130, 0, 5, 256, 77]
    ne, d, E = len(counts), 192, 128
    offs, tiles = _make_groups(counts)
    rows = offs[-1]
    x = torch.zeros(rows, d, dtype=torch.float16, device="cuda")
    for e, c in enumerate(counts):
        x[offs[e]:offs[e] + c] = _rand(c, d, seed=20 + e) if c else x[0:0]
    w = _rand(ne * E, d, seed=30) * 0.3            # K-major stacked [ne*E, d]
    tile_expert = torch.tensor(tiles + [0] * 4, dtype=torch.int32, device="cuda")
    ntiles = torch.tensor([len(tiles)], dtype=torch.int32, device="cuda")
    y = G.gemm_grouped_rows(x, w, tile_expert, ntiles, n=E, group_rows=E, out_dtype=torch.float32)
    L.check_status(what="grouped rows")
    for e, c in enumerate(counts):
        if c:
            ref = x[offs[e]:offs[e] + c].float() @ w[e * E:(e + 1) * E].float().t()
            rel, ok = _close(y[offs[e]:offs[e] + c], ref)
            assert ok, (e, rel)
    # N-major stacked B: dgrad dx = y16 @ W_e  with W_e stored [E, d] = [K, N]
    y16 = torch.zeros(rows, E, dtype=torch.float16, device="cuda")
    for e, c in enumerate(counts):
        if c:
            y16[offs[e]:offs[e] + c] = _rand(c, E, seed=40 + e)
    dx = G.gemm_grouped_rows(y16, w, tile_expert, ntiles, n=d, b_mn=True, group_rows=E, out_dtype=torch.float32)
    L.check_status(what="grouped rows N-major")
    for e, c in enumerate(counts):
        if c:
            ref = y16[offs[e]:offs[e] + c].float() @ w[e * E:(e + 1) * E].float()
            rel, ok = _close(dx[offs[e]:offs[e] + c], ref)
            assert ok, (e, rel)
    # wgrad: dW_e = y16_e^T @ x_e, accumulated into fp32
    seg = torch.tensor(offs, dtype=torch.int32, device="cuda")
    dw = torch.ones(ne, E, d, dtype=torch.float32, device="cuda")
    G.gemm_grouped_reduce(y16, x, seg, ne, dw, accumulate=True)
    L.check_status(what="grouped reduce")
    for e, c in enumerate(counts):
        ref = 1.0 + y16[offs[e]:offs[e] + c].float().t() @ x[offs[e]:offs[e] + c].float()
        rel, ok = _close(dw[e], ref)
        assert ok, (e, rel)
    # the same product with 256-wide tiles (N = 512)
    x2 = torch.zeros(rows, 512, dtype=torch.float16, device="cuda")
    for e, c in enumerate(counts):
        if c:
            x2[offs[e]:offs[e] + c] = _rand(c, 512, seed=50 + e)
    for bn in (128, 256):
        dw2 = torch.zeros(ne, E, 512, dtype=torch.float32, device="cuda")
        G.gemm_grouped_reduce(y16, x2, seg, ne, dw2, accumulate=False, block_n=bn)
        L.check_status(what="grouped reduce bn %d" % bn)
        for e, c in enumerate(counts):
            ref = y16[offs[e]:offs[e] + c].float().t() @ x2[offs[e]:offs[e] + c].float()
            rel, ok = _close(dw2[e], ref)
            assert ok, (bn, e, rel)


@pytest.mark.parametrize("M,N,K,splits", [(512, 768, 32000, 16), (100, 128, 600, 4)])
def test_split_k(M, N, K, splits):
    G, L = _ops()
    a = _rand(M, K, seed=60) * 0.2
    w = _rand(K, N, seed=61) * 0.2          # B stored [K, N]
    plan = G.SplitK(M, N, K, splits, torch.float16, "cuda")
    out = torch.empty(M, N, dtype=torch.float16, device="cuda")
    plan.run(a, w, out, b_mn=True)
    L.check_status(what="split-k")
    rel, ok = _close(out, a.float() @ w.float())
    assert ok, rel
    out2 = torch.empty_like(out)
    plan.run(a, w, out2, b_mn=True)
    assert torch.equal(out, out2)


def test_large_gemm_matches():
    G, L = _ops()
    a, b = _rand(4096, 1024, seed=50), _rand(2048, 1024, seed=51)
    out = G.gemm(a, b, out_dtype=torch.float32)
    L.check_status(what="gemm")
    rel, ok = _close(out, a.float() @ b.float().t())
    assert ok, rel


@pytest.mark.parametrize("M,N,K", [(768, 768, 8192), (1280, 768, 8192), (256, 128, 4096), (2560, 768, 2048), (128, 128, 1000)])
def test_weight_gradient_split_over_tokens(M, N, K):
    """gemm_wgrad splits the token dimension when the output has few tiles; either way grad += a^T b."""
    G, L = _ops()
    a = _rand(K, M, seed=70) * 0.2
    b = _rand(K, N, seed=71) * 0.2
    grad = torch.full((M, N), 0.5, dtype=torch.float32, device="cuda")
    G.gemm_wgrad(a, b, grad)
    G.gemm_wgrad(a, b, grad)                  # accumulates, and the cached plan is reused
    L.check_status(what="wgrad")
    ref = 0.5 + 2.0 * (a.float().t() @ b.float())
    rel, ok = _close(grad, ref)
    assert ok, rel


# ----------------------------------------------------------------------------- two-CTA 256 x 256 kernel (pair=True)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("out_dtype", [None, torch.float32])
@pytest.mark.parametrize("M,N,K", [(512, 512, 256), (300, 520, 320), (1024, 768, 512), (256, 256, 64), (2304, 1280, 768)])
def test_pair_dense(dtype, out_dtype, M, N, K):
    G, L = _ops()
    a = _rand(M, K, dtype=dtype, seed=1)
    b = _rand(N, K, dtype=dtype, seed=2)
    out = G.gemm(a, b, out_dtype=out_dtype, pair=True)
    L.check_status(what="pair gemm")
    rel, ok = _close(out, a.float() @ b.float().t())
    assert ok, rel
    out2 = G.gemm(a, b, out_dtype=out_dtype, pair=True)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
def test_pair_operand_majors(a_mn, b_mn):
    G, L = _ops()
    M, N, K = 640, 520, 448
    A = _rand(M, K, seed=3)
    B = _rand(N, K, seed=4)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, pair=True)
    L.check_status(what="pair gemm majors")
    rel, ok = _close(out, A.float() @ B.float().t())
    assert ok, rel


def test_pair_fp32_accumulate_and_residual():
    G, L = _ops()
    M, N, K = 520, 392, 128
    a, b = _rand(M, K, seed=5), _rand(N, K, seed=6)
    acc = torch.randn(M, N, device="cuda")
    ref = acc + a.float() @ b.float().t()
    G.gemm(a, b, out=acc, addend=acc, pair=True)            # TMA reduce-add into the matrix
    L.check_status(what="pair gemm accumulate")
    rel, ok = _close(acc, ref)
    assert ok, rel
    res = torch.randn(M, N, device="cuda")
    out = G.gemm(a, b, out_dtype=torch.float32, addend=res, pair=True)
    L.check_status(what="pair gemm residual")
    rel, ok = _close(out, res + a.float() @ b.float().t())
    assert ok, rel


@pytest.mark.parametrize("M,d,E,keep", [(4136, 256, 512, True), (520, 320, 192, True), (1024, 256, 256, False)])
def test_pair_swiglu_forward_backward_epilogues(M, d, E, keep):
    G, L = _ops()
    x = _rand(M, d, seed=7)
    wg, wu = _rand(E, d, seed=8) * 0.2, _rand(E, d, seed=9) * 0.2
    wgu = G.interleave_gate_up(wg, wu).contiguous()
    gu = torch.zeros(M, 2 * E, dtype=torch.float16, device="cuda") if keep else None
    act = G.gemm_swiglu(x, wgu, gu_out=gu, pair=True)
    L.check_status(what="pair swiglu fwd")
    g_ref = x.float() @ wg.float().t()
    u_ref = x.float() @ wu.float().t()
    rel, ok = _close(act, torch.nn.functional.silu(g_ref) * u_ref)
    assert ok, rel
    rel, ok = _close(act, G.gemm_swiglu(x, wgu, pair=False).float())    # the one-CTA epilogue agrees
    assert ok, rel
    if not keep:
        return
    g_got, u_got = G.deinterleave_cols(gu)
    assert _close(g_got, g_ref)[1] and _close(u_got, u_ref)[1]
    wd = _rand(d, E, seed=10) * 0.2
    dy = _rand(M, d, seed=11)
    dgu = G.gemm_swiglu_bwd(dy, wd, gu, pair=True)
    L.check_status(what="pair swiglu bwd")
    dact = dy.float() @ wd.float()
    gf, uf = g_got.float(), u_got.float()
    sg = torch.sigmoid(gf)
    dg, du = G.deinterleave_cols(dgu)
    assert _close(dg, dact * uf * (sg * (1 + gf * (1 - sg))))[1], _close(dg, dact * uf * (sg * (1 + gf * (1 - sg))))[0]
    assert _close(du, dact * gf * sg)[1], _close(du, dact * gf * sg)[0]
    dgu2 = G.gemm_swiglu_bwd(dy, wd, gu, pair=True)
    assert torch.equal(dgu, dgu2)


def test_pair_grouped_rows_and_grouped_reduce():
    G, L = _ops()
    counts = [130, 0, 5, 300, 77, 512]
    ne, d, E = len(counts), 320, 256
    offs, tiles = _make_groups(counts, pad_to=256)
    rows = offs[-1]
    x = torch.zeros(rows + 256, d, dtype=torch.float16, device="cuda")[:rows]
    for e, c in enumerate(counts):
        if c:
            x[offs[e]:offs[e] + c] = _rand(c, d, seed=20 + e)
    w = _rand(ne * E, d, seed=30) * 0.3
    tile_expert = torch.tensor(tiles + [0] * 4, dtype=torch.int32, device="cuda")
    ntiles = torch.tensor([len(tiles)], dtype=torch.int32, device="cuda")
    for od in (torch.float32, torch.float16):
        y = G.gemm_grouped_rows(x, w, tile_expert, ntiles, n=E, group_rows=E, out_dtype=od, pair=True)
        L.check_status(what="pair grouped rows")
        for e, c in enumerate(counts):
            if c:
                ref = x[offs[e]:offs[e] + c].float() @ w[e * E:(e + 1) * E].float().t()
                rel, ok = _close(y[offs[e]:offs[e] + c], ref)
                assert ok, (e, rel)
    y16 = torch.zeros(rows, E, dtype=torch.float16, device="cuda")
    for e, c in enumerate(counts):
        if c:
            y16[offs[e]:offs[e] + c] = _rand(c, E, seed=40 + e)
    dx = G.gemm_grouped_rows(y16, w, tile_expert, ntiles, n=d, b_mn=True, group_rows=E, out_dtype=torch.float32, pair=True)
    L.check_status(what="pair grouped rows N-major")
    for e, c in enumerate(counts):
        if c:
            ref = y16[offs[e]:offs[e] + c].float() @ w[e * E:(e + 1) * E].float()
            rel, ok = _close(dx[offs[e]:offs[e] + c], ref)
            assert ok, (e, rel)
    seg = torch.tensor(offs, dtype=torch.int32, device="cuda")
    dw = torch.ones(ne, E, d, dtype=torch.float32, device="cuda")
    G.gemm_grouped_reduce(y16, x, seg, ne, dw, accumulate=True, pair=True)
    L.check_status(what="pair grouped reduce")
    for e, c in enumerate(counts):
        ref = 1.0 + y16[offs[e]:offs[e] + c].float().t() @ x[offs[e]:offs[e] + c].float()
        rel, ok = _close(dw[e], ref)
        assert ok, (e, rel)
    dw2 = torch.full((ne, E, d), 7.0, dtype=torch.float32, device="cuda")
    G.gemm_grouped_reduce(y16, x, seg, ne, dw2, accumulate=False, pair=True)     # an empty group must store zeros
    L.check_status(what="pair grouped reduce store")
    assert torch.allclose(dw2, dw - 1.0, rtol=1e-5, atol=1e-5)
