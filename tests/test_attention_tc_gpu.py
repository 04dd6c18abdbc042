"""tcgen05 flash attention (forward, dQ, dK/dV) against the fp32 PyTorch attention of the oracle model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def near(got, ref, chain=True):
    """(ok, worst error / allowance, rule) under the suite's comparison rule (tests/tolerances.py): attention
    results pass through 16-bit probabilities, so 16-bit outputs take the "chain" rule of their type; fp32 outputs
    (the log-sum-exp) take the fp32 rule."""
    from tolerances import kind_of, worst
    k = kind_of(got.dtype, chain)
    ok, w, _ = worst(got, ref, k, floor=1.0)     # operands are N(0, 1): a gradient that cancels to zero keeps that scale
    return ok, w, k


def rnd(*shape, seed=0, dtype=torch.float16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, device="cuda", generator=g).to(dtype)


CASES = [
    # B, T, H, KV, hd, window, segments
    (1, 128, 2, 2, 64, 0, False),
    (2, 512, 12, 4, 64, 0, True),
    (1, 300, 4, 2, 64, 0, False),
    (2, 200, 4, 1, 64, 37, True),
    (1, 260, 2, 1, 128, 0, True),
    (1, 1, 2, 2, 64, 0, False),
    (1, 1024, 4, 4, 64, 0, False),
    (8, 512, 12, 4, 64, 0, True),       # more work items than resident CTAs: every CTA walks several
    (8, 384, 16, 4, 64, 100, True),
    (16, 512, 8, 4, 64, 0, True),       # more key-tile items than SMs too (the dK/dV kernel walks several per CTA)
]


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,T,H,KV,hd,window,use_seg", CASES)
def test_tc_attention_matches_oracle(dt, B, T, H, KV, hd, window, use_seg):
    from ghassan_b200.models import reference as R
    from ghassan_b200.ops import _lib, kernels as K
    n = B * T
    scale = hd ** -0.5
    qk = rnd(n, (H + KV) * hd, seed=1, dtype=dt)          # q and k share a buffer, v lives in a wider one
    qkv = rnd(n, (H + 2 * KV) * hd, seed=2, dtype=dt)
    q, k, v = qk[:, :H * hd], qk[:, H * hd:], qkv[:, (H + KV) * hd:]
    seg = None
    if use_seg:
        seg = (torch.arange(T, device="cuda") // 97).repeat(B).to(torch.int32)
    lo = torch.empty(n, dtype=torch.int32, device="cuda")
    o = torch.empty(n, H * hd, dtype=dt, device="cuda")
    lse = torch.empty(n, H, device="cuda")
    K.attn_tc_fwd(q, k, v, o, lse, seg, lo, B, T, H, KV, hd, window, scale)
    _lib.check_status(what="attn_tc_fwd")
    qf, kf, vf = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    ref = R.attention(qf.view(n, H, hd), kf.view(n, KV, hd), vf.view(n, KV, hd), B, T, scale, window, seg)
    ok, err, atol = near(o, ref.detach())
    assert ok, ("o", err, atol)
    g = rnd(n, H * hd, seed=3, dtype=dt)
    (ref * g.float()).sum().backward()
    dqk = torch.zeros_like(qk)
    dqkv = torch.zeros_like(qkv)
    delta = torch.empty(n, H, device="cuda")
    K.attn_tc_bwd(q, k, v, o, lse, seg, lo, g, delta, dqk[:, :H * hd], dqk[:, H * hd:], dqkv[:, (H + KV) * hd:], B, T, H,
                  KV, hd, window, scale)
    _lib.check_status(what="attn_tc_bwd")
    for got, want, name in ((dqk[:, :H * hd], qf.grad, "dq"), (dqk[:, H * hd:], kf.grad, "dk"),
                            (dqkv[:, (H + KV) * hd:], vf.grad, "dv")):
        ok, err, atol = near(got, want)
        assert ok, (name, err, atol)


def test_tc_attention_agrees_with_cuda_core_kernels():
    from ghassan_b200.ops import kernels as K
    B, T, H, KV, hd = 2, 384, 6, 2, 64
    n = B * T
    q, k, v = rnd(n, H * hd, seed=4), rnd(n, KV * hd, seed=5), rnd(n, KV * hd, seed=6)
    o1, o2 = torch.empty_like(q), torch.empty_like(q)
    l1, l2 = torch.empty(n, H, device="cuda"), torch.empty(n, H, device="cuda")
    lo = torch.empty(n, dtype=torch.int32, device="cuda")
    K.attn_fwd(q, k, v, o1, l1, None, B, T, H, KV, hd, 0, 0.125)
    K.attn_tc_fwd(q, k, v, o2, l2, None, lo, B, T, H, KV, hd, 0, 0.125)
    assert near(o2, o1)[0]
    assert near(l2, l1)[0]
    # bitwise reproducible from run to run
    o3 = torch.empty_like(q)
    K.attn_tc_fwd(q, k, v, o3, l2, None, lo, B, T, H, KV, hd, 0, 0.125)
    assert torch.equal(o2, o3)


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("use_seg", [False, True])
def test_tc_attention_forward_rescales_when_the_row_maximum_jumps(dt, use_seg):
    """The forward kernel keeps the output in tensor memory and rescales it only when a row's maximum has grown by
    more than 2^8 since it was last taken.  Keys that grow in magnitude along the sequence force that path in every
    later tile (unit-variance inputs never do); a second case makes only some rows of a warp jump."""
    from ghassan_b200.models import reference as R
    from ghassan_b200.ops import _lib, kernels as K
    B, T, H, KV, hd = 2, 512, 4, 2, 64
    n = B * T
    scale = hd ** -0.5
    for variant in range(2):
        q, k, v = rnd(n, H * hd, seed=11, dtype=dt), rnd(n, KV * hd, seed=12, dtype=dt), rnd(n, KV * hd, seed=13, dtype=dt)
        pos = torch.arange(T, device="cuda").repeat(B)
        if variant == 0:
            k = (k.float() * (1.0 + 5.0 * (pos // 128).float())[:, None]).to(dt)          # every tile louder than the last
        else:
            q = (q.float() * torch.where(pos % 7 == 0, 8.0, 1.0)[:, None]).to(dt)         # a few rows of each warp jump
            k = (k.float() * torch.where(pos >= 256, 4.0, 1.0)[:, None]).to(dt)
        seg = (pos // 200).to(torch.int32) if use_seg else None
        lo = torch.empty(n, dtype=torch.int32, device="cuda")
        o = torch.empty(n, H * hd, dtype=dt, device="cuda")
        lse = torch.empty(n, H, device="cuda")
        K.attn_tc_fwd(q, k, v, o, lse, seg, lo, B, T, H, KV, hd, 0, scale)
        _lib.check_status(what="attn_tc_fwd")
        ref = R.attention(q.float().view(n, H, hd), k.float().view(n, KV, hd), v.float().view(n, KV, hd), B, T, scale, 0, seg)
        ok, err, rule = near(o, ref)
        assert ok, ("o", variant, err, rule)
        sc = torch.einsum("bihd,bjhd->bhij", q.float().view(B, T, H, hd),
                          k.float().view(B, T, KV, hd).repeat_interleave(H // KV, dim=2)) * scale
        vis = pos[:T][None, :] <= pos[:T][:, None]
        if use_seg:
            vis = vis & ((pos[:T] // 200)[None, :] == (pos[:T] // 200)[:, None])
        want = torch.logsumexp(sc.masked_fill(~vis, float("-inf")), dim=-1).permute(0, 2, 1).reshape(n, H)
        ok, err, rule = near(lse, want, chain=False)
        assert ok, ("lse", variant, err, rule)


def test_tc_attention_leading_negative_segment_ids():
    """Rows with a negative segment id at the head of a sequence see every earlier key (the oracle's rule); the documents
    after them see only themselves."""
    from ghassan_b200.models import reference as R
    from ghassan_b200.ops import _lib, kernels as K
    B, T, H, KV, hd = 2, 300, 4, 2, 64
    n = B * T
    dt = torch.float16
    scale = hd ** -0.5
    q, k, v = rnd(n, H * hd, seed=21, dtype=dt), rnd(n, KV * hd, seed=22, dtype=dt), rnd(n, KV * hd, seed=23, dtype=dt)
    one = torch.cat([torch.full((40,), -1, device="cuda"), torch.arange(T - 40, device="cuda") // 97])
    seg = one.repeat(B).to(torch.int32)
    lo = torch.empty(n, dtype=torch.int32, device="cuda")
    o = torch.empty(n, H * hd, dtype=dt, device="cuda")
    lse = torch.empty(n, H, device="cuda")
    K.attn_tc_fwd(q, k, v, o, lse, seg, lo, B, T, H, KV, hd, 0, scale)
    _lib.check_status(what="attn_tc_fwd")
    assert int(lo.view(B, T)[:, :40].max()) == 0 and int(lo.view(B, T)[0, 40]) == 40
    assert bool((lo.view(B, T)[:, 1:] >= lo.view(B, T)[:, :-1]).all())       # non-decreasing along a sequence
    ref = R.attention(q.float().view(n, H, hd), k.float().view(n, KV, hd), v.float().view(n, KV, hd), B, T, scale, 0, seg)
    ok, err, rule = near(o, ref)
    assert ok, ("o", err, rule)
