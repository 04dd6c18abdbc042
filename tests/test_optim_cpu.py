"""Optimizers against their textbook formulas, the learning-rate schedules, the loss scaler, the balancing-bias
update and the router jitter seed."""
import math

import numpy as np
import pytest
import torch


def _params(shapes, seed=0):
    from ghassan_b200.training.optim import OptParam
    g = torch.Generator().manual_seed(seed)
    out = []
    for i, s in enumerate(shapes):
        w = torch.randn(*s, generator=g) * 0.1
        w.grad = torch.randn(*s, generator=g) * 0.01
        out.append(OptParam("p%d" % i, w, decay=(len(s) == 2)))
    return out


def test_adamw_matches_the_formula_and_torch():
    from ghassan_b200.training.optim import AdamW
    ps = _params([(8, 6), (6,)])
    ref_w = [p.w.clone().requires_grad_(True) for p in ps]
    opt = AdamW(ps, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, grad_clip=0.0)
    topt = torch.optim.AdamW([{"params": [ref_w[0]], "weight_decay": 0.1}, {"params": [ref_w[1]], "weight_decay": 0.0}],
                             lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for step in range(4):
        for p, r in zip(ps, ref_w):
            g = torch.randn_like(p.w) * 0.01
            p.w.grad = g.clone()
            r.grad = g.clone()
        gn = opt.step(1e-2, 1.0)
        topt.step()
        assert math.isfinite(gn)
    for p, r in zip(ps, ref_w):
        assert torch.allclose(p.w, r.detach(), rtol=2e-5, atol=1e-7)


def test_gradient_scale_and_clipping():
    from ghassan_b200.training.optim import AdamW, global_grad_norm
    ps = _params([(16, 16)])
    raw = float(ps[0].grad.double().pow(2).sum().sqrt())
    assert global_grad_norm(ps, 0.5) == pytest.approx(raw * 0.5, rel=1e-6)
    a, b = _params([(16, 16)]), _params([(16, 16)])
    b[0].w.grad = b[0].grad * 100.0                   # a 100x larger gradient, clipped back to the same norm
    oa = AdamW(a, 1e-2, grad_clip=1e-3)
    ob = AdamW(b, 1e-2, grad_clip=1e-3)
    ga, gb = oa.step(1e-2), ob.step(1e-2)
    assert gb == pytest.approx(100.0 * ga, rel=1e-5)   # the reported norm is the unclipped one
    assert torch.allclose(a[0].w, b[0].w, atol=1e-6)


def test_nonfinite_gradient_skips_the_step():
    from ghassan_b200.training.optim import AdamW, Lion
    for cls in (AdamW, Lion):
        ps = _params([(4, 4), (4,)])
        before = [p.w.clone() for p in ps]
        ps[1].grad[2] = float("inf")
        opt = cls(ps, 1e-2)
        gn = opt.step(1e-2)
        assert not math.isfinite(gn)
        for p, w0 in zip(ps, before):
            assert torch.equal(p.w, w0)
        assert opt.t == 0


def test_lion_sign_update():
    from ghassan_b200.training.optim import Lion
    ps = _params([(5, 5)])
    w0, g = ps[0].w.clone(), ps[0].grad.clone()
    Lion(ps, 1e-3, beta1=0.9, beta2=0.99, weight_decay=0.0, grad_clip=0.0).step(1e-3)
    assert torch.allclose(ps[0].w, w0 - 1e-3 * torch.sign(g), atol=1e-8)


def test_newton_schulz_orthogonalises():
    from ghassan_b200.training.optim import newton_schulz
    G = torch.randn(32, 16, generator=torch.Generator().manual_seed(1))
    O = newton_schulz(G, 10)
    s = torch.linalg.svdvals(O)
    assert float(s.max()) <= 1.01            # the cubic iteration is a contraction towards singular values of 1
    s5 = torch.linalg.svdvals(newton_schulz(G, 5))
    assert float((1 - s).abs().mean()) < float((1 - s5).abs().mean())     # more steps: closer to orthogonal
    assert torch.equal(newton_schulz(torch.zeros(4, 4), 5), torch.zeros(4, 4))


def test_muon_routes_parameters_by_shape():
    from ghassan_b200.training.optim import Muon
    ps = _params([(8, 8), (8,)])
    m = Muon(ps, min_ns_dim=0)
    assert m.uses_ns(ps[0]) and not m.uses_ns(ps[1])
    m2 = Muon(_params([(8, 4)]), min_ns_dim=8)
    assert not m2.uses_ns(m2.params[0])       # narrower than the threshold: Lion-style vector rule instead
    w0 = ps[0].w.clone()
    m.step(1e-2)
    assert not torch.equal(ps[0].w, w0)


@pytest.mark.parametrize("kind", ["cosine", "wsd"])
def test_schedules(kind):
    from ghassan_b200.training.optim import LrScheduler
    s = LrScheduler(1e-3, total=100, warmup=10, min_ratio=0.1, kind=kind, decay_frac=0.2)
    assert s.lr_at(0) == pytest.approx(1e-4)
    assert s.lr_at(9) == pytest.approx(1e-3)
    assert s.lr_at(100) == pytest.approx(1e-4, rel=1e-4)
    lrs = [s.lr_at(i) for i in range(10, 101)]
    assert all(a >= b - 1e-12 for a, b in zip(lrs, lrs[1:]))
    if kind == "wsd":
        assert s.lr_at(81) == pytest.approx(1e-3)        # stable until the last 20 % of post-warm-up steps
        assert s.lr_at(83) < 1e-3
    else:
        assert s.lr_at(55) == pytest.approx(1e-3 * (0.1 + 0.9 * 0.5), rel=1e-4)   # half-way down the cosine


def test_loss_scaler_rules():
    from ghassan_b200.training.optim import LossScaler
    s = LossScaler(65536.0, window=2, max_scale=0.0)
    assert s.scale == 16384.0 and s.for_step() == 16384.0          # hard cap
    s.update(float("nan"))
    assert s.scale == 8192.0 and s.overflows == 1
    s.update(1.0)
    s.update(1.0)
    assert s.scale == 16384.0 and s.clean_steps == 0
    s.update(1.0)
    s.update(1.0)
    assert s.scale == 16384.0                                      # never above the cap
    low = LossScaler(4.0, window=1, max_scale=8.0)
    low.update(1.0)
    low.update(1.0)
    assert low.scale == 8.0
    for _ in range(10):
        low.update(float("inf"))
    assert low.scale == 1.0                                        # floor
    off = LossScaler(1024.0, window=1, active=False)
    assert off.for_step() == 1.0 and off.scale == 1024.0           # recorded but not applied
    off.update(float("nan"))
    assert off.scale == 1024.0


def test_balancing_bias_update():
    from ghassan_b200.training.engine import moe_bias_update
    bias = torch.zeros(2, 4)
    counts = torch.tensor([[10.0, 30.0, 40.0, 20.0], [0.0, 0.0, 0.0, 0.0]])
    moe_bias_update(bias, counts)
    want = -0.001 * (torch.tensor([0.1, 0.3, 0.4, 0.2]) - 0.25)
    assert torch.allclose(bias[0], want, atol=1e-9)
    assert torch.equal(bias[1], torch.zeros(4))                    # a layer without routed slots is left alone
    big = torch.full((1, 4), 0.4999)
    for _ in range(10):
        moe_bias_update(big, torch.tensor([[0.0, 100.0, 100.0, 100.0]]))
    assert float(big.max()) <= 0.5


def test_jitter_seed_depends_on_step_and_rank():
    from ghassan_b200.training.engine import jitter_seed_for
    seen = {jitter_seed_for(42, s, r) for s in range(20) for r in range(4)}
    assert len(seen) == 80 and all(0 <= v < 2 ** 64 for v in seen)
    assert jitter_seed_for(42, 0, 0) == 42
