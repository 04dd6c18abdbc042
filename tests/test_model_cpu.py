"""The fp32 oracle model: initialisation order, causality, packing isolation, sliding window, routing rules,
jitter determinism, loss bookkeeping."""
import numpy as np
import pytest
import torch


def _cfg(**over):
    from ghassan_b200.models.config import ModelConfig
    base = dict(vocab_size=320, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=128,
                max_seq_len=32, use_moe=True, num_experts=4, moe_top_k=2, moe_expert_dim=64, moe_shared=True,
                use_qk_norm=True)
    base.update(over)
    c = ModelConfig(**base)
    c.validate()
    return c


def _model(cfg, seed=3):
    from ghassan_b200.models.reference import TorchModel
    m = TorchModel(cfg, "cpu")
    m.init_weights(seed)
    return m


def _ids(n, seed=0, vocab=320):
    return torch.randint(16, vocab, (n,), generator=torch.Generator().manual_seed(seed), dtype=torch.int32)


def test_init_is_seeded_and_bounded():
    from ghassan_b200.models.config import init_parameters
    cfg = _cfg()
    a, b, c = init_parameters(cfg, 5), init_parameters(cfg, 5), init_parameters(cfg, 6)
    assert set(a) == {s.name for s in cfg.param_specs()}
    for n in a:
        assert np.array_equal(a[n], b[n])
    assert not np.array_equal(a["tok_embeddings"], c["tok_embeddings"])
    for n, v in a.items():
        if n.endswith("norm"):
            assert np.all(v == 1.0), n
        else:
            assert np.abs(v).max() <= 2.0 * cfg.init_std + 1e-7, n     # truncated at two standard deviations
    # the random draws cover every matrix exactly once; norm gains are set to one without consuming the generator
    drawn = cfg.init_order()
    assert len(set(drawn)) == len(drawn)
    assert sorted(drawn) == sorted(s.name for s in cfg.param_specs() if not s.name.endswith("norm"))


def test_causality():
    cfg = _cfg()
    m = _model(cfg)
    ids = _ids(32)
    with torch.no_grad():
        a = m.logits(ids, 1, 32)
        ids2 = ids.clone()
        ids2[20] = (ids2[20] + 7) % 300 + 16
        b = m.logits(ids2, 1, 32)
    assert torch.allclose(a[:20], b[:20], atol=1e-6)
    assert not torch.allclose(a[20:], b[20:], atol=1e-6)


def test_packed_segments_do_not_see_each_other():
    cfg = _cfg(use_moe=False)
    m = _model(cfg)
    ids = _ids(32, seed=1)
    seg = torch.cat([torch.zeros(12), torch.ones(20)]).int()
    with torch.no_grad():
        packed = m.logits(ids, 1, 32, segment_ids=seg)
        ids2 = ids.clone()
        ids2[:12] = _ids(12, seed=9)
        packed2 = m.logits(ids2, 1, 32, segment_ids=seg)
    # tokens of the second document do not change when the first document does
    assert torch.allclose(packed[12:], packed2[12:], atol=1e-6)
    assert not torch.allclose(packed[:12], packed2[:12], atol=1e-6)


def test_sliding_window_limits_the_receptive_field():
    cfg = _cfg(use_moe=False, sliding_window=4, num_layers=1)
    m = _model(cfg)
    ids = _ids(32, seed=2)
    with torch.no_grad():
        a = m.logits(ids, 1, 32)
        ids2 = ids.clone()
        ids2[3] = (ids2[3] + 5) % 300 + 16
        b = m.logits(ids2, 1, 32)
    assert torch.allclose(a[7:], b[7:], atol=1e-6)        # one layer, window 4: position 3 reaches 3..6 only
    assert not torch.allclose(a[3:7], b[3:7], atol=1e-6)


def test_router_rules():
    from ghassan_b200.models.reference import route
    cfg = _cfg()
    x = torch.zeros(3, 64)                                # all logits equal: every expert ties
    rw = torch.randn(4, 64)
    probs, idx, w = route(x, rw, None, cfg, None)
    assert idx.tolist() == [[0, 1]] * 3                   # ties go to the lowest index
    assert torch.allclose(w.sum(-1), torch.ones(3))
    assert torch.allclose(probs.sum(-1), torch.ones(3))
    bias = torch.tensor([0.0, 0.0, 0.3, 0.0])
    _, idx_b, w_b = route(x, rw, bias, cfg, None)
    assert idx_b[:, 0].tolist() == [2, 2, 2]              # the bias steers selection ...
    assert torch.allclose(w_b, torch.full((3, 2), 0.5))   # ... but not the combine weights


def test_jitter_is_a_pure_function_of_the_seed_and_is_off_in_eval():
    from ghassan_b200.models.reference import jitter_u, route
    cfg = _cfg(moe_jitter=0.1)
    t, e = np.meshgrid(np.arange(50), np.arange(4), indexing="ij")
    u1, u2, u3 = jitter_u(t, e, 123), jitter_u(t, e, 123), jitter_u(t, e, 124)
    assert np.array_equal(u1, u2) and not np.array_equal(u1, u3)
    assert np.abs(u1).max() <= 0.5 + 1e-6 and abs(u1.mean()) < 0.1
    x = torch.randn(50, 64, generator=torch.Generator().manual_seed(0))
    rw = torch.randn(4, 64, generator=torch.Generator().manual_seed(1))
    p_eval, _, _ = route(x, rw, None, cfg, None)
    p_plain, _, _ = route(x, rw, None, _cfg(), 999)
    assert torch.equal(p_eval, p_plain)
    p_j, _, _ = route(x, rw, None, cfg, 999)
    assert not torch.equal(p_j, p_eval)


def test_loss_accounting_and_masked_targets():
    cfg = _cfg(z_loss_scale=1e-4, moe_aux_scale=0.01)
    m = _model(cfg)
    ids = _ids(64, seed=4)
    tg = torch.roll(ids, -1).clone()
    tg[10:30] = -100
    res = m.forward(ids, tg, 2, 32, None, jitter_seed=None, return_logits=True)
    assert res.ntok == 44
    lg = res.logits.float()
    keep = tg >= 0
    logz = torch.logsumexp(lg[keep], -1)
    ce = (logz - lg[keep].gather(1, tg[keep].long()[:, None])[:, 0] + 1e-4 * logz ** 2).sum()
    assert float(res.loss_sum) == pytest.approx(float(ce), rel=1e-5)
    assert res.slot_counts.shape == (2, 4) and float(res.slot_counts.sum()) == 2 * 2 * 64
    assert len(res.aux_raw) == 2 and all(float(a) >= 1.0 - 1e-4 for a in res.aux_raw)   # ne*sum(m*f) >= 1
    assert res.reported_loss(cfg) > float(res.loss_sum) / res.ntok
    all_masked = m.forward(ids, torch.full_like(tg, -100), 2, 32, None)
    assert all_masked.ntok == 0


def test_gradient_matches_finite_differences():
    cfg = _cfg(hidden_size=32, num_heads=2, num_kv_heads=1, intermediate_size=64, moe_expert_dim=32, vocab_size=64,
               max_seq_len=8)
    m = _model(cfg)
    for p in m.params.values():
        p.data = p.data.double()
    m.enable_grad(True)
    ids = _ids(8, seed=5, vocab=64)
    tg = torch.roll(ids, -1)
    res = m.forward(ids, tg, 1, 8, None)
    res.loss_sum.backward()
    for name in ("layers.0.wq", "layers.1.moe_down", "final_norm", "layers.0.moe_router"):
        p = m.params[name]
        flat = p.data.view(-1)
        k = int(torch.argmax(p.grad.view(-1).abs()))
        h = 1e-5
        old = float(flat[k])
        with torch.no_grad():
            flat[k] = old + h
            up = float(m.forward(ids, tg, 1, 8, None).loss_sum)
            flat[k] = old - h
            dn = float(m.forward(ids, tg, 1, 8, None).loss_sum)
            flat[k] = old
        assert (up - dn) / (2 * h) == pytest.approx(float(p.grad.view(-1)[k]), rel=2e-4), name
