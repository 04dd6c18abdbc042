"""The comparison rules that the CUDA parity tests use (tests/tolerances.py) are themselves tested: each must accept a
legal re-association of the same arithmetic in the precision it is used at, and reject three realistic mistakes (the
reference does the same for its oracle, tests/test_attention_cuda_parity.cpp:67-158).  The subject is d(loss)/dq of
causal attention, built by hand."""
import numpy as np
import pytest

from tolerances import RULES, near


def _round_to(x, kind):
    """Round an fp64 array the way a kernel's output type would."""
    if kind.startswith("bf16"):
        f = np.asarray(x, dtype=np.float32).copy()
        u = f.view(np.uint32)
        u += 0x7FFF + ((u >> 16) & 1)          # round to nearest even on the upper 16 bits
        u &= 0xFFFF0000
        return f.astype(np.float64)
    if kind.startswith("f16"):
        return np.asarray(x, dtype=np.float16).astype(np.float64)
    return np.asarray(x, dtype=np.float32).astype(np.float64)


def _attention_dq(q, k, v, do, scale, *, dtype=np.float64, reverse=False, drop_jacobian=False, drop_scale=False,
                  shift_k=0, p_kind=None):
    T, hd = q.shape
    q, k, v, do = (a.astype(dtype) for a in (q, k, v, do))
    dq = np.zeros((T, hd), dtype=dtype)
    for t in range(T):
        js = list(range(t + 1))
        s = np.array([float(q[t] @ k[j]) * scale for j in js], dtype=dtype)
        p = np.exp(s - s.max())
        p = p / p.sum()
        if p_kind:                                  # a kernel that keeps the probabilities in a 16-bit type
            p = _round_to(p, p_kind).astype(dtype)
        dp = np.array([float(do[t] @ v[j]) for j in js], dtype=dtype)
        rowdot = 0.0 if drop_jacobian else float((p * dp).sum())
        ds = p * (dp - rowdot) * (1.0 if drop_scale else scale)
        if p_kind:
            ds = _round_to(ds, p_kind).astype(dtype)
        order = reversed(range(len(js))) if reverse else range(len(js))
        acc = np.zeros(hd, dtype=dtype)
        for i in order:
            acc = acc + ds[i] * k[min(T - 1, js[i] + shift_k)]
        dq[t] = acc
    return dq


@pytest.fixture(scope="module")
def case():
    rng = np.random.default_rng(5)
    T, hd = 24, 16
    q, k, v, do = (rng.standard_normal((T, hd)) for _ in range(4))
    return q, k, v, do, hd ** -0.5


@pytest.mark.parametrize("kind", sorted(RULES))
def test_every_rule_accepts_legal_arithmetic_in_its_own_precision(case, kind):
    q, k, v, do, scale = case
    ref = _attention_dq(q, k, v, do, scale)
    chain = kind if kind.endswith("_chain") else None
    for reverse in (False, True):
        got = _attention_dq(q, k, v, do, scale, dtype=np.float32, reverse=reverse, p_kind=chain)
        assert near(_round_to(got, kind), ref, kind), (kind, reverse)


@pytest.mark.parametrize("kind", sorted(RULES))
def test_every_rule_rejects_real_mistakes_in_its_own_precision(case, kind):
    q, k, v, do, scale = case
    ref = _attention_dq(q, k, v, do, scale)
    chain = kind if kind.endswith("_chain") else None
    for mutation in (dict(drop_jacobian=True), dict(drop_scale=True), dict(shift_k=1)):
        got = _attention_dq(q, k, v, do, scale, dtype=np.float32, p_kind=chain, **mutation)
        assert not near(_round_to(got, kind), ref, kind), (kind, mutation)


def test_single_rounding_rules_reject_half_a_percent(case):
    q, k, v, do, scale = case
    ref = _attention_dq(q, k, v, do, scale)
    for kind in ("f32", "f16", "f16_chain"):
        assert not near(ref * (1 + 5e-3), ref, kind), kind          # half a percent is not noise
    assert near(ref * (1 + 5e-4), ref, "f32")
    assert not near(ref * (1 + 2e-2), ref, "bf16") and not near(ref * (1 + 4e-2), ref, "bf16_chain")


def test_rule_is_scale_invariant_and_handles_zeros():
    ref = np.array([0.0, 1e-9, 1.0, -2.0])
    assert near(ref + np.array([1e-5, 1e-5, 0, 0]), ref)          # absolute slack is tied to max|ref| = 2
    assert not near(ref + np.array([1e-3, 0, 0, 0]), ref)
    big = ref * 1e6
    assert near(big + np.array([10.0, 10.0, 0, 0]), big) and not near(big + np.array([1e3, 0, 0, 0]), big)
    assert not near(np.array([np.nan, 1.0]), np.array([0.0, 1.0]))
