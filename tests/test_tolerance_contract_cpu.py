"""The comparison rule that the CUDA parity tests rely on is itself tested: it must accept a legal re-association of
the same arithmetic and reject three realistic mistakes (the reference does the same for its oracle,
tests/test_attention_cuda_parity.cpp:67-158).  The subject is d(loss)/dq of causal attention, built by hand."""
import numpy as np
import pytest


def near_vec(got, ref, rtol=1e-3, atol_rel=1e-5):
    """|got - ref| <= atol + rtol*|ref| element-wise, with atol = atol_rel * max|ref| (the reference's near_vec)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    atol = atol_rel * float(np.abs(ref).max())
    return bool(np.all(np.abs(got - ref) <= atol + rtol * np.abs(ref)))


def _attention_dq(q, k, v, do, scale, *, dtype=np.float64, reverse=False, drop_jacobian=False, drop_scale=False, shift_k=0):
    T, hd = q.shape
    q, k, v, do = (a.astype(dtype) for a in (q, k, v, do))
    dq = np.zeros((T, hd), dtype=dtype)
    for t in range(T):
        js = list(range(t + 1))
        s = np.array([float(q[t] @ k[j]) * scale for j in js], dtype=dtype)
        p = np.exp(s - s.max())
        p = p / p.sum()
        dp = np.array([float(do[t] @ v[j]) for j in js], dtype=dtype)
        rowdot = 0.0 if drop_jacobian else float((p * dp).sum())
        ds = p * (dp - rowdot) * (1.0 if drop_scale else scale)
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


def test_rule_accepts_legal_reassociation(case):
    q, k, v, do, scale = case
    ref = _attention_dq(q, k, v, do, scale)
    assert near_vec(_attention_dq(q, k, v, do, scale, reverse=True), ref)                      # other summation order
    assert near_vec(_attention_dq(q, k, v, do, scale, dtype=np.float32), ref)                  # fp32 arithmetic
    assert near_vec(_attention_dq(q, k, v, do, scale, dtype=np.float32, reverse=True), ref)


def test_rule_rejects_real_mistakes(case):
    q, k, v, do, scale = case
    ref = _attention_dq(q, k, v, do, scale)
    assert not near_vec(_attention_dq(q, k, v, do, scale, drop_jacobian=True), ref)            # soft-max Jacobian forgotten
    assert not near_vec(_attention_dq(q, k, v, do, scale, drop_scale=True), ref)               # scale forgotten
    assert not near_vec(_attention_dq(q, k, v, do, scale, shift_k=1), ref)                     # key index off by one
    assert not near_vec(ref * (1 + 5e-3), ref)                                                  # half a percent is not noise
    assert near_vec(ref * (1 + 5e-4), ref)


def test_rule_is_scale_invariant_and_handles_zeros():
    ref = np.array([0.0, 1e-9, 1.0, -2.0])
    assert near_vec(ref + np.array([1e-5, 1e-5, 0, 0]), ref)          # absolute slack is tied to max|ref| = 2
    assert not near_vec(ref + np.array([1e-3, 0, 0, 0]), ref)
    big = ref * 1e6
    assert near_vec(big + np.array([10.0, 10.0, 0, 0]), big) and not near_vec(big + np.array([1e3, 0, 0, 0]), big)
