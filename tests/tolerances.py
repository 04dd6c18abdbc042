"""The one comparison rule of the test-suite, per kind of output.

Every CUDA-versus-oracle comparison goes through :func:`near`:  ``|got - ref| <= atol + rtol * |ref|`` element-wise
with ``atol`` tied to ``max|ref|`` (the form of the reference's ``near_vec``, tests/test_moe_cuda_parity.cpp:21-50,
tests/test_attention_cuda_parity.cpp:67-158).  The constants depend on what the kernel rounds:

``f32``      fp32 result of fp32 accumulation over exactly representable operands (GEMM with fp32 output, weight
             gradients, fp32 reductions).  Only the summation order differs from the oracle: the reference's own
             bound, rtol 1e-3 and atol 1e-5 * max|ref|.
``f16`` / ``bf16``
             the same fp32 result rounded once to a 16-bit type: half an ulp is ``u`` = 2^-11 (fp16) or 2^-8 (bf16)
             relative, so rtol = 2u on top of the fp32 slack.
``f16_chain`` / ``bf16_chain``
             results that pass through 16-bit intermediates before the final sum (attention probabilities, saved
             gate/up activations, normalised activations feeding a GEMM): the intermediate rounding is relative to the
             terms of a sum, not to its result, so the absolute slack grows to 4u * max|ref| and rtol to 4u.

``tests/test_tolerance_contract_cpu.py`` checks that each of these rules accepts a legal re-association and rejects a
dropped soft-max Jacobian, a dropped scale and a key index that is off by one, in the precision it is used at.
"""
from __future__ import annotations

import numpy as np

U16 = {"f16": 2.0 ** -11, "bf16": 2.0 ** -8}

RULES = {
    "f32": dict(rtol=1e-3, atol_rel=1e-5),
    "f16": dict(rtol=2 * U16["f16"], atol_rel=1e-5 + 2.0 ** -24),
    "bf16": dict(rtol=2 * U16["bf16"], atol_rel=1e-5),
    "f16_chain": dict(rtol=4 * U16["f16"], atol_rel=4 * U16["f16"]),
    "bf16_chain": dict(rtol=4 * U16["bf16"], atol_rel=4 * U16["bf16"]),
}


def _np(x):
    if hasattr(x, "detach"):
        x = x.detach().double().cpu().numpy()
    return np.asarray(x, dtype=np.float64)


def kind_of(dtype, chain=False) -> str:
    """Rule name for a torch dtype."""
    name = str(dtype).replace("torch.", "")
    base = {"float32": "f32", "float64": "f32", "float16": "f16", "bfloat16": "bf16"}[name]
    return base + "_chain" if (chain and base != "f32") else base


def worst(got, ref, kind="f32", floor=0.0):
    """(ok, worst ratio of error to allowance, index of the worst element).  ``floor``: magnitude of the terms that
    the result is a sum of, for results that cancel to (almost) zero: the absolute slack is tied to
    ``max(max|ref|, floor)``, since rounding noise scales with the terms, not with a sum that happens to vanish."""
    r = RULES[kind]
    got, ref = _np(got), _np(ref)
    if got.shape != ref.shape:
        raise AssertionError(f"shape {got.shape} vs {ref.shape}")
    if not np.all(np.isfinite(got)):
        return False, float("inf"), int(np.argmin(np.isfinite(got).ravel()))
    scale = float(np.abs(ref).max()) if ref.size else 0.0
    allow = r["atol_rel"] * max(scale, float(floor)) + r["rtol"] * np.abs(ref) + 1e-30
    ratio = np.abs(got - ref) / allow
    i = int(np.argmax(ratio)) if ratio.size else 0
    w = float(ratio.ravel()[i]) if ratio.size else 0.0
    return w <= 1.0, w, i


def near(got, ref, kind="f32", floor=0.0) -> bool:
    return worst(got, ref, kind, floor)[0]


def assert_near(got, ref, kind="f32", what="", floor=0.0):
    ok, w, i = worst(got, ref, kind, floor)
    assert ok, f"{what}: error is {w:.2f}x the '{kind}' allowance at flat index {i}"
