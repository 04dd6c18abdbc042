"""The allocation-free gradient-norm entry point (``gb_grad_norm_noalloc``), called through its exported C symbol,
against the two-kernel path that takes caller-provided scratch (``gb_sqnorm_partial`` + ``gb_finish_norm``).

Collected last on purpose (the file name sorts after the others): it has to pass both alone and after every other
test has used the device.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

PKG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "jdm-ghassan_v1_pro-_b200")
MAX_ELEMS = 4096 * 65536


def _lib():
    lib = ctypes.CDLL(os.path.join(PKG, "_gb200_cuda.so"))
    lib.gb_grad_norm_noalloc.restype = ctypes.c_int
    lib.gb_grad_norm_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float, ctypes.c_float,
                                         ctypes.c_void_p, ctypes.c_void_p]
    lib.gb_sqnorm_blocks.restype = ctypes.c_int
    lib.gb_sqnorm_blocks.argtypes = [ctypes.c_longlong]
    lib.gb_sqnorm_partial.restype = ctypes.c_int
    lib.gb_sqnorm_partial.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    lib.gb_finish_norm.restype = ctypes.c_int
    lib.gb_finish_norm.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_float, ctypes.c_float,
                                   ctypes.c_void_p, ctypes.c_void_p]
    lib.gb_noalloc_last_cuda_error.restype = ctypes.c_int
    return lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _existing(lib, g, grad_scale, clip):
    nb = lib.gb_sqnorm_blocks(g.numel())
    part = torch.empty(max(nb, 1), dtype=torch.float64, device="cuda")
    out = torch.empty(2, dtype=torch.float32, device="cuda")
    assert lib.gb_sqnorm_partial(g.data_ptr(), g.numel(), part.data_ptr(), _stream()) == 0
    assert lib.gb_finish_norm(part.data_ptr(), nb, None, grad_scale, clip, out.data_ptr(), _stream()) == 0
    torch.cuda.synchronize()
    return out.cpu()


@pytest.mark.parametrize("n", [1, 1000, 65536, 65537, 3_000_001, 40_000_000])
def test_matches_the_existing_entry_point_twice_in_a_row(n):
    lib = _lib()
    g = torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(n % 97)) * 3.0
    out = torch.full((2,), -1.0, device="cuda")
    for call, (gs, clip) in enumerate([(1.0 / 512, 1.0), (0.25, 0.0)]):     # second call right after the first
        rc = lib.gb_grad_norm_noalloc(g.data_ptr(), n, gs, clip, out.data_ptr(), _stream())
        assert rc == 0, (rc, lib.gb_noalloc_last_cuda_error())
        torch.cuda.synchronize()
        got = out.cpu()
        want = _existing(lib, g, gs, clip)
        assert torch.equal(got, want), (call, got, want)
        ref = float(g.double().pow(2).sum().sqrt()) * gs                      # and both agree with plain PyTorch
        assert float(got[1]) == pytest.approx(ref, rel=1e-5)
        g.mul_(1.5)


def test_nonfinite_input_gives_zero_scale():
    lib = _lib()
    g = torch.randn(100_000, device="cuda")
    g[77_777] = float("inf")
    out = torch.empty(2, device="cuda")
    assert lib.gb_grad_norm_noalloc(g.data_ptr(), g.numel(), 1.0, 1.0, out.data_ptr(), _stream()) == 0
    torch.cuda.synchronize()
    assert float(out[0]) == 0.0 and not torch.isfinite(out[1])
    g[77_777] = 0.0                                                          # the scratch carries nothing over
    assert lib.gb_grad_norm_noalloc(g.data_ptr(), g.numel(), 1.0, 0.0, out.data_ptr(), _stream()) == 0
    torch.cuda.synchronize()
    assert float(out[0]) == 1.0 and float(out[1]) == pytest.approx(float(g.norm()), rel=1e-5)


def test_rejects_what_the_static_scratch_cannot_hold():
    lib = _lib()
    g = torch.zeros(1024, device="cuda")
    out = torch.full((2,), 7.0, device="cuda")
    # size checks come before any access to g, so a count beyond the limit can be probed with a small buffer
    assert lib.gb_grad_norm_noalloc(g.data_ptr(), MAX_ELEMS + 1, 1.0, 1.0, out.data_ptr(), _stream()) == -3
    assert lib.gb_grad_norm_noalloc(g.data_ptr() + 4, 100, 1.0, 1.0, out.data_ptr(), _stream()) == -2
    assert lib.gb_grad_norm_noalloc(g.data_ptr(), -5, 1.0, 1.0, out.data_ptr(), _stream()) == -1
    assert lib.gb_grad_norm_noalloc(g.data_ptr(), 10, 1.0, 1.0, None, _stream()) == -1
    torch.cuda.synchronize()
    assert out.tolist() == [7.0, 7.0]                                        # rejected calls wrote nothing
    assert lib.gb_grad_norm_noalloc(g.data_ptr(), 0, 0.5, 1.0, out.data_ptr(), _stream()) == 0
    torch.cuda.synchronize()
    assert out.tolist() == [0.5, 0.0]
