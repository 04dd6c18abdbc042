"""ctypes access to the sm_100a kernel library and the device status word.

The library is built in-tree by ``ghassan_b200.build``.  On a machine with a GPU a missing or
stale library is a hard error (no silent PyTorch fallback on the CUDA path); on CPU-only
machines :func:`lib` raises only when it is actually called.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(_HERE, "_gb200_cuda.so")
_lock = threading.Lock()
_lib = None

c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_vp = ctypes.c_void_p
c_float = ctypes.c_float


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("A", c_vp), ("B", c_vp),
        ("M", c_int), ("N", c_int), ("K", c_int),
        ("a_rows", c_ll), ("a_cols", c_ll), ("lda", c_ll),
        ("b_rows", c_ll), ("b_cols", c_ll), ("ldb", c_ll),
        ("a_mn_major", c_int), ("b_mn_major", c_int), ("is_bf16", c_int), ("out_dtype", c_int),
        ("epilogue", c_int), ("block_n", c_int), ("mode", c_int),
        ("tile_expert", c_vp), ("num_m_tiles", c_vp), ("seg_offsets", c_vp),
        ("groups", c_int), ("b_group_rows", c_int),
        ("out", c_vp), ("ldo", c_int), ("out_group_stride", c_ll),
        ("addend", c_vp), ("ld_add", c_int),
        ("aux_out", c_vp), ("aux_in", c_vp), ("ld_aux", c_int),
        ("status", c_vp),
        ("tile_out", c_vp),
        ("pair", c_int),
    ]


def available() -> bool:
    return os.path.exists(_SO)


def lib():
    """Load (once) and return the kernel library."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(_SO):
                    raise RuntimeError(
                        f"{_SO} is missing: run `python -m ghassan_b200.build` (the CUDA path has no fallback)")
                _lib = ctypes.CDLL(_SO)
    return _lib


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    if t is None:
        return None
    return ctypes.c_void_p(t.data_ptr())


_status = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word that kernels write a non-zero code into when a bounded wait expires."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    key = (dev.type, dev.index)
    t = _status.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=dev)
        _status[key] = t
    return t


STATUS_NAMES = {
    0: "ok",
    101: "timeout waiting for TMA bytes (full barrier)",
    102: "timeout waiting for a free shared-memory stage (empty barrier)",
    103: "timeout waiting for the accumulator (tmem full barrier)",
    104: "timeout waiting for an accumulator buffer (tmem empty barrier)",
    105: "timeout waiting for an epilogue warp's own TMA load",
    201: "timeout waiting for a peer rank's flag",
    301: "bad argument detected on device",
    401: "decode step: a grid-wide barrier wait ran out",
    402: "decode step: a bulk copy of weight rows never signalled its barrier",
    302: "expert parallelism: more rows were routed to this rank's experts than its buffers hold (raise b200.ep_capacity)",
}


def check_status(device=None, what="kernel") -> None:
    """Synchronising check of the status word; raises RuntimeError on a recorded failure."""
    w = status_word(device)
    code = int(w[0].item())
    if code != 0:
        w.zero_()
        raise RuntimeError(f"{what}: device status {code} ({STATUS_NAMES.get(code, 'unknown')})")


def check_rc(rc: int, what: str) -> None:
    if rc <= -1000:            # the launch itself failed: -(1000 + cudaError_t)
        raise RuntimeError(f"{what}: CUDA launch error {-rc - 1000}")
    if rc != 0:
        raise RuntimeError(f"{what}: launcher returned {rc}")


DT_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
