"""Guard bands around device buffers: the stand-in for a memory checker on machines where none can run.

With ``GB200_CANARIES=1`` every buffer allocated through :func:`empty` / :func:`zeros` sits between two 4 KiB bands
filled with a byte pattern; :func:`check` names the buffers whose bands a kernel wrote into.  Without the variable
the functions are plain ``torch.empty`` / ``torch.zeros``.  The CUDA model, the MoE workspace, the optimizer state and
the inference engine allocate through here; ``tests/test_canaries_gpu.py`` runs training steps and decoding on
awkward sizes with the guards on.  Out-of-bounds reads are not caught by this (the argument checks of the launchers
and the fp32-oracle comparisons are what covers those).
"""
from __future__ import annotations

import os
from typing import List, Tuple

import torch

GUARD = 4096
PATTERN = 0xA5
_registry: List[Tuple[str, torch.Tensor, int]] = []


def enabled() -> bool:
    return os.environ.get("GB200_CANARIES", "") == "1"


def _alloc(shape, dtype, device, zero: bool, name: str) -> torch.Tensor:
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        shape = tuple(shape[0])
    if not enabled() or torch.device(device).type != "cuda":
        return (torch.zeros if zero else torch.empty)(*shape, dtype=dtype, device=device)
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    body = (nbytes + 255) // 256 * 256                   # keeps the 256-byte alignment kernels and TMA maps assume
    flat = torch.full((GUARD + body + GUARD,), PATTERN, dtype=torch.uint8, device=device)
    mid = flat[GUARD:GUARD + nbytes]
    if zero:
        mid.zero_()
    _registry.append((name or "buffer%d" % len(_registry), flat, nbytes))
    return mid.view(dtype).view(*shape)


def empty(*shape, dtype, device, name: str = "") -> torch.Tensor:
    return _alloc(shape, dtype, device, False, name)


def zeros(*shape, dtype, device, name: str = "") -> torch.Tensor:
    return _alloc(shape, dtype, device, True, name)


def check() -> List[str]:
    """Names (with the side that was hit) of the registered buffers whose guard bands no longer hold the pattern.
    The slack between the end of a buffer and its 256-byte boundary is part of the upper band."""
    bad = []
    for name, flat, nbytes in _registry:
        if not bool((flat[:GUARD] == PATTERN).all()):
            bad.append(name + ":below")
        if not bool((flat[GUARD + nbytes:] == PATTERN).all()):
            bad.append(name + ":above")
    return bad


def count() -> int:
    return len(_registry)


def reset():
    _registry.clear()
