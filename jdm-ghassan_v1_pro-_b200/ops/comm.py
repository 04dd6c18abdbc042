"""Launchers for the peer-memory gradient exchange kernels (``csrc/cuda/comm.cu``, protocol in ``gb_comm.h``)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

c_int, c_ll, c_vp, c_float, c_double, c_uint = (ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_float,
                                                ctypes.c_double, ctypes.c_uint)
CTL_WORDS = 1024
MAX_RANKS = 16
SYNC_BLOCKS = 592


class SyncArgs(ctypes.Structure):
    _fields_ = [
        ("rank", c_int), ("world", c_int),
        ("shard", c_ll), ("total", c_ll), ("decay_start", c_ll), ("f32_end", c_ll),
        ("peer_grad", c_vp), ("peer_master", c_vp), ("peer_w16", c_vp), ("peer_ctl", c_vp),
        ("m", c_vp), ("v", c_vp),
        ("kind", c_int), ("beta1", c_float), ("beta2", c_float), ("eps", c_float), ("wd", c_float),
        ("hyper", c_vp),
        ("loss_scale", c_float), ("clip", c_float),
        ("ntok_local", c_double),
        ("epoch", c_uint),
        ("partial", c_vp), ("ticket", c_vp), ("out", c_vp), ("status", c_vp),
        ("is_bf16", c_int), ("no_wait", c_int), ("local_only", c_int),
        ("mc_grad", c_vp), ("mc_master", c_vp), ("mc_w16", c_vp),
    ]


def pointer_table(ptrs, device) -> torch.Tensor:
    """Device array of raw pointers (int64) for a kernel's ``T* const*`` argument."""
    return torch.tensor([int(p) for p in ptrs], dtype=torch.int64, device=device)


def barrier(ctl_table: torch.Tensor, rank: int, world: int, epoch: int):
    rc = _lib.lib().gb_sync_barrier(c_vp(ctl_table.data_ptr()), c_int(rank), c_int(world), c_uint(epoch & 0xFFFFFFFF),
                                    c_vp(_lib.status_word(ctl_table.device).data_ptr()), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_sync_barrier")


def reduce(args: SyncArgs):
    _lib.check_rc(_lib.lib().gb_sync_reduce(ctypes.byref(args), _lib.stream_ptr()), "gb_sync_reduce")


def update(args: SyncArgs):
    _lib.check_rc(_lib.lib().gb_sync_update(ctypes.byref(args), _lib.stream_ptr()), "gb_sync_update")


def gather(peer_table: torch.Tensor, local: torch.Tensor, shard_elems: int, limit_elems: int, rank: int, world: int):
    """All-gather by peer loads: ``local[r*shard : (r+1)*shard]`` (below ``limit_elems``) from every other rank ``r``."""
    es = local.element_size()
    rc = _lib.lib().gb_sync_gather(c_vp(peer_table.data_ptr()), c_vp(local.data_ptr()), c_ll(shard_elems * es),
                                   c_ll(limit_elems * es), c_int(rank), c_int(world), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_sync_gather")


def small_allreduce(src_table: torch.Tensor, dst: torch.Tensor, n: int, world: int):
    rc = _lib.lib().gb_sync_small_allreduce(c_vp(src_table.data_ptr()), c_vp(dst.data_ptr()), c_int(n), c_int(world),
                                            _lib.stream_ptr())
    _lib.check_rc(rc, "gb_sync_small_allreduce")
