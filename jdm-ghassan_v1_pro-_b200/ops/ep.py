"""Launchers for the expert-parallel planning and dispatch kernels (``csrc/cuda/ep.cu``, protocol in ``gb_ep.h``)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

c_int, c_ll, c_vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
MAX_DESC = 160
MAX_EXPERTS = 128


class PlanBuffers(ctypes.Structure):
    _fields_ = [("recv_seg", c_vp), ("tile_expert", c_vp), ("num_tiles", c_vp), ("desc", c_vp), ("num_desc", c_vp),
                ("tile_out_a", c_vp), ("tile_out_b", c_vp)]


class PlanArgs(ctypes.Structure):
    _fields_ = [("rank", c_int), ("world", c_int), ("ne", c_int), ("has_shared", c_int), ("max_rows", c_int),
                ("peer_seg", c_vp), ("base_a", c_vp), ("base_b", c_vp), ("row_bytes_a", c_ll), ("row_bytes_b", c_ll),
                ("out", PlanBuffers), ("status", c_vp)]


class Plan:
    """Device buffers holding one layer's received layout on one rank."""

    def __init__(self, ne1: int, max_rows: int, device):
        i32 = dict(dtype=torch.int32, device=device)
        self.max_rows = max_rows
        self.recv_seg = torch.zeros(ne1 + 1, **i32)
        self.tile_expert = torch.zeros(max_rows // 128, **i32)
        self.num_tiles = torch.zeros(1, **i32)
        self.desc = torch.zeros(MAX_DESC * 4, **i32)
        self.num_desc = torch.zeros(1, **i32)
        self.tile_out_a = torch.zeros(max_rows // 128, dtype=torch.int64, device=device)
        self.tile_out_b = torch.zeros(max_rows // 128, dtype=torch.int64, device=device)

    def c_buffers(self) -> PlanBuffers:
        b = PlanBuffers()
        b.recv_seg, b.tile_expert, b.num_tiles = self.recv_seg.data_ptr(), self.tile_expert.data_ptr(), self.num_tiles.data_ptr()
        b.desc, b.num_desc = self.desc.data_ptr(), self.num_desc.data_ptr()
        b.tile_out_a, b.tile_out_b = self.tile_out_a.data_ptr(), self.tile_out_b.data_ptr()
        return b


def plan(p: Plan, rank: int, world: int, ne: int, has_shared: bool, peer_seg: torch.Tensor, base_a: torch.Tensor,
         base_b: torch.Tensor, row_bytes_a: int, row_bytes_b: int):
    a = PlanArgs()
    a.rank, a.world, a.ne, a.has_shared, a.max_rows = rank, world, ne, int(has_shared), p.max_rows
    a.peer_seg, a.base_a, a.base_b = peer_seg.data_ptr(), base_a.data_ptr(), base_b.data_ptr()
    a.row_bytes_a, a.row_bytes_b = row_bytes_a, row_bytes_b
    a.out = p.c_buffers()
    a.status = _lib.status_word(p.recv_seg.device).data_ptr()
    _lib.check_rc(_lib.lib().gb_ep_plan(ctypes.byref(a), _lib.stream_ptr()), "gb_ep_plan")


def pull(peer_src: torch.Tensor, dst: torch.Tensor, p: Plan):
    """Rows named by the plan's copy descriptors, from every rank's source buffer into ``dst`` (``[max_rows, width]``)."""
    row_bytes = dst.stride(0) * dst.element_size()
    rc = _lib.lib().gb_ep_pull(c_vp(peer_src.data_ptr()), c_vp(dst.data_ptr()), c_ll(row_bytes), c_vp(p.desc.data_ptr()),
                               c_vp(p.num_desc.data_ptr()), c_int(p.max_rows), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_ep_pull")


def barrier_auto(ctl_table: torch.Tensor, rank: int, world: int, counter: torch.Tensor, spin_limit: int = 0):
    rc = _lib.lib().gb_sync_barrier_auto(c_vp(ctl_table.data_ptr()), c_int(rank), c_int(world), c_vp(counter.data_ptr()),
                                         c_ll(spin_limit), c_vp(_lib.status_word(ctl_table.device).data_ptr()),
                                         _lib.stream_ptr())
    _lib.check_rc(rc, "gb_sync_barrier_auto")
