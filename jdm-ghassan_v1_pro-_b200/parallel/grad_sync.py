"""Fused gradient exchange + sharded optimizer + parameter all-gather over NVSwitch peer memory.

What the reference does per optimizer step with data parallelism (training/trainer.cpp:1835-1966): one NCCL
all-reduce per large gradient tensor plus one over a staging buffer of the small ones, an all-reduce of the token
count, one of the routing counts, a host-side gradient norm, and one optimizer launch per tensor on every rank.

Here the flat gradient, master-weight and 16-bit-shadow buffers live in symmetric memory, and one short kernel
sequence on each rank does all of it (``csrc/cuda/comm.cu``):

1. barrier: every rank's backward has finished;
2. reduce-scatter: rank r sums shard r of all ranks' gradients through peer loads (rank order, so the result is
   reproducible), accumulates Sum g^2 of the shard and mails {Sum g^2, its token count} to every rank;
3. update + all-gather: every rank folds the mailed numbers into the same global norm, clip factor and skip
   decision, updates its shard (moments stay sharded) and stores the new 16-bit weights, and the few tensors the
   kernels read in fp32, into every rank's buffers;
4. barrier: all stores have landed before anyone starts the next forward or clears its gradients.

Between steps a rank's fp32 master copy is current only for its own shard (and the fp32-consumed range);
:meth:`gather_full_state` completes it on every rank before a checkpoint is taken.
"""
from __future__ import annotations

import os

from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import comm as C

_F32 = np.float32


class SymmetricBuffers:
    """Symmetric-memory allocations of one process group and the peer pointer tables the kernels take."""

    def __init__(self, group=None, multicast: bool = False):
        # By default the kernels reach peers with plain loads and stores and never use a multicast address, so the
        # buffers are not bound to an NVLink multicast object: a rank that dies while its memory is bound to one (the
        # step watchdog exits hard, the launcher kills stragglers) can fault the other ranks' GPUs.  ``multicast``
        # (recipe key ``b200.grad_sync_nvls``) asks for the binding; it takes effect only if no buffer of this process
        # was created without it.  Set before the first rendezvous.
        if multicast:
            os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "0"
        else:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.multicast = multicast
        self.mc_ptrs = []
        import torch.distributed._symmetric_memory as symm
        self.symm = symm
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.handles = []

    def alloc(self, numel: int, dtype) -> "tuple[torch.Tensor, torch.Tensor]":
        """Returns (local tensor, device table of all ranks' base pointers)."""
        t = self.symm.empty(numel, dtype=dtype, device=self.device)
        t.zero_()
        h = self.symm.rendezvous(t, self.group.group_name)
        self.handles.append(h)          # keeps the mapping alive
        self.mc_ptrs.append(int(getattr(h, "multicast_ptr", 0) or 0) if self.multicast else 0)
        table = C.pointer_table(h.buffer_ptrs, self.device)
        return t, table


class LocalBuffers:
    """Same interface over plain device memory for world size 1 (a single rank still uses the fused kernels)."""

    def __init__(self):
        self.rank, self.world = 0, 1
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.multicast, self.mc_ptrs = False, []

    def alloc(self, numel: int, dtype):
        t = torch.zeros(numel, dtype=dtype, device=self.device)
        return t, C.pointer_table([t.data_ptr()], self.device)


class FusedGradSync:
    def __init__(self, engine, buffers=None, nvls: bool = False):
        """``nvls``: reduce and distribute through NVSwitch multicast (``multimem.ld_reduce`` / ``multimem.st``) when the
        symmetric buffers could be bound to a multicast object; otherwise, and by default, plain peer loads."""
        self.engine = engine
        m = engine.model
        L = m.layout
        if buffers is None:
            buffers = SymmetricBuffers(multicast=nvls) if (dist.is_available() and dist.is_initialized() and
                                                           dist.get_world_size() > 1) else LocalBuffers()
        self.buf = buffers
        self.rank, self.world = buffers.rank, buffers.world
        if self.world > C.MAX_RANKS:
            raise ValueError(f"fused gradient exchange supports up to {C.MAX_RANKS} ranks")
        self.total = L.total
        self.shard = ((self.total + self.world - 1) // self.world + 63) // 64 * 64
        padded = self.shard * self.world
        # re-home the flat buffers into symmetric memory (views into the first `total` elements keep their meaning)
        P, self.t_master = buffers.alloc(padded, torch.float32)
        W16, self.t_w16 = buffers.alloc(padded, m.dtype)
        Gr, self.t_grad = buffers.alloc(padded, torch.float32)
        mc = list(buffers.mc_ptrs[-3:]) if getattr(buffers, "multicast", False) else [0, 0, 0]
        self.mc_master, self.mc_w16, self.mc_grad = mc if all(mc) else (0, 0, 0)
        self.nvls = bool(self.mc_grad)
        if nvls and not self.nvls and buffers.rank == 0:
            from ..utils.log import log_warn
            log_warn("[sync] b200.grad_sync_nvls: no multicast address for the symmetric buffers; using peer loads")
        P[:self.total].copy_(m.P)
        W16[:self.total].copy_(m.W16)
        self._P_pad, self._W16_pad, self._Gr_pad = P, W16, Gr
        m.P, m.W16, m.Gr = P[:self.total], W16[:self.total], Gr[:self.total]
        ctl, self.t_ctl = buffers.alloc(C.CTL_WORDS, torch.int32)
        self.ctl = ctl
        self.counts_local = None
        if m.bias_counts is not None:
            n = m.bias_counts.numel()
            cs, self.t_counts = buffers.alloc((n + 63) // 64 * 64, torch.float32)
            self.counts_local = cs[:n].view_as(m.bias_counts)       # kernels accumulate here
            self.counts_global = torch.zeros_like(m.bias_counts)   # sum over ranks, read by the bias update
            m.bias_counts = self.counts_local
        dev = m.dev
        self.partial = torch.zeros(C.SYNC_BLOCKS, dtype=torch.float64, device=dev)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out = torch.zeros(4, dtype=torch.float32, device=dev)
        self.epoch = 0
        self.barrier_epoch = 0
        self.lo = self.rank * self.shard
        self.hi = min(self.total, self.lo + self.shard)
        # ZeRO-1 for real: only the owner ever touches the moments of a shard, so only the owner keeps them.  The
        # kernels index moments by global element, so they get the shard's address moved back by the shard's offset.
        self.m_own = self.v_own = None
        opt = engine.optimizer
        if self.world > 1 and opt.kind != "muon":
            own = slice(self.lo, self.hi)
            self.m_own = torch.zeros(self.shard, dtype=torch.float32, device=dev)
            self.m_own[:self.hi - self.lo].copy_(opt.m_flat[own])
            opt.m_flat = None
            if opt.v_flat is not None:
                self.v_own = torch.zeros(self.shard, dtype=torch.float32, device=dev)
                self.v_own[:self.hi - self.lo].copy_(opt.v_flat[own])
                opt.v_flat = None
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()

    # ------------------------------------------------------------------ one exchange
    def _args(self, lr_hyper: Optional[torch.Tensor], loss_scale: float, ntok_local: int, no_wait=False) -> C.SyncArgs:
        e, m, opt, t = self.engine, self.engine.model, self.engine.optimizer, self.engine.tcfg
        a = C.SyncArgs()
        a.rank, a.world = self.rank, self.world
        a.shard, a.total = self.shard, self.total
        a.decay_start, a.f32_end = m.layout.decay_start, m.layout.f32_end
        a.peer_grad, a.peer_master = self.t_grad.data_ptr(), self.t_master.data_ptr()
        a.peer_w16, a.peer_ctl = self.t_w16.data_ptr(), self.t_ctl.data_ptr()
        if opt.kind == "muon":           # norm and skip decision only; Muon itself runs after the gradient gather
            a.m, a.v, a.kind, a.hyper = None, None, 2, None
        else:
            if self.m_own is not None:
                a.m = self.m_own.data_ptr() - 4 * self.lo
                a.v = self.v_own.data_ptr() - 4 * self.lo if self.v_own is not None else None
            else:
                a.m = opt.m_flat.data_ptr()
                a.v = opt.v_flat.data_ptr() if opt.v_flat is not None else None
            a.kind = 0 if opt.kind == "adamw" else 1
            a.hyper = lr_hyper.data_ptr()
        a.beta1, a.beta2, a.eps, a.wd = opt.beta1, opt.beta2, opt.eps, opt.weight_decay
        a.loss_scale, a.clip = loss_scale, t.grad_clip
        a.ntok_local = float(ntok_local)
        a.epoch = self.epoch & 0xFFFFFFFF
        a.partial, a.ticket, a.out = self.partial.data_ptr(), self.ticket.data_ptr(), self.out.data_ptr()
        a.status = _lib.status_word(m.dev).data_ptr()
        a.is_bf16 = int(m.dtype == torch.bfloat16)
        a.no_wait = int(no_wait)
        a.local_only = 1                 # new values reach the peers by gb_sync_gather (loads), not by stores
        if self.nvls:
            a.mc_grad = self.mc_grad
            if opt.kind != "muon":       # Muon's update does not run in these kernels: only its reduction uses the switch
                a.mc_master, a.mc_w16 = self.mc_master, self.mc_w16
        return a

    def _barrier(self):
        if self.world > 1:
            self.barrier_epoch += 1
            C.barrier(self.t_ctl, self.rank, self.world, self.barrier_epoch)

    def step(self, lr: float, loss_scale: float, ntok_local: int):
        """Enqueue the whole exchange on the current stream; results land in ``self.out`` (scale, gnorm, ntok).

        AdamW / Lion: barrier, reduce-scatter + norm, update of the own shard, barrier, all-gather of the new 16-bit
        weights (and of the fp32 prefix) by peer loads; the next exchange's opening barrier is what keeps a rank from
        rewriting its shard under a peer that still reads it.  Muon: barrier, reduce-scatter + norm, barrier, all-gather
        of the reduced fp32 gradient, barrier (the next step zeroes the gradient buffer), then Muon on every rank: the
        Newton-Schulz matrices need whole gradients, and identical inputs give identical weights everywhere."""
        opt = self.engine.optimizer
        muon = opt.kind == "muon"
        hyper = None
        if not muon:
            t = opt.t + 1
            bc1 = float(_F32(1.0) - np.power(_F32(opt.beta1), _F32(t), dtype=_F32))
            bc2 = float(_F32(1.0) - np.power(_F32(opt.beta2), _F32(t), dtype=_F32))
            opt.hyper_host[0], opt.hyper_host[1], opt.hyper_host[2] = lr, bc1, bc2
            opt.hyper_dev.copy_(opt.hyper_host, non_blocking=True)
            hyper = opt.hyper_dev
        self.epoch += 1
        a = self._args(hyper, loss_scale, ntok_local)
        self._barrier()
        if self.counts_local is not None:
            C.small_allreduce(self.t_counts, self.counts_global, self.counts_global.numel(), self.world)
        C.reduce(a)
        C.update(a)
        self._barrier()
        if muon:
            C.gather(self.t_grad, self._Gr_pad, self.shard, self.total, self.rank, self.world)
            self._barrier()
            opt.launch(lr, self.out[0:1])
        elif not self.nvls:              # with multicast stores the new values are everywhere already
            C.gather(self.t_w16, self._W16_pad, self.shard, self.total, self.rank, self.world)
            C.gather(self.t_master, self._P_pad, self.shard, self.engine.model.layout.f32_end, self.rank, self.world)
        self._keep = a     # the struct is read at launch; kept only so that debugging can inspect the last call

    # ------------------------------------------------------------------ full state for checkpoints
    def gather_full_state(self):
        """Complete the master weights on every rank and the moments on rank 0, which writes the checkpoint
        (collective: all ranks must call it).  The full moments live in ``optimizer.m_flat`` / ``v_flat`` until
        :meth:`release_full_state`."""
        if self.world == 1:
            return
        opt = self.engine.optimizer
        own = slice(self.lo, self.lo + self.shard)
        if opt.kind == "muon":           # every rank ran the whole update: masters and state are complete already
            return
        dist.all_gather_into_tensor(self._P_pad, self._P_pad[own].clone())
        for name, mine in (("m_flat", self.m_own), ("v_flat", self.v_own)):
            if mine is None:
                continue
            pad = None
            if self.rank == 0:
                pad = torch.empty(self.shard * self.world, dtype=torch.float32, device=mine.device)
            dist.gather(mine, list(pad.view(self.world, self.shard).unbind(0)) if self.rank == 0 else None, dst=0)
            setattr(opt, name, pad[:self.total] if self.rank == 0 else None)
        ema = getattr(self.engine, "weight_ema", None)
        if ema is not None:
            pad = torch.zeros(self.shard * self.world, dtype=ema.dtype, device=ema.device)
            pad[:self.total].copy_(ema)
            dist.all_gather_into_tensor(pad, pad[own].clone())
            ema.copy_(pad[:self.total])

    def release_full_state(self):
        """Drop the gathered copy of the moments (after the checkpoint snapshot was taken)."""
        if self.m_own is not None:
            self.engine.optimizer.m_flat = None
            self.engine.optimizer.v_flat = None

    def load_full_moments(self, m_full: torch.Tensor, v_full: Optional[torch.Tensor]):
        """Resume: keep this rank's slice of moments read from a checkpoint (full, flat layout)."""
        n = self.hi - self.lo
        self.m_own[:n].copy_(m_full[self.lo:self.hi])
        if self.v_own is not None and v_full is not None:
            self.v_own[:n].copy_(v_full[self.lo:self.hi])
