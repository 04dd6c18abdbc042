"""Muon on the B200: the reference's update rule (training/optimizer.cpp:385-455; oracle: ``training/optim.py``) with
its Newton-Schulz products on the tcgen05 GEMM and everything else in CUDA kernels (``csrc/cuda/muon.cu``), no host
synchronisation and no per-matrix launch.

Which rule a parameter gets is the reference's: a 2-D matrix with weight decay whose smaller side is at least
``muon_min_ns_dim`` takes momentum + Newton-Schulz; a vector takes AdamW and any other matrix Lion, both at
``lr * muon_vec_ratio``.  The Newton-Schulz matrices are grouped into *classes* of equal shape; all matrices of a class
(one per layer, typically) are stacked in one buffer and iterate together: one grouped GEMM for every Gram matrix
``A = O^T O`` of the class and one for every product ``O A``.  Rows of a class are gathered from / scattered to the flat
compute-layout buffers through an offset table, so fused QKV rows and interleaved gate/up rows need no copies of the
weights.  GEMM operands are bf16 (fp32 accumulation, fp32 iterate and momentum): Newton-Schulz contracts rounding noise,
and a comparison with the fp32 oracle is part of the GPU tests.

Checkpoints hold the state in the reference's per-parameter form (momentum for every parameter, second moments for
vectors only), so a file written here resumes in the reference and the other way round.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..ops import _lib
from ..ops import gemm as G
from ..ops import kernels as K

_F32 = np.float32
ROW_PAD = 256            # class matrices start at multiples of this many rows (one two-CTA GEMM tile)


def _row_offsets(layout, cfg, name: str, shape) -> np.ndarray:
    """Flat-buffer offset of every row of the reference parameter ``name`` in the compute layout."""
    R, C = shape
    E, d, ne, qd, kvd = layout.Eff, cfg.hidden_size, cfg.num_experts, cfg.q_dim, cfg.kv_dim
    r = np.arange(R, dtype=np.int64)
    if name in ("tok_embeddings", "lm_head"):
        return layout.segments[name].offset + r * C
    _, li, leaf = name.split(".", 2)
    p = "L%s." % li
    seg = lambda key: layout.segments[p + key].offset
    if leaf == "wq":
        return seg("wqkv") + r * d
    if leaf == "wk":
        return seg("wqkv") + (qd + r) * d
    if leaf == "wv":
        return seg("wqkv") + (qd + kvd + r) * d
    if leaf == "wo":
        return seg("wo") + r * C
    if leaf == "moe_router":
        return seg("router") + r * C

    def gu(rows, first_expert, up):      # row j of expert e -> interleaved position inside w_gu
        e, j = first_expert + rows // E, rows % E
        return seg("w_gu") + ((e * 2 * E) + (j // 64) * 128 + (64 if up else 0) + (j % 64)) * d

    if leaf in ("moe_gate", "w_gate"):
        return gu(r, 0, False)
    if leaf in ("moe_up", "w_up"):
        return gu(r, 0, True)
    if leaf == "moe_sh_gate":
        return gu(r, ne, False)
    if leaf == "moe_sh_up":
        return gu(r, ne, True)
    if leaf in ("moe_down", "w_down"):
        return seg("w_down") + r * C
    if leaf == "moe_sh_down":
        return seg("w_down") + (ne * d + r) * C
    raise KeyError(name)


class _NsClass:
    """All Newton-Schulz matrices of one shape, stacked."""

    def __init__(self, shape, names: List[str], offsets: List[np.ndarray], decay: bool, device):
        self.R, self.C = shape
        self.names, self.decay = names, decay
        self.n = len(names)
        self.Rp = (self.R + ROW_PAD - 1) // ROW_PAD * ROW_PAD
        rows = self.n * self.Rp
        src = np.full(rows, -1, dtype=np.int64)
        for i, off in enumerate(offsets):
            src[i * self.Rp:i * self.Rp + self.R] = off
        self.rows = rows
        self.row_src = torch.from_numpy(src).to(device)
        self.m = torch.zeros(rows, self.C, dtype=torch.float32, device=device)      # momentum: the optimizer state
        self.partial = torch.zeros(rows // 8, dtype=torch.float64, device=device)
        self.skip = torch.zeros(self.n, dtype=torch.int32, device=device)
        self.tile_mat = torch.arange(self.n, dtype=torch.int32, device=device).repeat_interleave(self.Rp // 128).contiguous()
        self.num_tiles = torch.tensor([rows // 128], dtype=torch.int32, device=device)
        self.seg = (torch.arange(self.n + 1, dtype=torch.int32, device=device) * self.Rp).contiguous()


class MuonCuda:
    kind = "muon"

    def __init__(self, model, mcfg, tcfg):
        self.model, self.mcfg = model, mcfg
        dev = model.dev
        self.lr, self.vec_ratio = tcfg.learning_rate, tcfg.muon_vec_ratio
        self.beta1, self.beta2, self.eps = tcfg.beta1, tcfg.beta2, tcfg.eps
        self.weight_decay, self.grad_clip = tcfg.weight_decay, tcfg.grad_clip
        self.ns_steps = min(10, max(1, tcfg.muon_ns_steps))
        self.min_ns_dim = tcfg.muon_min_ns_dim
        self.t = 0
        L = model.layout
        self.specs = list(mcfg.param_specs())
        groups: Dict[Tuple, Tuple[List[str], List[np.ndarray]]] = {}
        small: List[Tuple[int, int, str, float]] = []          # (lo, hi, kind, wd) flat ranges of the other parameters
        self.rule: Dict[str, str] = {}
        for s in self.specs:
            if self.uses_ns(s):
                off = _row_offsets(L, mcfg, s.name, s.shape)
                names, offs = groups.setdefault((tuple(s.shape), bool(s.decay)), ([], []))
                names.append(s.name)
                offs.append(off)
                self.rule[s.name] = "ns"
                continue
            kind = "adamw" if len(s.shape) == 1 else "lion"
            self.rule[s.name] = kind
            wd = self.weight_decay if s.decay else 0.0
            if len(s.shape) == 1:
                key = "L" + s.name.split(".", 2)[1] + "." + s.name.split(".", 2)[2] if s.name.startswith("layers.") else s.name
                seg = L.segments[key]
                small.append((seg.offset, seg.offset + seg.numel, kind, wd))
            else:
                off = _row_offsets(L, mcfg, s.name, s.shape)
                C = s.shape[1]
                # contiguous runs of rows become ranges
                brk = np.nonzero(np.diff(off) != C)[0] + 1
                for a, b in zip(np.concatenate([[0], brk]), np.concatenate([brk, [len(off)]])):
                    small.append((int(off[a]), int(off[b - 1]) + C, kind, wd))
        self.classes = [_NsClass(shape, names, offs, decay, dev) for (shape, decay), (names, offs) in groups.items()]
        # merge neighbouring ranges of the same rule (alignment gaps between segments hold zeros and zero gradients)
        small.sort()
        merged: List[List] = []
        for lo, hi, kind, wd in small:
            if merged and merged[-1][2] == kind and merged[-1][3] == wd and lo - merged[-1][1] < 64:
                merged[-1][1] = hi
            else:
                merged.append([lo, hi, kind, wd])
        self.small = [tuple(x) for x in merged]
        span = max((hi for _, hi, _, _ in self.small), default=0)
        self.m_small = torch.zeros(span, dtype=torch.float32, device=dev)
        self.v_small = torch.zeros(span, dtype=torch.float32, device=dev)
        # scratch shared by all classes, sized for the largest
        rows_max = max((c.rows * c.C for c in self.classes), default=0)
        gram_max = max((c.n * c.C * c.C for c in self.classes), default=0)
        self.Y = torch.zeros(rows_max, dtype=torch.float32, device=dev)
        self.T = torch.zeros(rows_max, dtype=torch.float32, device=dev)
        self.Y16 = torch.zeros(rows_max, dtype=torch.bfloat16, device=dev)
        self.A = torch.zeros(gram_max, dtype=torch.float32, device=dev)
        self.B16 = torch.zeros(gram_max, dtype=torch.bfloat16, device=dev)
        self.hyper_vec = torch.zeros(3, dtype=torch.float32, device=dev)       # {lr * vec_ratio, bc1, bc2}
        self.lr_dev = torch.zeros(1, dtype=torch.float32, device=dev)
        self.hyper_host = torch.zeros(4, dtype=torch.float32).pin_memory()
        self.gemm_launches = 0

    # ------------------------------------------------------------------ rules
    def uses_ns(self, s) -> bool:
        if len(s.shape) != 2 or not s.decay:
            return False
        return self.min_ns_dim <= 0 or min(s.shape) >= self.min_ns_dim

    def hyper(self):
        return dict(lr=self.lr, vec_ratio=self.vec_ratio, beta1=self.beta1, beta2=self.beta2, eps=self.eps,
                    weight_decay=self.weight_decay, grad_clip=self.grad_clip, ns_steps=self.ns_steps,
                    min_ns_dim=self.min_ns_dim)

    # ------------------------------------------------------------------ one step (all launches asynchronous)
    def launch(self, lr: float, scale_dev: torch.Tensor):
        """Update every parameter from the gradients in ``model.Gr``; ``scale_dev[0]`` = grad_scale * clip factor of the
        step, 0 when the step is rejected (then nothing changes).  The caller advances ``t`` when the step applied."""
        m = self.model
        lib, st = _lib.lib(), _lib.stream_ptr()
        t = self.t + 1
        bc1 = float(_F32(1.0) - np.power(_F32(self.beta1), _F32(t), dtype=_F32))
        bc2 = float(_F32(1.0) - np.power(_F32(self.beta2), _F32(t), dtype=_F32))
        h = self.hyper_host
        h[0], h[1], h[2], h[3] = float(_F32(lr) * _F32(self.vec_ratio)), bc1, bc2, lr
        self.hyper_vec.copy_(h[:3], non_blocking=True)
        self.lr_dev.copy_(h[3:4], non_blocking=True)
        for lo, hi, kind, wd in self.small:
            K.optimizer_step(kind, m.P[lo:hi], m.Gr[lo:hi], self.m_small[lo:hi],
                             self.v_small[lo:hi] if kind == "adamw" else None, m.W16[lo:hi], self.hyper_vec, scale_dev,
                             self.beta1, self.beta2, self.eps, wd)
        p = lambda x: ctypes.c_void_p(x.data_ptr())
        sc = p(scale_dev)
        is_bf16 = int(m.W16.dtype == torch.bfloat16)
        for c in self.classes:
            rows, C, n = c.rows, c.C, c.n
            Y, T, Y16 = self.Y[:rows * C].view(rows, C), self.T[:rows * C].view(rows, C), self.Y16[:rows * C].view(rows, C)
            A, B16 = self.A[:n * C * C].view(n, C, C), self.B16[:n * C * C].view(n * C, C)
            _lib.check_rc(lib.gb_muon_momentum(p(c.m), p(m.Gr), p(c.row_src), ctypes.c_longlong(rows), C,
                                               ctypes.c_float(self.beta1), sc, p(c.partial), st), "muon_momentum")
            _lib.check_rc(lib.gb_muon_normalize(p(c.m), p(Y), p(T), p(Y16), p(c.partial), ctypes.c_longlong(rows), c.Rp, C,
                                                sc, p(c.skip), st), "muon_normalize")
            for _ in range(self.ns_steps):
                G.gemm_grouped_reduce(Y16, Y16, c.seg, n, A, accumulate=False)                  # A[g] = Y[g]^T Y[g]
                _lib.check_rc(lib.gb_muon_gram_cast(p(A), p(B16), ctypes.c_longlong(n * C * C), sc, st), "muon_gram_cast")
                G.gemm_grouped_rows(Y16, B16, c.tile_mat, c.num_tiles, n=C, group_rows=C, out=Y, addend=T)   # Y = 1.5 Y - 0.5 Y A
                _lib.check_rc(lib.gb_muon_refresh(p(Y), p(T), p(Y16), ctypes.c_longlong(rows), c.Rp, C, sc, p(c.skip), st),
                              "muon_refresh")
                self.gemm_launches += 2
            _lib.check_rc(lib.gb_muon_apply(p(m.P), p(m.W16), is_bf16, p(Y), p(c.row_src), ctypes.c_longlong(rows), C,
                                            p(self.lr_dev), ctypes.c_float(self.weight_decay if c.decay else 0.0), sc, st),
                          "muon_apply")

    # ------------------------------------------------------------------ state in the reference's per-parameter form
    def _small_named(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        pad = torch.zeros(self.model.layout.total - flat.numel(), dtype=flat.dtype, device=flat.device)
        return self.model.layout.from_internal(torch.cat([flat, pad]))

    def export_state(self) -> dict:
        cpu = lambda t: np.ascontiguousarray(t.detach().float().cpu().numpy().reshape(-1))
        m_named = self._small_named(self.m_small)
        v_named = self._small_named(self.v_small)
        ns = {}
        for c in self.classes:
            mm = c.m.view(c.n, c.Rp, c.C)
            for i, name in enumerate(c.names):
                ns[name] = mm[i, :c.R]
        ms, vs = [], []
        for s in self.specs:
            if self.rule[s.name] == "ns":
                ms.append(cpu(ns[s.name]))
                vs.append(None)
            else:
                ms.append(cpu(m_named[s.name]))
                vs.append(cpu(v_named[s.name]) if len(s.shape) == 1 else None)
        return {"kind": "muon", "t": int(self.t), "hyper": {k: (int(v) if isinstance(v, int) else float(v))
                                                            for k, v in self.hyper().items()}, "m": ms, "v": vs, "fmt": 1}

    def import_state(self, blob: dict) -> bool:
        if blob is None or blob.get("kind") != "muon" or len(blob["m"]) != len(self.specs):
            return False
        dev = self.model.dev
        L = self.model.layout
        m_named, v_named = {}, {}
        for i, s in enumerate(self.specs):
            mm = blob["m"][i]
            if mm is None:
                continue
            if np.asarray(mm).size != s.numel:
                return False
            t = torch.from_numpy(np.asarray(mm, dtype=np.float32).reshape(s.shape)).to(dev)
            if self.rule[s.name] == "ns":
                for c in self.classes:
                    if s.name in c.names:
                        c.m.view(c.n, c.Rp, c.C)[c.names.index(s.name), :c.R].copy_(t)
            else:
                m_named[s.name] = t
                vv = blob["v"][i] if i < len(blob.get("v", [])) else None
                if vv is not None and len(s.shape) == 1:
                    v_named[s.name] = torch.from_numpy(np.asarray(vv, dtype=np.float32).reshape(s.shape)).to(dev)
        if self.m_small.numel():
            full = torch.zeros(L.total, dtype=torch.float32, device=dev)
            full[:self.m_small.numel()] = self.m_small
            L.to_internal(m_named, full, missing_ok=True)
            self.m_small.copy_(full[:self.m_small.numel()])
            full.zero_()
            full[:self.v_small.numel()] = self.v_small
            L.to_internal(v_named, full, missing_ok=True)
            self.v_small.copy_(full[:self.v_small.numel()])
        self.t = int(blob["t"])
        h = blob.get("hyper", {})
        self.beta1, self.beta2 = float(h.get("beta1", self.beta1)), float(h.get("beta2", self.beta2))
        if "eps" in h:
            self.eps = float(h["eps"])
        return True
