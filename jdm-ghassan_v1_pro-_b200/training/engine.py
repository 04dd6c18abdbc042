"""Training engines: the object a :class:`Trainer` drives for one optimizer step.

``TorchEngine`` runs the fp32 PyTorch model (CPU, or any device) with the tensor-level optimizers; it
is the CPU path of the framework and the oracle the CUDA engine (``training/cuda_engine.py``) is
compared with.  Both expose the same protocol:

    begin_step(step, loss_scale)            zero gradients, set the router-jitter seed for the step
    micro_step(ids, targets, segments, B,T) forward + backward of one micro-batch (gradients accumulate)
    end_step(lr) -> StepResult              cross-rank sums, optimizer (or skip), router-bias update
    eval_batch(...) -> (loss_sum, ntok)     forward only, no jitter

Gradient semantics are the reference's (training/trainer.cpp:1476-1518): every rank back-propagates
the *sum* of per-token losses times the loss scale; after the cross-rank sum the optimizer applies
``grad_scale = 1 / (ntok_global * loss_scale)``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.reference import TorchModel
from . import optim as O

MOE_BIAS_LR = 0.001
MOE_BIAS_CLAMP = 0.5
_M64 = (1 << 64) - 1


def jitter_seed_for(seed: int, step: int, rank: int) -> int:
    """Per-step, per-rank seed of the router jitter hash (training/trainer.cpp:1462-1470)."""
    return (seed ^ ((step * 0x9E3779B97F4A7C15) & _M64) ^ ((rank * 0xBF58476D1CE4E5B9) & _M64)) & _M64


def moe_bias_update(bias: torch.Tensor, counts: torch.Tensor) -> None:
    """Aux-loss-free balancing: ``b[e] -= 0.001 * (share[e] - 1/ne)`` clamped to +-0.5, where ``share`` is the
    expert's part of all routed slots of the layer in this step (model/model.cpp:164-186, 233-262)."""
    ne = bias.shape[-1]
    row = counts.double().sum(dim=-1, keepdim=True)
    live = (row > 0).squeeze(-1)
    frac = (counts.double() / row.clamp_min(1.0)).float()
    upd = bias - MOE_BIAS_LR * (frac - 1.0 / ne)
    upd = upd.clamp_(-MOE_BIAS_CLAMP, MOE_BIAS_CLAMP)
    bias[live] = upd[live]


@dataclass
class StepResult:
    loss: float            # token-weighted mean of the micro-batch losses (incl. aux term)
    ntok_local: int
    ntok_global: int
    gnorm: float
    applied: bool          # False: skipped (non-finite norm) or all-masked step


def format_balance_report(acc, num_experts: int) -> str:
    """``expert load (share of routed slots): L0[min..max] L1[..]!`` from per-layer routed-slot counts accumulated
    since the last report; ``!`` marks a layer whose least (most) loaded expert is below a quarter of (above four
    times) the even share.  Same text as the reference prints at evaluation (model/model.cpp:107-127)."""
    if acc is None:
        return ""
    rows = acc.detach().double().cpu().tolist()
    out = []
    for l, row in enumerate(rows):
        tot = sum(row)
        if tot <= 0:
            continue
        mn, mx = min(row) / tot, max(row) / tot
        flag = "!" if (mn < 0.25 / num_experts or mx > 4.0 / num_experts) else ""
        out.append(" L%d[%.2f..%.2f]%s" % (l, mn, mx, flag))
    return ("expert load (share of routed slots):" + "".join(out)) if out else ""


class DistInfo:
    """Rank / world size and the small host-side collectives the engines need."""

    def __init__(self):
        import torch.distributed as dist
        self.dist = dist
        self.on = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank() if self.on else 0
        self.world = dist.get_world_size() if self.on else 1

    def all_reduce_sum_(self, t: torch.Tensor) -> torch.Tensor:
        if self.on and self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return t

    def broadcast_(self, t: torch.Tensor, src=0) -> torch.Tensor:
        if self.on and self.world > 1:
            self.dist.broadcast(t, src=src)
        return t

    def barrier(self):
        if self.on and self.world > 1:
            self.dist.barrier()


class TorchEngine:
    kind = "torch"

    def __init__(self, mcfg: ModelConfig, tcfg, device="cpu", seed: Optional[int] = None):
        self.mcfg, self.tcfg = mcfg, tcfg
        self.device = torch.device(device)
        self.dist = DistInfo()
        self.model = TorchModel(mcfg, self.device)
        self.model.init_weights(tcfg.seed if seed is None else seed)
        self.sync_model()
        self.model.enable_grad(True)
        specs = {s.name: s for s in mcfg.param_specs()}
        self.opt_params = [O.OptParam(n, p, specs[n].decay,
                                      frozen=(tcfg.freeze_embeddings and n == "tok_embeddings"))
                           for n, p in self.model.named_parameters()]
        self.optimizer = O.make_optimizer(tcfg, self.opt_params)
        self._bias_counts: Optional[torch.Tensor] = None
        self._load_acc: Optional[torch.Tensor] = None     # routed slots per (layer, expert) since the last report
        self._loss_num = 0.0
        self._ntok = 0
        self._loss_scale = 1.0
        self._jitter_seed = 0
        self.weight_ema: Optional[Dict[str, torch.Tensor]] = None
        if tcfg.weight_ema > 0:
            self.weight_ema = {n: p.detach().clone() for n, p in self.model.named_parameters()}

    # ------------------------------------------------------------------ distributed
    def sync_model(self):
        """Rank 0's weights everywhere (one broadcast per parameter)."""
        for _, p in self.model.named_parameters():
            self.dist.broadcast_(p.data, 0)

    # ------------------------------------------------------------------ step protocol
    def begin_step(self, step: int, loss_scale: float):
        self.model.zero_grad()
        self._loss_num, self._ntok = 0.0, 0
        self._loss_scale = float(loss_scale)
        self._jitter_seed = jitter_seed_for(self.tcfg.seed, step, self.dist.rank)

    def micro_step(self, ids, targets, segments, B, T):
        ids = torch.as_tensor(ids, device=self.device)
        targets = torch.as_tensor(targets, device=self.device)
        segments = torch.as_tensor(segments, device=self.device) if segments is not None else None
        seed = self._jitter_seed if self.mcfg.moe_jitter > 0 else None
        res = self.model.forward(ids, targets, B, T, segments, jitter_seed=seed)
        if res.ntok == 0:
            return 0.0, 0            # nothing supervised: no backward, no router counts
        (res.objective(self.mcfg) * self._loss_scale).backward()
        if self.tcfg.freeze_embeddings:
            self.model.params["tok_embeddings"].grad = None
        if res.slot_counts is not None:
            c = res.slot_counts.detach()
            self._load_acc = c.double() if self._load_acc is None else self._load_acc + c.double()
            if self.model.moe_bias is not None:
                self._bias_counts = c if self._bias_counts is None else self._bias_counts + c
        loss = res.reported_loss(self.mcfg)
        self._loss_num += loss * res.ntok
        self._ntok += res.ntok
        return loss, res.ntok

    def end_step(self, lr: float) -> StepResult:
        d = self.dist
        if d.world > 1:
            for _, p in self.model.named_parameters():
                if p.grad is None:
                    p.grad = torch.zeros_like(p)
                d.all_reduce_sum_(p.grad)
        ntok_global = int(d.all_reduce_sum_(torch.tensor([self._ntok], dtype=torch.int64, device=self.device))[0])
        loss = self._loss_num / self._ntok if self._ntok > 0 else 0.0
        applied, gnorm = False, 0.0
        if ntok_global > 0:
            grad_scale = float(np.float32(1.0) / (np.float32(ntok_global) * np.float32(self._loss_scale)))
            gnorm = self.optimizer.step(lr, grad_scale)
            applied = math.isfinite(gnorm)
        else:
            self.model.zero_grad()
        if self.model.moe_bias is not None:
            counts = self._bias_counts
            if counts is None:
                counts = torch.zeros_like(self.model.moe_bias)
            counts = d.all_reduce_sum_(counts.clone())
            if applied:   # rows without any routed slot (nothing supervised anywhere) are left untouched
                moe_bias_update(self.model.moe_bias, counts)
            self._bias_counts = None
        if applied and self.weight_ema is not None:
            beta = self.tcfg.weight_ema
            with torch.no_grad():
                for n, p in self.model.named_parameters():
                    self.weight_ema[n].mul_(beta).add_(p.detach(), alpha=1.0 - beta)
        return StepResult(loss, self._ntok, ntok_global, gnorm, applied)

    def balance_report(self) -> str:
        """Expert-load line for the evaluation log; resets the accumulation."""
        rep = format_balance_report(self._load_acc, self.mcfg.num_experts) if self.mcfg.use_moe else ""
        self._load_acc = None
        return rep

    @torch.no_grad()
    def eval_batch(self, ids, targets, segments, B, T):
        ids = torch.as_tensor(ids, device=self.device)
        targets = torch.as_tensor(targets, device=self.device)
        segments = torch.as_tensor(segments, device=self.device) if segments is not None else None
        res = self.model.forward(ids, targets, B, T, segments, jitter_seed=None)
        return float(res.loss_sum), res.ntok

    # ------------------------------------------------------------------ state for checkpoints
    def export_weights(self) -> List:
        return [(n, np.ascontiguousarray(p.detach().cpu().numpy())) for n, p in self.model.named_parameters()]

    def import_weights(self, named: Dict[str, np.ndarray], strict=True) -> List[str]:
        missing = []
        with torch.no_grad():
            for n, p in self.model.named_parameters():
                if n in named:
                    p.copy_(torch.from_numpy(np.asarray(named[n], dtype=np.float32)).view_as(p))
                else:
                    missing.append(n)
        if missing and strict:
            raise KeyError(f"checkpoint lacks param {missing[0]}")
        return missing

    def export_moe_bias(self) -> List[np.ndarray]:
        if self.model.moe_bias is None:
            return []
        return [np.ascontiguousarray(r.cpu().numpy()) for r in self.model.moe_bias]

    def import_moe_bias(self, rows) -> None:
        if self.model.moe_bias is None:
            return
        for l, r in enumerate(rows):
            if len(r) != self.model.moe_bias.shape[1]:
                raise ValueError("checkpoint moe bias shape mismatch")
            self.model.moe_bias[l].copy_(torch.as_tensor(np.asarray(r, dtype=np.float32)))

    def export_optimizer(self) -> dict:
        opt = self.optimizer
        cpu = lambda t: None if t is None else np.ascontiguousarray(t.detach().cpu().numpy().reshape(-1))
        return {"kind": opt.kind, "t": int(opt.t), "hyper": {k: float(v) if not isinstance(v, int) else v
                                                            for k, v in opt.hyper().items()},
                "m": [cpu(t) for t in opt.m], "v": [cpu(t) for t in opt.v], "fmt": 1}

    def import_optimizer(self, blob: dict) -> bool:
        """Restore moments and the applied-update counter; False when the blob does not fit this optimizer."""
        opt = self.optimizer
        if blob is None or blob.get("kind") != opt.kind or len(blob["m"]) != len(opt.m):
            return False
        for i, (m, v) in enumerate(zip(blob["m"], blob["v"])):
            if m is not None and opt.m[i] is not None:
                if m.size != opt.m[i].numel():
                    return False
                opt.m[i].copy_(torch.from_numpy(np.asarray(m)).view_as(opt.m[i]))
            if v is not None and opt.v[i] is not None:
                opt.v[i].copy_(torch.from_numpy(np.asarray(v)).view_as(opt.v[i]))
        opt.t = int(blob["t"])
        h = blob["hyper"]
        opt.beta1, opt.beta2 = float(h["beta1"]), float(h["beta2"])
        if "eps" in h and hasattr(opt, "eps"):
            opt.eps = float(h["eps"])
        return True

    def optimizer_hyper(self) -> dict:
        return self.optimizer.hyper()

    def set_opt_step(self, t: int):
        self.optimizer.t = int(t)
