"""Optimizers, learning-rate schedule and the dynamic loss scaler (tensor-level reference versions).

These run on any device with plain PyTorch ops and define the arithmetic the fused sm_100a
optimizer kernels are tested against.  Semantics follow the reference engine
(training/optimizer.cpp:82-135, 295-336, 385-455; core/ops_cpu_dense.cpp:997-1030;
training/scheduler.h:17-46; training/trainer.cpp:1051-1084):

* one global gradient norm over all parameters in float64, ``gnorm = sqrt(sum g^2) * grad_scale``;
  clip factor ``clip / (gnorm + 1e-6)`` when ``gnorm > clip``; a non-finite norm skips the update and
  does not advance the applied-update counter ``t``;
* AdamW with decoupled weight decay inside the update and float32 bias corrections ``1 - beta^t``;
* Lion: ``c = b1*m + (1-b1)*g; w -= lr*(sign(c) + wd*w); m = b2*m + (1-b2)*g``;
* Muon: decayed 2-D matrices (min(rows, cols) >= min_ns_dim) take momentum -> Frobenius
  normalisation -> ``ns_steps`` x ``O <- 1.5 O - 0.5 O (O^T O)`` in fp32 -> ``w += -lr*O; w *= 1-lr*wd``;
  vectors take AdamW and the remaining matrices Lion, both at ``lr * vec_ratio``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

_F32 = np.float32


@dataclass
class OptParam:
    name: str
    w: torch.Tensor          # fp32 master weight
    decay: bool
    frozen: bool = False

    @property
    def grad(self) -> Optional[torch.Tensor]:
        return self.w.grad


def global_grad_norm(params: List[OptParam], grad_scale: float) -> float:
    sq = 0.0
    for p in params:
        if p.frozen or p.grad is None or p.w.numel() == 0:
            continue
        sq += float(p.grad.double().pow(2).sum())
    return math.sqrt(sq) * float(grad_scale) if math.isfinite(sq) else float("nan")


def _clip_scale(gnorm: float, clip: float) -> float:
    if clip > 0.0 and gnorm > clip:
        return float(_F32(clip / (gnorm + 1e-6)))
    return 1.0


def _adamw_update(w, g, m, v, lr, b1, b2, eps, wd, bc1, bc2, scale):
    gi = g * scale
    m.mul_(b1).add_(gi, alpha=1.0 - b1)
    v.mul_(b2).addcmul_(gi, gi, value=1.0 - b2)
    upd = (m / bc1) / ((v / bc2).sqrt() + eps)
    if wd != 0.0:
        upd = upd + wd * w
    w.sub_(upd, alpha=lr)


def _lion_update(w, g, m, lr, b1, b2, wd, scale):
    gi = g * scale
    c = m * b1 + gi * (1.0 - b1)
    upd = torch.sign(c)
    if wd != 0.0:
        upd = upd + wd * w
    w.sub_(upd, alpha=lr)
    m.mul_(b2).add_(gi, alpha=1.0 - b2)


def _adamw_update_many(ws, gs, ms, vs, decay, lr, b1, b2, eps, wd, bc1, bc2, scale):
    """``_adamw_update`` over lists of tensors: the same operations in the same order, one multi-tensor call per operation
    instead of one call per tensor and operation (a step of a small model is mostly call overhead on a CPU)."""
    if not ws:
        return
    gi = torch._foreach_mul(gs, scale)
    torch._foreach_mul_(ms, b1)
    torch._foreach_add_(ms, gi, alpha=1.0 - b1)
    torch._foreach_mul_(vs, b2)
    torch._foreach_addcmul_(vs, gi, gi, value=1.0 - b2)
    den = torch._foreach_div(vs, bc2)
    torch._foreach_sqrt_(den)
    torch._foreach_add_(den, eps)
    upd = list(torch._foreach_div(torch._foreach_div(ms, bc1), den))
    if wd != 0.0:
        idx = [i for i, d in enumerate(decay) if d]
        if idx:
            dec = torch._foreach_add([upd[i] for i in idx], torch._foreach_mul([ws[i] for i in idx], wd))
            for i, t in zip(idx, dec):
                upd[i] = t
    torch._foreach_sub_(ws, upd, alpha=lr)


def _lion_update_many(ws, gs, ms, decay, lr, b1, b2, wd, scale):
    """``_lion_update`` over lists of tensors, operation by operation."""
    if not ws:
        return
    gi = torch._foreach_mul(gs, scale)
    c = torch._foreach_add(torch._foreach_mul(ms, b1), torch._foreach_mul(gi, 1.0 - b1))
    upd = list(torch._foreach_sign(c))
    if wd != 0.0:
        idx = [i for i, d in enumerate(decay) if d]
        if idx:
            dec = torch._foreach_add([upd[i] for i in idx], torch._foreach_mul([ws[i] for i in idx], wd))
            for i, t in zip(idx, dec):
                upd[i] = t
    torch._foreach_sub_(ws, upd, alpha=lr)
    torch._foreach_mul_(ms, b2)
    torch._foreach_add_(ms, gi, alpha=1.0 - b2)


class Optimizer:
    kind = "none"

    def __init__(self, params: List[OptParam]):
        self.params = params
        self.t = 0                     # applied updates (skipped steps do not count)
        self.last_grad_norm = 0.0

    def _begin(self, grad_scale: float, clip: float) -> Tuple[float, Optional[float]]:
        self.t += 1
        gnorm = global_grad_norm(self.params, grad_scale)
        self.last_grad_norm = gnorm
        if not math.isfinite(gnorm):
            self.t -= 1
            return gnorm, None
        return gnorm, float(_F32(grad_scale) * _F32(_clip_scale(gnorm, clip)))

    def _bias_corrections(self, b1, b2):
        return (float(_F32(1.0) - np.power(_F32(b1), _F32(self.t), dtype=_F32)),
                float(_F32(1.0) - np.power(_F32(b2), _F32(self.t), dtype=_F32)))


class AdamW(Optimizer):
    kind = "adamw"

    def __init__(self, params, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, grad_clip=1.0):
        super().__init__(params)
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.weight_decay, self.grad_clip = weight_decay, grad_clip
        self.m = [None if p.frozen else torch.zeros_like(p.w) for p in params]
        self.v = [None if p.frozen else torch.zeros_like(p.w) for p in params]

    @torch.no_grad()
    def step(self, lr: float, grad_scale: float = 1.0) -> float:
        gnorm, eff = self._begin(grad_scale, self.grad_clip)
        if eff is None:
            return gnorm
        bc1, bc2 = self._bias_corrections(self.beta1, self.beta2)
        live = [i for i, p in enumerate(self.params) if not p.frozen and p.grad is not None]
        _adamw_update_many([self.params[i].w for i in live], [self.params[i].grad for i in live], [self.m[i] for i in live],
                           [self.v[i] for i in live], [self.params[i].decay for i in live], lr, self.beta1, self.beta2,
                           self.eps, self.weight_decay, bc1, bc2, eff)
        return gnorm

    def hyper(self):
        return dict(lr=self.lr, beta1=self.beta1, beta2=self.beta2, eps=self.eps, weight_decay=self.weight_decay,
                    grad_clip=self.grad_clip)


class Lion(Optimizer):
    kind = "lion"

    def __init__(self, params, lr=3e-5, beta1=0.9, beta2=0.99, weight_decay=0.1, grad_clip=1.0):
        super().__init__(params)
        self.lr, self.beta1, self.beta2 = lr, beta1, beta2
        self.weight_decay, self.grad_clip = weight_decay, grad_clip
        self.m = [None if p.frozen else torch.zeros_like(p.w) for p in params]
        self.v = [None for _ in params]

    @torch.no_grad()
    def step(self, lr: float, grad_scale: float = 1.0) -> float:
        gnorm, eff = self._begin(grad_scale, self.grad_clip)
        if eff is None:
            return gnorm
        live = [i for i, p in enumerate(self.params) if not p.frozen and p.grad is not None]
        _lion_update_many([self.params[i].w for i in live], [self.params[i].grad for i in live], [self.m[i] for i in live],
                          [self.params[i].decay for i in live], lr, self.beta1, self.beta2, self.weight_decay, eff)
        return gnorm

    def hyper(self):
        return dict(lr=self.lr, beta1=self.beta1, beta2=self.beta2, weight_decay=self.weight_decay,
                    grad_clip=self.grad_clip)


def newton_schulz(G: torch.Tensor, steps: int) -> torch.Tensor:
    """Frobenius-normalise then iterate ``O <- 1.5 O - 0.5 O (O^T O)`` in fp32 (no transpose trick)."""
    O = G.float().clone()
    frob = float(O.double().pow(2).sum().sqrt())
    if not math.isfinite(frob) or frob < 1e-12:
        return O
    O.mul_(float(_F32(1.0 / frob)))
    for _ in range(steps):
        A = O.t() @ O
        O = 1.5 * O - 0.5 * (O @ A)
    return O


class Muon(Optimizer):
    kind = "muon"

    def __init__(self, params, lr=3e-4, vec_ratio=0.1, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                 grad_clip=1.0, ns_steps=5, min_ns_dim=0):
        super().__init__(params)
        self.lr, self.vec_ratio, self.beta1, self.beta2, self.eps = lr, vec_ratio, beta1, beta2, eps
        self.weight_decay, self.grad_clip = weight_decay, grad_clip
        self.ns_steps = min(10, max(1, ns_steps))
        self.min_ns_dim = min_ns_dim
        self.m, self.v = [], []
        for p in params:
            if p.frozen:
                self.m.append(None)
                self.v.append(None)
                continue
            self.m.append(torch.zeros_like(p.w))
            self.v.append(torch.zeros_like(p.w) if (not self.uses_ns(p) and p.w.dim() == 1) else None)

    def uses_ns(self, p: OptParam) -> bool:
        if p.frozen or p.w.dim() != 2 or not p.decay:
            return False
        if self.min_ns_dim <= 0:
            return True
        return min(p.w.shape) >= self.min_ns_dim

    @torch.no_grad()
    def step(self, lr: float, grad_scale: float = 1.0) -> float:
        gnorm, eff = self._begin(grad_scale, self.grad_clip)
        if eff is None:
            return gnorm
        bc1, bc2 = self._bias_corrections(self.beta1, self.beta2)
        vec_lr = float(_F32(lr) * _F32(self.vec_ratio))
        for i, p in enumerate(self.params):
            if p.frozen or p.grad is None:
                continue
            wd = self.weight_decay if p.decay else 0.0
            if self.uses_ns(p):
                self.m[i].mul_(self.beta1).add_(p.grad, alpha=eff * (1.0 - self.beta1))
                O = newton_schulz(self.m[i], self.ns_steps)
                p.w.add_(O, alpha=-lr)
                if wd != 0.0:
                    p.w.mul_(1.0 - lr * wd)
            elif p.w.dim() == 1:
                _adamw_update(p.w, p.grad, self.m[i], self.v[i], vec_lr, self.beta1, self.beta2, self.eps, wd, bc1,
                              bc2, eff)
            else:
                _lion_update(p.w, p.grad, self.m[i], vec_lr, self.beta1, self.beta2, wd, eff)
        return gnorm

    def hyper(self):
        return dict(lr=self.lr, vec_ratio=self.vec_ratio, beta1=self.beta1, beta2=self.beta2, eps=self.eps,
                    weight_decay=self.weight_decay, grad_clip=self.grad_clip, ns_steps=self.ns_steps,
                    min_ns_dim=self.min_ns_dim)


def make_optimizer(tcfg, params: List[OptParam]) -> Optimizer:
    """Build the optimizer a recipe names (Lion runs at a tenth of the recipe's learning rate)."""
    if tcfg.optimizer == "adamw":
        return AdamW(params, tcfg.learning_rate, tcfg.beta1, tcfg.beta2, tcfg.eps, tcfg.weight_decay, tcfg.grad_clip)
    if tcfg.optimizer == "lion":
        return Lion(params, tcfg.effective_peak_lr(), tcfg.beta1, tcfg.beta2, tcfg.weight_decay, tcfg.grad_clip)
    if tcfg.optimizer == "muon":
        return Muon(params, tcfg.learning_rate, tcfg.muon_vec_ratio, tcfg.beta1, tcfg.beta2, tcfg.eps,
                    tcfg.weight_decay, tcfg.grad_clip, tcfg.muon_ns_steps, tcfg.muon_min_ns_dim)
    raise ValueError(f"unknown optimizer {tcfg.optimizer}")


# ---------------------------------------------------------------------------------------- schedule
class LrScheduler:
    """Linear warm-up ``(step+1)/warmup`` then cosine to ``min_ratio`` or WSD (stable, then a linear decay over
    the last ``decay_frac`` of the post-warm-up steps).  float32 arithmetic throughout."""

    KINDS = {"cosine": 0, "wsd": 1}

    def __init__(self, peak, total, warmup, min_ratio=0.1, kind="cosine", decay_frac=0.2):
        self.peak, self.total, self.warmup = _F32(peak), int(total), int(warmup)
        self.min_ratio, self.kind, self.decay_frac = _F32(min_ratio), kind, _F32(decay_frac)

    def lr_at(self, step: int) -> float:
        if self.total <= 0:
            return float(self.peak)
        step = min(max(int(step), 0), self.total)
        if self.warmup > 0 and step < self.warmup:
            return float(self.peak * (_F32(step + 1) / _F32(self.warmup)))
        one = _F32(1.0)
        if self.kind == "wsd":
            stable_end = self.total - int(float(self.decay_frac) * float(self.total - self.warmup))
            stable_end = max(stable_end, self.warmup)
            if step < stable_end:
                return float(self.peak)
            decay_steps = self.total - stable_end
            if decay_steps <= 0:
                return float(self.peak)
            p = min(1.0, (step - stable_end) / decay_steps)
            return float(self.peak * (one - (one - self.min_ratio) * _F32(p)))
        decay_steps = self.total - self.warmup
        if decay_steps <= 0:
            return float(self.peak)
        t = min(step - self.warmup, decay_steps)
        progress = _F32(t) / _F32(decay_steps)
        cos_out = _F32(0.5) * (one + np.cos(_F32(3.14159265358979) * progress, dtype=_F32))
        return float(self.peak * (self.min_ratio + (one - self.min_ratio) * cos_out))


# ---------------------------------------------------------------------------------------- loss scaler
LOSS_SCALE_HARD_CAP = 16384.0


class LossScaler:
    """Dynamic loss scale: halve (floor 1) on a non-finite gradient norm, double after ``window`` clean steps up
    to ``min(loss_scale_max or inf, 16384)``.  Inactive (scale 1) when ``init <= 0`` or 16-bit GEMMs are off."""

    def __init__(self, init: float, window: int, max_scale: float = 0.0, active: bool = True):
        self.active = bool(active and init > 0)
        self.window = int(window)
        self.max_scale = float(max_scale)
        # the stored scale follows the recipe even while scaling is inactive (checkpoints record it)
        self.scale = min(float(init), self.cap()) if init > 0 else 1.0
        self.clean_steps = 0
        self.overflows = 0
        self.skipped = 0

    def cap(self) -> float:
        return LOSS_SCALE_HARD_CAP if not self.max_scale > 0 else min(self.max_scale, LOSS_SCALE_HARD_CAP)

    def for_step(self) -> float:
        if not self.active:
            return 1.0
        return float(_F32(min(self.scale, self.cap())))

    def update(self, gnorm: float) -> None:
        if not self.active:
            return
        if not math.isfinite(gnorm):
            self.scale = max(1.0, self.scale * 0.5)
            self.clean_steps = 0
            self.overflows += 1
        else:
            self.clean_steps += 1
            if self.clean_steps >= self.window:
                self.clean_steps = 0
                self.scale = min(self.cap(), self.scale * 2.0)
