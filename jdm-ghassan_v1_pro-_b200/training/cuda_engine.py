"""Training engine for a B200: drives :class:`CudaModel` and the flat-buffer optimizer kernels.

Same protocol as ``TorchEngine`` (begin_step / micro_step / end_step / eval_batch).  Differences that matter:

* one micro-batch = one CUDA-graph replay (captured after two eager warm-up runs), inputs staged from pinned
  host memory into static device buffers, per-launch scalars (loss scale, aux coefficient, jitter seed) in
  device memory so the captured graph follows them;
* the host reads back exactly one small record per optimizer step (gradient norm / skip flag, loss sum, token
  count, aux sum) instead of the reference's per-layer and per-tensor round trips
  (training/trainer.cpp:1476-1536, cuda/moe.cu:601-676, cuda/kernels.cu:1108-1128);
* gradients of all ranks are combined by ``parallel.grad_sync`` (peer-memory reduce-scatter fused with the
  optimizer and the parameter all-gather) or, with ``b200.grad_sync: nccl``, by one NCCL all-reduce.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.cuda_model import CudaModel
from ..ops import _lib
from ..ops import kernels as K
from ..utils import canary as CA
from ..utils.log import log_info, log_warn
from ..utils.telemetry import PERF
from . import optim as O
from .engine import (MOE_BIAS_CLAMP, MOE_BIAS_LR, DistInfo, StepResult, format_balance_report, jitter_seed_for,
                     moe_bias_update)

_F32 = np.float32


class _FlatOptimizer:
    """AdamW / Lion over the flat [no-decay | decay] layout; moments are flat fp32 buffers."""

    def __init__(self, kind, model: CudaModel, tcfg):
        self.kind = kind
        self.model = model
        self.t = 0
        self.beta1, self.beta2, self.eps = tcfg.beta1, tcfg.beta2, tcfg.eps
        self.weight_decay, self.grad_clip = tcfg.weight_decay, tcfg.grad_clip
        self.lr = tcfg.effective_peak_lr()
        n = model.layout.total
        self.m_flat = CA.zeros(n, dtype=torch.float32, device=model.dev, name="moment m")
        self.v_flat = CA.zeros(n, dtype=torch.float32, device=model.dev, name="moment v") if kind == "adamw" else None
        self.hyper_dev = torch.zeros(3, dtype=torch.float32, device=model.dev)
        self.hyper_host = torch.zeros(3, dtype=torch.float32).pin_memory()

    def hyper(self):
        h = dict(lr=self.lr, beta1=self.beta1, beta2=self.beta2, weight_decay=self.weight_decay, grad_clip=self.grad_clip)
        if self.kind == "adamw":
            h["eps"] = self.eps
        return h

    def launch(self, lr: float, scale_dev: torch.Tensor, lo: int = 0, hi: Optional[int] = None):
        """Update elements [lo, hi) of the flat buffers (both regions, each with its own weight decay)."""
        m = self.model
        hi = m.layout.total if hi is None else hi
        t = self.t + 1   # applied count if this step is accepted; a rejected step leaves everything untouched
        bc1 = float(_F32(1.0) - np.power(_F32(self.beta1), _F32(t), dtype=_F32))
        bc2 = float(_F32(1.0) - np.power(_F32(self.beta2), _F32(t), dtype=_F32))
        self.hyper_host[0], self.hyper_host[1], self.hyper_host[2] = lr, bc1, bc2
        self.hyper_dev.copy_(self.hyper_host, non_blocking=True)
        ds = m.layout.decay_start
        for a, b, wd in ((lo, min(hi, ds), 0.0), (max(lo, ds), hi, self.weight_decay)):
            if b > a:
                K.optimizer_step(self.kind, m.P[a:b], m.Gr[a:b], self.m_flat[a:b],
                                 None if self.v_flat is None else self.v_flat[a:b], m.W16[a:b], self.hyper_dev,
                                 scale_dev, self.beta1, self.beta2, self.eps, wd)


class CudaEngine:
    kind = "cuda"

    def __init__(self, mcfg: ModelConfig, tcfg, seed: Optional[int] = None, device=None, fused_sync_single=False):
        if not torch.cuda.is_available():
            raise RuntimeError("CudaEngine needs a CUDA device")
        if not _lib.available():
            raise RuntimeError("the sm_100a kernel library is not built: run `python -m ghassan_b200.build`")
        self.mcfg, self.tcfg = mcfg, tcfg
        self.dist = DistInfo()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.dtype = torch.bfloat16 if tcfg.operand_dtype() == "bf16" else torch.float16
        self.uses_loss_scaling = self.dtype == torch.float16 and tcfg.gemm_fp16
        micro = getattr(tcfg, "micro_tokens", 0)      # set by the trainer when it fuses micro-batches into one pass
        if micro and mcfg.use_moe and not _lib.lib().gb_moe_seg_ok(tcfg.batch_size * tcfg.seq_len, micro):
            log_warn("[cuda] micro-batches of %d tokens do not line up with the routing blocks: balance statistics and "
                     "router jitter are taken over the whole pass" % micro)
            micro = 0
        self.model = CudaModel(mcfg, tcfg.batch_size, tcfg.seq_len, self.dtype, self.device, tcfg.ce_chunks,
                               use_segments=tcfg.pack_sequences, train=True, micro_tokens=micro)
        self.model.init_weights(tcfg.seed if seed is None else seed)
        self.sync_model()
        self.muon = None
        if tcfg.optimizer == "muon":
            self.optimizer = self._make_muon()
        else:
            self.optimizer = _FlatOptimizer(tcfg.optimizer, self.model, tcfg)
        n = self.model.layout.total
        self.sq_partial = torch.zeros(K.sqnorm_blocks(n), dtype=torch.float64, device=self.device)
        self.norm_out = torch.zeros(4, dtype=torch.float32, device=self.device)   # [scale or 0, gnorm, -, -]
        self.gs_dev = torch.zeros(1, dtype=torch.float32, device=self.device)     # 1 / (ntok_global * loss_scale)
        self.ntok_dev = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.aux_weighted = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.readback = torch.zeros(6, dtype=torch.float64).pin_memory()
        # per-launch scalars go through a pinned ring with one slot per micro-batch of a step (plus slack): the copy is
        # asynchronous and nothing syncs the host between micro-batches, so a single pinned buffer would be rewritten
        # before an earlier micro-batch's copy has run.  end_step() synchronises once per step.
        self.dyn_ring = torch.zeros(max(4, tcfg.grad_accum + 2), self.model.dyn.numel(), dtype=torch.float32).pin_memory()
        self._dyn_slot = 0
        self.seed_host = torch.zeros(1, dtype=torch.int64).pin_memory()
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.eval_graph: Optional[torch.cuda.CUDAGraph] = None
        self._warm = 0
        self._ntok = 0
        self._loss_scale = 1.0
        self.weight_ema = torch.empty_like(self.model.P).copy_(self.model.P) if tcfg.weight_ema > 0 else None
        self.grad_sync = None
        fused_ok = tcfg.tokens_per_step_global(self.dist.world) < (1 << 24)
        if fused_ok and ((self.dist.world > 1 and tcfg.grad_sync == "fused") or fused_sync_single):
            from ..parallel.grad_sync import FusedGradSync
            # moves P / W16 / Gr (and routing counts) into symmetric memory
            self.grad_sync = FusedGradSync(self, nvls=bool(getattr(tcfg, "grad_sync_nvls", False)))
            if self.weight_ema is not None:
                self.weight_ema = torch.empty_like(self.model.P).copy_(self.model.P)
        self.expert_parallel = None
        if tcfg.ep_size > 1:
            if not mcfg.use_moe:
                raise ValueError("b200.ep_size > 1 needs a mixture-of-experts model")
            if tcfg.ep_size != self.dist.world:
                raise ValueError("b200.ep_size must equal the number of ranks (%d): the expert group is the whole job" % self.dist.world)
            self.expert_parallel = self.model.enable_expert_parallel(capacity=tcfg.ep_capacity)
        # routed slots per (layer, expert) since the last expert-load report (this rank's tokens)
        self.load_acc = (torch.zeros(mcfg.num_layers, mcfg.num_experts, dtype=torch.float64, device=self.device)
                         if mcfg.use_moe else None)
        self.last_step_ms = None
        self._ev0, self._ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.kernel_launches = 0
        log_info("[cuda] %s operands, %s activations+workspace, %s parameters (flat)" % (
            "bf16" if self.dtype == torch.bfloat16 else "fp16",
            _human(self.model.activation_bytes()), _human(n * 4)))

    # ------------------------------------------------------------------ distributed
    def sync_model(self):
        if self.dist.world > 1:
            self.dist.broadcast_(self.model.P, 0)
            if self.model.moe_bias is not None:
                self.dist.broadcast_(self.model.moe_bias, 0)
            self.model.refresh_shadows()

    # ------------------------------------------------------------------ muon (training/muon_cuda.py)
    def _make_muon(self):
        from .muon_cuda import MuonCuda
        return MuonCuda(self.model, self.mcfg, self.tcfg)

    # ------------------------------------------------------------------ step protocol
    def begin_step(self, step: int, loss_scale: float):
        m = self.model
        self._ev0.record()
        m.zero_grad()
        m.ce_acc.zero_()
        m.aux_acc.zero_()
        self.aux_weighted.zero_()
        if m.bias_counts is not None:
            m.bias_counts.zero_()
        self._ntok = 0
        self._loss_scale = float(loss_scale)
        seed = jitter_seed_for(self.tcfg.seed, step, self.dist.rank)
        self.seed_host[0] = seed - (1 << 64) if seed >= (1 << 63) else seed
        m.seed_dev.copy_(self.seed_host, non_blocking=True)

    def _run_micro(self):
        m = self.model
        freeze = self.tcfg.freeze_embeddings
        if not self.tcfg.cuda_graphs:
            m.forward_backward(freeze)
        elif self.graph is not None:
            self.graph.replay()
        elif self._warm < 2:
            m.forward_backward(freeze)
            self._warm += 1
        else:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):   # other threads (prefetch, checkpoint writer) may call CUDA
                m.forward_backward(freeze)
            self.graph = g
            g.replay()   # capture does not execute: run the micro-batch that triggered it
        self.kernel_launches += m.launches_per_micro_batch()

    def micro_step(self, ids, targets, segments, B, T):
        m = self.model
        ntok = int((targets.view(-1) >= 0).sum()) if not targets.is_cuda else int((targets >= 0).sum().item())
        if ntok == 0 and self.expert_parallel is None:
            return 0.0, 0    # nothing supervised: no forward/backward, no router counts
        # With experts divided among the ranks every layer holds peer barriers and row exchanges, so a rank may not
        # skip on its own: an all-masked micro-batch runs anyway (zero loss and gradient; its rows still serve the
        # peers' experts, and its routed slots do enter the balancing counts, unlike the skipped case above).
        cfg = self.mcfg
        dyn_host = self.dyn_ring[self._dyn_slot]
        self._dyn_slot = (self._dyn_slot + 1) % self.dyn_ring.shape[0]
        dyn_host.zero_()
        dyn_host[0] = self._loss_scale
        if cfg.use_moe:
            # per micro-batch of the pass: its supervised tokens weight its balance loss, and scale the coefficient
            # of that loss's gradient (the reference does both per micro-batch: training/trainer.cpp:1476-1490)
            n_seg = m.n_seg
            seg_ntok = ((targets.view(n_seg, -1) >= 0).sum(dim=1).to(torch.float32) if n_seg > 1
                        else torch.tensor([float(ntok)]))
            seg_tokens = float(B * T) / n_seg
            dyn_host[2:2 + n_seg] = seg_ntok.cpu() * (cfg.moe_aux_scale * self._loss_scale / cfg.num_layers *
                                                      cfg.num_experts / seg_tokens)
            dyn_host[2 + n_seg:2 + 2 * n_seg] = seg_ntok.cpu()
        m.dyn.copy_(dyn_host, non_blocking=True)
        m.set_inputs(ids, targets, segments)
        PERF.add("h2d_bytes", ids.numel() * 4 * (3 if m.use_segments else 2))
        self._run_micro()
        if cfg.use_moe and cfg.moe_aux_scale > 0:
            self.aux_weighted.add_(m.aux_acc)      # already weighted by each micro-batch's supervised tokens
            m.aux_acc.zero_()
        self._ntok += ntok
        return None, ntok

    def end_step(self, lr: float) -> StepResult:
        m, d, cfg = self.model, self.dist, self.mcfg
        ntok_global = self._ntok
        fused = self.grad_sync is not None
        if d.world > 1 and not fused:
            self.ntok_dev[0] = self._ntok
            d.all_reduce_sum_(self.ntok_dev)
            if m.bias_counts is not None:
                d.all_reduce_sum_(m.bias_counts)
        gnorm, applied = 0.0, False
        if d.world > 1 and not fused:
            ntok_global = int(self.ntok_dev.item())   # small host read; also orders the step on every rank
        if fused:
            # token count, routing counts, gradients, norm, clip, skip decision, optimizer and the parameter
            # all-gather are one kernel sequence; nothing is read on the host until the step's single read-back
            if self.tcfg.freeze_embeddings:
                m.g("tok_embeddings").zero_()
            self.grad_sync.step(lr, self._loss_scale, self._ntok)
        elif ntok_global > 0:
            grad_scale = float(_F32(1.0) / (_F32(ntok_global) * _F32(self._loss_scale)))
            if self.tcfg.freeze_embeddings:
                m.g("tok_embeddings").zero_()
            if d.world > 1:
                d.all_reduce_sum_(m.Gr)
            K.sqnorm_partial(m.Gr, self.sq_partial)
            K.finish_norm(self.sq_partial, self.sq_partial.numel(), None, grad_scale, self.tcfg.grad_clip, self.norm_out)
            self.optimizer.launch(lr, self.norm_out[0:1])      # AdamW / Lion flat kernel, or Muon (NS on the GEMM)
        if self.load_acc is not None and m.bias_counts is not None:
            self.load_acc.add_(m.bias_counts)      # this rank's counts (the fused exchange keeps the global sum apart)
        # ---- the one host read-back of the step
        self._ev1.record()
        norm_src = self.grad_sync.out if fused else self.norm_out
        rb = torch.cat([norm_src[:2].double(), m.ce_acc, self.aux_weighted.double(), norm_src[2:3].double()])
        self.readback[:6].copy_(rb, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        PERF.add("sync")
        PERF.add("d2h_bytes", 40)
        _lib.check_status(self.device, "training step")
        self.last_step_ms = self._ev0.elapsed_time(self._ev1)
        _, gn, loss_sum, rows, aux_w, ntok_dev = (float(x) for x in self.readback[:6])
        if fused:
            ntok_global = int(round(ntok_dev))
        if ntok_global > 0:
            gnorm = gn
            applied = math.isfinite(gnorm)
            if applied:
                self.optimizer.t += 1
        loss = 0.0
        if self._ntok > 0:
            loss = loss_sum / self._ntok
            if cfg.use_moe and cfg.moe_aux_scale > 0:
                loss += cfg.moe_aux_scale * aux_w / cfg.num_layers / self._ntok
        if m.moe_bias is not None and applied:
            moe_bias_update(m.moe_bias, self.grad_sync.counts_global if fused else m.bias_counts)
        if applied and self.weight_ema is not None:
            if fused and self.tcfg.optimizer != "muon":   # master current on the owned shard only; checkpoints gather
                own = slice(self.grad_sync.lo, self.grad_sync.hi)
                self.weight_ema[own].lerp_(m.P[own], 1.0 - self.tcfg.weight_ema)
            else:
                self.weight_ema.lerp_(m.P, 1.0 - self.tcfg.weight_ema)
        PERF.add("opt_steps")
        return StepResult(loss, self._ntok, ntok_global, gnorm, applied)

    @torch.no_grad()
    def eval_batch(self, ids, targets, segments, B, T):
        m = self.model
        m.ce_acc.zero_()
        m.set_inputs(ids, targets, segments)
        m.forward(False)
        acc = m.ce_acc.cpu()
        return float(acc[0]), int(acc[1])

    def balance_report(self) -> str:
        """Expert-load line for the evaluation log (model/model.cpp:107-127 in the reference); resets the counts."""
        if self.load_acc is None:
            return ""
        rep = format_balance_report(self.load_acc, self.mcfg.num_experts)
        self.load_acc.zero_()
        return rep

    # ------------------------------------------------------------------ checkpoint state
    def prepare_export(self):
        """Collective: every rank calls this before rank 0 captures a checkpoint."""
        if self.grad_sync is not None:
            self.grad_sync.gather_full_state()

    def finish_export(self):
        """After the snapshot was captured: drop what prepare_export() gathered only for it."""
        if self.grad_sync is not None:
            self.grad_sync.release_full_state()

    def export_weights(self) -> List:
        named = self.model.export_named()
        return [(s.name, named[s.name]) for s in self.mcfg.param_specs()]

    def import_weights(self, named: Dict[str, np.ndarray], strict=True) -> List[str]:
        missing = self.model.load_named(named, missing_ok=not strict)
        return missing

    def export_moe_bias(self):
        if self.model.moe_bias is None:
            return []
        return [np.ascontiguousarray(r.cpu().numpy()) for r in self.model.moe_bias]

    def import_moe_bias(self, rows):
        if self.model.moe_bias is None:
            return
        for l, r in enumerate(rows):
            self.model.moe_bias[l].copy_(torch.as_tensor(np.asarray(r, dtype=np.float32)))

    def export_optimizer(self) -> dict:
        """Moments in the reference's per-parameter order and layout (replicated view of the flat state)."""
        opt = self.optimizer
        specs = self.mcfg.param_specs()
        if self.tcfg.optimizer == "muon":
            return opt.export_state()
        if opt.m_flat is None:
            raise RuntimeError("the moments are sharded over the ranks: prepare_export() must run first (rank 0 exports)")
        m_named = self.model.export_named(opt.m_flat)
        v_named = self.model.export_named(opt.v_flat) if opt.v_flat is not None else None
        if self.grad_sync is not None:
            self.grad_sync.release_full_state()
        return {"kind": opt.kind, "t": int(opt.t), "hyper": {k: float(v) for k, v in opt.hyper().items()},
                "m": [m_named[s.name].reshape(-1) for s in specs],
                "v": [v_named[s.name].reshape(-1) if v_named is not None else None for s in specs], "fmt": 1}

    def import_optimizer(self, blob: dict) -> bool:
        opt = self.optimizer
        specs = self.mcfg.param_specs()
        if blob is None or blob.get("kind") != opt.kind or len(blob["m"]) != len(specs):
            return False
        if self.tcfg.optimizer == "muon":
            return opt.import_state(blob)
        else:
            for i, s in enumerate(specs):
                if blob["m"][i] is not None and blob["m"][i].size != s.numel:
                    return False
            sharded = self.grad_sync is not None and self.grad_sync.m_own is not None
            n = self.model.layout.total
            m_flat = torch.zeros(n, dtype=torch.float32, device=self.device) if sharded else opt.m_flat
            has_v = opt.kind == "adamw"
            v_flat = (torch.zeros(n, dtype=torch.float32, device=self.device) if sharded else opt.v_flat) if has_v else None
            self.model.layout.to_internal({s.name: blob["m"][i].reshape(s.shape) for i, s in enumerate(specs)
                                           if blob["m"][i] is not None}, m_flat, missing_ok=True)
            if v_flat is not None:
                self.model.layout.to_internal({s.name: blob["v"][i].reshape(s.shape) for i, s in enumerate(specs)
                                               if blob["v"][i] is not None}, v_flat, missing_ok=True)
            if sharded:                  # every rank reads the whole state and keeps its own slice
                self.grad_sync.load_full_moments(m_flat, v_flat)
        opt.t = int(blob["t"])
        h = blob["hyper"]
        opt.beta1, opt.beta2 = float(h["beta1"]), float(h["beta2"])
        if "eps" in h:
            opt.eps = float(h["eps"])
        return True

    def optimizer_hyper(self) -> dict:
        return self.optimizer.hyper()

    def set_opt_step(self, t: int):
        self.optimizer.t = int(t)


def _human(n):
    from ..utils.log import human_bytes
    return human_bytes(n)
