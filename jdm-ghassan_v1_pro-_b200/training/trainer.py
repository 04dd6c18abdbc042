"""Training loop: schedule, loss scaling, gradient accumulation, evaluation, checkpoints, resume gates.

The loop, its guards and its log lines follow the reference trainer (training/trainer.cpp:382-1028 for
construction and resume, :1316-1594 for the loop, :1179-1207 for the step line) while the heavy work is
delegated to an engine (``TorchEngine`` on CPU, ``CudaEngine`` on a B200).  Step times are measured
on the device (CUDA events) when a GPU engine is used and reported next to the host wall time.
"""
from __future__ import annotations

import dataclasses
import json
import math
import os
import time
from typing import Optional

import numpy as np
import torch

from ..data.loader import RANK_SEED_STRIDE, DataLoader, Prefetcher, state_from_dict, state_to_dict
from ..models.config import ModelConfig
from ..utils.log import (human_bytes, human_count, human_duration, log_debug, log_error, log_info, log_warn)
from ..parallel.watchdog import PeerFailure, StepWatchdog
from ..utils.telemetry import PERF, STOP, PhaseTimers
from . import checkpoint as C
from .config import TrainerConfig
from .optim import LossScaler, LrScheduler


class TrainerError(RuntimeError):
    pass


def _rel_same(a: float, b: float, tol=1e-6) -> bool:
    return abs(a - b) <= tol * abs(a) + 1e-30


class Trainer:
    def __init__(self, mcfg: ModelConfig, tcfg: TrainerConfig, engine=None, device: Optional[str] = None):
        self.mcfg, self.cfg = mcfg, tcfg
        self._check_ranges()
        self.fuse = 1
        self.segments = 1          # row slices a micro-batch is run in (training.ckpt_segments), see _pick_segments
        self.engine = engine if engine is not None else self._make_engine(device)
        self.dist = self.engine.dist
        self.rank, self.world = self.dist.rank, self.dist.world
        self.state = C.TrainState(seed=tcfg.seed, tok_vocab=mcfg.vocab_size, tok_fingerprint=tcfg.tok_fingerprint,
                                  ddp_world=self.world)
        scaling = tcfg.loss_scale_init > 0 and getattr(self.engine, "uses_loss_scaling", False)
        self.scaler = LossScaler(tcfg.loss_scale_init, tcfg.loss_scale_window, tcfg.loss_scale_max, active=scaling)
        log_info("[prec] loss_scaling=%s (init %.0f, scaler now %.0f)" % (
            "ENABLED (fp16 GEMMs active)" if scaling else "DISABLED", tcfg.loss_scale_init, self.scaler.for_step()))
        self.ema_loss = 0.0
        self.skipped_steps = 0
        self.total_steps = 0
        self.stopped_by_signal = False
        self.heartbeat = None           # set by run() when there are peers (parallel/watchdog.py)
        self.phases = PhaseTimers(cuda=getattr(self.engine, "kind", "") == "cuda")
        self.writer = C.CheckpointWriter()
        self.jsonl_path = os.environ.get("GB200_JSONL", "")
        self._snapshot_cache = None
        self._open_loaders()
        self._preflight()
        self._resume()

    # ------------------------------------------------------------------ construction helpers
    def _check_ranges(self):
        c = self.cfg
        if c.batch_size <= 0 or c.seq_len <= 0 or c.grad_accum <= 0:
            raise TrainerError("batch_size, seq_len and grad_accum must be positive")
        if c.seq_len > self.mcfg.max_seq_len:
            raise TrainerError(f"training.seq_len {c.seq_len} exceeds model.max_seq_len {self.mcfg.max_seq_len}")
        if c.ddp_grad_compression:
            raise TrainerError("training.ddp_grad_compression is not supported (gradients are exchanged exactly)")
        if not (0.0 < c.sched_decay_frac <= 1.0):
            raise TrainerError("training.sched_decay_frac must be in (0,1]")

    def _preflight(self, probe=None):
        """Host RAM, free disk and output quota before anything is trained (training/guards.py); the device-memory
        guard ran in _make_engine, ahead of the allocations."""
        from . import guards
        c = self.cfg
        try:
            guards.preflight(self.mcfg.count_parameters(), c.optimizer, c.checkpoint_dir, c.output_budget_mb,
                             self.writer.budget, probe=probe, main=self.is_main(),
                             pretrained=c.pretrained_checkpoint if c.stage == "sft" else "")
        except guards.GuardError as e:
            raise TrainerError(str(e)) from None

    def _make_engine(self, device):
        dev = device or self.cfg.device
        if dev == "auto":
            dev = "cuda" if torch.cuda.is_available() else "cpu"
        if dev == "cuda":
            from .cuda_engine import CudaEngine
            self.fuse = self._pick_fuse()
            self.segments = self._pick_segments()
            ecfg = self.cfg
            if self.segments > 1:
                ecfg = dataclasses.replace(self.cfg, batch_size=self.cfg.batch_size // self.segments,
                                           grad_accum=self.cfg.grad_accum * self.segments)
            if self.fuse > 1:
                ecfg = dataclasses.replace(self.cfg, batch_size=self.cfg.batch_size * self.fuse,
                                           grad_accum=self.cfg.grad_accum // self.fuse)
                ecfg.micro_tokens = self.cfg.batch_size * self.cfg.seq_len   # MoE statistics stay per micro-batch
                log_info("[cuda] %d micro-batches of %d x %d tokens run as one pass of %d tokens (%d passes per step)" % (
                    self.fuse, self.cfg.batch_size, self.cfg.seq_len, ecfg.batch_size * ecfg.seq_len, ecfg.grad_accum))
            from . import guards
            from .memory_plan import memory_plan
            world = int(os.environ.get("WORLD_SIZE", "1") or 1)
            try:
                guards.check_device_memory(memory_plan(self.mcfg, self.cfg, world, self.fuse)["total"],
                                           int(torch.cuda.memory_allocated()), world, guards.Probe(), True)
            except guards.GuardError as e:
                raise TrainerError(str(e)) from None
            return CudaEngine(self.mcfg, ecfg)
        if dev != "cpu":
            log_warn(f"device '{dev}' is not supported; falling back to cpu")
        from .engine import TorchEngine
        self.segments = self._pick_segments()
        return TorchEngine(self.mcfg, self.cfg, "cpu")

    def _pick_segments(self) -> int:
        """``training.activation_checkpointing`` with ``ckpt_segments: S`` runs every micro-batch as S row slices one
        after another (the reference's "checkpointing" is this segmenting, not recomputation:
        training/trainer.cpp:1122-1146): same gradient sum, 1/S of the activation memory.  When micro-batches are
        fused into larger passes instead, the pass size is already chosen by the memory plan and the key has nothing
        left to do; that is logged, not silent."""
        c = self.cfg
        if not c.activation_checkpointing or c.ckpt_segments <= 1:
            return 1
        if self.fuse > 1:
            log_info("[ckpt] ckpt_segments=%d not applied: %d micro-batches already run as one pass whose size the "
                     "memory plan chose (b200.fuse_micro_batches: 1 brings segmenting back)" % (c.ckpt_segments, self.fuse))
            return 1
        if c.batch_size % c.ckpt_segments:
            log_warn("[ckpt] ckpt_segments=%d does not divide batch_size=%d: micro-batches run unsegmented" % (
                c.ckpt_segments, c.batch_size))
            return 1
        log_info("[ckpt] every micro-batch runs as %d slices of %d sequences" % (c.ckpt_segments, c.batch_size // c.ckpt_segments))
        return c.ckpt_segments

    def _pick_fuse(self) -> int:
        """How many of the recipe's micro-batches one forward/backward pass covers.  The gradient of a step is a sum
        over its micro-batches, so running F of them as one batch of F*batch_size rows gives the same sum with F times
        fewer, F times larger kernels.  What the reference defines per micro-batch stays per micro-batch inside the
        pass: the MoE kernels keep the balance statistics (mean router probability, routed share) and the token index
        of the router-jitter hash per segment of batch_size x seq_len tokens (``micro_tokens``)."""
        c = self.cfg
        f = c.fuse_micro_batches
        if f <= 0:
            # auto: the largest divisor of grad_accum whose pass stays within a token cap and whose predicted memory
            # (closed form of cli/train.py) fits the device with room to spare.  Measured on pro_1b, one B200:
            # 113.6 k tokens/s at 8192 tokens per pass, 122.7 k at 16384, 126.7 k at 32768 (activations 80 GB).
            from .memory_plan import memory_plan
            total = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory if torch.cuda.is_available() else 0
            cap = 32768 if total >= 120 * (1 << 30) else 8192
            if c.ep_size > 1:
                cap = 8192          # the expert-parallel receive buffers grow with the pass and are not in the plan
            world = 1               # the plan does not shrink with the number of ranks
            f = 1
            for cand in range(1, min(c.grad_accum, 64) + 1):
                if c.grad_accum % cand or c.batch_size * cand * c.seq_len > cap:
                    continue
                if cand > 1 and total and memory_plan(self.mcfg, c, world, cand)["total"] > 0.6 * total:
                    continue
                f = cand
        if c.grad_accum % f:
            raise TrainerError("b200.fuse_micro_batches=%d must divide training.grad_accum=%d" % (f, c.grad_accum))
        return f

    def _fused(self, batches):
        """Concatenate up to ``self.fuse`` loader batches into one pinned buffer triple (missing rows unsupervised)."""
        if self.fuse == 1:
            b = batches[0]
            return b.ids, b.targets, b.segments, b.B, b.T
        c = self.cfg
        n = c.batch_size * c.seq_len
        if not hasattr(self, "_fuse_ring"):
            pin = torch.cuda.is_available()
            mk = lambda: (torch.zeros(self.fuse * n, dtype=torch.int32).pin_memory() if pin
                          else torch.zeros(self.fuse * n, dtype=torch.int32))
            self._fuse_ring = [(mk(), mk(), mk()) for _ in range(c.grad_accum // self.fuse + 3)]
            self._fuse_pos = 0
        ids, tg, sg = self._fuse_ring[self._fuse_pos]
        self._fuse_pos = (self._fuse_pos + 1) % len(self._fuse_ring)
        for j, b in enumerate(batches):
            ids[j * n:(j + 1) * n].copy_(b.ids.view(-1))
            tg[j * n:(j + 1) * n].copy_(b.targets.view(-1))
            sg[j * n:(j + 1) * n].copy_(b.segments.view(-1))
        if len(batches) < self.fuse:
            tg[len(batches) * n:].fill_(-100)
            ids[len(batches) * n:].zero_()
            sg[len(batches) * n:].zero_()
        return ids, tg, sg, c.batch_size * self.fuse, c.seq_len

    def _open_loaders(self):
        c = self.cfg
        seed = (c.seed + self.rank * RANK_SEED_STRIDE) & (2 ** 64 - 1)
        self.train_loader = DataLoader(c.batch_size, c.seq_len, c.pack_sequences, seed, self.mcfg.vocab_size)
        ok = False
        if c.mix:
            ok = self.train_loader.open_mix(c.data_dir, c.mix)
            if not ok:
                raise TrainerError(f"data.mix is configured but no matching shards (train_<domain>_*.gbin) exist in {c.data_dir}")
            log_info("[data] " + self.train_loader.mix_report())
        else:
            ok = self.train_loader.open_glob(c.data_dir, c.train_prefix)
        if not ok:
            raise TrainerError(f"no training shards found in {c.data_dir} (prefix '{c.train_prefix}')")
        if c.stage == "sft" and not self.train_loader.all_have_mask:
            raise TrainerError("SFT needs shards with loss masks (assistant spans)")
        self.val_loader = DataLoader(c.batch_size, c.seq_len, c.pack_sequences, (c.seed + 1) & (2 ** 64 - 1),
                                     self.mcfg.vocab_size)
        self.have_val = self.val_loader.open_glob(c.data_dir, c.val_prefix)
        if getattr(self.engine, "kind", "") == "cuda":
            self.train_loader.set_ring(c.grad_accum + 6)
            self.val_loader.set_ring(4)
        self.prefetch = Prefetcher(self.train_loader)
        log_info("[data] %d train shard(s), %s tokens%s" % (self.train_loader.num_shards,
                                                          human_count(self.train_loader.total_tokens),
                                                          "" if self.have_val else " (no validation shards)"))

    # ------------------------------------------------------------------ resume
    def _resume(self):
        c = self.cfg
        if c.stage == "sft" and c.pretrained_checkpoint:
            self._load_pretrained(c.pretrained_checkpoint)
        elif c.stage == "sft" and not c.allow_no_pretrained and c.resume == "none":
            raise TrainerError("SFT needs training.pretrained_checkpoint (or allow_no_pretrained: true)")
        path = ""
        if c.resume == "auto":
            path = C.latest_in(c.checkpoint_dir)
        elif c.resume != "none":
            path = c.resume
        if not path or not os.path.exists(path):
            return
        exact = c.resume_exact()
        log_info(f"[ckpt] resume_mode={c.resume_mode} from {path}")
        pk = C.peek(path)
        if pk is not None:
            ck, st, _ = pk
            cur = self.mcfg
            math_same = all(getattr(ck, k) == getattr(cur, k) for k in (
                "rope_theta", "rope_scale", "rope_yarn_mscale", "rope_yarn_low", "rope_yarn_high", "rope_type",
                "rms_eps", "max_seq_len", "sliding_window", "moe_aux_free"))
            if not math_same and not c.allow_recipe_drift:
                raise TrainerError("resume recipe drift: checkpoint was saved with different math (rope/yarn/type, "
                                   "sliding_window, aux_free, rms_eps, max_seq_len); restore the original recipe or "
                                   "pass --allow-recipe-drift")
            if not math_same:
                log_warn("[ckpt] resuming WITH recipe drift (--allow-recipe-drift): numerics differ from save time")
            same, why = ck.same_architecture_as(cur)
            if not same and exact:
                raise TrainerError(f"exact resume refused: checkpoint architecture differs: {why}")
            if not same:
                log_warn(f"[ckpt] resuming WITH architecture drift (migrate): {why}")
            if st.tok_fingerprint and c.tok_fingerprint and st.tok_fingerprint != c.tok_fingerprint:
                raise TrainerError("tokenizer mismatch: checkpoint was trained with a different .gtok "
                                   "(fingerprint %016x vs %016x)" % (st.tok_fingerprint, c.tok_fingerprint))
            if not st.tok_fingerprint and c.tok_fingerprint:
                if exact:
                    raise TrainerError("exact resume refused: checkpoint predates tokenizer fingerprints")
                log_warn("[ckpt] checkpoint predates tokenizer fingerprints: cannot verify the tokenizer identity")
            if st.sched_total > 0:
                want_peak = c.effective_peak_lr()
                kind = 1 if c.scheduler == "wsd" else 0
                same_s = (st.sched_kind == kind and _rel_same(st.sched_peak, want_peak) and
                          st.sched_warmup == c.warmup_steps and abs(st.sched_min_ratio - c.min_lr_ratio) <= 1e-9 and
                          abs(st.sched_decay_frac - c.sched_decay_frac) <= 1e-9)
                if not same_s:
                    why = ("scheduler recipe differs from the checkpoint: ckpt(kind=%d peak=%.6e warmup=%d min=%.4f "
                           "decay=%.4f) vs cur(kind=%d peak=%.6e warmup=%d min=%.4f decay=%.4f)" % (
                               st.sched_kind, st.sched_peak, st.sched_warmup, st.sched_min_ratio, st.sched_decay_frac,
                               kind, want_peak, c.warmup_steps, c.min_lr_ratio, c.sched_decay_frac))
                    if exact:
                        raise TrainerError("exact resume: " + why)
                    log_warn("[ckpt] resuming WITH scheduler drift: " + why)
        ok, moments = self._load_checkpoint(path, strict=exact)
        if not ok and exact:
            raise TrainerError(f"exact resume rejected: {path} is not an exact continuation of this recipe")
        if not ok:
            self.state = C.TrainState(seed=c.seed, tok_vocab=self.mcfg.vocab_size, tok_fingerprint=c.tok_fingerprint,
                                      ddp_world=self.world)
            self.engine.set_opt_step(0)
            log_warn(f"[ckpt] failed to load {path}; starting from scratch")
            return
        if not moments:
            self.engine.set_opt_step(0)
            log_warn("[ckpt] moments NOT restored (kind switch/corrupt/legacy); optimizer t=0 with weights at step %d"
                     % self.state.step)
        self.train_loader.set_state(state_from_dict(self.state.loader))
        self.prefetch.last_consumed_state = self.train_loader.get_state()
        if self.have_val and self.state.val_loader.get("batches", -1) >= 0:
            self.val_loader.set_state(state_from_dict(self.state.val_loader))
        if self.scaler.active and self.state.loss_scale >= 1.0:
            self.scaler.scale = float(self.state.loss_scale)
            self.scaler.clean_steps = int(self.state.clean_steps)
        saved_ws = self.state.ddp_world if self.state.ddp_world > 0 else 1
        if self.world > 1 or saved_ws > 1:
            if saved_ws != self.world:
                raise TrainerError("DDP resume world mismatch: checkpoint saved with %d ranks but now %d" % (
                    saved_ws, self.world))
            if self.rank > 0:
                # only rank 0's stream is stored; the others replay theirs from the seed
                nb = int(self.state.loader["batches"])
                self.train_loader.reseed((c.seed + self.rank * RANK_SEED_STRIDE) & (2 ** 64 - 1))
                if nb > 0:
                    self.train_loader.skip_batches(nb)
                self.prefetch.last_consumed_state = self.train_loader.get_state()
        log_info("[ckpt] resumed from %s at step %d (%s tokens seen, scaler %.0f)" % (
            path, self.state.step, human_count(self.state.tokens_seen), self.scaler.scale))

    def _load_pretrained(self, path):
        if not os.path.exists(path):
            if self.cfg.allow_no_pretrained:
                log_warn(f"[sft ] pretrained checkpoint {path} not found; training from the initialisation")
                return
            raise TrainerError(f"pretrained checkpoint not found: {path}")
        pk = C.peek(path)
        if pk is None:
            raise TrainerError(f"cannot read pretrained checkpoint: {path}")
        same, why = pk[0].same_architecture_as(self.mcfg)
        if not same:
            raise TrainerError(f"pretrained checkpoint does not match the SFT recipe: {why}")
        d = C.read(path, with_optimizer=False)
        self.engine.import_weights(dict(d["params"]))
        if d["moe_bias"]:
            self.engine.import_moe_bias(d["moe_bias"])
        log_info(f"[sft ] initialised from {path}")

    def _load_checkpoint(self, path, strict):
        """Returns (ok, moments_restored)."""
        try:
            d = C.read(path)
        except Exception as e:
            log_error(f"[ckpt] cannot read {path}: {e}")
            return False, False
        ck = C.config_from_dict(d["config"])
        cur = self.mcfg
        struct = ("vocab_size", "hidden_size", "num_layers", "num_heads", "num_kv_heads", "intermediate_size",
                  "tie_embeddings", "use_moe", "num_experts", "moe_top_k", "moe_expert_dim", "moe_shared", "use_qk_norm")
        if any(getattr(ck, k) != getattr(cur, k) for k in struct):
            log_error("checkpoint architecture does not match the current model config")
            return False, False
        st = C.TrainState.from_dict(d["state"])
        if st.tok_vocab not in (0, cur.vocab_size):
            log_error("checkpoint vocab %d != model vocab %d; refusing resume" % (st.tok_vocab, cur.vocab_size))
            return False, False
        if not d["payload_finite"]:
            if strict:
                log_error("exact resume: checkpoint tensor '%s' contains non-finite payload" % d["first_nonfinite"])
                return False, False
            log_warn("checkpoint tensor '%s' contains non-finite payload (corrupt file?)" % d["first_nonfinite"])
        named = dict(d["params"])
        specs = {s.name: s.numel for s in cur.param_specs()}
        for n, a in named.items():
            if n not in specs or specs[n] != a.size:
                log_error("checkpoint tensor mismatch: " + n)
                return False, False
        missing = [n for n in specs if n not in named]
        if missing and strict:
            log_error("exact resume: checkpoint lacks param " + missing[0])
            return False, False
        for n in missing:
            log_warn(f"checkpoint lacks param {n}; keeping fresh init")
        for row in d["moe_bias"]:
            if not np.all(np.isfinite(row)) or len(row) != cur.num_experts:
                return False, False
        self.engine.import_weights(named, strict=False)
        if d["moe_bias"]:
            self.engine.import_moe_bias(d["moe_bias"])
        moments = False
        blob = d["optimizer"]
        if d["has_optimizer"]:
            if blob is None:
                if strict:
                    log_error("exact resume: optimizer state unreadable")
                    return False, False
                log_warn("optimizer state could not be restored; continuing with fresh moments")
            elif blob["kind"] != self.engine.optimizer.kind:
                if strict:
                    log_error("exact resume: checkpoint holds a different optimizer kind")
                    return False, False
                log_warn("checkpoint holds %s moments but trainer uses %s; starting fresh moments" % (
                    blob["kind"], self.engine.optimizer.kind))
            else:
                if strict and not self._hyper_same(blob):
                    return False, False
                moments = self.engine.import_optimizer(blob)
                if not moments and strict:
                    log_error("exact resume: optimizer state does not fit the parameter table")
                    return False, False
        if d["trailing_bytes"]:
            if strict:
                log_error("exact resume: checkpoint has trailing bytes after the optimizer state")
                return False, False
            log_warn("[ckpt] checkpoint has trailing bytes after the optimizer state (ignored)")
        self.state = st
        return True, moments

    def _hyper_same(self, blob) -> bool:
        cur = self.engine.optimizer_hyper()
        h = blob["hyper"]
        keys = [k for k in ("beta1", "beta2", "eps", "weight_decay", "grad_clip", "vec_ratio") if k in cur and k in h]
        for k in keys:
            if abs(float(h[k]) - float(cur[k])) > 1e-9 * (1 + abs(float(h[k]))):
                log_error("exact resume: %s hyperparams differ from checkpoint (%s: %g vs %g)" % (
                    blob["kind"], k, h[k], cur[k]))
                return False
        if "ns_steps" in cur and int(h.get("ns_steps", cur["ns_steps"])) != int(cur["ns_steps"]):
            log_error("exact resume: muon ns_steps differ from checkpoint")
            return False
        if "min_ns_dim" in h and "min_ns_dim" in cur and int(h["min_ns_dim"]) != int(cur["min_ns_dim"]):
            log_error("exact resume: muon min_ns_dim differs from checkpoint")
            return False
        return True

    # ------------------------------------------------------------------ schedule
    def _plan_schedule(self):
        c, st = self.cfg, self.state
        if c.max_steps > 0:
            self.total_steps = c.max_steps
            log_info("[sched] steps mode: %d optimizer steps (per-rank %s tok/step, global %s tok/step x%d)" % (
                self.total_steps, human_count(c.tokens_per_step_local()), human_count(c.tokens_per_step_global(self.world)),
                self.world))
        else:
            self.total_steps = c.epoch_steps(self.train_loader.total_tokens, self.world)
            if self.total_steps <= 0:
                raise TrainerError("epochs mode needs data: no training tokens found in " + c.data_dir)
            log_info("[sched] epochs mode: %d epochs x %s tokens = %d steps" % (
                c.epochs, human_count(self.train_loader.total_tokens), self.total_steps))
        exact = c.resume_exact()
        if exact and st.sched_total > 0 and st.sched_total != self.total_steps:
            raise TrainerError("exact resume refused: checkpoint planned total %d steps but this session budgets %d" % (
                st.sched_total, self.total_steps))
        if st.sched_total > 0 and st.sched_total > self.total_steps:
            log_warn("[sched] continuation: keeping the checkpoint's %d-step plan (this session stops early)" % st.sched_total)
            self.total_steps = st.sched_total
            if not c.warmup_steps < self.total_steps:
                c.warmup_steps = max(1, self.total_steps // 10)
        if not (0 <= c.warmup_steps < self.total_steps):
            raise TrainerError("training.warmup_steps=%d must be in [0,total=%d)" % (c.warmup_steps, self.total_steps))
        peak = c.effective_peak_lr()
        self.sched = LrScheduler(peak, self.total_steps, c.warmup_steps, c.min_lr_ratio, c.scheduler, c.sched_decay_frac)
        log_info("[sched] %s warmup %d total %d min %.0f%% decay_frac %.2f" % (
            c.scheduler, c.warmup_steps, self.total_steps, c.min_lr_ratio * 100.0, c.sched_decay_frac))
        checks = [(st.sched_total > 0 and st.sched_total != self.total_steps, "planned total %d but now %d" % (st.sched_total, self.total_steps)),
                  (st.sched_warmup > 0 and st.sched_warmup != c.warmup_steps, "warmup %d but now %d" % (st.sched_warmup, c.warmup_steps)),
                  (st.sched_peak > 0 and abs(st.sched_peak - peak) > 1e-9, "peak %.3e but now %.3e" % (st.sched_peak, peak))]
        for bad, why in checks:
            if bad:
                if exact:
                    raise TrainerError("exact resume refused: [sched] RESUME MISMATCH: checkpoint " + why)
                log_warn("[sched] RESUME MISMATCH: checkpoint " + why)
        st.sched_total, st.sched_warmup, st.sched_peak = self.total_steps, c.warmup_steps, float(np.float32(peak))
        st.sched_min_ratio, st.sched_decay_frac = c.min_lr_ratio, c.sched_decay_frac
        st.sched_kind = 1 if c.scheduler == "wsd" else 0
        st.ddp_world = self.world

    # ------------------------------------------------------------------ evaluation / saving
    def evaluate(self, max_batches: int) -> float:
        if not self.have_val:
            return 0.0
        total, ntok = 0.0, 0
        left = max_batches
        while left > 0:
            group = [self.val_loader.next() for _ in range(min(self.fuse, left))]
            left -= len(group)
            s, n = self.engine.eval_batch(*self._fused(group))
            total += s
            ntok += n
        return total / ntok if ntok > 0 else 0.0

    def is_main(self) -> bool:
        return self.rank == 0

    def save(self, name: str):
        """Snapshot on rank 0 (loader quiesced so its cursor equals the consumed batches), publish in background."""
        ok = torch.ones(1, dtype=torch.uint8)
        prep = getattr(self.engine, "prepare_export", None)
        if prep is not None:
            prep()          # sharded state is completed on every rank before rank 0 captures it
        if self.is_main():
            try:
                self.prefetch.quiesce()
                self.state.loader = state_to_dict(self.prefetch.last_consumed_state)
                self.state.val_loader = state_to_dict(self.val_loader.get_state()) if self.have_val else \
                    {"rng": (0, 0, 0, 0), "batches": -1, "rng_spare": 0.0, "rng_has_spare": 0}
                self.state.loss_scale = float(self.scaler.scale)
                self.state.clean_steps = int(self.scaler.clean_steps)
                if self._snapshot_cache is None or self._snapshot_cache[0] != self.state.step:
                    self._snapshot_cache = (self.state.step, C.capture(self.engine, self.state))
                else:
                    self._snapshot_cache[1].state = self.state.to_dict()
                self.writer.submit(self._snapshot_cache[1], os.path.join(self.cfg.checkpoint_dir, name))
            except Exception as e:
                log_error(f"[ckpt] capture failed: {e}")
                ok[0] = 0
            finally:
                self.prefetch.start()
        else:
            self.prefetch.quiesce()
            self.prefetch.start()
        fin = getattr(self.engine, "finish_export", None)
        if fin is not None:
            fin()           # what prepare_export gathered only for the snapshot is dropped again
        if self.world > 1:
            dev = getattr(self.engine, "device", torch.device("cpu"))
            flag = ok.to(dev) if dev.type == "cuda" else ok
            self.dist.broadcast_(flag, 0)
            ok = flag.cpu()
            self.dist.barrier()
        if int(ok[0]) == 0:
            raise TrainerError("checkpoint capture failed on rank 0")

    # ------------------------------------------------------------------ logging
    def _log_step(self, loss, lr, gnorm, dt, ntok, dev_ms):
        tps = ntok / dt if dt > 0 else 0.0
        remaining = self.total_steps - self.state.step
        eta = remaining * dt if remaining > 0 else 0.0
        dense = self.cfg.tokens_per_step_global(self.world)
        sup = ntok / dense if dense > 0 else 0.0
        log_info("step %6d | loss %7.4f | ema %7.4f | ppl %8.2f | lr %.3e | gnorm %6.3f | %7.0f tok/s | %s | eta %s "
                 "| sup %4.1f%% | ckptq %d (%s) | perf [%s] | %s" % (
                     self.state.step, loss, self.ema_loss, math.exp(min(20.0, self.ema_loss)), lr, gnorm, tps,
                     human_count(self.state.tokens_seen), human_duration(eta), sup * 100.0, self.writer.queue_depth(),
                     human_bytes(self.writer.queued_bytes()), PERF.report(), self.phases.report()))
        if self.jsonl_path:
            with open(self.jsonl_path, "a") as f:
                f.write(json.dumps({"step": self.state.step, "loss": loss, "ema": self.ema_loss, "lr": lr,
                                    "gnorm": gnorm, "tok_s_host": tps, "ntok": ntok, "device_ms": dev_ms,
                                    "loss_scale": self.scaler.for_step(), "tokens_seen": self.state.tokens_seen}) + "\n")

    # ------------------------------------------------------------------ one optimizer step
    def prepare(self):
        """Plan the schedule and start the loader thread; ``run`` calls this, step-wise callers call it once."""
        if self.total_steps == 0:
            self._plan_schedule()
        self.prefetch.start()

    def train_step(self):
        """One optimizer step: ``grad_accum`` micro-batches, gradient exchange, optimizer, scaler and state
        bookkeeping.  Returns ``(StepResult, lr, host_seconds)``."""
        c = self.cfg
        t0 = time.perf_counter()
        dscale = self.scaler.for_step()
        self.engine.begin_step(self.state.step, dscale)
        for _ in range(c.grad_accum // self.fuse):
            self.phases.start("load")
            group = [self.prefetch.get() for _ in range(self.fuse)]
            self.phases.stop("load")
            ids, tg, sg, Bm, Tm = self._fused(group)
            if self.segments == 1:
                self.engine.micro_step(ids, tg, sg, Bm, Tm)
            else:
                rows = Bm // self.segments
                cut = lambda t, k: None if t is None else t.view(Bm, Tm)[k * rows:(k + 1) * rows]
                for k in range(self.segments):
                    self.engine.micro_step(cut(ids, k), cut(tg, k), cut(sg, k), rows, Tm)
        lr = self.sched.lr_at(self.state.step)
        res = self.engine.end_step(lr)
        loss = res.loss
        self.ema_loss = loss if (self.state.step == 0 and self.ema_loss == 0.0) else 0.98 * self.ema_loss + 0.02 * loss
        if res.ntok_global > 0 and not res.applied:
            self.skipped_steps += 1
        if res.ntok_global == 0:
            log_warn("[train] all-masked step (ntok=0): optimizer skipped")
        before = self.scaler.scale
        self.scaler.update(res.gnorm)
        if self.scaler.scale != before:
            log_info("[scaler] step %d: scale %.0f -> %.0f" % (self.state.step, before, self.scaler.scale))
        self.state.step += 1
        self.state.tokens_seen += res.ntok_global
        self.state.last_loss = loss
        return res, lr, time.perf_counter() - t0

    # ------------------------------------------------------------------ the loop
    def run(self):
        STOP.install()
        self._plan_schedule()
        c = self.cfg
        sft = c.stage == "sft"
        log_info("---------------- %s ----------------" % ("SFT (instruction tuning)" if sft else "pretraining"))
        log_info("  steps %d | micro-batch %d x %d tok | accum %d | %s tok/step | opt %s | sched %s | peak lr %.2e" % (
            self.total_steps, c.batch_size, c.seq_len, c.grad_accum, human_count(c.tokens_per_step_local()),
            c.optimizer, c.scheduler, self.sched.peak))
        t_wall = time.perf_counter()
        self.prefetch.start()
        self.writer.start()
        deadline = float(os.environ.get("GB200_STEP_DEADLINE_S", "0") or 0) or c.step_deadline_s
        watchdog = None
        if deadline > 0:                         # host thread: ends the process when a step (a peer) never arrives
            watchdog = StepWatchdog(deadline, describe=lambda: "rank %d step %d/%d" % (self.rank, self.state.step, self.total_steps)).start()
        if self.world > 1 and c.heartbeat_stale_s > 0:
            # liveness through the job's key-value store: a peer that failed or left is reported here, on the host,
            # before this rank launches another collective towards it
            import torch.distributed as tdist
            from ..parallel.watchdog import Heartbeat
            store = tdist.PrefixStore("gb200_heartbeat", tdist.distributed_c10d._get_default_store())
            self.heartbeat = Heartbeat(store, self.rank, self.world, stale_s=c.heartbeat_stale_s)
        try:
            while self.state.step < self.total_steps:
                if self.heartbeat is not None:
                    self.heartbeat.beat()
                    try:
                        self.heartbeat.check()
                    except PeerFailure as pf:
                        raise TrainerError("peer failure before step %d: %s" % (self.state.step + 1, pf))
                res, lr, dt = self.train_step()
                loss = res.loss
                if watchdog is not None:
                    watchdog.beat()
                main = self.is_main()
                if main and c.log_every > 0 and self.state.step % c.log_every == 0:
                    self._log_step(loss, lr, res.gnorm, dt, res.ntok_global, getattr(self.engine, "last_step_ms", None))
                    self.writer.check_health()
                if watchdog is not None and ((self.have_val and c.eval_every > 0 and self.state.step % c.eval_every == 0) or
                                             (c.save_every > 0 and self.state.step % c.save_every == 0)):
                    watchdog.hold()              # evaluation and checkpoint capture have no step cadence
                if self.have_val and c.eval_every > 0 and self.state.step % c.eval_every == 0:
                    best = torch.zeros(2, dtype=torch.int64)
                    if main:
                        vl = self.evaluate(c.eval_batches)
                        rep = getattr(self.engine, "balance_report", lambda: "")()
                        if rep:
                            log_info("  >> " + rep)
                        log_info("  >> val loss %.4f  (ppl %.2f)  [best %s]" % (
                            vl, math.exp(min(20.0, vl)), ("%.4f" % self.state.best_val) if self.state.best_val < 1e29 else "-"))
                        if vl < self.state.best_val:
                            self.state.best_val = vl
                            best[0] = 1
                        best[1] = int(np.float64(self.state.best_val).view(np.int64))
                    if self.world > 1:
                        dev = getattr(self.engine, "device", torch.device("cpu"))
                        bb = best.to(dev) if dev.type == "cuda" else best
                        self.dist.broadcast_(bb, 0)
                        best = bb.cpu()
                        self.state.best_val = float(np.int64(int(best[1])).view(np.float64))
                    if int(best[0]):
                        self.save("best.ckpt")
                if c.save_every > 0 and self.state.step % c.save_every == 0:
                    self.save("last.ckpt")
                self.writer.check_health()
                if watchdog is not None:
                    watchdog.release()
                if STOP.requested:
                    self.stopped_by_signal = True
                if main:
                    self._snapshot_cache = None
                if self.stopped_by_signal:
                    break
            self.prefetch.stop()
            if self.stopped_by_signal:
                log_warn("[stop] %s received at step %d/%d: saving last.ckpt and exiting cleanly" % (
                    STOP.reason, self.state.step, self.total_steps))
                self.save("last.ckpt")
            elif not (c.save_every > 0 and self.state.step % c.save_every == 0):
                self.save("last.ckpt")
            self.writer.wait()
        except BaseException as e:
            if self.heartbeat is not None and not isinstance(e, TrainerError):
                try:
                    self.heartbeat.fail("%s: %s" % (type(e).__name__, e))
                except Exception:
                    pass
            raise
        finally:
            if watchdog is not None:
                watchdog.stop()
            self.prefetch.stop()
            self.writer.stop()
        log_info("---------------- %s done: %d steps, %s tokens, %s --------------------" % (
            "sft" if sft else "pretrain", self.state.step, human_count(self.state.tokens_seen),
            human_duration(time.perf_counter() - t_wall)))
        if self.scaler.active and self.state.step > 0:
            log_info("[scaler] %d/%d optimizer steps skipped (%.2f%%), %d overflow(s), final scale %.0f" % (
                self.skipped_steps, self.state.step, 100.0 * self.skipped_steps / self.state.step,
                self.scaler.overflows, self.scaler.scale))
        return self.state
