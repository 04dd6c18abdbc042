"""Training recipe (``training.*`` / ``data.*`` keys) with the reference's defaults, derived rules
and typo allow-list (training/trainer.h:24-94, training/trainer.cpp:106-321).

Keys under ``b200.*`` are this framework's additions (expert parallelism, fused gradient sync,
weight EMA, micro-batch fusion); recipes written for the reference engine never contain them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict

import numpy as np

from ..utils.config import Config, ConfigError
from ..utils.log import log_info, log_warn


def _f32(x) -> float:
    return float(np.float32(x))


def split_shard_glob(glob: str):
    """``<dir>/<prefix>*.gbin`` -> (dir, prefix) or None."""
    if not glob.endswith("*.gbin"):
        return None
    stem = glob[: -len("*.gbin")]
    if "*" in stem or "?" in stem:
        return None
    slash = max(stem.rfind("/"), stem.rfind("\\"))
    if slash < 0:
        return ".", stem
    d, p = stem[:slash], stem[slash + 1:]
    return (d or "/"), p


MODEL_KEYS = [
    "vocab_size", "hidden_size", "num_layers", "num_heads", "num_kv_heads", "intermediate_size", "max_seq_len",
    "rope_theta", "rms_eps", "tie_embeddings", "init_std", "use_moe", "num_experts", "moe_top_k", "moe_expert_dim",
    "moe_shared", "moe_aux_scale", "moe_jitter", "moe_allow_dense", "moe_aux_free", "use_qk_norm", "z_loss_scale",
    "rope_scale", "rope_yarn_mscale", "rope_yarn_low", "rope_yarn_high", "sliding_window", "rope_type",
]
TRAINING_KEYS = [
    "data_dir", "batch_size", "seq_len", "grad_accum", "max_steps", "epochs", "learning_rate", "min_lr_ratio",
    "warmup_steps", "optimizer", "scheduler", "sched_decay_frac", "weight_decay", "beta1", "beta2", "eps", "grad_clip",
    "ns_steps", "muon_min_ns_dim", "muon_vec_ratio", "output_budget_mb", "tok_fingerprint", "precision", "gemm_fp16",
    "fp16_weight_cache", "loss_scale_init", "loss_scale_max", "loss_scale_window", "log_every", "eval_every",
    "eval_batches", "save_every", "checkpoint_dir", "resume", "seed", "device", "stage", "pretrained_checkpoint",
    "allow_no_pretrained", "allow_recipe_drift", "resume_mode", "freeze_embeddings", "activation_checkpointing",
    "ckpt_segments", "ce_chunks", "pack_sequences", "ddp", "ddp_grad_compression",
]
KNOWN_KEYS = ([f"model.{k}" for k in MODEL_KEYS] + ["tokenizer.path", "tokenizer.vocab_size"] +
              [f"training.{k}" for k in TRAINING_KEYS] +
              ["data.data_dir", "data.train_glob", "data.val_glob", "data.train_prefix", "data.val_prefix"])
KNOWN_PREFIXES = ["data.mix.", "b200."]


@dataclass
class TrainerConfig:
    data_dir: str = "artifacts/shards"
    train_prefix: str = "train"
    val_prefix: str = "val"
    mix: Dict[str, float] = field(default_factory=dict)
    batch_size: int = 8
    seq_len: int = 1024
    grad_accum: int = 16
    max_steps: int = 0
    epochs: int = 0
    learning_rate: float = 3e-4
    min_lr_ratio: float = 0.1
    warmup_steps: int = 2000
    optimizer: str = "adamw"
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    grad_clip: float = 1.0
    muon_ns_steps: int = 5
    muon_min_ns_dim: int = 0
    muon_vec_ratio: float = 0.1
    scheduler: str = "cosine"
    sched_decay_frac: float = 0.2
    precision: str = "fp32"           # fp32 | fp16 | bf16 (selects the 16-bit GEMM operand type when != fp32)
    gemm_fp16: bool = True
    fp16_weight_cache: bool = False
    loss_scale_init: float = 65536.0
    loss_scale_window: int = 2000
    loss_scale_max: float = 0.0
    activation_checkpointing: bool = False
    ckpt_segments: int = 2
    ce_chunks: int = 4
    pack_sequences: bool = False
    ddp: bool = False
    ddp_grad_compression: bool = False
    log_every: int = 10
    eval_every: int = 500
    eval_batches: int = 20
    save_every: int = 1000
    checkpoint_dir: str = "artifacts/checkpoints/200m"
    resume: str = "auto"
    tok_fingerprint: int = 0
    seed: int = 42
    device: str = "auto"
    pretrained_checkpoint: str = ""
    allow_no_pretrained: bool = False
    freeze_embeddings: bool = False
    allow_recipe_drift: bool = False
    output_budget_mb: int = 0
    resume_mode: str = "migrate"
    stage: str = "pretrain"
    # ---- b200.* additions
    ep_size: int = 1                  # expert-parallel degree (num_experts % ep_size == 0; 1 or the number of ranks)
    ep_capacity: float = 2.0          # receive-buffer rows per rank, in units of its own routed rows (balanced load = 1)
    grad_sync: str = "fused"          # fused (peer-memory reduce-scatter + optimizer + all-gather) | nccl
    grad_sync_nvls: bool = False      # fused exchange through NVSwitch multicast (multimem) where the buffers allow it
    weight_ema: float = 0.0           # > 0: keep an exponential moving average of the weights with this decay
    fuse_micro_batches: int = 0       # micro-batches run as one forward/backward pass (same gradient sum); 0 = choose
    cuda_graphs: bool = True
    heartbeat_stale_s: float = 600.0  # multi-rank: a peer without progress for this long (or one that posted a failure) ends the run; 0 = off
    step_deadline_s: float = 0.0      # > 0: a host watchdog ends the process when no step finishes within this many seconds
    compute_dtype: str = ""           # "" = derive from precision/gemm_fp16; fp16 | bf16

    def resume_exact(self) -> bool:
        return self.resume_mode == "exact"

    # ------------------------------------------------------------------ derived
    def tokens_per_step_local(self) -> int:
        return self.batch_size * self.seq_len * self.grad_accum

    def tokens_per_step_global(self, world_size: int = 1) -> int:
        return self.tokens_per_step_local() * max(1, world_size)

    def epoch_steps(self, total_tokens: int, world_size: int = 1) -> int:
        tps = self.tokens_per_step_global(world_size)
        if tps <= 0 or total_tokens <= 0:
            return 0
        per_epoch = (total_tokens + tps - 1) // tps
        steps = per_epoch * self.epochs
        if steps >= 2 ** 63:
            raise ConfigError("training schedule overflow in epoch_steps")
        return steps

    def effective_peak_lr(self) -> float:
        """Lion runs at a tenth of the configured learning rate (training/trainer.cpp:349-358)."""
        if self.optimizer == "lion":
            return _f32(np.float32(self.learning_rate) * np.float32(0.1))
        return self.learning_rate

    def operand_dtype(self) -> str:
        """16-bit GEMM operand type for the CUDA path."""
        if self.compute_dtype:
            return self.compute_dtype
        if self.precision == "bf16":
            return "bf16"
        return "fp16"

    def loss_scaling_active(self) -> bool:
        return self.loss_scale_init > 0 and self.gemm_fp16 and self.operand_dtype() == "fp16"

    @classmethod
    def from_config(cls, c: Config, strict: bool = False) -> "TrainerConfig":
        t = cls()
        t.data_dir = c.get_str("training.data_dir", t.data_dir)
        t.train_prefix = c.get_str("data.train_prefix", t.train_prefix)
        t.val_prefix = c.get_str("data.val_prefix", t.val_prefix)
        t.batch_size = c.get_int("training.batch_size", t.batch_size)
        t.seq_len = c.get_int("training.seq_len", t.seq_len)
        t.grad_accum = c.get_int("training.grad_accum", t.grad_accum)
        t.max_steps = c.get_int("training.max_steps", 0)
        t.epochs = c.get_int("training.epochs", 0)
        if t.max_steps > 0 and t.epochs > 0:
            raise ConfigError("ambiguous schedule: set EITHER training.max_steps OR training.epochs, not both")
        if t.max_steps <= 0 and t.epochs <= 0:
            raise ConfigError("no schedule: set training.max_steps (>0) or training.epochs (>0)")
        t.learning_rate = _f32(c.get_float("training.learning_rate", t.learning_rate))
        t.min_lr_ratio = _f32(c.get_float("training.min_lr_ratio", t.min_lr_ratio))
        t.warmup_steps = c.get_int("training.warmup_steps", t.warmup_steps)
        t.optimizer = c.get_str("training.optimizer", t.optimizer)
        if t.optimizer not in ("adamw", "lion", "muon"):
            raise ConfigError(f"unknown training.optimizer '{t.optimizer}' (adamw|lion|muon)")
        t.scheduler = c.get_str("training.scheduler", t.scheduler)
        if t.scheduler not in ("cosine", "wsd"):
            raise ConfigError(f"unknown training.scheduler '{t.scheduler}' (cosine|wsd)")
        t.sched_decay_frac = _f32(c.get_float("training.sched_decay_frac", t.sched_decay_frac))
        t.weight_decay = _f32(c.get_float("training.weight_decay", t.weight_decay))
        t.beta1 = _f32(c.get_float("training.beta1", t.beta1))
        t.beta2 = _f32(c.get_float("training.beta2", 0.99 if t.optimizer == "lion" else t.beta2))
        t.eps = _f32(c.get_float("training.eps", t.eps))
        t.grad_clip = _f32(c.get_float("training.grad_clip", t.grad_clip))
        t.muon_ns_steps = c.get_int("training.ns_steps", t.muon_ns_steps)
        t.muon_min_ns_dim = c.get_int("training.muon_min_ns_dim", t.muon_min_ns_dim)
        t.muon_vec_ratio = _f32(c.get_float("training.muon_vec_ratio", t.muon_vec_ratio))
        if not 1 <= t.muon_ns_steps <= 10:
            raise ConfigError("training.ns_steps must be in 1..10")
        if t.muon_min_ns_dim < 0:
            raise ConfigError("training.muon_min_ns_dim must be >= 0")
        if not (0.0 < t.muon_vec_ratio <= 1.0):
            raise ConfigError("training.muon_vec_ratio must be in (0,1]")
        t.precision = c.get_str("training.precision", "fp32")
        if t.precision not in ("fp32", "fp16", "bf16"):
            raise ConfigError(f"training.precision must be one of: fp32, fp16, bf16 (got '{t.precision}')")
        t.gemm_fp16 = c.get_bool("training.gemm_fp16", t.gemm_fp16)
        t.fp16_weight_cache = c.get_bool("training.fp16_weight_cache", t.fp16_weight_cache)
        t.loss_scale_init = _f32(c.get_float("training.loss_scale_init", t.loss_scale_init))
        t.loss_scale_max = _f32(c.get_float("training.loss_scale_max", t.loss_scale_max))
        if not (t.loss_scale_max >= 0.0) or not math.isfinite(t.loss_scale_max):
            raise ConfigError("training.loss_scale_max must be finite and >= 0 (0 = fp16-safe max)")
        t.loss_scale_window = c.get_int("training.loss_scale_window", t.loss_scale_window)
        t.log_every = c.get_int("training.log_every", t.log_every)
        t.eval_every = c.get_int("training.eval_every", t.eval_every)
        t.eval_batches = c.get_int("training.eval_batches", t.eval_batches)
        t.save_every = c.get_int("training.save_every", t.save_every)
        t.checkpoint_dir = c.get_str("training.checkpoint_dir", t.checkpoint_dir)
        t.resume = c.get_str("training.resume", t.resume)
        t.tok_fingerprint = c.get_int("training.tok_fingerprint", t.tok_fingerprint) & (2 ** 64 - 1)
        t.seed = c.get_int("training.seed", t.seed) & (2 ** 64 - 1)
        t.output_budget_mb = c.get_int("training.output_budget_mb", t.output_budget_mb)
        t.device = c.get_str("training.device", t.device)
        t.stage = c.get_str("training.stage", t.stage)
        if t.stage not in ("pretrain", "sft", "cpt"):
            raise ConfigError(f"unknown training.stage '{t.stage}' (pretrain|sft|cpt)")
        t.pretrained_checkpoint = c.get_str("training.pretrained_checkpoint", t.pretrained_checkpoint)
        t.allow_no_pretrained = c.get_bool("training.allow_no_pretrained", t.allow_no_pretrained)
        t.freeze_embeddings = c.get_bool("training.freeze_embeddings", t.freeze_embeddings)
        t.allow_recipe_drift = c.get_bool("training.allow_recipe_drift", t.allow_recipe_drift)
        t.resume_mode = c.get_str("training.resume_mode", t.resume_mode)
        if t.resume_mode not in ("migrate", "exact"):
            raise ConfigError(f"unknown training.resume_mode '{t.resume_mode}' (exact|migrate)")
        for k, v in sorted(c.kv.items()):
            if k.startswith("data.mix.") and len(k) > len("data.mix."):
                try:
                    w = float(v.strip())
                    if not math.isfinite(w) or not w > 0.0:
                        raise ValueError
                    t.mix[k[len("data.mix."):]] = w
                except ValueError:
                    log_warn(f"config: ignoring malformed data.mix weight for '{k}': '{v}' (want positive number)")
        if c.get_bool("training.activation_checkpointing", False):
            t.activation_checkpointing = True
            t.ckpt_segments = min(8, max(1, c.get_int("training.ckpt_segments", 2)))
        t.ce_chunks = min(32, max(1, c.get_int("training.ce_chunks", t.ce_chunks)))
        t.pack_sequences = c.get_bool("training.pack_sequences", False)
        t.ddp = c.get_bool("training.ddp", False)
        t.ddp_grad_compression = c.get_bool("training.ddp_grad_compression", False)

        has_tg, has_vg = c.has("data.train_glob"), c.has("data.val_glob")
        if has_tg or has_vg:
            tsplit = split_shard_glob(c.get_str("data.train_glob")) if has_tg else None
            vsplit = split_shard_glob(c.get_str("data.val_glob")) if has_vg else None
            if has_tg and tsplit is None:
                raise ConfigError("cannot parse data.train_glob (want <dir>/<prefix>*.gbin): " + c.get_str("data.train_glob"))
            if has_vg and vsplit is None:
                raise ConfigError("cannot parse data.val_glob (want <dir>/<prefix>*.gbin): " + c.get_str("data.val_glob"))
            if has_tg and has_vg and tsplit[0] != vsplit[0]:
                raise ConfigError(f"data.train_glob and data.val_glob span different shard dirs ({tsplit[0]} vs {vsplit[0]})")
            gdir = tsplit[0] if has_tg else vsplit[0]
            if c.has("training.data_dir") and c.get_str("training.data_dir") != gdir:
                raise ConfigError(f"training.data_dir '{c.get_str('training.data_dir')}' conflicts with the shard glob dir '{gdir}'")
            t.data_dir = gdir
            if has_tg:
                if c.has("data.train_prefix") and c.get_str("data.train_prefix") != tsplit[1]:
                    raise ConfigError("data.train_prefix conflicts with data.train_glob")
                t.train_prefix = tsplit[1]
            if has_vg:
                if c.has("data.val_prefix") and c.get_str("data.val_prefix") != vsplit[1]:
                    raise ConfigError("data.val_prefix conflicts with data.val_glob")
                t.val_prefix = vsplit[1]
            log_info(f"[data] shard globs honored: dir={t.data_dir} train_prefix={t.train_prefix} val_prefix={t.val_prefix}")
        if c.has("data.data_dir"):
            dd = c.get_str("data.data_dir")
            if dd and dd != t.data_dir:
                raise ConfigError(f"data.data_dir '{dd}' conflicts with training.data_dir '{t.data_dir}'")
            if dd:
                log_warn("[cfg ] data.data_dir duplicates training.data_dir (legacy; ignored)")

        # framework additions
        t.ep_size = max(1, c.get_int("b200.ep_size", t.ep_size))
        t.ep_capacity = max(1.0, c.get_float("b200.ep_capacity", t.ep_capacity))
        t.grad_sync = c.get_str("b200.grad_sync", t.grad_sync)
        t.grad_sync_nvls = c.get_bool("b200.grad_sync_nvls", t.grad_sync_nvls)
        if t.grad_sync not in ("fused", "nccl"):
            raise ConfigError(f"unknown b200.grad_sync '{t.grad_sync}' (fused|nccl)")
        t.weight_ema = c.get_float("b200.weight_ema", t.weight_ema)
        t.fuse_micro_batches = max(0, c.get_int("b200.fuse_micro_batches", t.fuse_micro_batches))
        t.cuda_graphs = c.get_bool("b200.cuda_graphs", t.cuda_graphs)
        t.step_deadline_s = max(0.0, c.get_float("b200.step_deadline_s", t.step_deadline_s))
        t.heartbeat_stale_s = max(0.0, c.get_float("b200.heartbeat_stale_s", t.heartbeat_stale_s))
        t.compute_dtype = c.get_str("b200.compute_dtype", t.compute_dtype)
        if t.compute_dtype not in ("", "fp16", "bf16"):
            raise ConfigError("b200.compute_dtype must be fp16 or bf16")
        c.check_known(KNOWN_KEYS, KNOWN_PREFIXES, strict)
        return t
