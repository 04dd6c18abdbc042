"""Training entry point (the reference's ``gai_train``, tools/training_cli.cpp:36-400): a YAML recipe plus flag
overrides, a pricing-only dry run, pre-flight memory / disk gates, training, optional GGUF export at the end.

    python -m ghassan_b200.cli.train --config configs/pro_1b_2xt4.yaml [flags]
    torchrun --nproc-per-node 8 -m ghassan_b200.cli.train --config ...        # one process per GPU

Flags (all optional): --data --checkpoint-dir --resume auto|none|<path> --resume-mode exact|migrate
--allow-recipe-drift --batch-size --seq-len --grad-accum --max-steps --lr --warmup --seed --optimizer
adamw|lion|muon --scheduler cosine|wsd --ce-chunks --gemm-fp16 0|1 --device auto|cpu|cuda --log-every --eval-every
--save-every --vocab --layers --hidden --heads --kv-heads --tokenizer --strict-config --strict-args --dry-run
--max-vram-mb --output-budget-mb --export <path> --export-profile fp16|q8_k|q4_0 --set KEY VALUE (any recipe key).
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List, Optional

from ..models.config import ModelConfig
from ..training.config import TrainerConfig
from ..training.memory_plan import memory_plan
from ..utils.config import Config, ConfigError
from ..utils.log import human_bytes, human_count, log_error, log_info, log_warn
from .common import add_common_flags, apply_common_flags


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="gai_train", description="MoE decoder-LLM trainer (B200)")
    ap.add_argument("--config", default="configs/flash_480m_single.yaml")
    for name in ("data", "checkpoint-dir", "resume", "resume-mode", "optimizer", "scheduler", "device", "tokenizer", "export",
                 "export-profile"):
        ap.add_argument("--" + name)
    for name in ("batch-size", "seq-len", "grad-accum", "max-steps", "warmup", "seed", "ce-chunks", "gemm-fp16", "log-every",
                 "eval-every", "save-every", "vocab", "layers", "hidden", "heads", "kv-heads", "max-vram-mb",
                 "output-budget-mb", "ckpt-segments", "threads"):
        ap.add_argument("--" + name)
    ap.add_argument("--lr")
    for name in ("strict-config", "strict-args", "dry-run", "allow-recipe-drift", "verbose"):
        ap.add_argument("--" + name, action="store_true")
    ap.add_argument("--set", nargs=2, action="append", metavar=("KEY", "VALUE"))
    add_common_flags(ap)
    return ap


def _num(args, name, strict, cast=int):
    raw = getattr(args, name.replace("-", "_"))
    if raw is None:
        return None
    try:
        return cast(raw)
    except ValueError:
        if strict:
            raise ConfigError(f"--{name}: '{raw}' is not a number")
        log_warn(f"--{name}: '{raw}' is not a number; ignored")
        return None


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    apply_common_flags(args)
    try:
        return _run(args)
    except (ConfigError, ValueError) as e:
        log_error(str(e))
        return 2
    except Exception as e:            # TrainerError and friends: message, no traceback, non-zero exit
        from ..training.trainer import TrainerError
        if isinstance(e, TrainerError):
            log_error("training aborted: " + str(e))
            return 1
        raise


def _run(args) -> int:
    cfg = Config()
    if os.path.exists(args.config):
        cfg = Config.from_file(args.config)
        log_info("[cfg ] " + args.config)
    else:
        log_warn("[cfg ] " + args.config + " not found, using built-in defaults")
    for k, v in (args.set or []):
        cfg.set(k, v)
    mcfg = ModelConfig.from_config(cfg)
    tcfg = TrainerConfig.from_config(cfg, strict=args.strict_config)
    strict = args.strict_args
    if cfg.has("tokenizer.vocab_size") and cfg.get_int("tokenizer.vocab_size", mcfg.vocab_size) != mcfg.vocab_size:
        log_warn("[cfg ] tokenizer.vocab_size %d != model.vocab_size %d (embedding/tokenizer mismatch; training would "
                 "corrupt)" % (cfg.get_int("tokenizer.vocab_size", 0), mcfg.vocab_size))
    if args.data:
        tcfg.data_dir = args.data
    if args.checkpoint_dir:
        tcfg.checkpoint_dir = args.checkpoint_dir
    if args.resume:
        tcfg.resume = args.resume
    if args.allow_recipe_drift:
        tcfg.allow_recipe_drift = True
    if args.resume_mode:
        if args.resume_mode not in ("exact", "migrate"):
            raise ConfigError("--resume-mode must be 'exact' or 'migrate' (got '%s')" % args.resume_mode)
        tcfg.resume_mode = args.resume_mode
    for flag, attr in (("batch-size", "batch_size"), ("seq-len", "seq_len"), ("grad-accum", "grad_accum"),
                       ("warmup", "warmup_steps"), ("seed", "seed"), ("log-every", "log_every"),
                       ("eval-every", "eval_every"), ("save-every", "save_every"), ("output-budget-mb", "output_budget_mb")):
        v = _num(args, flag, strict)
        if v is not None:
            setattr(tcfg, attr, v)
    v = _num(args, "max-steps", strict)
    if v is not None:
        if tcfg.epochs > 0:
            log_warn("[cfg ] --max-steps overrides yaml epochs (epochs ignored)")
        tcfg.max_steps, tcfg.epochs = v, 0
    v = _num(args, "gemm-fp16", strict)
    if v is not None:
        tcfg.gemm_fp16 = v != 0
    v = _num(args, "lr", strict, float)
    if v is not None:
        tcfg.learning_rate = v
    if args.optimizer:
        if args.optimizer not in ("adamw", "lion", "muon"):
            raise ConfigError("unknown --optimizer (adamw|lion|muon)")
        tcfg.optimizer = args.optimizer
        if tcfg.optimizer == "lion" and abs(tcfg.beta2 - 0.95) < 1e-9:
            tcfg.beta2 = 0.99
    if args.scheduler:
        if args.scheduler not in ("cosine", "wsd"):
            raise ConfigError("unknown --scheduler (cosine|wsd)")
        tcfg.scheduler = args.scheduler
    v = _num(args, "ckpt-segments", strict)
    if v is not None:
        if v < 1:
            raise ConfigError("--ckpt-segments must be >= 1")
        tcfg.ckpt_segments, tcfg.activation_checkpointing = v, v > 1
    v = _num(args, "threads", strict)
    if v is not None and v > 0:
        import torch as _torch
        _torch.set_num_threads(v)
    v = _num(args, "ce-chunks", strict)
    if v is not None:
        tcfg.ce_chunks = min(32, max(1, v))
    if args.device:
        tcfg.device = args.device
    for flag, attr in (("vocab", "vocab_size"), ("layers", "num_layers"), ("hidden", "hidden_size"), ("heads", "num_heads"),
                       ("kv-heads", "num_kv_heads")):
        v = _num(args, flag, strict)
        if v is not None:
            setattr(mcfg, attr, v)
    mcfg.validate()
    # tokenizer identity: fingerprint pinned into checkpoints and verified on resume
    tok_path = args.tokenizer or cfg.get_str("tokenizer.path", "")
    if tok_path and not os.path.isabs(tok_path):
        cand = os.path.join(os.path.dirname(os.path.abspath(args.config)), tok_path)
        if os.path.exists(cand):
            tok_path = cand
    from .. import _gb200_host as H
    if tcfg.tok_fingerprint == 0 and tok_path:
        fp = H.fingerprint_file(tok_path)
        tcfg.tok_fingerprint = fp
        if fp:
            log_info("[tok ] fingerprint %s (%s) pinned for resume verification" % (H.fingerprint_hex(fp), tok_path))
        else:
            log_warn("[tok ] cannot read %s: resume will not verify tokenizer identity" % tok_path)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    import torch
    dev = tcfg.device
    if dev == "auto":
        dev = "cuda" if torch.cuda.is_available() else "cpu"
    if dev == "cuda" and not torch.cuda.is_available() and not args.dry_run:
        raise ConfigError("--device cuda requested but no CUDA device is available")
    fuse = 1
    if dev == "cuda":
        f = tcfg.fuse_micro_batches
        if f <= 0:
            f = max(c for c in range(1, min(tcfg.grad_accum, 64) + 1)
                    if tcfg.grad_accum % c == 0 and (c == 1 or tcfg.batch_size * c * tcfg.seq_len <= 8192))
        fuse = f
    plan = memory_plan(mcfg, tcfg, world, fuse)
    log_info("---------------- memory estimate ----------------")
    log_info("  model       : " + mcfg.summary())
    log_info("  parameters  : %s (%s active per token)" % (human_count(plan["parameters"]), human_count(plan["active_per_token"])))
    log_info("  weights     : %s (fp32 master + 16-bit shadow)" % human_bytes(plan["weights"]))
    log_info("  gradients   : %s" % human_bytes(plan["gradients"]))
    log_info("  optimizer   : %s (%s)" % (human_bytes(plan["optimizer"]), tcfg.optimizer))
    log_info("  activations : %s (%d tokens per pass, %d micro-batches per pass)" % (
        human_bytes(plan["activations"]), plan["tokens_per_pass"], fuse))
    log_info("  total       : %s per GPU" % human_bytes(plan["total"]))
    steps = tcfg.max_steps if tcfg.max_steps > 0 else 0
    log_info("  schedule    : %s tokens/step per rank, %s global (x%d), %s" % (
        human_count(tcfg.tokens_per_step_local()), human_count(tcfg.tokens_per_step_global(world)), world,
        ("%d steps" % steps) if steps else ("%d epochs" % tcfg.epochs)))
    log_info("  checkpoint  : %s each" % human_bytes(plan["checkpoint_bytes"]))
    v = _num(args, "max-vram-mb", strict)
    if v is not None:
        if v <= 0:
            raise ConfigError("--max-vram-mb needs a positive MiB value")
        if plan["total"] > v * (1 << 20):
            raise ConfigError("predicted peak %s exceeds --max-vram-mb %d MiB" % (human_bytes(plan["total"]), v))
    if tcfg.output_budget_mb > 0:
        # two snapshots on disk while a save is in flight, plus the exported GGUF (the trainer's own quota guard adds
        # what is already in the output tree: training/guards.py)
        from ..training.guards import snapshot_bytes
        per = snapshot_bytes(plan["parameters"], tcfg.optimizer)
        proj = 2 * per + plan["parameters"] + per // 8
        budget = tcfg.output_budget_mb * (1 << 20)
        log_info("  output budget       : %s (proj snapshots+gguf %s, %s left for existing data)" % (
            human_bytes(budget), human_bytes(proj), human_bytes(max(0, budget - proj))))
        if proj > budget:
            raise ConfigError("projected output %s exceeds budget %s (2 snapshots %.1fGB + GGUF). Raise --output-budget-mb "
                              "knowingly or shrink the model." % (human_bytes(proj), human_bytes(budget), 2 * per / 1e9))
    if args.dry_run:
        log_info("[dry ] nothing was allocated; exiting")
        return 0

    if world > 1 and not torch.distributed.is_initialized():
        local = int(os.environ.get("LOCAL_RANK", "0"))
        if dev == "cuda":
            torch.cuda.set_device(local)
            torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            torch.distributed.init_process_group("gloo")
    from ..training.trainer import Trainer
    trainer = Trainer(mcfg, tcfg, device=dev)
    state = trainer.run()
    if args.export and trainer.is_main():
        from ..formats.gguf import export_gguf
        if not tok_path:
            raise ConfigError("--export needs --tokenizer (the vocabulary is embedded in the file)")
        named = dict(trainer.engine.export_weights())
        info = export_gguf(args.export, mcfg, named, tok_path, args.export_profile or "fp16",
                           moe_bias=trainer.engine.export_moe_bias(), extra_meta={"steps": str(state.step)})
        log_info("[gguf] exported %s profile=%s tensors=%d" % (info["path"], info["profile"], info["tensors"]))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
