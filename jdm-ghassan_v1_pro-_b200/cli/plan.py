"""Session planning: measure what a recipe really does on this machine, then size a run from the measurement.

Two commands (the roles of the reference's pilot cell and time estimator, configs/kaggle/measure_training_throughput.sh
and configs/kaggle/estimate_t4_time.py, which quote fixed Tesla T4 rates; here the rate is measured or given):

``pilot``     run a few optimizer steps of the real recipe (guards, loaders, engine and optimizer as in training, no
              checkpoints kept), report the steady device-timed rate, whether a resource guard would fire, and how
              many steps / tokens / epochs fit into 2, 4, 6, 8 and 10 hours.
``estimate``  no run: hours for a corpus of a given size at a given rate, and whether it fits the session budget.

Both print a table for people and, with ``--json``, one JSON object for scripts.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import time
from typing import List, Optional

from ..models.config import ModelConfig
from ..training.config import TrainerConfig
from ..utils.config import Config, ConfigError
from ..utils.log import human_count, human_duration, log_error, log_info, log_warn
from .common import add_common_flags, apply_common_flags

HOUR_MARKS = (2, 4, 6, 8, 10)


def budget_table(tokens_per_step: int, tok_per_s: float, corpus_tokens: int = 0, hours=HOUR_MARKS) -> List[dict]:
    """Rows {hours, steps, tokens, epochs}: what fits into each time budget at ``tok_per_s``."""
    rows = []
    for h in hours:
        steps = int(h * 3600.0 * tok_per_s / tokens_per_step) if tokens_per_step > 0 else 0
        toks = steps * tokens_per_step
        rows.append({"hours": h, "steps": steps, "tokens": toks,
                     "epochs": (toks / corpus_tokens) if corpus_tokens > 0 else None})
    return rows


def estimate(tokens_per_step: int, corpus_tokens: float, epochs: float, tok_per_s: float, budget_hours: float) -> dict:
    total = corpus_tokens * max(epochs, 0.0)
    secs = total / tok_per_s if tok_per_s > 0 else float("inf")
    return {"tokens_per_step": tokens_per_step, "corpus_tokens": corpus_tokens, "epochs": epochs, "total_tokens": total,
            "steps": int(total / tokens_per_step) if tokens_per_step > 0 else 0, "tok_per_s": tok_per_s,
            "seconds": secs, "hours": secs / 3600.0, "budget_hours": budget_hours, "fits": secs <= budget_hours * 3600.0}


def _format_table(rows) -> str:
    out = ["  %-8s %10s %12s %10s" % ("budget", "steps", "tokens", "epochs")]
    for r in rows:
        out.append("  %-8s %10d %12s %10s" % ("%dh" % r["hours"], r["steps"], human_count(r["tokens"]),
                                             "-" if r["epochs"] is None else "%.2f" % r["epochs"]))
    return "\n".join(out)


def _load(args):
    if not os.path.exists(args.config):
        raise ConfigError("config %s not found" % args.config)
    cfg = Config.from_file(args.config)
    for k, v in (args.set or []):
        cfg.set(k, v)
    return ModelConfig.from_config(cfg), TrainerConfig.from_config(cfg, strict=False)


def run_pilot(mcfg: ModelConfig, tcfg: TrainerConfig, steps: int, warm: int, device: str, probe=None) -> dict:
    """``steps`` optimizer steps of the recipe; the rate is the median of the steps after the first ``warm``."""
    import torch
    from ..training.guards import GuardError
    from ..training.trainer import Trainer, TrainerError
    if steps <= warm:
        raise ConfigError("pilot needs more steps (%d) than warm-up steps (%d)" % (steps, warm))
    tcfg.max_steps, tcfg.epochs = steps, 0
    tcfg.save_every, tcfg.eval_every, tcfg.resume = 0, 0, "none"
    tcfg.warmup_steps = min(tcfg.warmup_steps, max(1, steps // 4))
    out = {"steps": steps, "warm": warm, "guard": None}
    with tempfile.TemporaryDirectory(prefix="gb200_pilot_") as tmp:
        tcfg.checkpoint_dir = tmp
        t_start = time.perf_counter()
        try:
            tr = Trainer(mcfg, tcfg, device=device)
        except (GuardError, TrainerError) as e:
            if isinstance(e, GuardError) or "guard" in str(e):
                out["guard"] = str(e)
                return out
            raise
        tr.prepare()
        world = tr.world
        per_step, dev_ms, losses, ntoks = [], [], [], []
        try:
            for _ in range(steps):
                res, _lr, dt = tr.train_step()
                per_step.append(dt)
                ms = getattr(tr.engine, "last_step_ms", None)
                dev_ms.append(ms if ms is not None else dt * 1e3)
                losses.append(res.loss)
                ntoks.append(res.ntok_global)
        finally:
            tr.prefetch.stop()
            tr.writer.stop()
        if torch.cuda.is_available() and device == "cuda":
            torch.cuda.synchronize()
        wall = time.perf_counter() - t_start
        steady_ms = statistics.median(dev_ms[warm:])
        dense = tcfg.tokens_per_step_global(world)
        out.update({
            "world": world, "tokens_per_step": dense, "wall_s": wall, "steady_ms_per_step": steady_ms,
            "tok_per_s": dense / (steady_ms / 1e3) if steady_ms > 0 else 0.0,
            "tok_per_s_with_startup": dense * steps / wall if wall > 0 else 0.0,
            "supervised_share": (sum(ntoks) / (dense * steps)) if dense > 0 else 0.0,
            "first_loss": losses[0], "last_loss": losses[-1], "finite": all(x == x and abs(x) < 1e30 for x in losses),
            "corpus_tokens": int(tr.train_loader.total_tokens),
            "segments": tr.segments, "fuse": tr.fuse,
        })
    return out


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="gai_plan", description="measure a recipe's rate and plan a session from it")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("pilot", help="run a few real steps and print the plan table")
    p.add_argument("--config", required=True)
    p.add_argument("--data")
    p.add_argument("--device", default="auto")
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warm", type=int, default=5, help="steps left out of the steady rate")
    p.add_argument("--set", nargs=2, action="append", metavar=("KEY", "VALUE"))
    p.add_argument("--json", action="store_true")
    e = sub.add_parser("estimate", help="hours for a corpus at a rate (no run)")
    e.add_argument("--config", required=True)
    e.add_argument("--tps", type=float, required=True, help="tokens per second (from `pilot`, or a known rate)")
    e.add_argument("--corpus-tokens", type=float, default=0.0)
    e.add_argument("--corpus-gb", type=float, default=0.0, help="size of the text corpus; with --tokens-per-gb")
    e.add_argument("--tokens-per-gb", type=float, default=150e6)
    e.add_argument("--budget-hours", type=float, default=10.0)
    e.add_argument("--set", nargs=2, action="append", metavar=("KEY", "VALUE"))
    e.add_argument("--json", action="store_true")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    ap = build_parser()
    add_common_flags(ap)
    args = ap.parse_args(argv)
    apply_common_flags(args)
    try:
        mcfg, tcfg = _load(args)
        mcfg.validate()
        if args.cmd == "estimate":
            corpus = args.corpus_tokens or args.corpus_gb * args.tokens_per_gb
            if corpus <= 0:
                raise ConfigError("estimate needs --corpus-tokens or --corpus-gb")
            if args.tps <= 0:
                raise ConfigError("--tps must be positive")
            world = int(os.environ.get("WORLD_SIZE", "1"))
            r = estimate(tcfg.tokens_per_step_global(world), corpus, max(1, tcfg.epochs), args.tps, args.budget_hours)
            if args.json:
                print(json.dumps(r))
                return 0 if r["fits"] else 3
            log_info("config       : %s (B=%d T=%d accum=%d -> %s tokens/step)" % (
                args.config, tcfg.batch_size, tcfg.seq_len, tcfg.grad_accum, human_count(r["tokens_per_step"])))
            log_info("corpus       : %s tokens x %g epoch(s) = %s tokens, %d steps" % (
                human_count(int(corpus)), r["epochs"], human_count(int(r["total_tokens"])), r["steps"]))
            log_info("rate         : %s tokens/s" % human_count(int(args.tps)))
            log_info("time         : %s (%.1f h)" % (human_duration(r["seconds"]), r["hours"]))
            if r["fits"]:
                log_info("verdict      : fits the %.0f h budget" % args.budget_hours)
                return 0
            log_warn("verdict      : does NOT fit the %.0f h budget (%.1fx over): fewer epochs, a smaller corpus or a "
                     "smaller model" % (args.budget_hours, r["hours"] / args.budget_hours))
            return 3
        # ---- pilot
        import torch
        dev = args.device
        if dev == "auto":
            dev = "cuda" if torch.cuda.is_available() else "cpu"
        if args.data:
            tcfg.data_dir = args.data
        r = run_pilot(mcfg, tcfg, args.steps, args.warm, dev)
        if r["guard"]:
            log_error("a resource guard fired on this recipe: " + r["guard"])
            if args.json:
                print(json.dumps(r))
            return 1
        r["table"] = budget_table(r["tokens_per_step"], r["tok_per_s"], r["corpus_tokens"])
        if args.json:
            print(json.dumps(r))
            return 0
        log_info("pilot        : %d steps in %s (start-up included); no resource guard fired" % (
            r["steps"], human_duration(r["wall_s"])))
        log_info("steady       : %.1f ms/step, %s tokens/s (median of the last %d steps, device-timed on a GPU)" % (
            r["steady_ms_per_step"], human_count(int(r["tok_per_s"])), r["steps"] - r["warm"]))
        log_info("budget       : %s tokens/step over %d rank(s); %.0f %% of them supervised" % (
            human_count(r["tokens_per_step"]), r["world"], 100.0 * r["supervised_share"]))
        log_info("loss         : %.4f -> %.4f%s" % (r["first_loss"], r["last_loss"], "" if r["finite"] else "  (NOT finite)"))
        log_info("corpus       : %s tokens in the training shards" % human_count(r["corpus_tokens"]))
        print(_format_table(r["table"]))
        return 0 if r["finite"] else 1
    except (ConfigError, ValueError) as e:
        log_error(str(e))
        return 2


if __name__ == "__main__":
    sys.exit(main())
