#!/usr/bin/env python
"""Training-throughput benchmark: train tokens/s on the pro_1b recipe (configs/pro_1b_2xt4.yaml), synthetic
uniform token data, random-initialised weights.

    python bench.py --gpus N --steps K --warmup W                  # this framework
    python bench.py --impl reference --gpus N --steps K --warmup W  # the unmodified reference binary

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...``; rank,
world size and rendezvous come from the environment.  A "step" is one optimizer step of the recipe
(grad_accum micro-batches of batch_size x seq_len tokens per rank, gradient exchange, optimizer).  Rank 0
prints one JSON line.  ``value`` is device-timed (CUDA events, max over ranks); ``e2e`` is host-timed through
``Trainer.train_step()`` including the pinned-host -> device input copies and the loss read-back.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import shutil
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
DEFAULT_CONFIG = os.path.join(ROOT, "configs", "pro_1b_2xt4.yaml")
REF_BIN = os.path.join(ROOT, "baseline", "_ref", "bin", "gai_train")


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0, period_ms=200):
        self.index, self.period_ms = index, period_ms
        self.proc = None
        self.lines = []
        self._t = None

    def start(self):
        smi = shutil.which("nvidia-smi")
        if not smi:
            return
        try:
            self.proc = subprocess.Popen([smi, "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self._t = threading.Thread(target=self._read, daemon=True)
        self._t.start()

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()      # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 7:
                continue
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for n, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def load_recipe(path, data_dir, ckpt_dir, tok_path, total_steps):
    """The recipe as shipped, with only paths and run-length keys replaced (they do not change the step's work)."""
    from ghassan_b200.utils.config import Config
    c = Config.from_file(path)
    for k in ("data.train_glob", "data.val_glob", "data.data_dir"):
        c.kv.pop(k, None)
    c.set("training.data_dir", data_dir)
    c.set("data.train_prefix", "train")
    c.set("data.val_prefix", "val")
    c.set("training.checkpoint_dir", ckpt_dir)
    c.set("tokenizer.path", tok_path)
    c.set("training.resume", "none")
    c.set("training.max_steps", total_steps)
    c.set("training.epochs", 0)
    c.set("training.warmup_steps", 1)          # LR schedule only
    c.set("training.save_every", 1000000)
    c.set("training.eval_every", 0)
    c.set("training.log_every", 1)
    c.set("training.output_budget_mb", 0)
    return c


def dump_yaml(c, path):
    """Write the flat recipe back as nested YAML (maps only; list values are not used by training recipes)."""
    tree = {}
    for k, v in sorted(c.kv.items()):
        if v == "":          # section headers carry no value of their own
            continue
        parts = k.split(".")
        node = tree
        for p in parts[:-1]:
            node = node.setdefault(p, {})
        node[parts[-1]] = v
    lines = []

    def walk(n, ind):
        for k, v in n.items():
            if isinstance(v, dict):
                if v:
                    lines.append(" " * ind + k + ":")
                    walk(v, ind + 2)
            else:
                lines.append(" " * ind + "%s: %s" % (k, v))

    walk(tree, 0)
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")


def make_data(work, mcfg_vocab, mix):
    from ghassan_b200.data import synthetic as S
    data = os.path.join(work, "shards")
    S.make_corpus(data, mcfg_vocab, mix=mix or None, train_tokens=4_000_000, val_tokens=200_000, mean_doc=512)
    tok = os.path.join(work, "tok", "synthetic.gtok")
    if not os.path.exists(tok):
        S.write_placeholder_gtok(tok, mcfg_vocab)
    return data, tok


def recipe_label(path, mcfg, tcfg, world):
    return {"model": os.path.splitext(os.path.basename(path))[0],
            "params": mcfg.count_parameters(),
            "global_batch": tcfg.batch_size * tcfg.grad_accum * world,
            "micro_batch": tcfg.batch_size, "grad_accum": tcfg.grad_accum, "seq_len": tcfg.seq_len,
            "optimizer": tcfg.optimizer, "parallelism": ("dp%d" % world) + ("+ep%d" % tcfg.ep_size if tcfg.ep_size > 1 else ""),
            "l2": "per-step working set (weights, gradients, moments: several GB) exceeds the 126 MB L2"}


# ------------------------------------------------------------------------------------------ this framework
def run_ours(args):
    import torch
    import torch.distributed as dist
    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer
    from ghassan_b200.utils import log as L
    from ghassan_b200.utils.config import Config
    if not args.verbose:
        L.set_log_level(L.WARN)
    base = Config.from_file(args.config)
    vocab = ModelConfig.from_config(base).vocab_size
    mix = TrainerConfig.from_config(base).mix
    work = os.path.join(args.workdir, "rank%d" % rank)
    data, tok = make_data(work, vocab, mix)
    total = args.settle_max + args.warmup + 2 * args.steps + 1
    c = load_recipe(args.config, data, os.path.join(work, "ckpt"), tok, total)
    for k, v in (args.set or []):
        c.set(k, v)
    mcfg, tcfg = ModelConfig.from_config(c), TrainerConfig.from_config(c)
    tr = Trainer(mcfg, tcfg, device="cuda")
    tr.prepare()
    eng = tr.engine
    # The recipe's dynamic loss scale starts high and halves on every overflowing step (those steps skip the
    # optimizer).  Run untimed steps until one applies, so that the warm-up and the timed steps all do the full work.
    settle = 0
    while settle < args.settle_max:
        res, _, _ = tr.train_step()
        settle += 1
        ok = torch.tensor([1.0 if res.applied else 0.0], device="cuda")
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) > 0:
            break
    for _ in range(args.warmup):
        tr.train_step()

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- phase A: device-timed
    sampler = ClockSampler(local)
    fence()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = eng.kernel_launches
    ev0.record()
    toks = 0
    losses = []
    applied = 0
    for _ in range(args.steps):
        res, _, _ = tr.train_step()
        toks += res.ntok_global
        losses.append(res.loss)
        applied += int(res.applied)
    ev1.record()
    fence()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1)
    launches = eng.kernel_launches - launches0 + args.steps * 6
    # ---- phase B: end to end through the public step API, host clock
    fence()
    t0 = time.perf_counter()
    toks_e = 0
    for _ in range(args.steps):
        res, _, _ = tr.train_step()
        toks_e += res.ntok_global
    fence()
    sec_e = time.perf_counter() - t0
    t = torch.tensor([ms, sec_e], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, sec_e = float(t[0]), float(t[1])
    tr.prefetch.stop()
    value = toks / (ms / 1e3)
    n_in = 3 if tcfg.pack_sequences else 2
    out = {"metric": "train tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16" if tcfg.operand_dtype() == "bf16" else "fp16", "data": "synthetic",
           "impl": "ours", "config": dict(recipe_label(args.config, mcfg, tcfg, world), fuse_micro_batches=tr.fuse,
                                            grad_sync=("fused peer-memory" if eng.grad_sync is not None else
                                                       ("nccl" if world > 1 else "none"))), "clocks": clocks,
           "e2e": {"value": toks_e / sec_e, "unit": "tokens/s",
                   "h2d_bytes_per_step": tcfg.grad_accum * tcfg.batch_size * tcfg.seq_len * 4 * n_in + 64,
                   "d2h_bytes_per_step": 40},
           "gpu_launches": int(launches), "optimizer_steps_applied": applied, "settle_steps": settle,
           "loss_first": losses[0], "loss_last": losses[-1],
           "supervised_tokens_per_step": toks / args.steps}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


# ------------------------------------------------------------------------------------------ the reference
STEP_RE = re.compile(r"step\s+(\d+) \| loss\s+([0-9.eE+-]+|nan|inf).*?\|\s+([0-9.]+) tok/s \|")


def run_reference(args):
    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0

    if not os.path.exists(REF_BIN):
        return unavailable("baseline/_ref/bin/gai_train is not built (cmake build of the reference for sm_100)")
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.utils import log as L
    from ghassan_b200.utils.config import Config
    L.set_log_level(L.WARN)
    base = Config.from_file(args.config)
    mcfg0 = ModelConfig.from_config(base)
    tcfg0 = TrainerConfig.from_config(base)
    work = os.path.join(args.workdir, "ref_rank%d" % rank)
    data, tok = make_data(work, mcfg0.vocab_size, tcfg0.mix)
    total = args.warmup + args.steps
    c = load_recipe(args.config, data, os.path.join(work, "ckpt"), tok, total)
    for k in [k for k in c.kv if k.startswith("b200.")]:
        c.kv.pop(k)
    c.set("data.train_glob", os.path.join(data, "train_*.gbin"))
    c.set("data.val_glob", os.path.join(data, "val_*.gbin"))
    c.kv.pop("data.train_prefix", None)
    c.kv.pop("data.val_prefix", None)
    c.kv.pop("training.data_dir", None)
    c.set("training.ddp", "true" if world > 1 else "false")   # the binary refuses ddp with one visible rank
    for k, v in (args.ref_set or []):      # explicit, non-default reference settings (reported in the JSON line)
        if k == "training.gemm_fp16" and str(v).lower() in ("false", "0", "no", "off"):
            # measured once on a B200: with fp32 GEMMs the reference's own code raised "an illegal memory access was
            # encountered" (cuda/cuda_utils.cu:99); a path that faults the GPU is not run again
            return unavailable("the reference's gemm_fp16=false path faults on B200 (illegal memory access in its own "
                               "code); its default fp16 path aborts with cuBLAS status 15 in cuda/attention.cu:362")
        c.set(k, v)
    yml = os.path.join(work, "bench_recipe.yaml")
    dump_yaml(c, yml)
    shutil.rmtree(os.path.join(work, "ckpt"), ignore_errors=True)
    env = dict(os.environ)
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    sampler = ClockSampler(local)
    sampler.start()
    t0 = time.perf_counter()
    try:
        p = subprocess.run([REF_BIN, "--config", yml, "--device", "cuda", "--resume", "none", "--log-every", "1"],
                           env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                           timeout=args.ref_timeout)
    except subprocess.TimeoutExpired:
        sampler.stop()
        return unavailable("reference run exceeded %d s" % args.ref_timeout)
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    log_path = os.path.join(work, "reference.log")
    with open(log_path, "w") as f:
        f.write(p.stdout)
    if p.returncode != 0:
        tail = " | ".join(p.stdout.strip().splitlines()[-3:])[:300]
        return unavailable("reference exited %d: %s" % (p.returncode, tail))
    if rank != 0:
        return 0
    steps = [(int(m.group(1)), float(m.group(3))) for m in STEP_RE.finditer(p.stdout)]
    timed = [s for s in steps if s[0] > args.warmup]
    if len(timed) < args.steps:
        return unavailable("could not find %d timed step lines in the reference log (%d found)" % (args.steps, len(timed)))
    # the reference reports global supervised tokens / host seconds of each step
    tok_per_step = tcfg0.batch_size * tcfg0.seq_len * tcfg0.grad_accum * world
    secs = sum(tok_per_step / max(tps, 1e-9) for _, tps in timed[:args.steps])
    value = tok_per_step * args.steps / secs
    out = {"metric": "train tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": 1e3 * secs / args.steps, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "fp16 GEMM inputs, fp32 accumulate/activations",
           "data": "synthetic", "impl": "reference", "config": recipe_label(args.config, mcfg0, tcfg0, world),
           "clocks": clocks, "timing": "the reference's own per-step tok/s (host wall clock), steps after warm-up",
           "reference_overrides": {k: v for k, v in (args.ref_set or [])},
           "wall_seconds_total": wall}
    print(json.dumps(out), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=DEFAULT_CONFIG)
    ap.add_argument("--workdir", default=os.environ.get("GB200_BENCH_DIR", "/tmp/gb200_bench"))
    ap.add_argument("--set", nargs=2, action="append", metavar=("KEY", "VALUE"), help="override a recipe key")
    ap.add_argument("--ref-timeout", type=int, default=1500)
    ap.add_argument("--ref-set", nargs=2, action="append", metavar=("KEY", "VALUE"),
                    help="recipe override for the reference arm only (e.g. training.gemm_fp16 false); default: none")
    ap.add_argument("--settle-max", type=int, default=12,
                    help="untimed steps allowed before warm-up for the dynamic loss scale to stop overflowing")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    world = env_int("WORLD_SIZE", 1)
    if world != args.gpus and env_int("RANK", 0) == 0:
        sys.stderr.write("[bench] note: --gpus %d but WORLD_SIZE=%d; using WORLD_SIZE\n" % (args.gpus, world))
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
