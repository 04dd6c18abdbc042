#!/usr/bin/env python
"""Training-throughput benchmark: train tokens/s on the pro_1b recipe (configs/pro_1b_2xt4.yaml), synthetic
uniform token data, random-initialised weights.

    python bench.py --gpus N --steps K --warmup W                  # this framework
    python bench.py --impl reference --gpus N --steps K --warmup W  # the unmodified reference binary
    python bench.py --profile-passes 2 [--fuse F] [--layers L] [--end-step]   # a few eager passes, for use under ncu
    python bench.py --sync-only                                     # the gradient exchange alone (one process per GPU)

With one GPU the JSON line also carries a ``decode`` object: batch-1 decode tokens/s of the same model for f16, q8_0 and
q4_0 weights (device-timed; ``--no-decode`` skips it, ``bench_decode.py`` has the full table with batch 32).

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

    def __init__(self, index=0, period_ms=100):
        self.index, self.period_ms = index, period_ms
        self.proc = None
        self.lines = []            # (host time of arrival, line)
        self._t = None
        self._begin = 0.0

    def begin(self):
        """The timed region starts now: samples that arrived earlier (the tool takes a few hundred milliseconds to
        print its first line, so it is started ahead of the region) are not counted."""
        self._begin = time.time()

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
            self.lines.append((time.time(), ln.strip()))

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
        for at, ln in self.lines:
            if at < self._begin:
                continue
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
    sampler = ClockSampler(local)
    for i in range(args.warmup):
        if i == args.warmup - 1:
            sampler.start()        # running by the time the timed region starts
        tr.train_step()

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- phase A: device-timed
    fence()
    if sampler.proc is None:
        sampler.start()
    sampler.begin()
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
                                            grad_sync=(("fused NVSwitch multicast" if getattr(eng.grad_sync, "nvls", False)
                                                        else "fused peer-memory") if eng.grad_sync is not None else
                                                       ("nccl" if world > 1 else "none"))), "clocks": clocks,
           "e2e": {"value": toks_e / sec_e, "unit": "tokens/s",
                   "h2d_bytes_per_step": tcfg.grad_accum * tcfg.batch_size * tcfg.seq_len * 4 * n_in + 64,
                   "d2h_bytes_per_step": 40},
           "gpu_launches": int(launches), "optimizer_steps_applied": applied, "settle_steps": settle,
           "loss_first": losses[0], "loss_last": losses[-1],
           "supervised_tokens_per_step": toks / args.steps}
    if world == 1 and not args.no_decode:
        del tr, eng
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        try:
            out["decode"] = run_decode(args, local)
        except Exception as e:        # the training number stands on its own
            out["decode"] = {"error": "%s: %s" % (type(e).__name__, str(e)[:200])}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_decode(args, local):
    """Decode of the recipe's model (random-initialised): one sequence for three weight formats and 32 sequences for
    two, tokens/s with CUDA events around the decode steps, SM clocks sampled meanwhile.  Runs after the training
    measurement has released the GPU."""
    import torch
    from ghassan_b200.inference.engine import InferenceEngine, SamplingParams
    from ghassan_b200.inference.generator import Generator
    from ghassan_b200.models.config import ModelConfig, init_parameters
    from ghassan_b200.utils.config import Config
    cfg = ModelConfig.from_config(Config.from_file(args.config))
    named = init_parameters(cfg, 1234)
    sp = SamplingParams(temperature=0.8, top_k=40, top_p=0.9, min_p=0.0, repetition_penalty=1.0, seed=1234)
    out = {"batch": 1, "prompt_len": args.decode_prompt, "new_tokens": args.decode_new, "kv_cache": "fp16",
           "sampling": "top_p 0.9 top_k 40 temperature 0.8 seed 1234", "timing": "CUDA events around the decode steps"}
    sampler = ClockSampler(local)
    sampler.start()
    for fmt in ("f16", "q8_0", "q4_0"):
        eng = InferenceEngine(cfg, named, fmt=fmt, batch=1, max_len=args.decode_prompt + args.decode_new + 8,
                              prefill_chunk=args.decode_prompt)
        r = Generator(eng).benchmark(args.decode_prompt, args.decode_new, sp, 1234)
        out[fmt] = {"tokens_per_s": r["decode_tokens_per_s"], "ms_per_token": r["decode_ms_per_token"],
                    "stored_weight_bytes": r["stored_weight_bytes"], "prefill_ms": r["prefill_ms"],
                    "token_step": "one cooperative kernel" if eng.mega is not None else "kernel chain"}
        del eng
        torch.cuda.empty_cache()
    # 32 sequences: the token step runs its projections and experts as tensor-core GEMMs over 16-bit weight copies
    out["batch_32"] = {"token_step": "tcgen05 GEMMs over 16-bit weight copies, attention per sequence over the cache",
                       "new_tokens": min(args.decode_new, 128)}
    for fmt in ("f16", "q4_0"):
        eng = InferenceEngine(cfg, named, fmt=fmt, batch=32, max_len=args.decode_prompt + args.decode_new + 8,
                              prefill_chunk=args.decode_prompt)
        r = Generator(eng).benchmark(args.decode_prompt, min(args.decode_new, 128), sp, 1234)
        out["batch_32"][fmt] = {"tokens_per_s": r["decode_tokens_per_s"], "ms_per_step": r["decode_ms_per_token"],
                                "prefill_ms": r["prefill_ms"]}
        del eng
        torch.cuda.empty_cache()
    out["clocks"] = sampler.stop()
    return out


def run_sync(args):
    """The gradient exchange alone on buffers of the recipe's size (default: the 1.04 G parameters of pro_1b), one
    process per GPU: barrier, reduce-scatter + norm by peer loads, Lion update of the own shard, barrier, all-gather of
    the 16-bit weights and the fp32 prefix by peer loads.  Device time, max over ranks, against one NCCL all-reduce of
    the same fp32 gradient (which does no norm and no optimizer).  Launch like the training bench:

        python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench.py --sync-only
    """
    import torch
    import torch.distributed as dist
    from ghassan_b200.ops import _lib, comm as C
    from ghassan_b200.parallel.grad_sync import SymmetricBuffers
    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    torch.cuda.set_device(local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    total = (args.sync_elements + 63) // 64 * 64
    buf = SymmetricBuffers(multicast=bool(args.nvls))
    shard = ((total + world - 1) // world + 63) // 64 * 64
    pad = shard * world
    P, tP = buf.alloc(pad, torch.float32)
    W16, tW = buf.alloc(pad, torch.float16)
    Gr, tG = buf.alloc(pad, torch.float32)
    ctl, tC = buf.alloc(C.CTL_WORDS, torch.int32)
    Gr.normal_()
    m = torch.zeros(pad, device=dev)
    partial = torch.zeros(C.SYNC_BLOCKS, dtype=torch.float64, device=dev)
    ticket = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(4, device=dev)
    hyper = torch.tensor([1e-5, 0.1, 0.01], device=dev)
    f32_end = min(total, 25_400_000 // 64 * 64)
    a = C.SyncArgs()
    a.rank, a.world, a.shard, a.total = rank, world, shard, total
    a.decay_start, a.f32_end = min(total, 25_000_000 // 64 * 64), f32_end
    a.peer_grad, a.peer_master, a.peer_w16, a.peer_ctl = tG.data_ptr(), tP.data_ptr(), tW.data_ptr(), tC.data_ptr()
    a.m, a.v, a.kind = m.data_ptr(), None, 1
    a.beta1, a.beta2, a.eps, a.wd = 0.9, 0.99, 1e-8, 0.1
    a.hyper, a.loss_scale, a.clip, a.ntok_local = hyper.data_ptr(), 1024.0, 1.0, 32768.0
    a.partial, a.ticket, a.out = partial.data_ptr(), ticket.data_ptr(), out.data_ptr()
    a.status = _lib.status_word(dev).data_ptr()
    a.is_bf16, a.no_wait, a.local_only = 0, 0, 1
    nvls = bool(args.nvls) and all(buf.mc_ptrs[:3])
    if nvls:                       # reduce in the switch, distribute with multicast stores: no gather afterwards
        a.mc_master, a.mc_w16, a.mc_grad = buf.mc_ptrs[0], buf.mc_ptrs[1], buf.mc_ptrs[2]
    elif args.nvls and rank == 0:
        print("[sync] no multicast address for the symmetric buffers: peer loads", file=sys.stderr, flush=True)
    state = {"be": 0}

    def bar():
        state["be"] += 1
        C.barrier(tC, rank, world, state["be"])

    def exchange(epoch, ev=None):
        a.epoch = epoch
        bar()
        if ev: ev[0].record()
        C.reduce(a)
        if ev: ev[1].record()
        C.update(a)
        if ev: ev[2].record()
        bar()
        if ev: ev[3].record()
        if not nvls:
            C.gather(tW, W16, shard, total, rank, world)
            C.gather(tP, P, shard, f32_end, rank, world)
        if ev: ev[4].record()

    torch.cuda.synchronize()
    dist.barrier()
    for e in range(1, 4):
        exchange(e)
    torch.cuda.synchronize()
    _lib.check_status(dev, "exchange")
    dist.barrier()
    iters = max(3, args.steps)
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for e in range(4, 4 + iters):
        exchange(e)
    bar()                         # the barrier that opens the next exchange belongs to the cycle
    e1.record()
    torch.cuda.synchronize()
    fused_ms = e0.elapsed_time(e1) / iters
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(iters)]
    for k in range(iters):
        exchange(4 + iters + k, evs[k])
    torch.cuda.synchronize()
    clocks = sampler.stop()
    phase = lambda i, j: sum(x[i].elapsed_time(x[j]) for x in evs) / iters
    reduce_ms, update_ms, gather_ms = phase(0, 1), phase(1, 2), phase(3, 4)
    g2 = torch.randn(total, device=dev)
    for _ in range(2):
        dist.all_reduce(g2)
    torch.cuda.synchronize()
    dist.barrier()
    e0.record()
    for _ in range(iters):
        dist.all_reduce(g2)
    e1.record()
    torch.cuda.synchronize()
    nccl_ms = e0.elapsed_time(e1) / iters
    t = torch.tensor([fused_ms, nccl_ms, reduce_ms, update_ms, gather_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    fused_ms, nccl_ms, reduce_ms, update_ms, gather_ms = (float(x) for x in t)
    # Bytes that cross each direction of a GPU's NVLink per exchange: it reads W-1 peer shards of fp32 gradient and
    # W-1 peer shards of new weights (16-bit everywhere, fp32 below f32_end), and serves the same amounts to its peers.
    per_dir = (world - 1) * (shard * 4 + shard * 2) + max(0, min(f32_end, total) - shard) * 4
    if nvls:                       # the switch adds and copies: a GPU receives one reduced shard and every new weight once
        per_dir = shard * 4 + (world - 1) * shard * 2 + max(0, min(f32_end, total) - shard) * 4
    roof_ms = per_dir / 770e9 * 1e3
    if rank == 0:
        print(json.dumps({"bench": "fused_grad_sync", "world": world, "path": "NVSwitch multicast (multimem)" if nvls else "peer loads", "elements": total, "fused_ms": fused_ms,
                          "reduce_scatter_phase_ms": reduce_ms, "update_phase_ms": update_ms,
                          "allgather_phase_ms": gather_ms, "nccl_allreduce_only_ms": nccl_ms,
                          "nvlink_bytes_per_direction": per_dir, "roofline_ms_at_770GBs_per_direction": roof_ms,
                          "fraction_of_roofline": roof_ms / fused_ms if world > 1 else None, "clocks": clocks,
                          "note": "fused = barrier + reduce-scatter + norm + mailbox + Lion update + barrier + all-gather "
                                  "of 16-bit weights and fp32 prefix by peer loads; the NCCL figure is the all-reduce "
                                  "alone (no norm, no optimizer, fp32 result only)"}), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


def run_profile_passes(args):
    """A few training passes launched eagerly (no CUDA graph) so that a profiler sees every kernel:

        CMD="python bench.py --profile-passes 2 --fuse 64"
        $CMD > plain.log 2>&1 && ncu --metrics gpu__time_duration.sum --clock-control none -c 6000 --csv \
            --log-file launches.csv $CMD

    Prints the launches and device milliseconds per pass.  ``--layers`` shrinks the model for ``--set full`` captures."""
    import torch
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer
    from ghassan_b200.utils import log as L
    from ghassan_b200.utils.config import Config
    L.set_log_level(L.WARN)
    torch.cuda.set_device(env_int("LOCAL_RANK", 0))
    base = Config.from_file(args.config)
    work = os.path.join(args.workdir, "profile")
    data, tok = make_data(work, ModelConfig.from_config(base).vocab_size, TrainerConfig.from_config(base).mix)
    c = load_recipe(args.config, data, os.path.join(work, "ckpt"), tok, 10)
    c.set("b200.cuda_graphs", "true" if args.graphs else "false")
    c.set("b200.fuse_micro_batches", args.fuse)
    if args.layers > 0:
        c.set("model.num_layers", args.layers)
    for k, v in (args.set or []):
        c.set(k, v)
    tr = Trainer(ModelConfig.from_config(c), TrainerConfig.from_config(c), device="cuda")
    tr.prepare()
    eng = tr.engine
    eng.begin_step(0, 64.0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(args.profile_passes):
        fused = tr._fused([tr.prefetch.get() for _ in range(tr.fuse)])
        e0.record()
        eng.micro_step(*fused)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    print("launches per pass: %d | tokens per pass: %d | device ms per pass: %s" % (
        eng.model.launches_per_micro_batch(), eng.model.N, " ".join("%.2f" % t for t in times)), flush=True)
    if args.end_step:
        e0.record()
        r = eng.end_step(1e-5)
        e1.record()
        torch.cuda.synchronize()
        print("end_step: %.2f ms %s" % (e0.elapsed_time(e1), r), flush=True)
    tr.prefetch.stop()
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
    ap.add_argument("--no-decode", action="store_true", help="skip the batch-1 decode measurement of the 1-GPU run")
    ap.add_argument("--decode-prompt", type=int, default=1024)
    ap.add_argument("--decode-new", type=int, default=256)
    ap.add_argument("--profile-passes", type=int, default=0, help="run this many eager passes and exit (for profilers)")
    ap.add_argument("--fuse", type=int, default=0, help="--profile-passes: micro-batches per pass (0 = automatic)")
    ap.add_argument("--layers", type=int, default=0, help="--profile-passes: override model.num_layers")
    ap.add_argument("--graphs", action="store_true", help="--profile-passes: replay CUDA graphs instead of eager launches")
    ap.add_argument("--end-step", action="store_true", help="--profile-passes: also run the optimizer step")
    ap.add_argument("--sync-only", action="store_true", help="time the gradient exchange alone (see run_sync)")
    ap.add_argument("--nvls", action="store_true", help="--sync-only: reduce and distribute through NVSwitch multicast")
    ap.add_argument("--sync-elements", type=int, default=1_036_995_840)
    args = ap.parse_args()
    if args.profile_passes > 0:
        return run_profile_passes(args)
    if args.sync_only:
        return run_sync(args)
    world = env_int("WORLD_SIZE", 1)
    if world != args.gpus and env_int("RANK", 0) == 0:
        sys.stderr.write("[bench] note: --gpus %d but WORLD_SIZE=%d; using WORLD_SIZE\n" % (args.gpus, world))
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
