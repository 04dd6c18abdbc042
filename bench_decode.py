#!/usr/bin/env python
"""Decode-throughput benchmark: random-initialised weights of a recipe's model, a synthetic uniform-random prompt,
autoregressive decoding with top-p / temperature sampling and a fixed seed, KV cache in fp16, one B200.

    python bench_decode.py [--config configs/pro_1b_2xt4.yaml] [--formats f16,q8_0,q4_0] [--batches 1,32]
                           [--prompt 1024] [--new 512]

Prints one JSON line per (format, batch): tokens/s timed on the device with CUDA events around the decode steps
(no host reads inside the timed region; the prompt pass is timed separately).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def run_reference(a):
    """The unmodified reference binary (``ghassan-ai bench``, greedy, batch 1 — it has no batched decode and no seeded
    sampling in its benchmark) on a GGUF file of the same random-initialised model, written by this repository's
    exporter (byte-compatible with the reference's own)."""
    import re
    import subprocess
    ref = os.path.join(ROOT, "baseline", "_ref", "bin", "ghassan-ai")

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0

    if not os.path.exists(ref):
        return unavailable("baseline/_ref/bin/ghassan-ai is not built")
    if re.search(r"--gemm-fp16\s+(0|false)", a.ref_args):
        # measured once on a B200: with its fp32 GEMM option the reference's own code raised "an illegal memory
        # access was encountered" (cuda/cuda_utils.cu:99); a path that faults the GPU is not run again
        return unavailable("the reference's --gemm-fp16 0 path faults on B200 (illegal memory access in its own code); not run")
    from ghassan_b200.data import synthetic as S
    from ghassan_b200.formats import gguf as G
    from ghassan_b200.models.config import ModelConfig, init_parameters
    from ghassan_b200.utils import log as L
    from ghassan_b200.utils.config import Config
    L.set_log_level(L.WARN)
    cfg = ModelConfig.from_config(Config.from_file(a.config))
    os.makedirs(a.workdir, exist_ok=True)
    tok = os.path.join(a.workdir, "synthetic.gtok")
    S.write_placeholder_gtok(tok, cfg.vocab_size)
    named = init_parameters(cfg, a.seed)
    prof = {"f16": "fp16", "q8_0": "q8_k", "q4_0": "q4_0"}
    for fmt in a.formats.split(","):
        if fmt not in prof:
            continue
        path = os.path.join(a.workdir, "model_%s.gguf" % fmt)
        G.export_gguf(path, cfg, named, tok, prof[fmt])
        cmd = [ref, "bench", "--model", path, "--device", "cuda", "--ctx", str(a.prompt + a.new + 8), "--tokens", str(a.new),
               "--prompt-tokens", str(a.prompt)] + a.ref_args.split()
        try:
            p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1500)
        except subprocess.TimeoutExpired:
            unavailable("reference bench exceeded 1500 s (%s)" % fmt)
            continue
        m = re.search(r"decode\s*:\s*(\d+) tok in .*? = ([0-9.]+) tok/s", p.stdout)
        pm = re.search(r"prefill\s*:\s*(\d+) tok in .*? = ([0-9.]+) tok/s", p.stdout)
        if p.returncode != 0 or not m:
            unavailable("reference exited %d (%s): %s" % (p.returncode, fmt, " | ".join(p.stdout.strip().splitlines()[-3:])[:300]))
            continue
        print(json.dumps({"impl": "reference", "metric": "decode tokens/s", "batch": 1, "weight_format": fmt,
                          "prompt_len": a.prompt, "new_tokens": int(m.group(1)), "decode_tokens_per_s": float(m.group(2)),
                          "prefill_tokens_per_s": float(pm.group(2)) if pm else None, "sampling": "greedy", "reference_args": a.ref_args,
                          "timing": "the reference's own host clock", "model": os.path.splitext(os.path.basename(a.config))[0]}),
              flush=True)
        os.remove(path)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=os.path.join(ROOT, "configs", "pro_1b_2xt4.yaml"))
    ap.add_argument("--formats", default="f16,q8_0,q4_0")
    ap.add_argument("--batches", default="1,32")
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new", type=int, default=512)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-args", default="", help="extra arguments for the reference binary (default: none)")
    ap.add_argument("--workdir", default=os.environ.get("GB200_BENCH_DIR", "/tmp/gb200_bench_decode"))
    ap.add_argument("--single-kernel", type=int, default=-1, help="1 / 0: force the one-kernel token step on or off (default: the engine's)")
    ap.add_argument("--trace-phases", type=int, default=0,
                    help="with the one-kernel step: print the mean time of each phase and barrier over this many tokens")
    a = ap.parse_args()
    if a.impl == "reference":
        return run_reference(a)
    import torch
    from ghassan_b200.inference.engine import InferenceEngine, SamplingParams
    from ghassan_b200.inference.generator import Generator
    from ghassan_b200.models.config import ModelConfig, init_parameters
    from ghassan_b200.utils import log as L
    from ghassan_b200.utils.config import Config
    L.set_log_level(L.WARN)
    cfg = ModelConfig.from_config(Config.from_file(a.config))
    named = init_parameters(cfg, a.seed)
    sp = SamplingParams(temperature=0.8, top_k=40, top_p=0.9, min_p=0.0, repetition_penalty=1.0, seed=a.seed)
    for fmt in a.formats.split(","):
        for B in (int(x) for x in a.batches.split(",")):
            eng = InferenceEngine(cfg, named, fmt=fmt, batch=B, max_len=a.prompt + a.new + 8, prefill_chunk=a.prompt,
                                  single_kernel=None if a.single_kernel < 0 else bool(a.single_kernel))
            r = Generator(eng).benchmark(a.prompt, a.new, sp, a.seed)
            r["token_step"] = ("one cooperative kernel" if eng.mega is not None else
                               "tensor-core GEMMs over 16-bit weight copies" if eng.batched else "GEMV kernel chain over the stored bytes")
            if a.trace_phases > 0 and eng.mega is not None:
                r["phase_us"] = eng.trace_phases(a.trace_phases)
            r.update({"metric": "decode tokens/s", "model": os.path.splitext(os.path.basename(a.config))[0],
                      "params": cfg.count_parameters(), "weight_format": fmt, "kv_cache": "fp16",
                      "sampling": "top_p 0.9 top_k 40 temperature 0.8 seed %d" % a.seed, "data": "synthetic"})
            print(json.dumps(r), flush=True)
            del eng
            torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    sys.exit(main())
