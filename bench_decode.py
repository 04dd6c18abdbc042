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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=os.path.join(ROOT, "configs", "pro_1b_2xt4.yaml"))
    ap.add_argument("--formats", default="f16,q8_0,q4_0")
    ap.add_argument("--batches", default="1,32")
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new", type=int, default=512)
    ap.add_argument("--seed", type=int, default=1234)
    a = ap.parse_args()
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
            eng = InferenceEngine(cfg, named, fmt=fmt, batch=B, max_len=a.prompt + a.new + 8, prefill_chunk=a.prompt)
            r = Generator(eng).benchmark(a.prompt, a.new, sp, a.seed)
            r.update({"metric": "decode tokens/s", "model": os.path.splitext(os.path.basename(a.config))[0],
                      "params": cfg.count_parameters(), "weight_format": fmt, "kv_cache": "fp16",
                      "sampling": "top_p 0.9 top_k 40 temperature 0.8 seed %d" % a.seed, "data": "synthetic"})
            print(json.dumps(r), flush=True)
            del eng
            torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    sys.exit(main())
