"""Run a few training passes of a recipe on synthetic data, eagerly (no CUDA graph), for use under a profiler:

    python -m ghassan_b200.utils.profile_step --config configs/pro_1b_2xt4.yaml --passes 2 --fuse 16
    ncu --metrics gpu__time_duration.sum --clock-control none -s <launches of pass 1> -c <launches of pass 2> \\
        --csv --log-file launches.csv python -m ghassan_b200.utils.profile_step --passes 2 --fuse 16

Prints the number of kernel launches per pass (so that ``-s`` / ``-c`` can be set) and the device time per pass.
``--layers`` shrinks the model for ``--set full`` captures, which replay every kernel many times.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=os.path.join(ROOT, "configs", "pro_1b_2xt4.yaml"))
    ap.add_argument("--passes", type=int, default=2)
    ap.add_argument("--fuse", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override model.num_layers (0 = recipe)")
    ap.add_argument("--graphs", action="store_true", help="replay CUDA graphs instead of launching eagerly")
    ap.add_argument("--end-step", action="store_true", help="also run the optimizer step")
    ap.add_argument("--workdir", default=os.path.join(tempfile.gettempdir(), "gb200_profile"))
    a = ap.parse_args(argv)
    sys.path.insert(0, ROOT)
    import torch
    import bench
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer
    from ghassan_b200.utils import log as L
    from ghassan_b200.utils.config import Config
    L.set_log_level(L.WARN)
    base = Config.from_file(a.config)
    vocab = ModelConfig.from_config(base).vocab_size
    data, tok = bench.make_data(a.workdir, vocab, TrainerConfig.from_config(base).mix)
    c = bench.load_recipe(a.config, data, os.path.join(a.workdir, "ckpt"), tok, 10)
    c.set("b200.cuda_graphs", "true" if a.graphs else "false")
    c.set("b200.fuse_micro_batches", a.fuse)
    if a.layers > 0:
        c.set("model.num_layers", a.layers)
    tr = Trainer(ModelConfig.from_config(c), TrainerConfig.from_config(c), device="cuda")
    tr.prepare()
    eng = tr.engine
    eng.begin_step(0, 64.0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(a.passes):
        group = [tr.prefetch.get() for _ in range(tr.fuse)]
        fused = tr._fused(group)
        e0.record()
        eng.micro_step(*fused)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    print("launches per pass: %d | tokens per pass: %d | device ms per pass: %s" % (
        eng.model.launches_per_micro_batch(), eng.model.N, " ".join("%.2f" % t for t in times)), flush=True)
    if a.end_step:
        e0.record()
        r = eng.end_step(1e-5)
        e1.record()
        torch.cuda.synchronize()
        print("end_step: %.2f ms %s" % (e0.elapsed_time(e1), r), flush=True)
    tr.prefetch.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
