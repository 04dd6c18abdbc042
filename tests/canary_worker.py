"""Run by tests/test_canaries_gpu.py with GB200_CANARIES=1: training steps and decoding on awkward sizes, then the
guard bands of every buffer are checked.  Prints ``CANARIES OK <buffers>`` or the names of the buffers that were
written out of bounds."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.data.loader import write_shard
    from ghassan_b200.inference.engine import InferenceEngine, SamplingParams
    from ghassan_b200.models.config import ModelConfig, init_parameters
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer
    from ghassan_b200.utils import canary as CA
    from ghassan_b200.utils import log as L
    from ghassan_b200.utils.config import Config
    assert CA.enabled()
    L.set_log_level(L.WARN)
    work = sys.argv[1]
    r = H.Rng(3)
    docs = []
    for _ in range(160):
        a = np.empty(25 + int(r.below(140)), dtype=np.int32)
        r.fill_uniform_ids(a, 600 - 16)
        docs.append(a + 16)
    write_shard(os.path.join(work, "train_0000.gbin"), docs, 600, None)
    bad = []
    # sizes that are not multiples of the tile shapes: vocabulary 600, expert width 192, 5 + 1 experts, odd batch
    for opt, moe, B, T in (("adamw", True, 3, 96), ("lion", False, 2, 160), ("muon", True, 1, 128)):
        c = Config.from_string("""
model:
  vocab_size: 600
  hidden_size: 256
  num_layers: 2
  num_heads: 4
  num_kv_heads: 2
  intermediate_size: 320
  max_seq_len: 160
  use_moe: %s
  num_experts: 5
  moe_top_k: 2
  moe_expert_dim: 192
  moe_shared: true
  use_qk_norm: true
training:
  optimizer: %s
  batch_size: %d
  seq_len: %d
  grad_accum: 2
  warmup_steps: 1
  max_steps: 3
  eval_every: 0
  save_every: 0
""" % ("true" if moe else "false", opt, B, T))
        c.set("training.data_dir", work)
        c.set("training.checkpoint_dir", os.path.join(work, "ck_" + opt))
        tr = Trainer(ModelConfig.from_config(c), TrainerConfig.from_config(c), device="cuda")
        tr.prepare()
        for _ in range(3):
            res, _, _ = tr.train_step()
            assert np.isfinite(res.loss)
        tr.prefetch.stop()
        tr.writer.stop()
        torch.cuda.synchronize()
        bad += ["train/%s/%s" % (opt, b) for b in CA.check()]
    n_train = CA.count()
    # decoding: per-sequence kernels, the tensor-core token step, and the one-kernel step
    for kw, moe, E in ((dict(batch=1, fmt="q4_0"), True, 192), (dict(batch=3, fmt="q8_0", gemm_min_batch=2), True, 192),
                       (dict(batch=1, fmt="f16", single_kernel=True), True, 256)):
        cfg = ModelConfig(vocab_size=600, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=320,
                          max_seq_len=96, use_moe=moe, num_experts=5, moe_top_k=2, moe_expert_dim=E, moe_shared=True, use_qk_norm=True)
        cfg.validate()
        eng = InferenceEngine(cfg, init_parameters(cfg, 5), max_len=40, prefill_chunk=32, **kw)
        eng.reset(1)
        prompt = torch.randint(16, 600, (eng.B, 70), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
        eng.prefill(prompt[:, :38].contiguous())
        sp = SamplingParams(seed=3, top_k=20)
        eng.sample_first(sp)
        eng.decode_steps(30, sp)                               # past the cache size: the ring wraps
        torch.cuda.synchronize()
        bad += ["decode/%s/%s" % (kw, b) for b in CA.check()]
    if bad:
        print("CANARIES HIT", bad, flush=True)
        return 1
    print("CANARIES OK %d buffers (%d from training)" % (CA.count(), n_train), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
