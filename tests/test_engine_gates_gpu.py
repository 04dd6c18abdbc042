"""Engine gates of the reference's verification suite (configs/kaggle/verify_engine_suite.sh:135-226), as tests:
perplexity drift of the quantised decode path, and the memory plan against what the CUDA engine really allocates."""
import math
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
VOCAB = 608


def _learnable_shards(d, n_docs=400, seed=3):
    """Documents a small model can learn: arithmetic progressions of token ids with one of four strides."""
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.data.loader import write_shard
    rng = H.Rng(seed)

    def docs(n):
        out = []
        for _ in range(n):
            L = 40 + int(rng.below(80))
            start, stride = 16 + int(rng.below(VOCAB - 16)), (1, 3, 7, 11)[int(rng.below(4))]
            out.append(((start - 16 + stride * np.arange(L)) % (VOCAB - 16) + 16).astype(np.int32))
        return out

    write_shard(os.path.join(d, "train_0000.gbin"), docs(n_docs), VOCAB, None)
    val = docs(12)
    write_shard(os.path.join(d, "val_0000.gbin"), val, VOCAB, None)
    return val


def test_quantised_decode_perplexity_drift(tmp_path):
    """Train a small model, then score held-out documents through the decode kernels with f16, q8_0 and q4_0 weights:
    q8 may cost at most +15 % perplexity, q4 at most +60 %, and q4 must not come out better than fp16 (the reference's
    thresholds, verify_engine_suite.sh:164-195)."""
    from ghassan_b200.inference.engine import InferenceEngine
    from ghassan_b200.inference.generator import Generator
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer
    from ghassan_b200.utils.config import Config
    tmp = str(tmp_path)
    val = _learnable_shards(tmp)
    c = Config.from_string(
        "model:\n  vocab_size: %d\n  hidden_size: 128\n  num_layers: 2\n  num_heads: 4\n  num_kv_heads: 2\n"
        "  max_seq_len: 128\n  use_moe: true\n  num_experts: 4\n  moe_top_k: 2\n  moe_expert_dim: 64\n  moe_shared: true\n"
        "  use_qk_norm: true\n  moe_aux_scale: 0.01\n"
        "training:\n  optimizer: adamw\n  learning_rate: 0.004\n  batch_size: 8\n  seq_len: 64\n  grad_accum: 1\n"
        "  warmup_steps: 10\n  max_steps: 300\n  save_every: 100000\n  eval_every: 0\n  log_every: 100\n"
        "  loss_scale_init: 1024\n  loss_scale_max: 1024\n  pack_sequences: true\n" % VOCAB)
    c.set("training.data_dir", tmp)
    c.set("training.checkpoint_dir", os.path.join(tmp, "ckpt"))
    c.set("training.resume", "none")
    mcfg = ModelConfig.from_config(c)
    tr = Trainer(mcfg, TrainerConfig.from_config(c), device="cuda")
    tr.run()
    assert tr.state.last_loss < 2.5, tr.state.last_loss          # it learned the progressions (ln 608 = 6.4)
    named = dict(tr.engine.export_weights())
    ids = [int(t) for d in val for t in d][:700]
    ppl = {}
    for fmt in ("f16", "q8_0", "q4_0"):
        eng = InferenceEngine(mcfg, named, fmt=fmt, batch=1, max_len=len(ids) + 8, prefill_chunk=64)
        ppl[fmt] = Generator(eng).perplexity(ids)
        del eng
    assert all(math.isfinite(v) and v > 1.0 for v in ppl.values()), ppl
    assert ppl["f16"] < 12.0, ppl
    assert ppl["q8_0"] <= 1.15 * ppl["f16"], ppl
    assert ppl["q4_0"] <= 1.60 * ppl["f16"], ppl
    assert ppl["q4_0"] >= 0.98 * ppl["f16"], ppl                  # 4-bit weights must not look better than 16-bit


@pytest.mark.parametrize("recipe,fuse", [("flash_109m_compact_2xt4.yaml", 4), ("cpu_smoke_test.yaml", 1)])
def test_memory_plan_matches_what_the_engine_allocates(recipe, fuse):
    """The dry run's closed form against the bytes the CUDA engine holds after construction (within 5 % for a real
    recipe; the smoke recipe is so small that fixed scratch dominates and only an upper bound is checked)."""
    import dataclasses
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.cuda_engine import CudaEngine
    from ghassan_b200.training.memory_plan import memory_plan
    from ghassan_b200.utils.config import Config
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    c = Config.from_file(os.path.join(root, "configs", recipe))
    c.set("training.device", "cuda")
    mcfg, tcfg = ModelConfig.from_config(c), TrainerConfig.from_config(c)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    before = torch.cuda.memory_allocated()
    ecfg = dataclasses.replace(tcfg, batch_size=tcfg.batch_size * fuse, grad_accum=max(1, tcfg.grad_accum // fuse))
    ecfg.micro_tokens = tcfg.batch_size * tcfg.seq_len
    eng = CudaEngine(mcfg, ecfg)
    torch.cuda.synchronize()
    held = torch.cuda.memory_allocated() - before
    plan = memory_plan(mcfg, tcfg, 1, fuse)["total"]
    if recipe.startswith("flash"):
        assert abs(held - plan) <= 0.05 * held, (held, plan, held / plan)
    else:
        assert held <= plan + (64 << 20), (held, plan)
    del eng
