"""The CUDA training engine against the fp32 PyTorch engine on the same data and recipe."""
import math
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _make_shards(tmp, vocab, n_docs=120, lo=30, hi=200, seed=5):
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.data.loader import write_shard
    rng = H.Rng(seed)

    def docs(n):
        out = []
        for _ in range(n):
            a = np.empty(lo + int(rng.below(hi - lo)), dtype=np.int32)
            rng.fill_uniform_ids(a, vocab - 16)
            out.append(a + 16)
        return out

    write_shard(os.path.join(tmp, "train_0000.gbin"), docs(n_docs), vocab, None)
    write_shard(os.path.join(tmp, "val_0000.gbin"), docs(30), vocab, None)


def _recipe(tmp, **over):
    from ghassan_b200.utils.config import Config
    c = Config.from_string("""
model:
  vocab_size: 608
  hidden_size: 128
  num_layers: 2
  num_heads: 4
  num_kv_heads: 2
  intermediate_size: 256
  max_seq_len: 64
  use_moe: true
  num_experts: 4
  moe_top_k: 2
  moe_expert_dim: 64
  moe_shared: true
  use_qk_norm: true
  moe_aux_scale: 0.01
  z_loss_scale: 0.0001
training:
  optimizer: adamw
  batch_size: 2
  seq_len: 64
  grad_accum: 2
  warmup_steps: 2
  max_steps: 6
  save_every: 100
  eval_every: 100
  log_every: 1
  loss_scale_init: 1024
  loss_scale_max: 1024
  ce_chunks: 2
b200:
  fuse_micro_batches: 1
""")
    c.set("training.data_dir", tmp)
    c.set("training.checkpoint_dir", os.path.join(tmp, "ckpt"))
    c.set("training.resume", "none")
    for k, v in over.items():
        c.set(k, v)
    return c


def _run(c, device, steps=None):
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer
    m, t = ModelConfig.from_config(c), TrainerConfig.from_config(c)
    tr = Trainer(m, t, device=device)
    log = []
    orig = tr.engine.end_step

    def spy(lr):
        r = orig(lr)
        log.append((r.loss, r.gnorm, r.ntok_global, r.applied))
        return r

    tr.engine.end_step = spy
    tr.run()
    return tr, log


@pytest.mark.parametrize("opt,extra", [("adamw", {}), ("lion", {"model.moe_jitter": "0.01"}),
                                       ("adamw", {"model.use_moe": "false", "training.pack_sequences": "true"}),
                                       ("adamw", {"model.moe_aux_free": "true", "model.moe_aux_scale": "0.0",
                                                  "b200.cuda_graphs": "false"}),
                                       ("lion", {"model.hidden_size": "256", "training.pack_sequences": "true",
                                                 "model.moe_expert_dim": "128"}),     # head_dim 64: tcgen05 attention
                                       ("muon", {})])
def test_cuda_engine_tracks_fp32_engine(tmp_path, opt, extra):
    tmp = str(tmp_path)
    _make_shards(tmp, 608)
    over = {"training.optimizer": opt}
    over.update(extra)
    _, ref = _run(_recipe(tmp, **over), "cpu")
    tr, got = _run(_recipe(tmp, **over), "cuda")
    assert tr.engine.kind == "cuda"
    assert len(ref) == len(got) == 6
    for (l0, g0, n0, a0), (l1, g1, n1, a1) in zip(ref, got):
        assert n0 == n1 and a0 == a1
        assert abs(l0 - l1) < 2e-2 * abs(l0), (l0, l1)
        assert abs(g0 - g1) < 8e-2 * abs(g0) + 1e-3, (g0, g1)
    # weights after 6 steps agree to fp16 accuracy
    ref_tr, _ = _run(_recipe(tmp, **over), "cpu")
    a = dict(ref_tr.engine.export_weights())
    b = dict(tr.engine.export_weights())
    for name in a:
        err = np.abs(a[name] - b[name]).max()
        assert err < 5e-3, (name, err)


def test_fused_micro_batches_give_the_same_step(tmp_path):
    """Two micro-batches run as one pass of twice the rows: same gradient sum, hence the same trajectory as the
    unfused fp32 engine (no auxiliary loss or jitter here, whose statistics are defined per pass)."""
    tmp = str(tmp_path)
    _make_shards(tmp, 608)
    over = {"model.moe_aux_free": "true", "model.moe_aux_scale": "0.0", "training.pack_sequences": "true",
            "training.grad_accum": "4"}
    _, ref = _run(_recipe(tmp, **over), "cpu")
    for fuse in ("2", "0"):         # explicit, and chosen automatically (4 here: 4 x 2 x 64 tokens fit easily)
        tr, got = _run(_recipe(tmp, **dict(over, **{"b200.fuse_micro_batches": fuse})), "cuda")
        assert tr.fuse == (2 if fuse == "2" else 4)
        assert tr.engine.model.B == 2 * tr.fuse
        for (l0, g0, n0, a0), (l1, g1, n1, a1) in zip(ref, got):
            assert n0 == n1 and a0 == a1
            assert abs(l0 - l1) < 2e-2 * abs(l0), (l0, l1)
            assert abs(g0 - g1) < 8e-2 * abs(g0) + 1e-3, (g0, g1)


def test_fused_pass_keeps_balance_loss_and_jitter_per_micro_batch(tmp_path):
    """With the auxiliary balance loss and router jitter on, a pass of several micro-batches still follows the unfused
    fp32 engine: the statistics and the jitter token index are kept per micro-batch inside the pass."""
    tmp = str(tmp_path)
    _make_shards(tmp, 608)
    over = {"model.moe_aux_scale": "0.05", "model.moe_jitter": "0.02", "training.pack_sequences": "true",
            "training.grad_accum": "4", "training.optimizer": "adamw"}
    _, ref = _run(_recipe(tmp, **over), "cpu")
    tr, got = _run(_recipe(tmp, **dict(over, **{"b200.fuse_micro_batches": "4"})), "cuda")
    assert tr.fuse == 4 and tr.engine.model.n_seg == 4 and tr.engine.model.micro_tokens == 2 * 64
    for (l0, g0, n0, a0), (l1, g1, n1, a1) in zip(ref, got):
        assert n0 == n1 and a0 == a1
        assert abs(l0 - l1) < 2e-2 * abs(l0), (l0, l1)
        assert abs(g0 - g1) < 8e-2 * abs(g0) + 1e-3, (g0, g1)
    # the routing itself is the unfused one: same experts for (almost) every token of the last pass
    ws = tr.engine.model.layers[0].ws
    assert ws.f_frac.shape == (4, 4) and float(ws.f_frac.sum(dim=1).min()) > 0.99


def test_cuda_checkpoint_roundtrip_and_resume(tmp_path):
    """A checkpoint written by the CUDA engine resumes on the CPU engine (same file format, same layout)."""
    tmp = str(tmp_path)
    _make_shards(tmp, 608)
    c = _recipe(tmp)
    c.set("training.save_every", 3)
    tr, got = _run(c, "cuda")
    path = os.path.join(tmp, "ckpt", "last.ckpt")
    assert os.path.exists(path)
    from ghassan_b200.training import checkpoint as C
    d = C.read(path)
    assert d["version"] == 12 and d["state"]["step"] == 6 and d["optimizer"]["kind"] == "adamw"
    assert d["optimizer"]["t"] == sum(1 for r in got if r[3])
    names = [n for n, _ in d["params"]]
    from ghassan_b200.models.config import ModelConfig
    assert names == [s.name for s in ModelConfig.from_config(c).param_specs()]
    c2 = _recipe(tmp)
    c2.set("training.resume", path)
    c2.set("training.max_steps", 8)
    c2.set("training.resume_mode", "migrate")
    tr2, more = _run(c2, "cpu")
    assert tr2.state.step == 8 and len(more) == 2 and all(math.isfinite(r[0]) for r in more)


def test_overflow_skips_step_and_halves_scale(tmp_path):
    tmp = str(tmp_path)
    _make_shards(tmp, 608)
    c = _recipe(tmp)
    tr, _ = _run(c, "cuda")
    eng = tr.engine
    before = eng.model.P.clone()
    t_before = eng.optimizer.t
    eng.begin_step(99, 1024.0)
    b = tr.train_loader.next()
    eng.micro_step(b.ids, b.targets, b.segments, b.B, b.T)
    eng.model.Gr[123] = float("inf")
    r = eng.end_step(1e-3)
    assert not r.applied and not math.isfinite(r.gnorm)
    assert torch.equal(eng.model.P, before) and eng.optimizer.t == t_before
    tr.scaler.scale = 1024.0
    tr.scaler.update(r.gnorm)
    assert tr.scaler.scale == 512.0
