"""Trainer behaviour on the CPU engine: learning, bit-exact resume, resume gates, checkpoint publication."""
import os
import shutil
import threading
import time

import numpy as np
import pytest
import torch

VOCAB = 320


def _docs(seed, n, lo, hi):
    from ghassan_b200 import _gb200_host as H
    r = H.Rng(seed)
    out = []
    for _ in range(n):
        a = np.empty(lo + int(r.below(hi - lo)), dtype=np.int32)
        r.fill_uniform_ids(a, 40)          # a small alphabet so that a tiny model learns something
        out.append(a + 16)
    return out


@pytest.fixture(scope="module")
def data_dir(tmp_path_factory):
    from ghassan_b200.data.loader import write_shard
    d = str(tmp_path_factory.mktemp("shards"))
    write_shard(os.path.join(d, "train_0000.gbin"), _docs(1, 150, 20, 120), VOCAB, None)
    write_shard(os.path.join(d, "val_0000.gbin"), _docs(2, 30, 20, 120), VOCAB, None)
    return d


def _recipe(data_dir, ckpt_dir, **over):
    from ghassan_b200.utils.config import Config
    c = Config.from_string("""
model:
  vocab_size: %d
  hidden_size: 64
  num_layers: 2
  num_heads: 4
  num_kv_heads: 2
  intermediate_size: 128
  max_seq_len: 32
  use_moe: true
  num_experts: 4
  moe_top_k: 2
  moe_expert_dim: 64
  moe_shared: true
  use_qk_norm: true
  moe_aux_free: true
  moe_aux_scale: 0.0
training:
  optimizer: adamw
  learning_rate: 0.003
  batch_size: 2
  seq_len: 32
  grad_accum: 2
  warmup_steps: 2
  max_steps: 8
  save_every: 100
  eval_every: 4
  eval_batches: 2
  log_every: 100
  pack_sequences: true
  resume: none
  resume_mode: exact
""" % VOCAB)
    c.set("training.data_dir", data_dir)
    c.set("training.checkpoint_dir", ckpt_dir)
    for k, v in over.items():
        c.set(k if "." in k else "training." + k, v)
    return c


def _trainer(c):
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer
    return Trainer(ModelConfig.from_config(c), TrainerConfig.from_config(c), device="cpu")


def _params(path):
    from ghassan_b200.training import checkpoint as C
    return C.read(path)


def test_loss_goes_down(data_dir, tmp_path):
    tr = _trainer(_recipe(data_dir, str(tmp_path / "ck"), max_steps=30))
    tr.prepare()
    losses = [tr.train_step()[0].loss for _ in range(30)]
    tr.prefetch.stop()
    assert all(np.isfinite(losses))
    assert np.mean(losses[-5:]) < np.mean(losses[:5]) - 0.3


@pytest.mark.parametrize("opt", ["adamw", "lion", "muon"])
def test_exact_resume_is_bit_identical(data_dir, tmp_path, opt):
    ck = str(tmp_path / "ck")
    a = _trainer(_recipe(data_dir, ck, optimizer=opt))
    a.prepare()
    a.writer.start()
    for _ in range(4):
        a.train_step()
    a.save("mid.ckpt")
    a.writer.wait()
    shutil.copy(os.path.join(ck, "mid.ckpt"), str(tmp_path / "mid.ckpt"))
    for _ in range(4):
        a.train_step()
    a.save("end.ckpt")
    a.writer.wait()
    a.prefetch.stop()
    a.writer.stop()
    ck2 = str(tmp_path / "ck2")
    b = _trainer(_recipe(data_dir, ck2, optimizer=opt, resume=str(tmp_path / "mid.ckpt"), eval_every=0))
    assert b.state.step == 4
    b.run()
    A, B = _params(os.path.join(ck, "end.ckpt")), _params(os.path.join(ck2, "last.ckpt"))
    assert B["state"]["step"] == 8 and A["state"]["tokens_seen"] == B["state"]["tokens_seen"]
    for (n, x), (m, y) in zip(A["params"], B["params"]):
        assert n == m and np.array_equal(np.asarray(x), np.asarray(y)), n
    assert A["state"]["loader"] == B["state"]["loader"]
    for x, y in zip(A["moe_bias"], B["moe_bias"]):
        assert np.array_equal(np.asarray(x), np.asarray(y))


@pytest.fixture()
def saved(data_dir, tmp_path):
    ck = str(tmp_path / "ck")
    tr = _trainer(_recipe(data_dir, ck, max_steps=8, eval_every=0))
    tr.prepare()
    tr.writer.start()
    for _ in range(3):
        tr.train_step()
    tr.save("last.ckpt")
    tr.writer.wait()
    tr.prefetch.stop()
    tr.writer.stop()
    return ck


def test_auto_resume_picks_last(data_dir, saved):
    tr = _trainer(_recipe(data_dir, saved, resume="auto"))
    assert tr.state.step == 3
    tr.prefetch.stop()


@pytest.mark.parametrize("change,fragment", [
    ({"model.num_layers": 3}, "architecture"),
    ({"learning_rate": 0.001}, "scheduler"),
    ({"warmup_steps": 3}, "scheduler"),
    ({"scheduler": "wsd"}, "scheduler"),
    ({"optimizer": "lion"}, "exact"),
    ({"beta2": 0.99}, "exact"),
    ({"model.rope_theta": 50000}, "drift"),
])
def test_exact_resume_refusals(data_dir, saved, change, fragment):
    from ghassan_b200.training.trainer import TrainerError
    with pytest.raises(TrainerError) as e:
        _trainer(_recipe(data_dir, saved, resume="auto", **change))
    assert fragment in str(e.value)


def test_exact_resume_refuses_a_different_step_budget(data_dir, saved):
    from ghassan_b200.training.trainer import TrainerError
    tr = _trainer(_recipe(data_dir, saved, resume="auto", max_steps=12))
    with pytest.raises(TrainerError) as e:
        tr.prepare()
    assert "planned total" in str(e.value)
    tr.prefetch.stop()


def test_migrate_mode_accepts_what_exact_refuses(data_dir, saved):
    tr = _trainer(_recipe(data_dir, saved, resume="auto", resume_mode="migrate", optimizer="lion", learning_rate=0.0005))
    assert tr.state.step == 3          # weights and counters restored, moments fresh
    tr.prepare()
    res = tr.train_step()[0]
    assert np.isfinite(res.loss)
    tr.prefetch.stop()


def test_trailing_bytes_and_truncation(data_dir, saved):
    from ghassan_b200.training.trainer import TrainerError
    p = os.path.join(saved, "last.ckpt")
    blob = open(p, "rb").read()
    open(p, "ab").write(b"\0" * 7)
    with pytest.raises(TrainerError):
        _trainer(_recipe(data_dir, saved, resume="auto"))
    open(p, "wb").write(blob[:len(blob) // 2])
    with pytest.raises(TrainerError):
        _trainer(_recipe(data_dir, saved, resume="auto"))
    # migrate mode falls back to a fresh start on an unreadable file
    tr = _trainer(_recipe(data_dir, saved, resume="auto", resume_mode="migrate"))
    assert tr.state.step == 0
    tr.prefetch.stop()


def test_tokenizer_fingerprint_gate(data_dir, tmp_path):
    from ghassan_b200.training.trainer import TrainerError
    ck = str(tmp_path / "ck")
    tr = _trainer(_recipe(data_dir, ck, eval_every=0, tok_fingerprint=1234))
    tr.prepare()
    tr.train_step()
    tr.save("last.ckpt")
    tr.writer.wait()
    tr.prefetch.stop()
    with pytest.raises(TrainerError) as e:
        _trainer(_recipe(data_dir, ck, resume="auto", tok_fingerprint=99))
    assert "tokenizer mismatch" in str(e.value)
    ok = _trainer(_recipe(data_dir, ck, resume="auto", tok_fingerprint=1234))
    assert ok.state.step == 1
    ok.prefetch.stop()


def test_sft_needs_a_pretrained_checkpoint(data_dir, tmp_path):
    from ghassan_b200.training.trainer import TrainerError
    with pytest.raises(TrainerError) as e:
        _trainer(_recipe(data_dir, str(tmp_path / "ck"), stage="sft"))
    assert "pretrained" in str(e.value) or "loss masks" in str(e.value)
    # with the pretrained gate waived the next gate is the data: SFT shards must carry assistant-span masks
    with pytest.raises(TrainerError) as e:
        _trainer(_recipe(data_dir, str(tmp_path / "ck"), stage="sft", allow_no_pretrained="true"))
    assert "loss masks" in str(e.value)
    from ghassan_b200.data.loader import write_shard
    d = str(tmp_path / "sft")
    os.makedirs(d)
    docs = _docs(9, 40, 20, 60)
    write_shard(os.path.join(d, "train_0000.gbin"), docs, VOCAB, [np.arange(len(x)) % 2 for x in docs])
    tr = _trainer(_recipe(d, str(tmp_path / "ck"), stage="sft", allow_no_pretrained="true", eval_every=0))
    tr.prepare()
    res = tr.train_step()[0]
    tr.prefetch.stop()
    assert 0 < res.ntok_global < 2 * 2 * 32          # only masked-in positions are supervised


def test_writer_links_second_name_and_applies_back_pressure(tmp_path):
    from ghassan_b200.training import checkpoint as C

    class Snap:
        def __init__(self, n):
            self.n, self.state = n, {}

        def nbytes(self):
            return self.n

    written, gate = [], threading.Event()
    w = C.CheckpointWriter(ram_budget=100)

    def slow_write(snap, path):
        gate.wait(5)
        written.append(path)

    w._write = slow_write
    w.start()
    a, b = Snap(80), Snap(80)
    w.submit(a, "a1")
    w.submit(a, "a2")                      # same snapshot twice: counted once
    assert w.queued_bytes() == 80
    blocked = threading.Event()

    def later():
        w.submit(b, "b1")                  # 80 + 80 > 100: must wait for the first to drain
        blocked.set()

    t = threading.Thread(target=later)
    t.start()
    time.sleep(0.4)
    assert not blocked.is_set()
    gate.set()
    t.join(5)
    assert blocked.is_set()
    w.wait()
    w.stop()
    assert written == ["a1", "a2", "b1"]


def test_writer_never_links_a_new_snapshot_to_an_old_file(tmp_path, monkeypatch):
    """last.ckpt at step A, snapshot freed, best.ckpt from a new snapshot at step B: best must hold step B even when
    the new object reuses the old one's id()."""
    import gc
    from ghassan_b200.training import checkpoint as C

    saved = {}

    def fake_save(snap, path):
        with open(path, "w") as f:
            f.write(str(snap.state["step"]))
        saved[path] = snap.state["step"]

    monkeypatch.setattr(C, "save_snapshot", fake_save)

    class Snap:
        def __init__(self, step):
            self.state = {"step": step}

        def nbytes(self):
            return 8

    for trial in range(20):
        w = C.CheckpointWriter(ram_budget=1 << 20)
        last, best = str(tmp_path / ("last%d" % trial)), str(tmp_path / ("best%d" % trial))
        a = Snap(100 + trial)
        w.submit(a, last)
        del a
        gc.collect()
        b = Snap(200 + trial)              # often gets the id of the freed object
        w.submit(b, best)
        w.submit(b, last + ".second")      # the same snapshot under a second name is still a link to its own file
        assert open(best).read() == str(200 + trial)
        assert open(last + ".second").read() == str(200 + trial)
        assert os.path.samefile(best, last + ".second")


def test_latest_in_order(tmp_path):
    from ghassan_b200.training import checkpoint as C
    d = str(tmp_path)
    assert C.latest_in(d) == ""
    open(os.path.join(d, "step_0001.ckpt"), "w").close()
    open(os.path.join(d, "step_0002.ckpt"), "w").close()
    assert C.latest_in(d).endswith("step_0002.ckpt")
    open(os.path.join(d, "last.ckpt.bak"), "w").close()
    assert C.latest_in(d).endswith("last.ckpt.bak")
    open(os.path.join(d, "last.ckpt"), "w").close()
    assert C.latest_in(d).endswith("last.ckpt")


def test_expert_load_report_text_and_reset(data_dir, tmp_path):
    """The evaluation log's expert-load line: shares of routed slots per layer, '!' on a lopsided layer
    (model/model.cpp:107-127 in the reference), accumulated over training steps and reset by the report."""
    import torch
    from ghassan_b200.training.engine import format_balance_report
    acc = torch.tensor([[10.0, 10.0, 10.0, 10.0], [1.0, 0.0, 30.0, 9.0], [0.0, 0.0, 0.0, 0.0]])
    assert format_balance_report(acc, 4) == "expert load (share of routed slots): L0[0.25..0.25] L1[0.00..0.75]!"
    assert format_balance_report(None, 4) == "" and format_balance_report(acc[2:], 4) == ""
    tr = _trainer(_recipe(data_dir, str(tmp_path / "ck"), eval_every=0))
    tr.prepare()
    tr.train_step()
    tr.prefetch.stop()
    rep = tr.engine.balance_report()
    assert rep.startswith("expert load (share of routed slots): L0[") and " L1[" in rep
    assert tr.engine.balance_report() == ""            # reset by the report
