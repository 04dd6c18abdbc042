"""Trainer resource guards against faked machine sizes (the reference's guards: training/trainer.cpp:672-836)."""
import os

import pytest

from ghassan_b200.training import guards as G

GIB = 1 << 30


def _probe(**kw):
    base = dict(gpu_total=lambda: 180 * GIB, gpu_free_live=lambda: 170 * GIB, ram_total=lambda: 64 * GIB,
                disk_free=lambda p: 500 * GIB, tree_size=lambda root, skip: (0, 0), file_size=lambda p: 0,
                same_file=lambda a, b: False, exists=lambda p: False)
    base.update(kw)
    return G.Probe(**base)


def test_device_memory_guard_static_and_live():
    G.check_device_memory(100 * GIB, 0, 1, _probe(), True)                          # 56 %: fine
    with pytest.raises(G.GuardError, match="OOM guard: need"):
        G.check_device_memory(175 * GIB, 0, 1, _probe(), True)                      # above 95 % with slack
    with pytest.raises(G.GuardError, match=r"OOM guard \(live\)"):
        G.check_device_memory(100 * GIB, 0, 1, _probe(gpu_free_live=lambda: 60 * GIB), True)
    # what is already allocated by this process does not count against the live figure
    G.check_device_memory(100 * GIB, 50 * GIB, 1, _probe(gpu_free_live=lambda: 60 * GIB), True)
    G.check_device_memory(10 ** 15, 0, 1, _probe(gpu_total=lambda: 0), True)        # unknown device size: passes
    G.check_device_memory(10 ** 15, 0, 1, _probe(), False)                          # CPU engine: not checked


def test_more_slack_with_peers():
    p = _probe(gpu_total=lambda: 100 * GIB, gpu_free_live=lambda: 100 * GIB)
    core = int(0.95 * 100 * GIB) - 1024 * G.MIB - 8 * G.MIB
    G.check_device_memory(core, 0, 1, p, True)
    with pytest.raises(G.GuardError):
        G.check_device_memory(core, 0, 8, p, True)


def test_host_ram_guard_needs_two_snapshots():
    per = G.snapshot_bytes(1_000_000_000, "lion")                                  # 8 GB
    assert per == 8_000_000_000 and G.snapshot_bytes(1_000_000_000, "adamw") == 12_000_000_000
    G.check_host_ram(per, 8 * GIB, _probe(ram_total=lambda: 32 * GIB))
    with pytest.raises(G.GuardError, match="host RAM guard"):
        G.check_host_ram(per, 8 * GIB, _probe(ram_total=lambda: 15 * GIB))
    G.check_host_ram(per, 8 * GIB, _probe(ram_total=lambda: 0))                     # unknown: passes


def test_disk_guard_counts_published_checkpoints_once_when_linked():
    per = 8 * GIB
    d = "/x/ckpt"
    G.check_disk(d, per, _probe(disk_free=lambda p: 11 * GIB))                      # nothing published: 1.25 snapshots
    with pytest.raises(G.GuardError, match="disk guard"):
        G.check_disk(d, per, _probe(disk_free=lambda p: 9 * GIB))
    both = dict(exists=lambda p: True)
    with pytest.raises(G.GuardError):                                               # two files + .tmp + margin = 26 GiB
        G.check_disk(d, per, _probe(disk_free=lambda p: 20 * GIB, **both))
    G.check_disk(d, per, _probe(disk_free=lambda p: 20 * GIB, same_file=lambda a, b: True, **both))   # one inode: 18 GiB
    G.check_disk(d, per, _probe(disk_free=lambda p: 0))                             # cannot stat: warns, passes


def test_output_quota_guard(tmp_path):
    per, n = 8 * GIB, 1_000_000_000
    d = str(tmp_path / "working" / "run" / "ckpt")
    os.makedirs(d)
    assert G.quota_root(d) == str(tmp_path / "working")
    assert G.quota_root(str(tmp_path / "elsewhere" / "ckpt")) == os.path.abspath(".")
    used = {"v": 1 * GIB}
    p = _probe(tree_size=lambda root, skip: (used["v"], 3))
    G.check_output_quota(0, d, per, n, p)                                           # no budget: off
    G.check_output_quota(20 * 1024, d, per, n, p)                                   # 1 + 16 + ~1.9 GiB < 20 GiB
    used["v"] = 3 * GIB
    with pytest.raises(G.GuardError, match="output quota guard"):
        G.check_output_quota(20 * 1024, d, per, n, p)
    # a pre-trained checkpoint inside the tree is loaded, not kept: its size is taken off
    G.check_output_quota(20 * 1024, d, per, n, _probe(tree_size=lambda r, s: (used["v"], 3), file_size=lambda f: 2 * GIB),
                         pretrained="/x/pre.ckpt")


def test_native_probes_on_a_real_tree(tmp_path):
    from ghassan_b200 import _gb200_host as H
    a = tmp_path / "a"
    (a / "build").mkdir(parents=True)
    (a / "keep").mkdir()
    (a / "keep" / "f1").write_bytes(b"x" * 1000)
    os.link(a / "keep" / "f1", a / "keep" / "f1_again")                             # a second name: counted once
    (a / "build" / "junk").write_bytes(b"y" * 5000)
    os.symlink(a / "keep" / "f1", a / "link")
    assert tuple(H.tree_size_bytes(str(a), ["build"])) == (1000, 1)
    assert tuple(H.tree_size_bytes(str(a), [])) == (6000, 2)
    assert tuple(H.tree_size_bytes(str(a / "missing"), [])) == (0, 0)
    assert H.free_disk_bytes(str(a / "not" / "yet" / "made")) > 0
    assert H.physical_ram_bytes() > (1 << 28)


def test_trainer_refuses_before_training(tmp_path, monkeypatch):
    """The guards run inside the Trainer constructor, after the loaders open and before a resume."""
    import numpy as np
    from ghassan_b200.data.synthetic import make_corpus
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer, TrainerError
    from ghassan_b200.utils.config import Config
    data = str(tmp_path / "shards")
    make_corpus(data, 600, train_tokens=6000, val_tokens=600, mean_doc=40)
    c = Config.from_string(
        "model:\n  vocab_size: 600\n  hidden_size: 32\n  num_layers: 1\n  num_heads: 2\n  num_kv_heads: 1\n"
        "  max_seq_len: 32\n  num_experts: 4\n  moe_top_k: 2\n  moe_expert_dim: 32\n"
        "training:\n  batch_size: 2\n  seq_len: 16\n  grad_accum: 1\n  max_steps: 2\n  optimizer: adamw\n  device: cpu\n")
    c.set("training.data_dir", data)
    c.set("training.checkpoint_dir", str(tmp_path / "ck"))
    c.set("training.resume", "none")
    real = G.Probe
    small, fine = _probe(disk_free=lambda p: 1000), _probe()
    monkeypatch.setattr(G, "Probe", lambda *a, **k: real(*a, **k) if (a or k) else small)
    with pytest.raises(TrainerError, match="disk guard"):
        Trainer(ModelConfig.from_config(c), TrainerConfig.from_config(c), device="cpu")
    monkeypatch.setattr(G, "Probe", lambda *a, **k: real(*a, **k) if (a or k) else fine)
    tr = Trainer(ModelConfig.from_config(c), TrainerConfig.from_config(c), device="cpu")
    tr.prefetch.stop()
    assert np.isfinite(tr.scaler.for_step())
