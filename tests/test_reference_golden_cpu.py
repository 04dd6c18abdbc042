"""The CPU trainer against values recorded from the reference trainer binary.

``tests/golden/cpu_smoke_20steps.json`` holds what the reference's ``gai_train`` (CPU build) left in its ``last.ckpt``
after 20 steps of ``configs/cpu_smoke_test.yaml`` over the two shards regenerated below: the training state (step,
tokens, losses, loss scale), the sampler's generator state, the balancing biases and per-tensor summaries of every
weight.  The data stream must match exactly (same generator state, same token count); weights and losses match up to
the summation order of the matrix products.
"""
import hashlib
import json
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden", "cpu_smoke_20steps.json")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _docs(rng, n, lo, hi, vocab):
    out = []
    for _ in range(n):
        a = np.empty(lo + int(rng.below(hi - lo)), dtype=np.int32)
        rng.fill_uniform_ids(a, vocab - 16)
        out.append(a + 16)
    return out


@pytest.fixture(scope="module")
def run(tmp_path_factory):
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.data.loader import write_shard
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training import checkpoint as C
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer
    from ghassan_b200.utils.config import Config
    tmp = str(tmp_path_factory.mktemp("golden"))
    rng = H.Rng(7)
    write_shard(os.path.join(tmp, "train_0000.gbin"), _docs(rng, 200, 20, 200, 600), 600, None)
    write_shard(os.path.join(tmp, "val_0000.gbin"), _docs(rng, 40, 20, 200, 600), 600, None)
    c = Config.from_file(os.path.join(ROOT, "configs", "cpu_smoke_test.yaml"))
    for k, v in (("max_steps", 20), ("log_every", 5), ("save_every", 10), ("eval_every", 10),
                 ("data_dir", tmp), ("checkpoint_dir", os.path.join(tmp, "ckpt")), ("resume", "none")):
        c.set("training." + k, v)
    Trainer(ModelConfig.from_config(c), TrainerConfig.from_config(c), device="cpu").run()
    got = C.read(os.path.join(tmp, "ckpt", "last.ckpt"))
    return tmp, got, json.load(open(GOLD))


def test_shards_are_the_recorded_ones(run):
    tmp, _, gold = run
    for name, md5 in gold["shard_md5"].items():
        assert hashlib.md5(open(os.path.join(tmp, name), "rb").read()).hexdigest() == md5


def test_data_stream_matches_exactly(run):
    _, got, gold = run
    st = got["state"]
    assert st["step"] == gold["state"]["step"]
    assert st["tokens_seen"] == gold["state"]["tokens_seen"]
    assert [str(x) for x in st["loader"]["rng"]] == gold["loader_rng"]
    assert st["loader"]["batches"] == gold["loader_batches"]
    assert [str(x) for x in st["val_loader"]["rng"]] == gold["val_loader_rng"]
    assert st["loss_scale"] == gold["state"]["loss_scale"]
    assert st["clean_steps"] == gold["state"]["clean_steps"]


def test_losses_match(run):
    _, got, gold = run
    assert got["state"]["last_loss"] == pytest.approx(gold["state"]["last_loss"], rel=2e-6)
    assert got["state"]["best_val"] == pytest.approx(gold["state"]["best_val"], rel=2e-6)


def test_weights_match(run):
    _, got, gold = run
    names = [n for n, _ in got["params"]]
    assert names == list(gold["params"].keys())
    for n, a in got["params"]:
        a = np.asarray(a, dtype=np.float64).ravel()
        g = gold["params"][n]
        assert np.sqrt((a * a).sum()) == pytest.approx(g["l2"], rel=1e-5), n
        assert np.allclose(a[:4], g["head"], rtol=1e-3, atol=2e-6), n
    for row, grow in zip(got["moe_bias"], gold["moe_bias"]):
        assert np.allclose(np.asarray(row), np.asarray(grow), atol=1e-7)
