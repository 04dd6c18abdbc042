"""Checkpoints cross between the two trainers: the reference's CPU build resumes a run that this trainer started, and
this trainer resumes a run that the reference started (same recipe, same shards, strict resume).  Runs where a build
of the reference trainer sits under baseline/_ref/bin; the byte-level format tests do not need it
(tests/test_formats_cpu.py)."""
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_BIN = os.path.join(ROOT, "baseline", "_ref", "bin", "gai_train")
RECIPE = os.path.join(ROOT, "configs", "cpu_smoke_test.yaml")

pytestmark = pytest.mark.skipif(not os.path.exists(REF_BIN), reason="no build of the reference trainer here")


def _docs(rng, n, lo, hi, vocab):
    out = []
    for _ in range(n):
        a = np.empty(lo + int(rng.below(hi - lo)), dtype=np.int32)
        rng.fill_uniform_ids(a, vocab - 16)
        out.append(a + 16)
    return out


@pytest.fixture(scope="module")
def shards(tmp_path_factory):
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.data.loader import write_shard
    tmp = str(tmp_path_factory.mktemp("cross"))
    rng = H.Rng(7)
    write_shard(os.path.join(tmp, "train_0000.gbin"), _docs(rng, 200, 20, 200, 600), 600, None)
    write_shard(os.path.join(tmp, "val_0000.gbin"), _docs(rng, 40, 20, 200, 600), 600, None)
    return tmp


def _ours(shards, ckpt, steps, resume):
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.run(["python", "-m", "ghassan_b200.cli.train", "--config", RECIPE, "--device", "cpu", "--max-steps", str(steps),
                        "--data", shards, "--checkpoint-dir", ckpt, "--resume", resume, "--save-every", "10", "--log-every", "10"],
                       capture_output=True, cwd=ROOT, env=env, timeout=300)
    return p.returncode, (p.stdout + p.stderr).decode("utf-8", "replace")


def _theirs(shards, ckpt, steps, resume):
    p = subprocess.run([REF_BIN, "--config", RECIPE, "--device", "cpu", "--max-steps", str(steps), "--data", shards,
                        "--checkpoint-dir", ckpt, "--resume", resume, "--save-every", "10", "--log-every", "10"],
                       capture_output=True, cwd=ROOT, timeout=300)
    return p.returncode, (p.stdout + p.stderr).decode("utf-8", "replace")


def _loss(log, step):
    m = re.search(r"step +%d \| loss +([0-9.]+)" % step, log)
    return float(m.group(1)) if m else None


def test_the_reference_resumes_a_run_of_this_trainer(shards, tmp_path):
    ck = str(tmp_path / "a")
    rc, log = _ours(shards, ck, 20, "none")
    assert rc == 0, log[-600:]
    rc, log = _theirs(shards, ck, 40, "auto")          # a longer schedule: the reference migrates and goes on
    assert rc == 0, log[-600:]
    assert re.search(r"resumed from .*last\.ckpt at step 20", log), log[-800:]
    assert _loss(log, 30) is not None and _loss(log, 40) is not None


def test_this_trainer_resumes_a_run_of_the_reference(shards, tmp_path):
    ck = str(tmp_path / "b")
    rc, log = _theirs(shards, ck, 20, "none")
    assert rc == 0, log[-600:]
    rc, log = _ours(shards, ck, 40, "auto")
    assert rc == 0, log[-600:]
    assert re.search(r"resumed from .*last\.ckpt at step 20", log), log[-800:]
    assert _loss(log, 30) is not None and _loss(log, 40) is not None


def test_both_continuations_agree(shards, tmp_path):
    """From one checkpoint of the reference (step 20), the next 20 steps of either trainer report the same losses to the
    printed precision up to summation order."""
    ck1, ck2 = str(tmp_path / "c1"), str(tmp_path / "c2")
    rc, log = _theirs(shards, ck1, 20, "none")
    assert rc == 0, log[-600:]
    os.makedirs(ck2)
    with open(os.path.join(ck1, "last.ckpt"), "rb") as f, open(os.path.join(ck2, "last.ckpt"), "wb") as g:
        g.write(f.read())
    rc, a = _theirs(shards, ck1, 40, "auto")
    assert rc == 0, a[-600:]
    rc, b = _ours(shards, ck2, 40, "auto")
    assert rc == 0, b[-600:]
    for step in (30, 40):
        la, lb = _loss(a, step), _loss(b, step)
        assert la is not None and lb is not None
        assert abs(la - lb) <= 2e-3, (step, la, lb)
