"""Data-parallel host logic on two gloo ranks: identical weights on every rank, equality with a one-process emulation
of both rank streams, exact resume of a 2-rank run, world-size gate, and a rank that leaves between steps."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "ddp_worker.py")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _launch(world, args, extra_env=None, timeout=240):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, WORKER] + [str(a) for a in args], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()                       # the exact child started above
            o, _ = p.communicate()
        outs.append((p.returncode, o))
    return outs


@pytest.fixture(scope="module")
def data_dir(tmp_path_factory):
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.data.loader import write_shard
    d = str(tmp_path_factory.mktemp("ddp_shards"))
    r = H.Rng(3)
    docs = []
    for _ in range(200):
        a = np.empty(20 + int(r.below(80)), dtype=np.int32)
        r.fill_uniform_ids(a, 40)
        docs.append(a + 16)
    write_shard(os.path.join(d, "train_0000.gbin"), docs, 320, None)
    return d


@pytest.fixture(scope="module")
def two_rank_run(data_dir, tmp_path_factory):
    out = str(tmp_path_factory.mktemp("ddp_out"))
    res = _launch(2, [out, data_dir, 6])
    for rc, o in res:
        assert rc == 0, o[-2000:]
    return out


def test_ranks_hold_identical_weights(two_rank_run):
    a = np.load(os.path.join(two_rank_run, "rank0_train.npz"))
    b = np.load(os.path.join(two_rank_run, "rank1_train.npz"))
    for k in a.files:
        assert np.array_equal(a[k], b[k]), k


def test_two_ranks_equal_one_process_over_both_streams(two_rank_run, data_dir, tmp_path):
    """Sum of both ranks' micro-batch gradients divided by the global token count: the same update as one process
    that draws rank 0's and rank 1's batches itself (up to the order of the floating-point sums)."""
    sys.path.insert(0, HERE)
    import ddp_worker as W
    from ghassan_b200.data.loader import RANK_SEED_STRIDE, DataLoader
    tr = W.build(data_dir, str(tmp_path / "ck"), False)
    tr.prepare()
    tr.prefetch.stop()
    c = tr.cfg
    loaders = []
    for r in range(2):
        ld = DataLoader(c.batch_size, c.seq_len, c.pack_sequences, c.seed + r * RANK_SEED_STRIDE, vocab_size=320, pin=False)
        assert ld.open_glob(data_dir, "train")
        loaders.append(ld)
    eng = tr.engine
    for step in range(6):
        eng.begin_step(step, 1.0)
        for ld in loaders:
            for _ in range(c.grad_accum):
                b = ld.next()
                eng.micro_step(b.ids, b.targets, b.segments, b.B, b.T)
        eng.end_step(tr.sched.lr_at(step))
    got = np.load(os.path.join(two_rank_run, "rank0_train.npz"))
    for n, p in eng.model.named_parameters():
        ref = p.detach().numpy()
        # Adam divides by sqrt(v): a last-bit difference in a tiny gradient moves the update by more than a bit
        assert np.abs(got[n] - ref).max() <= 2e-4 * (np.abs(ref).max() + 1e-6), n


def test_two_rank_exact_resume(two_rank_run, data_dir):
    res = _launch(2, [two_rank_run, data_dir, 6, "resume"])
    for rc, o in res:
        assert rc == 0, o[-2000:]
    for r in range(2):
        a = np.load(os.path.join(two_rank_run, "rank%d_train.npz" % r))
        b = np.load(os.path.join(two_rank_run, "rank%d_resume.npz" % r))
        for k in a.files:
            assert np.array_equal(a[k], b[k]), (r, k)


def test_resume_refuses_another_world_size(two_rank_run, data_dir):
    sys.path.insert(0, HERE)
    import ddp_worker as W
    from ghassan_b200.training.trainer import TrainerError
    with pytest.raises(TrainerError) as e:
        W.build(data_dir, os.path.join(two_rank_run, "ckpt"), False, resume=os.path.join(two_rank_run, "ckpt", "last.ckpt"))
    assert "world mismatch" in str(e.value)


def test_a_rank_that_leaves_between_steps_is_an_error_not_a_hang(data_dir, tmp_path):
    out = str(tmp_path)
    res = _launch(2, [out, data_dir, 3, "absent"], extra_env={"PG_TIMEOUT_S": "8"}, timeout=120)
    assert res[1][0] == 0                      # the leaving rank exits cleanly
    assert res[0][0] == 17, res[0][1][-1500:]  # the survivor got an exception from its next collective
    assert os.path.exists(os.path.join(out, "rank0.err"))


def test_a_failed_rank_is_reported_through_the_heartbeat_before_the_next_collective(data_dir, tmp_path):
    import time
    out = str(tmp_path)
    t0 = time.time()
    res = _launch(2, [out, data_dir, 6, "peer_raises"], extra_env={"PG_TIMEOUT_S": "60"}, timeout=120)
    assert res[1][0] == 21 and "injected" in open(os.path.join(out, "rank1.err")).read()
    assert res[0][0] == 22, res[0][1][-1500:]
    msg = open(os.path.join(out, "rank0.err")).read()
    assert "peer failure before step 3" in msg and "rank 1" in msg and "device lost" in msg
    assert time.time() - t0 < 45                      # learned on the host, not through the 60 s collective timeout
