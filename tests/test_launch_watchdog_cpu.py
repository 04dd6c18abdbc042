"""Launcher supervision rules, rank-environment parsing, the step watchdog and the heartbeat — every failure is made
on the host, among CPU processes."""
import os
import sys
import threading
import time

import pytest

WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "launch_worker.py")


def _launch(mode, tmp_path, nproc=2, **kw):
    from ghassan_b200.parallel.launch import launch
    lines = []
    res = launch([WORKER, mode, str(tmp_path)], nproc, poll_s=0.05, echo=lines.append, **kw)
    return res, "\n".join(lines)


def _notes(tmp_path, rank):
    p = tmp_path / ("rank%d.txt" % rank)
    return p.read_text() if p.exists() else ""


# ------------------------------------------------------------------------------------------ environment
def test_rank_environment_parsing():
    from ghassan_b200.parallel.env import EnvError, parse_env
    assert parse_env({}).world == 1 and parse_env({}).source == "single" and not parse_env({}).distributed
    e = parse_env({"WORLD_SIZE": "8", "RANK": "3", "LOCAL_RANK": "3", "MASTER_ADDR": "10.0.0.2", "MASTER_PORT": "1234"})
    assert (e.world, e.rank, e.local_rank, e.source, e.init_method()) == (8, 3, 3, "env", "tcp://10.0.0.2:1234")
    s = parse_env({"SLURM_NTASKS": "4", "SLURM_PROCID": "2", "SLURM_LOCALID": "0"})
    assert (s.world, s.rank, s.local_rank, s.source, s.master_addr, s.master_port) == (4, 2, 0, "slurm", "127.0.0.1", 29500)
    both = parse_env({"WORLD_SIZE": "2", "RANK": "1", "SLURM_NTASKS": "16", "SLURM_PROCID": "9"})
    assert both.world == 2 and both.rank == 1 and both.local_rank == 1          # explicit variables win
    for bad in ({"WORLD_SIZE": "2", "RANK": "2"}, {"WORLD_SIZE": "0"}, {"WORLD_SIZE": "two"}, {"WORLD_SIZE": "2", "RANK": "0", "MASTER_PORT": "70000"}):
        with pytest.raises(EnvError):
            parse_env(bad)


def test_launcher_exports_one_environment_per_rank():
    from ghassan_b200.parallel.launch import rank_environment
    e = rank_environment(3, 8, "127.0.0.1", 4242, {"PATH": "/bin"})
    assert (e["RANK"], e["LOCAL_RANK"], e["WORLD_SIZE"], e["MASTER_ADDR"], e["MASTER_PORT"]) == ("3", "3", "8", "127.0.0.1", "4242")
    assert e["PATH"] == "/bin" and int(e["OMP_NUM_THREADS"]) >= 1


# ------------------------------------------------------------------------------------------ supervision rules
def test_all_ranks_finish(tmp_path):
    res, log = _launch("ok", tmp_path, nproc=3)
    assert res.ok and res.exit_codes == {0: 0, 1: 0, 2: 0} and "all ranks finished" in log
    assert all("done" in _notes(tmp_path, r) for r in range(3))


def test_failed_rank_ends_the_job(tmp_path):
    t0 = time.time()
    res, log = _launch("fail", tmp_path)
    assert not res.ok and res.exit_codes[1] == 1 and "rank 1 exited" in res.reason
    assert res.exit_codes[0] not in (None, 0)                 # the waiting sibling was stopped, by PID
    assert time.time() - t0 < 30 and "stopping 1 rank(s)" in log


def test_survivor_that_outlives_its_sibling_is_killed(tmp_path):
    t0 = time.time()
    res, log = _launch("straggler", tmp_path, grace_s=1.0)
    assert not res.ok and "outlived" in res.reason and res.exit_codes[0] == 0 and res.exit_codes[1] not in (None, 0)
    assert 1.0 <= time.time() - t0 < 30 and "collective desync" in log


def test_job_deadline(tmp_path):
    res, _ = _launch("fail", tmp_path, nproc=1, max_seconds=1.0)        # a single rank 0 that only sleeps
    assert not res.ok and "exceeded" in res.reason


def test_sigterm_is_forwarded_once_and_ranks_save(tmp_path):
    from ghassan_b200.parallel.launch import Supervisor, rank_environment
    envs = [rank_environment(r, 2, "127.0.0.1", 1, None) for r in range(2)]
    sup = Supervisor([[sys.executable, WORKER, "sigterm", str(tmp_path)]] * 2, envs, poll_s=0.05, echo=lambda s: None)
    sup.start()
    for _ in range(200):
        if all("ready" in _notes(tmp_path, r) for r in range(2)):
            break
        time.sleep(0.05)
    import signal
    threading.Timer(0.1, lambda: (sup.forward(signal.SIGTERM), sup.forward(signal.SIGTERM))).start()
    res = sup.wait()
    assert res.ok and all("saved" in _notes(tmp_path, r) for r in range(2))


# ------------------------------------------------------------------------------------------ gloo ranks
def test_gloo_job_under_the_launcher(tmp_path):
    res, _ = _launch("allreduce", tmp_path, nproc=3)
    assert res.ok
    assert all("sum=6" in _notes(tmp_path, r) for r in range(3))


def test_absent_rank_times_the_collective_out(tmp_path):
    res, _ = _launch("absent", tmp_path)
    assert not res.ok and res.exit_codes[0] == 3 and "collective failed" in _notes(tmp_path, 0)
    assert "unexpected" not in _notes(tmp_path, 0)


def test_heartbeat_reports_a_rank_that_left(tmp_path):
    res, _ = _launch("heartbeat", tmp_path, master_port=0)
    assert res.ok, res
    assert "peer failure: rank 1: left the job" in _notes(tmp_path, 0) and "left" in _notes(tmp_path, 1)


def test_watchdog_ends_a_stuck_process(tmp_path):
    from ghassan_b200.parallel.watchdog import EXIT_WATCHDOG
    t0 = time.time()
    res, _ = _launch("watchdog", tmp_path, nproc=1)
    assert not res.ok and res.exit_codes[0] == EXIT_WATCHDOG and time.time() - t0 < 20


# ------------------------------------------------------------------------------------------ in-process pieces
def test_watchdog_deadline_pause_and_report():
    from ghassan_b200.parallel.watchdog import StepWatchdog
    fired = []
    wd = StepWatchdog(0.3, describe=lambda: "step 12", on_expire=fired.append, first_step_factor=3.0).start()
    time.sleep(0.5)
    assert not fired                                           # the first step gets three deadlines
    wd.beat()
    for _ in range(4):
        time.sleep(0.15)
        wd.beat()
    assert not fired
    with wd.pause():
        time.sleep(0.6)                                        # evaluation / checkpoint: no cadence expected
    assert not fired
    time.sleep(0.7)
    assert fired and "step 12" in fired[0] and "deadline 0.3" in fired[0] and wd.expired
    wd.stop()
    with pytest.raises(ValueError):
        StepWatchdog(0)


def test_heartbeat_states_with_a_local_store():
    import torch.distributed as dist
    from ghassan_b200.parallel.watchdog import Heartbeat, PeerFailure
    store = dist.HashStore()
    a, b, c = (Heartbeat(store, r, 3, stale_s=0.3) for r in range(3))
    for h in (a, b, c):
        h.beat()
    a.check()
    time.sleep(0.2)
    b.beat()
    c.beat()
    a.check()
    time.sleep(0.4)
    c.beat()
    with pytest.raises(PeerFailure) as ei:                     # b made no progress for longer than stale_s
        for _ in range(3):
            a.check()
            time.sleep(0.2)
            c.beat()
    assert ei.value.rank == 1 and "no heartbeat" in ei.value.why
    c.fail("cuda error 700 in step 9")
    with pytest.raises(PeerFailure) as ei:
        b.check()
    assert ei.value.rank == 2 and "cuda error 700" in str(ei.value)
    assert [p["state"] for p in a.peers()] == ["alive", "alive", "failed:cuda error 700 in step 9"]
