"""Child process for the launcher / watchdog tests (CPU only, gloo).  Usage: launch_worker.py <mode> [out_dir]."""
import datetime
import os
import sys
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def main():
    mode = sys.argv[1]
    out = sys.argv[2] if len(sys.argv) > 2 else ""
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])

    def note(text):
        if out:
            with open(os.path.join(out, "rank%d.txt" % rank), "a") as f:
                f.write(text + "\n")

    if mode == "ok":
        note("done")
        return 0
    if mode == "fail":                      # one rank raises; the others would wait forever
        if rank == 1:
            raise RuntimeError("injected failure on rank 1")
        time.sleep(600)
        return 0
    if mode == "straggler":                 # rank 0 finishes; rank 1 never does
        if rank == 0:
            note("done")
            return 0
        time.sleep(600)
        return 0
    if mode == "sigterm":                   # finish the step and save on SIGTERM, as the trainer does
        import signal
        stop = []
        signal.signal(signal.SIGTERM, lambda *a: stop.append(1))
        note("ready")
        t0 = time.time()
        while not stop and time.time() - t0 < 60:
            time.sleep(0.05)
        note("saved" if stop else "timeout")
        return 0

    import torch
    import torch.distributed as dist
    import ghassan_b200  # noqa: F401
    from ghassan_b200.parallel.env import init_process_group
    from ghassan_b200.parallel.watchdog import Heartbeat, PeerFailure, StepWatchdog

    if mode == "allreduce":
        e = init_process_group("gloo", timeout_s=30)
        t = torch.tensor([float(e.rank + 1)])
        dist.all_reduce(t)
        note("sum=%g" % float(t))
        dist.destroy_process_group()
        return 0
    if mode == "absent":                    # rank 1 never joins the second collective: a short timeout ends it with an error
        init_process_group("gloo", timeout_s=3)
        t = torch.ones(1)
        dist.all_reduce(t)
        if rank == 1:
            note("leaving")
            time.sleep(30)                  # alive but absent
            return 0
        try:
            dist.all_reduce(t)
            note("unexpected: collective returned")
            return 0
        except Exception as ex:
            note("collective failed: " + type(ex).__name__)
            return 3
    if mode == "heartbeat":                 # rank 1 leaves between steps; rank 0 learns of it before its next collective
        e = init_process_group("gloo", timeout_s=30)
        store = dist.PrefixStore("hb_test", dist.distributed_c10d._get_default_store())    # the job's own store
        hb = Heartbeat(store, rank, world, stale_s=30)
        t = torch.ones(1)
        for step in range(3):
            hb.beat()
            dist.all_reduce(t)
        dist.barrier()
        if rank == 1:
            hb.leave()
            note("left")
            time.sleep(1.0)                 # keep the store reachable while rank 0 looks
            return 0
        for _ in range(100):
            try:
                hb.check()
            except PeerFailure as pf:
                note("peer failure: %s" % pf)
                return 0                    # stop cleanly: nothing was launched towards the missing rank
            time.sleep(0.05)
        note("never noticed")
        return 4
    if mode == "watchdog":                  # the step never finishes: the watchdog ends the process with its exit code
        wd = StepWatchdog(0.5, describe=lambda: "step 7 micro-batch 3", first_step_factor=1.0).start()
        wd.beat()
        note("armed")
        time.sleep(30)
        return 0
    raise SystemExit("unknown mode " + mode)


if __name__ == "__main__":
    sys.exit(main())
