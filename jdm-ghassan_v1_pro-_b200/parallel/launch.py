"""One process per GPU on one node, with the supervision rules of the reference's launch scripts
(``wait_ddp_ranks``, configs/kaggle/train_2xt4.sh:134-182):

* a rank that exits non-zero ends the job: its siblings are terminated and the job fails;
* after the first rank exits cleanly, the others get ``grace`` seconds to finish; one that outlives the grace
  period is taken to be stuck in a collective with a peer that is gone, and is killed (job fails);
* no rank exiting within ``max_seconds`` ends the job too;
* SIGINT/SIGTERM are forwarded once, so that every rank finishes its step and saves (trainer semantics), then the
  same rules apply.

Children are started in their own process group and are only ever signalled by PID.

    python -m ghassan_b200.parallel.launch --nproc 8 [--master-port 29500] [--grace 180] [--log-dir logs] -- \\
        -m ghassan_b200.cli.train --config configs/pro_1b_2xt4.yaml
"""
from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


@dataclass
class LaunchResult:
    ok: bool
    reason: str
    exit_codes: Dict[int, Optional[int]] = field(default_factory=dict)
    seconds: float = 0.0


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def rank_environment(rank: int, world: int, master_addr: str, master_port: int, base: Optional[dict] = None) -> dict:
    env = dict(os.environ if base is None else base)
    env.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_WORLD_SIZE": str(world),
                "MASTER_ADDR": master_addr, "MASTER_PORT": str(master_port)})
    env.setdefault("OMP_NUM_THREADS", str(max(1, (os.cpu_count() or 8) // max(1, world))))
    return env            # every GPU stays visible; a rank binds the one its LOCAL_RANK names


class Supervisor:
    """Owns the child processes of one job.  ``poll_s`` is the supervision period."""

    def __init__(self, commands: Sequence[Sequence[str]], envs: Sequence[dict], grace_s: float = 180.0, max_seconds: float = 46000.0,
                 poll_s: float = 0.5, kill_wait_s: float = 10.0, log_dir: str = "", echo=print):
        if len(commands) != len(envs) or not commands:
            raise ValueError("need one environment per command")
        self.commands, self.envs = [list(c) for c in commands], list(envs)
        self.grace, self.max_seconds, self.poll, self.kill_wait = grace_s, max_seconds, poll_s, kill_wait_s
        self.log_dir, self.echo = log_dir, echo
        self.procs: List[subprocess.Popen] = []
        self._logs = []
        self._forwarded = False

    # -- process control (by PID only)
    def start(self):
        if self.log_dir:
            os.makedirs(self.log_dir, exist_ok=True)
        for r, (cmd, env) in enumerate(zip(self.commands, self.envs)):
            out = None
            if self.log_dir and r > 0:                       # rank 0 keeps the terminal, the others log to files
                out = open(os.path.join(self.log_dir, "rank%d.log" % r), "wb")
                self._logs.append(out)
            self.procs.append(subprocess.Popen(cmd, env=env, stdout=out, stderr=subprocess.STDOUT if out else None,
                                               start_new_session=True))

    def _signal(self, p: subprocess.Popen, sig: int):
        if p.poll() is None:
            try:
                os.kill(p.pid, sig)
            except ProcessLookupError:
                pass

    def terminate_all(self, why: str):
        alive = [p for p in self.procs if p.poll() is None]
        if alive:
            self.echo("[launch] %s - stopping %d rank(s)" % (why, len(alive)))
        for p in alive:
            self._signal(p, signal.SIGTERM)
        end = time.monotonic() + self.kill_wait
        while time.monotonic() < end and any(p.poll() is None for p in alive):
            time.sleep(min(0.1, self.poll))
        for p in alive:
            if p.poll() is None:
                self._signal(p, signal.SIGKILL)
        for p in alive:
            try:
                p.wait(timeout=self.kill_wait)
            except subprocess.TimeoutExpired:
                pass

    def forward(self, sig: int):
        if not self._forwarded:
            self._forwarded = True
            self.echo("[launch] signal %d: asking every rank to finish its step and save" % sig)
            for p in self.procs:
                self._signal(p, sig)

    def codes(self) -> Dict[int, Optional[int]]:
        return {r: p.poll() for r, p in enumerate(self.procs)}

    # -- the rules
    def wait(self) -> LaunchResult:
        t0 = time.monotonic()
        first_clean: Optional[float] = None
        try:
            while True:
                now = time.monotonic()
                codes = self.codes()
                bad = [(r, c) for r, c in codes.items() if c not in (None, 0)]
                if bad:
                    r, c = bad[0]
                    self.terminate_all("rank %d exited with code %d" % (r, c))
                    return LaunchResult(False, "rank %d exited %d" % (r, c), self.codes(), now - t0)
                if all(c == 0 for c in codes.values()):
                    return LaunchResult(True, "all ranks finished", codes, now - t0)
                if any(c == 0 for c in codes.values()):
                    if first_clean is None:
                        first_clean = now
                    elif now - first_clean > self.grace:
                        left = [r for r, c in codes.items() if c is None]
                        self.terminate_all("rank(s) %s still running %.0f s after a sibling finished (collective desync)" % (left, self.grace))
                        return LaunchResult(False, "survivor outlived sibling by %.0f s" % self.grace, self.codes(), now - t0)
                if now - t0 > self.max_seconds:
                    self.terminate_all("no result after %.0f s" % self.max_seconds)
                    return LaunchResult(False, "job exceeded %.0f s" % self.max_seconds, self.codes(), now - t0)
                time.sleep(self.poll)
        finally:
            for f in self._logs:
                f.close()


def launch(argv_after: Sequence[str], nproc: int, master_addr: str = "127.0.0.1", master_port: int = 0, grace_s: float = 180.0,
           max_seconds: float = 46000.0, log_dir: str = "", poll_s: float = 0.5, extra_env: Optional[dict] = None, echo=print) -> LaunchResult:
    if nproc < 1:
        raise ValueError("--nproc must be >= 1")
    port = master_port or free_port()
    base = dict(os.environ)
    base.update(extra_env or {})
    envs = [rank_environment(r, nproc, master_addr, port, base) for r in range(nproc)]
    cmds = [[sys.executable] + list(argv_after) for _ in range(nproc)]
    sup = Supervisor(cmds, envs, grace_s, max_seconds, poll_s, log_dir=log_dir, echo=echo)
    echo("[launch] %d rank(s), rendezvous %s:%d" % (nproc, master_addr, port))
    sup.start()
    old = {}
    for s in (signal.SIGINT, signal.SIGTERM):
        try:
            old[s] = signal.signal(s, lambda signum, frame: sup.forward(signum))
        except ValueError:                                   # not the main thread (tests): no forwarding
            pass
    try:
        res = sup.wait()
    finally:
        for s, h in old.items():
            signal.signal(s, h)
    echo("[launch] %s (%.1f s) exit codes %s" % (res.reason, res.seconds, res.exit_codes))
    return res


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="launch")
    ap.add_argument("--nproc", type=int, default=0, help="ranks to start (default: one per visible GPU)")
    ap.add_argument("--master-addr", default="127.0.0.1")
    ap.add_argument("--master-port", type=int, default=0)
    ap.add_argument("--grace", type=float, default=180.0)
    ap.add_argument("--max-seconds", type=float, default=46000.0)
    ap.add_argument("--log-dir", default="")
    ap.add_argument("rest", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    rest = a.rest[1:] if a.rest[:1] == ["--"] else a.rest
    if not rest:
        ap.error("give the program after '--', e.g.  -- -m ghassan_b200.cli.train --config recipe.yaml")
    n = a.nproc
    if n <= 0:
        import torch
        n = max(1, torch.cuda.device_count())
    res = launch(rest, n, a.master_addr, a.master_port, a.grace, a.max_seconds, a.log_dir)
    return 0 if res.ok else 1


if __name__ == "__main__":
    sys.exit(main())
