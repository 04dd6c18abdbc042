"""Process-wide performance counters, phase timers, signal flags and a step watchdog.

Counters mirror what the reference prints in every step line (core/ops.h:21-51, core/ops.cpp:86-240):
GEMM launches, host<->device bytes, synchronisations, MoE / CE / optimizer call counts and time.
Phase timers bracket the hot regions with CUDA events on the launching stream (or wall clock on CPU)
and are summed once per log line (cuda/cuda_utils.cu:196-255 in the reference).
"""
from __future__ import annotations

import os
import signal
import sys
import threading
import time
from collections import defaultdict
from typing import Dict, List, Optional

import torch


class PerfCounters:
    def __init__(self):
        self._mu = threading.Lock()
        self.c: Dict[str, float] = defaultdict(float)

    def add(self, key: str, v: float = 1.0):
        with self._mu:
            self.c[key] += v

    def snapshot(self) -> Dict[str, float]:
        with self._mu:
            return dict(self.c)

    def report(self) -> str:
        s = self.snapshot()
        return ("gemm %d | h2d %.1fMB d2h %.1fMB | sync %d | moe %d | ce %d | opt %d (%.1fms)" % (
            s.get("gemm", 0), s.get("h2d_bytes", 0) / 1e6, s.get("d2h_bytes", 0) / 1e6, s.get("sync", 0),
            s.get("moe", 0), s.get("ce", 0), s.get("opt_steps", 0), s.get("opt_us", 0) / 1e3))


PERF = PerfCounters()


class PhaseTimers:
    """start/stop pairs per phase; CUDA events when a device is in use, wall clock otherwise."""

    PHASES = ("attnF", "moeF", "attnB", "moeB", "load", "sync", "opt")

    def __init__(self, cuda: bool = False, max_pairs: int = 16384):
        self.cuda = cuda and torch.cuda.is_available()
        self.max_pairs = max_pairs
        self.pairs: Dict[str, List] = defaultdict(list)
        self.wall: Dict[str, float] = defaultdict(float)
        self._open: Dict[str, object] = {}
        self.enabled = True
        # GB200_NVTX=1: every phase is also an NVTX range, so a timeline profiler shows the step's structure
        self.nvtx = self.cuda and os.environ.get("GB200_NVTX", "") == "1"

    def start(self, phase: str):
        if not self.enabled:
            return
        if self.nvtx:
            torch.cuda.nvtx.range_push(phase)
        if self.cuda and phase != "load":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open[phase] = ev
        else:
            self._open[phase] = time.perf_counter()

    def stop(self, phase: str):
        if not self.enabled or phase not in self._open:
            return
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        t0 = self._open.pop(phase)
        if self.cuda and phase != "load":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            if len(self.pairs[phase]) < self.max_pairs:
                self.pairs[phase].append((t0, ev))
        else:
            self.wall[phase] += (time.perf_counter() - t0) * 1e3

    def report(self, reset=True) -> str:
        """``ph [attnF a moeF b attnB c moeB d] load e ms`` (milliseconds since the previous report)."""
        ms = dict(self.wall)
        if self.cuda:
            torch.cuda.synchronize()
            for ph, prs in self.pairs.items():
                ms[ph] = ms.get(ph, 0.0) + sum(a.elapsed_time(b) for a, b in prs)
        if reset:
            self.pairs.clear()
            self.wall.clear()
        inner = " ".join("%s %.1f" % (p, ms.get(p, 0.0)) for p in ("attnF", "moeF", "attnB", "moeB"))
        return "ph [%s] load %.1f ms" % (inner, ms.get("load", 0.0))


# ---------------------------------------------------------------------------------------- stop signals
class StopFlag:
    """First SIGINT/SIGTERM asks the trainer to finish the step and save; a second one exits at once (130)."""

    def __init__(self):
        self.requested = False
        self.reason = ""
        self._installed = False

    def install(self):
        if self._installed or threading.current_thread() is not threading.main_thread():
            return

        def handler(signum, frame):
            if self.requested:
                os._exit(130)
            self.requested = True
            self.reason = signal.Signals(signum).name

        signal.signal(signal.SIGINT, handler)
        signal.signal(signal.SIGTERM, handler)
        self._installed = True

    def reset(self):
        self.requested = False
        self.reason = ""


STOP = StopFlag()
