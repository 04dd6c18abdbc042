"""Levelled line logger and human-readable formatters.

Line shape matches the reference so scripts that scrape its output keep working
(core/common.cpp:33-96): ``[info ] msg`` / ``[warn ] msg`` ..., info and debug to stdout, warnings
and errors to stderr, whole lines serialised across threads.
"""
from __future__ import annotations

import sys
import threading
import time

DEBUG, INFO, WARN, ERROR, SILENT = 0, 1, 2, 3, 4
_TAGS = {DEBUG: "[debug] ", INFO: "[info ] ", WARN: "[warn ] ", ERROR: "[error] "}
_level = INFO
_mu = threading.Lock()


def set_log_level(level: int) -> None:
    global _level
    _level = int(level)


def log_level() -> int:
    return _level


def log_raw(level: int, msg: str) -> None:
    if level >= SILENT or level < _level:
        return
    stream = sys.stderr if level >= WARN else sys.stdout
    with _mu:
        stream.write(_TAGS.get(level, "") + msg + "\n")
        stream.flush()


def log_debug(msg: str) -> None:
    log_raw(DEBUG, msg)


def log_info(msg: str) -> None:
    log_raw(INFO, msg)


def log_warn(msg: str) -> None:
    log_raw(WARN, msg)


def log_error(msg: str) -> None:
    log_raw(ERROR, msg)


def human_bytes(n: int) -> str:
    units = ["B", "KiB", "MiB", "GiB", "TiB"]
    v = float(n)
    i = 0
    while v >= 1024.0 and i < 4:
        v /= 1024.0
        i += 1
    return ("%.0f %s" if i == 0 else "%.2f %s") % (v, units[i])


def human_count(n: int) -> str:
    if n < 1000:
        return str(int(n))
    units = ["", "K", "M", "B", "T"]
    v = float(n)
    i = 0
    while v >= 1000.0 and i < 4:
        v /= 1000.0
        i += 1
    return "%.2f%s" % (v, units[i])


def human_duration(s: float) -> str:
    if s < 1.0:
        return "%.0fms" % (s * 1000.0)
    if s < 60.0:
        return "%.1fs" % s
    si = int(s)
    if s < 3600:
        return "%dm%02ds" % (si // 60, si % 60)
    if s < 86400:
        return "%dh%02dm" % (si // 3600, (si % 3600) // 60)
    return "%dd%02dh" % (si // 86400, (si % 86400) // 3600)


class Timer:
    """Wall-clock stopwatch (seconds)."""

    def __init__(self):
        self.t0 = time.perf_counter()

    def reset(self) -> None:
        self.t0 = time.perf_counter()

    def seconds(self) -> float:
        return time.perf_counter() - self.t0

    def millis(self) -> float:
        return self.seconds() * 1000.0
