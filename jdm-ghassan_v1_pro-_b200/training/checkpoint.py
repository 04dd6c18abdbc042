"""Checkpoint capture, asynchronous publishing and loading on top of the native codec (``csrc/host/ckpt.cpp``).

Behaviour follows the reference trainer (training/checkpoint.cpp, training/trainer.cpp:1229-1311,
2014-2170): a snapshot is a host copy of weights + optimizer moments + train state taken at a step
boundary; a writer thread publishes it (``.tmp`` -> rename, previous file parked as ``.bak``); ``best`` and
``last`` of the same step share one snapshot and the second file is a hard link of the first; the queue
is bounded by a RAM budget (back-pressure on the training thread); a failed write surfaces at the next
health check instead of being lost.
"""
from __future__ import annotations

import os
import queue
import shutil
import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np

from .. import _gb200_host as H
from ..models.config import ModelConfig
from ..utils.log import log_error, log_info, log_warn

CKPT_VERSION = 12


@dataclass
class TrainState:
    step: int = 0
    tokens_seen: int = 0
    best_val: float = 1e30
    last_loss: float = 0.0
    seed: int = 42
    loader: dict = field(default_factory=lambda: {"rng": (0, 0, 0, 0), "batches": 0, "rng_spare": 0.0, "rng_has_spare": 0})
    loss_scale: float = 65536.0
    clean_steps: int = 0
    tok_vocab: int = 0
    tok_fingerprint: int = 0
    val_loader: dict = field(default_factory=lambda: {"rng": (0, 0, 0, 0), "batches": 0, "rng_spare": 0.0, "rng_has_spare": 0})
    sched_total: int = 0
    sched_warmup: int = 0
    sched_peak: float = 0.0
    sched_min_ratio: float = 0.1
    sched_decay_frac: float = 0.2
    sched_kind: int = 0
    ddp_world: int = 1

    def to_dict(self) -> dict:
        return dict(self.__dict__)

    @classmethod
    def from_dict(cls, d: dict) -> "TrainState":
        s = cls()
        for k, v in d.items():
            if hasattr(s, k):
                setattr(s, k, v)
        return s


def config_to_dict(c: ModelConfig) -> dict:
    return {k: getattr(c, k) for k in c.__dataclass_fields__}


def config_from_dict(d: dict) -> ModelConfig:
    c = ModelConfig()
    for k, v in d.items():
        if k in c.__dataclass_fields__:
            setattr(c, k, v)
    c.__post_init__()
    return c


@dataclass
class Snapshot:
    config: dict
    state: dict
    moe_bias: List[np.ndarray]
    params: List            # [(name, float32 array)]
    optimizer: Optional[dict]

    def nbytes(self) -> int:
        n = sum(a.nbytes for _, a in self.params)
        if self.optimizer:
            n += sum(a.nbytes for a in self.optimizer["m"] if a is not None)
            n += sum(a.nbytes for a in self.optimizer.get("v", []) if a is not None)
        return n


def capture(engine, state: TrainState) -> Snapshot:
    """Host copy of everything a checkpoint stores (call at a step boundary with the loader quiesced)."""
    return Snapshot(config_to_dict(engine.mcfg), state.to_dict(), engine.export_moe_bias(), engine.export_weights(),
                    engine.export_optimizer())


def save_snapshot(snap: Snapshot, path: str) -> None:
    H.write_checkpoint(path, snap.config, snap.state, list(snap.moe_bias), list(snap.params), snap.optimizer)


def peek(path: str):
    """(ModelConfig, TrainState, version) from the header only; None when unreadable."""
    try:
        d = H.read_checkpoint(path, True, False)
    except Exception:
        return None
    return config_from_dict(d["config"]), TrainState.from_dict(d["state"]), int(d["version"])


def read(path: str, with_optimizer=True) -> dict:
    return H.read_checkpoint(path, False, with_optimizer)


def latest_in(directory: str) -> str:
    """``last.ckpt``, else its ``.bak``, else the lexicographically last ``*.ckpt``; empty when none."""
    if not os.path.isdir(directory):
        return ""
    last = os.path.join(directory, "last.ckpt")
    if os.path.exists(last):
        return last
    if os.path.exists(last + ".bak"):
        return last + ".bak"
    found = sorted(os.path.join(directory, f) for f in os.listdir(directory)
                   if f.endswith(".ckpt") and os.path.isfile(os.path.join(directory, f)))
    return found[-1] if found else ""


def physical_ram_bytes() -> int:
    try:
        return os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
    except (ValueError, OSError):
        return 0


def snapshot_ram_budget() -> int:
    """clamp(physical RAM - 8 GiB, 8 GiB, 32 GiB)."""
    gib = 1 << 30
    return min(32 * gib, max(8 * gib, physical_ram_bytes() - 8 * gib))


class CheckpointWriter:
    """Background publisher with RAM back-pressure and hard-link reuse for same-snapshot files."""

    def __init__(self, ram_budget: Optional[int] = None):
        self.budget = snapshot_ram_budget() if ram_budget is None else ram_budget
        self._q: "queue.Queue" = queue.Queue()
        self._cv = threading.Condition()
        self._pending: List[Snapshot] = []     # queued or being written (unique snapshots)
        self._err: Optional[BaseException] = None
        self._thread: Optional[threading.Thread] = None
        # (serial of the snapshot, first path it was written to) of the last full write.  Every snapshot gets a serial
        # from this writer the first time it is submitted; id() is not used, because the id of a freed snapshot can be
        # taken by a later one, which would then be published as a hard link to the earlier file.
        self._written = None
        self._serial = 0

    def start(self):
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="ckpt-writer", daemon=True)
            self._thread.start()

    def queue_depth(self) -> int:
        with self._cv:
            return self._q.qsize()

    def queued_bytes(self) -> int:
        with self._cv:
            seen, total = set(), 0
            for s in self._pending:
                if id(s) not in seen:
                    seen.add(id(s))
                    total += s.nbytes()
            return total

    def submit(self, snap: Snapshot, path: str):
        """Blocks while the unique queued snapshots would exceed the RAM budget."""
        self.check_health()
        self._serial_of(snap)
        if self._thread is None:
            self._write(snap, path)
            return
        need = snap.nbytes()
        with self._cv:
            while True:
                ids = {id(s) for s in self._pending}
                cur = 0
                seen = set()
                for s in self._pending:
                    if id(s) not in seen:
                        seen.add(id(s))
                        cur += s.nbytes()
                if id(snap) in ids or cur == 0 or cur + need <= self.budget:
                    break
                self._cv.wait(timeout=0.2)
                if self._err:
                    break
            self._pending.append(snap)
        self._q.put((snap, path))

    def _write(self, snap: Snapshot, path: str):
        serial = self._serial_of(snap)
        prior = self._written[1] if (self._written is not None and self._written[0] == serial) else None
        if prior and os.path.exists(prior) and os.path.abspath(prior) != os.path.abspath(path):
            # same step, second name: link (or copy) the file that is already on disk
            tmp = path + ".lnk"
            try:
                if os.path.exists(tmp):
                    os.remove(tmp)
                try:
                    os.link(prior, tmp)
                except OSError:
                    shutil.copyfile(prior, tmp)
                H.publish_file(path, tmp)
                return
            except Exception:
                if os.path.exists(tmp):
                    os.remove(tmp)
        save_snapshot(snap, path)
        self._written = (serial, path)

    def _serial_of(self, snap) -> int:
        s = getattr(snap, "_writer_serial", None)
        if s is None:
            with self._cv:
                self._serial += 1
                s = self._serial
            snap._writer_serial = s
        return s

    def _run(self):
        while True:
            item = self._q.get()
            if item is None:
                return
            snap, path = item
            try:
                self._write(snap, path)
            except BaseException as e:
                self._err = e
                log_error(f"[ckpt] background write failed for {path}: {e}")
            finally:
                with self._cv:
                    for i, s in enumerate(self._pending):
                        if s is snap:
                            del self._pending[i]
                            break
                    self._cv.notify_all()

    def check_health(self):
        if self._err is not None:
            e, self._err = self._err, None
            raise RuntimeError(f"checkpoint writer failed: {e}") from e

    def wait(self):
        if self._thread is None:
            return
        with self._cv:
            while self._pending:
                self._cv.wait(timeout=0.2)
        self.check_health()

    def stop(self):
        if self._thread is not None:
            self.wait()
            self._q.put(None)
            self._thread.join()
            self._thread = None
