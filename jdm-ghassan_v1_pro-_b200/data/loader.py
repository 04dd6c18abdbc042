"""Batch loading: the native sampler (``csrc/host/shards.cpp``) plus pinned staging and a prefetch thread.

The stream is the reference's (training/dataloader.cpp:475-756): rank ``r`` samples with seed
``seed + r * 1000003``, the validation stream with ``seed + 1``; the committed state (full generator
state + batch count) of the *last consumed* batch is what a checkpoint stores, so a resumed run sees
the batches it would have seen.
"""
from __future__ import annotations

import queue
import threading
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import _gb200_host as H

RANK_SEED_STRIDE = 1000003


@dataclass
class Batch:
    ids: torch.Tensor        # int32 [B*T] (pinned when CUDA is available)
    targets: torch.Tensor    # int32 [B*T], -100 = not supervised
    segments: torch.Tensor   # int32 [B*T]
    B: int
    T: int
    supervised: int
    state: tuple             # sampler state after this batch (for checkpoints)


def write_shard(path: str, docs: List[np.ndarray], vocab_size: int, masks: Optional[List[np.ndarray]] = None):
    w = H.ShardWriter(path, vocab_size, masks is not None)
    for i, d in enumerate(docs):
        w.add_document(np.asarray(d, dtype=np.int32), None if masks is None else np.asarray(masks[i], dtype=np.uint8))
    w.close()
    return w.token_count, w.doc_count


class DataLoader:
    """Synchronous loader over ``<dir>/<prefix>*.gbin`` or a domain mix."""

    def __init__(self, batch_size: int, seq_len: int, pack: bool, seed: int, vocab_size: int = 0, pin: bool = None):
        self.B, self.T, self.pack = batch_size, seq_len, pack
        self.s = H.BatchSampler()
        self.seed = seed
        self.vocab = vocab_size
        self.pin = torch.cuda.is_available() if pin is None else pin
        self._opened = False

    def open_glob(self, directory: str, prefix: str) -> bool:
        ok = self.s.open_glob(directory, prefix, self.B, self.T, self.pack, self.seed)
        return self._after_open(ok)

    def open_paths(self, paths: List[str]) -> bool:
        return self._after_open(self.s.open(list(paths), self.B, self.T, self.pack, self.seed))

    def open_mix(self, directory: str, mix: Dict[str, float]) -> bool:
        return self._after_open(self.s.open_mix(directory, dict(mix), self.B, self.T, self.pack, self.seed))

    def _after_open(self, ok):
        self._opened = bool(ok)
        if ok and self.vocab:
            self.s.set_vocab(self.vocab)
        return self._opened

    def set_ring(self, n: int):
        """Stage batches in a ring of ``n`` pre-pinned buffer triples instead of pinning fresh memory per batch
        (pinning allocates through the driver and stalls the device).  ``n`` must exceed the number of batches
        that can be in flight between two host synchronisations (grad_accum + prefetch depth + 1)."""
        self._ring = [tuple(self._new_buf() for _ in range(3)) for _ in range(max(1, n))]
        self._ring_pos = 0

    def _new_buf(self):
        t = torch.empty(self.B * self.T, dtype=torch.int32)
        return t.pin_memory() if self.pin else t

    def _bufs(self):
        ring = getattr(self, "_ring", None)
        if not ring:
            return self._new_buf(), self._new_buf(), self._new_buf()
        out = ring[self._ring_pos]
        self._ring_pos = (self._ring_pos + 1) % len(ring)
        return out

    def next(self) -> Batch:
        if not self._opened:
            raise RuntimeError("dataloader has no shards")
        ids, tgt, seg = self._bufs()
        sup = self.s.next(ids.numpy(), tgt.numpy(), seg.numpy())
        return Batch(ids, tgt, seg, self.B, self.T, int(sup), self.s.get_state())

    # ---- pass-throughs
    def fast_forward(self, n: int):
        self.s.fast_forward(n)

    skip_batches = fast_forward

    def reseed(self, seed: int):
        self.seed = seed
        self.s.reseed(seed)

    def get_state(self):
        return self.s.get_state()

    def set_state(self, st):
        self.s.set_state(tuple(st))

    @property
    def total_tokens(self):
        return self.s.total_tokens

    @property
    def num_shards(self):
        return self.s.num_shards

    @property
    def batches_seen(self):
        return self.s.batches_seen

    @property
    def all_have_mask(self):
        return self.s.all_have_mask

    def mix_report(self):
        return self.s.mix_report()


def state_to_dict(st) -> dict:
    return {"rng": tuple(int(x) for x in st[0]), "batches": int(st[1]), "rng_spare": float(st[2]),
            "rng_has_spare": int(st[3])}


def state_from_dict(d) -> tuple:
    return (tuple(int(x) for x in d["rng"]), int(d["batches"]), float(d["rng_spare"]), int(d["rng_has_spare"]))


class Prefetcher:
    """One background thread keeps ``depth`` batches ready.  ``quiesce()`` drains it so that the loader state
    equals the state after the last *consumed* batch (what a checkpoint must record); an exception in the
    thread is re-raised on the training thread at the next ``get()``."""

    def __init__(self, loader: DataLoader, depth: int = 2):
        self.loader = loader
        self.q: "queue.Queue" = queue.Queue(maxsize=depth)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.last_consumed_state = loader.get_state()
        self._err: Optional[BaseException] = None

    def start(self):
        if self._thread is not None:
            return
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, name="prefetch", daemon=True)
        self._thread.start()

    def _run(self):
        try:
            while not self._stop.is_set():
                b = self.loader.next()
                while not self._stop.is_set():
                    try:
                        self.q.put(b, timeout=0.05)
                        break
                    except queue.Full:
                        continue
        except BaseException as e:  # surfaced by get()
            self._err = e
            try:
                self.q.put_nowait(None)
            except queue.Full:
                pass

    def get(self) -> Batch:
        if self._thread is None:
            b = self.loader.next()
        else:
            while True:
                if self._err is not None and self.q.empty():
                    raise RuntimeError(f"prefetch thread failed: {self._err}") from self._err
                try:
                    b = self.q.get(timeout=0.1)
                    break
                except queue.Empty:
                    continue
            if b is None:
                raise RuntimeError(f"prefetch thread failed: {self._err}") from self._err
        self.last_consumed_state = b.state
        return b

    def quiesce(self):
        """Stop the thread, drop batches that were produced but not consumed and rewind the sampler."""
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None
            while not self.q.empty():
                self.q.get_nowait()
        self.loader.set_state(self.last_consumed_state)

    def stop(self):
        self.quiesce()
