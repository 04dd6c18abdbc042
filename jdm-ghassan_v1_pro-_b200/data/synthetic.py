"""Synthetic corpora for benchmarks and tests: uniform token ids with an end-of-sequence token closing every
document, written as ``.gbin`` shards under the names a recipe expects (one ``train_<domain>_0000.gbin`` per
``data.mix`` domain, or ``train_0000.gbin``, plus ``val_0000.gbin``), and a placeholder ``.gtok`` vocabulary of
the right size (16 special tokens, 256 byte tokens, ``<|unusedN|>`` padding, no merges).
"""
from __future__ import annotations

import os
import struct
from typing import Dict, Iterable, Optional

import numpy as np

from .. import _gb200_host as H

SPECIAL_TOKENS = ["<pad>", "<s>", "</s>", "<unk>", "<|system|>", "<|user|>", "<|assistant|>", "<|end|>", "<|nl|>",
                  "<|fr|>", "<|ar|>", "<|darija|>", "<|latin|>", "<|tool|>", "<|mask|>", "<|reserved|>"]
EOS_ID = 2
GTOK_MAGIC = 0x4B4F5447


def write_uniform_shard(path: str, vocab_size: int, n_tokens: int, mean_doc: int = 512, seed: int = 0,
                        with_mask: bool = True) -> int:
    """Documents of ``mean_doc * [0.75, 1.25)`` tokens, ids uniform in [16, vocab), last token of a document = EOS."""
    rng = np.random.default_rng(seed)
    w = H.ShardWriter(path, vocab_size, with_mask)
    written = 0
    lo, hi = max(2, int(mean_doc * 0.75)), max(3, int(mean_doc * 1.25))
    while written < n_tokens:
        n = int(rng.integers(lo, hi))
        doc = rng.integers(16, vocab_size, size=n, dtype=np.int32)
        doc[-1] = EOS_ID
        w.add_document(doc, None)
        written += n
    w.close()
    return written


def write_placeholder_gtok(path: str, vocab_size: int, normalizer_bits: int = 0) -> None:
    """A structurally valid tokenizer file with ``vocab_size`` entries and no merges."""
    if vocab_size < 272:
        raise ValueError("a tokenizer needs at least 16 special + 256 byte tokens")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        f.write(struct.pack("<IIII", GTOK_MAGIC, 1, normalizer_bits, vocab_size))
        for s in SPECIAL_TOKENS:
            b = s.encode()
            f.write(struct.pack("<I", len(b)) + b)
        for i in range(256):
            f.write(struct.pack("<I", 1) + bytes([i]))
        for i in range(vocab_size - 272):
            b = ("<|unused%d|>" % i).encode()
            f.write(struct.pack("<I", len(b)) + b)
        f.write(struct.pack("<I", 0))


def make_corpus(directory: str, vocab_size: int, mix: Optional[Dict[str, float]] = None, train_tokens: int = 4_000_000,
                val_tokens: int = 400_000, mean_doc: int = 512, seed: int = 1234, train_prefix: str = "train",
                val_prefix: str = "val") -> Dict[str, int]:
    """Create the shard set of a recipe; returns ``{file name: tokens}``.  Existing complete sets are reused."""
    os.makedirs(directory, exist_ok=True)
    stamp = os.path.join(directory, ".complete")
    want = f"{vocab_size}:{sorted((mix or {}).items())}:{train_tokens}:{val_tokens}:{mean_doc}:{seed}"
    if os.path.exists(stamp) and open(stamp).read() == want:
        return {}
    out = {}
    tp = train_prefix.rstrip("_")
    vp = val_prefix.rstrip("_")
    if mix:
        total = sum(mix.values())
        for i, (dom, w) in enumerate(sorted(mix.items())):
            name = f"{tp}_{dom}_0000.gbin"
            out[name] = write_uniform_shard(os.path.join(directory, name), vocab_size,
                                            max(mean_doc * 8, int(train_tokens * w / total)), mean_doc, seed + 1 + i)
    else:
        name = f"{tp}_0000.gbin"
        out[name] = write_uniform_shard(os.path.join(directory, name), vocab_size, train_tokens, mean_doc, seed + 1)
    name = f"{vp}_0000.gbin"
    out[name] = write_uniform_shard(os.path.join(directory, name), vocab_size, val_tokens, mean_doc, seed + 99)
    with open(stamp, "w") as f:
        f.write(want)
    return out
