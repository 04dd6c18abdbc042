"""Tokenizer trainer (the reference's ``train_tokenizer``, tools/tokenizer_trainer_cli.cpp:13-270).

    python -m ghassan_b200.cli.train_tokenizer --input <file|dir> [--output tok.gtok] [--vocab 32000] [--keep-case]
    python -m ghassan_b200.cli.train_tokenizer --study --input <file|dir> [--eval heldout.txt]   # compare 16k/24k/32k
    python -m ghassan_b200.cli.train_tokenizer --synth 20000 --output tok.gtok                   # generated Darija

The corpus is one document per line (.txt/.text/.jsonl under a directory).  ``--keep-case`` keeps Latin capitals and
is stored in the .gtok, so shards and inference follow it.  The report after training is fertility (tokens per word)
per script slice of the held-out file, or of the head of the corpus when none is given.
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List, Optional
from .common import add_common_flags, apply_common_flags

from .. import _gb200_host as H
from ..data import synth as S
from ..data import tokenizer as T
from ..utils.log import log_error, log_info


def collect_inputs(path: str) -> List[str]:
    if not path:
        return []
    if os.path.isdir(path):
        out = []
        for root, _, names in os.walk(path):
            out += [os.path.join(root, n) for n in names if os.path.splitext(n)[1] in (".txt", ".jsonl", ".text")]
        return sorted(out)
    return [path] if os.path.exists(path) else []


def read_lines(path: str, limit: int = 0) -> List[str]:
    out = []
    with open(path, encoding="utf-8", errors="replace") as f:
        for line in f:
            line = line.rstrip("\r\n")
            if line:
                out.append(line)
                if limit and len(out) >= limit:
                    break
    return out


def fertility_report(tok: T.Tokenizer, lines: List[str], label: str) -> dict:
    """Tokens per whitespace word overall and per language slice of ``lines``."""
    slices = {"all": lines}
    for ln in lines:
        slices.setdefault(H.classify_language(ln)["tag"], []).append(ln)
    log_info("  ---- fertility: " + label + " ----")
    out = {}
    for name, group in slices.items():
        words = sum(len(g.split()) for g in group)
        toks = sum(len(tok.encode(g)) for g in group)
        out[name] = toks / words if words else 0.0
        log_info("    %-12s docs %6d  words %8d  tokens %8d  tokens/word %.3f" % (name, len(group), words, toks, out[name]))
    return out


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="train_tokenizer")
    ap.add_argument("--input", default="")
    ap.add_argument("--output", default="artifacts/tokenizer/english32k.gtok")
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--min-freq", type=int, default=2)
    ap.add_argument("--synth", type=int, default=0)
    ap.add_argument("--eval", default="")
    ap.add_argument("--seed", type=int, default=1)
    for f in ("study", "keep-diacritics", "fold-letters", "keep-case"):
        ap.add_argument("--" + f, action="store_true")
    add_common_flags(ap)
    a = ap.parse_args(argv)
    apply_common_flags(a)
    if not (0 < a.vocab <= 10_000_000):
        log_error("--vocab is out of range")
        return 2
    if a.min_freq < 0 or a.synth < 0:
        log_error("--min-freq and --synth must be >= 0")
        return 2
    files = collect_inputs(a.input)
    texts: List[str] = []
    if a.synth:
        for row in S.darija_conversations(a.synth, seed=a.seed):
            texts += [m["content"] for m in row["messages"]]
        log_info("[synth] %d generated lines" % len(texts))
    if not files and not texts:
        log_error("no corpus data. use --input <path> and/or --synth <n>")
        return 1
    norm = H.NormalizerConfig()
    norm.strip_diacritics = not a.keep_diacritics
    norm.fold_letters = bool(a.fold_letters)
    norm.lowercase_latin = not a.keep_case
    held = read_lines(a.eval) if a.eval else ((read_lines(files[0], 2000) if files else texts[:2000]))
    sizes = [16000, 24000, 32000] if a.study else [a.vocab]
    for v in sizes:
        log_info("[bpe ] training vocab=%d min_freq=%d on %d file(s)%s" % (v, a.min_freq, len(files), " + synthetic" if texts else ""))
        tok = T.train_bpe(files, v, a.min_freq, normalizer_bits=norm.pack(), texts=texts)
        log_info("[bpe ] learned %d tokens" % tok.vocab_size)
        fertility_report(tok, held, "vocab %d" % v)
        if not a.study:
            os.makedirs(os.path.dirname(os.path.abspath(a.output)), exist_ok=True)
            tok.save(a.output)
            log_info("[bpe ] wrote %s (fingerprint %s)" % (a.output, H.fingerprint_hex(H.fingerprint_file(a.output))))
            log_info("  ---- sample encodings ----")
            for ln in held[:3]:
                ids = tok.encode(ln)
                log_info("    %s\n      -> %s" % (ln[:80], " | ".join(tok.token_bytes(int(i)).decode("utf-8", "replace") for i in ids[:24])))
    return 0


if __name__ == "__main__":
    sys.exit(main())
