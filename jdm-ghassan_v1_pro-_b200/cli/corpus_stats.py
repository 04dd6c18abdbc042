"""Corpus measurement (the reference's ``corpus_stats``, tools/corpus_inspector_cli.cpp:13-160).

    python -m ghassan_b200.cli.corpus_stats --input <file|dir> [--tokenizer tok.gtok] [--dedup] [--pii] [--quality]
                                            [--limit n] [--sample n]

One document per line (text files) or per record (json/jsonl/parquet).  Reports documents, words, the language and
script mix, length percentiles; with a tokenizer also tokens and tokens per word; optionally the duplicate ratio,
personal-data counts and how many documents the quality filter would reject.
"""
from __future__ import annotations

import argparse
import itertools
import sys
from collections import Counter, defaultdict
from typing import List, Optional
from .common import add_common_flags, apply_common_flags

from .. import _gb200_host as H
from ..data import pipeline as P
from ..data import tokenizer as T
from ..utils.log import human_count, log_error, log_info


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="corpus_stats")
    ap.add_argument("--input", default="")
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--limit", type=int, default=0)
    ap.add_argument("--sample", type=int, default=0)
    for f in ("dedup", "pii", "quality"):
        ap.add_argument("--" + f, action="store_true")
    add_common_flags(ap)
    a = ap.parse_args(argv)
    apply_common_flags(a)
    if not a.input:
        log_error("--input is required")
        return 2
    tok = None
    if a.tokenizer:
        try:
            tok = T.Tokenizer.load(a.tokenizer)
        except T.TokenizerError as e:
            log_error("cannot load tokenizer: %s (%s)" % (a.tokenizer, e))
            return 1
        log_info("[tok] loaded vocab=%d" % tok.vocab_size)
    recs = P.iter_inputs(a.input)
    if a.limit > 0:
        recs = itertools.islice(recs, a.limit)
    dd = H.Deduplicator() if a.dedup else None
    pii = Counter()
    rejected = Counter()
    samples = defaultdict(list)
    qcfg = H.QualityConfig()

    def watch(stream):
        for r in stream:
            text = r.text if r.messages is None else "\n".join(m.content for m in r.messages)
            if dd is not None:
                dd.add(text)
            if a.pii:
                rep = H.scan_pii(text)
                for k, v in rep.items():
                    if k != "total" and v:
                        pii[k] += v
            if a.quality:
                ok, why = H.quality_check(text, qcfg)
                if not ok:
                    rejected[why] += 1
            if a.sample:
                tag = H.classify_language(text)["tag"]
                if len(samples[tag]) < a.sample:
                    samples[tag].append(text[:160].replace("\n", " "))
            yield r

    st = P.corpus_stats(watch(recs), tok)
    if st["documents"] == 0:
        log_error("no documents found under " + a.input)
        return 1
    log_info("documents : %s" % human_count(st["documents"]))
    log_info("words     : %s   characters: %s" % (human_count(st["words"]), human_count(st["characters"])))
    log_info("words/doc : p50 %d  p90 %d  p99 %d" % (st["words_p50"], st["words_p90"], st["words_p99"]))
    if tok is not None:
        log_info("tokens    : %s   tokens/word %.3f" % (human_count(st["tokens"]), st["tokens_per_word"] or 0.0))
    log_info("---- language mix ----")
    for k, v in st["languages"].items():
        log_info("  %-12s %8d  %6.2f%%" % (k, v, 100.0 * v / st["documents"]))
    sc = st["scripts"]
    total = max(1, sum(sc.values()))
    log_info("---- script mix (letters) ----")
    for k in ("arabic", "latin", "digits", "emoji"):
        log_info("  %-8s %10d  %6.2f%%" % (k, sc[k], 100.0 * sc[k] / total))
    if dd is not None:
        log_info("duplicates: exact %d  near %d  (%.2f%% of %d)" % (dd.exact_dups, dd.near_dups,
                                                                    100.0 * (dd.exact_dups + dd.near_dups) / max(1, dd.seen), dd.seen))
    if a.pii:
        log_info("personal data: " + (" ".join("%s=%d" % kv for kv in sorted(pii.items())) or "none found"))
    if a.quality:
        log_info("quality filter would reject %d document(s): %s" % (sum(rejected.values()),
                                                                     " ".join("%s=%d" % kv for kv in rejected.most_common())))
    for tag, rows in samples.items():
        log_info("---- sample: %s ----" % tag)
        for r in rows:
            log_info("  " + r)
    return 0


if __name__ == "__main__":
    sys.exit(main())
