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
from ..utils.log import human_bytes, human_count, log_error, log_info


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
    # the report goes to stdout as the reference's does (dataset/corpus_stats.cpp:92-140): totals, share of documents
    # per language (by name), per script and style, lengths, vocabulary use
    docs = st["documents"]
    share = lambda k: 100.0 * k / docs
    out = ["", "==================== corpus statistics ====================",
           "  documents          : %s" % human_count(docs),
           "  lines              : %s" % human_count(st["lines"]),
           "  bytes              : %s" % human_bytes(st["bytes"]),
           "  characters         : %s" % human_count(st["characters"]),
           "  words              : %s" % human_count(st["words"])]
    if tok is not None:
        out += ["  tokens             : %s" % human_count(st["tokens"]),
                "  tokens / word      : %.3f" % (st["tokens_per_word"] or 0.0),
                "  bytes / token      : %.3f" % (st["bytes_per_token"] or 0.0)]
    out += ["", "  -- language distribution (share of documents) --"]
    out += ["    %-14s %8s  %6.2f%%" % (k, human_count(v), share(v)) for k, v in sorted(st["languages"].items())]
    sy = st["style"]
    out += ["", "  -- script / style --",
            "    arabic script    %6.2f%%" % share(sy["arabic_script"]), "    latin script     %6.2f%%" % share(sy["latin_script"]),
            "    arabizi          %6.2f%%" % share(sy["arabizi"]), "    french-mixed     %6.2f%%" % share(sy["french_mixed"]),
            "    contains emoji   %6.2f%%" % share(sy["emoji"])]
    sc = st["scripts"]
    total = max(1, sum(sc.values()))
    out += ["    letters by script: " + "  ".join("%s %.2f%%" % (k, 100.0 * sc[k] / total) for k in ("arabic", "latin", "digits", "emoji"))]
    out += ["", "  -- length --", "    avg chars/doc    %.1f" % st["avg_chars"], "    avg words/doc    %.1f" % st["avg_words"],
            "    words p50/p90/p99  %d / %d / %d" % (st["words_p50"], st["words_p90"], st["words_p99"])]
    if "avg_tokens" in st:
        out += ["    avg tokens/doc   %.1f" % st["avg_tokens"], "    median tokens    %d" % st["median_tokens"],
                "    p10/p50/p90/p99  %d / %d / %d / %d" % (st["tokens_p10"], st["tokens_p50"], st["tokens_p90"], st["tokens_p99"]),
                "", "  -- vocabulary --",
                "    distinct tokens  %s / %d  (%.1f%% coverage)" % (human_count(st["vocab_used"]), tok.vocab_size,
                                                                      100.0 * st["vocab_used"] / max(1, tok.vocab_size)),
                "    byte-fallback    %.2f%% of used vocab" % (100.0 * st["byte_fallback"])]
    if dd is not None and dd.seen:
        out += ["", "  duplicate ratio    : %.2f%%" % (100.0 * (dd.exact_dups + dd.near_dups) / dd.seen)]
    out += ["==========================================================="]
    print("\n".join(out))
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
