"""Dataset construction (the reference's ``data_pipeline``, tools/data_pipeline_cli.cpp:30-1720).

    data_pipeline parquet        --lake <dir|file.parquet> --tokenizer tok.gtok --out shards [--match s] [--domain d] [--mode auto|qa|text|chat]
    data_pipeline parquet-corpus --lake <dir> --out corpus.txt [--limit n]
    data_pipeline build          --tokenizer tok.gtok --out shards [--text path] [--chat file.jsonl] [--synth n]
    data_pipeline synth          --out synth.jsonl --n 50000 [--config configs/synthesis_large_200k.yaml [--section synth|sft_synth]]
    data_pipeline synth-en       --out synth_en.jsonl --n 20000 [--seed 4321]
    data_pipeline inspect        --shards shards [--tokenizer tok.gtok]
    data_pipeline tok-info       --tokenizer tok.gtok
    data_pipeline csvs           --dir <csv-root> --out corpus_csv.txt [--with-english]
    data_pipeline csv2json       --dir <csv-root> --out json_shards [--docs-per-file n] [--id-start n]
    data_pipeline jsons          --dir <json-root> --out corpus_json.txt
    data_pipeline json           --input <file.json|jsonl> [--limit n]          # show how records are read
    data_pipeline retrieve       --index <json file|dir> --query "salam labas" [--top 3] [--min-score f]

(run as ``python -m ghassan_b200.cli.data_pipeline <command> ...``).  Shard-building commands share: --val-ratio
--shard-tokens --seq-len --domain --min-keep --keep-robotic --style-mode darija|en|off --no-dedup --expect-vocab
--blocklist <file>.
"""
from __future__ import annotations

import argparse
import glob
import itertools
import json
import os
import sys
from typing import Iterator, List, Optional

from .common import add_common_flags, apply_common_flags

from .. import _gb200_host as H
from ..data import pipeline as P
from ..data import retrieval as R
from ..data import synth as S
from ..data import tokenizer as T
from ..utils.log import human_count, log_error, log_info, log_warn

COMMANDS = ["parquet", "parquet-corpus", "build", "synth", "synth-en", "inspect", "tok-info", "csvs", "csv2json", "jsons", "json",
            "json-inspect", "dump-text", "retrieve"]


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="data_pipeline")
    ap.add_argument("command", choices=COMMANDS)
    ap.add_argument("rest", nargs="*")
    for n in ("lake", "dir", "match", "tokenizer", "out", "domain", "style-mode", "mode", "text", "chat", "shards", "index", "query",
              "input", "blocklist", "config", "section"):
        ap.add_argument("--" + n, default="")
    for n, d in (("val-ratio", 0.005), ("min-score", 0.0)):
        ap.add_argument("--" + n, type=float, default=d)
    for n, d in (("shard-tokens", 50_000_000), ("seq-len", 4096), ("min-keep", 1), ("expect-vocab", 0), ("limit", 0), ("n", None),
                 ("synth", 0), ("seed", None), ("top", 3), ("docs-per-file", 20000), ("id-start", 1_000_000), ("min-chars", 2)):
        ap.add_argument("--" + n, type=int, default=d)
    for n in ("keep-robotic", "keep-case", "no-dedup", "probe", "with-english", "english"):
        ap.add_argument("--" + n, action="store_true")
    return ap


def _load_tok(a) -> T.Tokenizer:
    if not a.tokenizer:
        raise SystemExit("--tokenizer <path> is required")
    tok = T.Tokenizer.load(a.tokenizer)
    if a.expect_vocab and tok.vocab_size != a.expect_vocab:
        raise SystemExit("tokenizer vocab %d != --expect-vocab %d" % (tok.vocab_size, a.expect_vocab))
    lower = bool(H.NormalizerConfig.unpack(tok.normalizer_bits).lowercase_latin)
    if a.keep_case and lower:
        raise SystemExit("--keep-case given but the tokenizer lowercases Latin; retrain it with --keep-case")
    if not a.keep_case and not lower:
        log_warn("[tok ] the tokenizer keeps Latin case; pass --keep-case to acknowledge (shards follow the tokenizer)")
    return tok


def _build_cfg(a) -> P.BuildConfig:
    # the reference's defaults: `build` works in the English style, the Parquet reader in the Darija one
    style = a.style_mode or ("en" if getattr(a, "command", "") == "build" else "darija")
    if style not in ("darija", "en", "off"):
        raise SystemExit("--style-mode must be darija|en|off")
    block: List[str] = []
    if a.blocklist:
        block = [ln.strip() for ln in open(a.blocklist, encoding="utf-8") if ln.strip()]
    if a.seq_len < 8 or a.shard_tokens < a.seq_len or not (0.0 <= a.val_ratio < 1.0):
        raise SystemExit("--seq-len must be >= 8, --shard-tokens >= --seq-len and --val-ratio in [0, 1)")
    return P.BuildConfig(seq_len=a.seq_len, shard_tokens=a.shard_tokens, val_ratio=a.val_ratio, domain=a.domain, style_mode=style,
                         keep_robotic=a.keep_robotic, min_keep=a.min_keep, dedup=not a.no_dedup, blocklist=block)


def _mode_filter(recs: Iterator[P.Record], mode: str) -> Iterator[P.Record]:
    """--mode of the parquet command: qa/chat keep conversations only, text flattens everything to lines."""
    any_chat = False
    for r in recs:
        if mode in ("qa", "chat"):
            if r.messages is None:
                continue
            any_chat = True
            yield r
        elif mode == "text":
            yield r if r.messages is None else P.Record(text="\n".join(m.content for m in r.messages), source=r.source)
        else:
            yield r
    if mode in ("qa", "chat") and not any_chat:
        raise SystemExit("--mode %s: no question/answer or message rows in the input" % mode)


def _csv_files(root: str) -> List[str]:
    if os.path.isfile(root):
        return [root]
    return sorted(p for p in glob.glob(os.path.join(root, "**", "*"), recursive=True) if p.endswith(".csv") and os.path.isfile(p))


# How the vocabulary and grammar tables are read (the reference's tools/data_pipeline_cli.cpp:894-926, 928-1030, 1099-1215):
# a first row counts as a header only when it names one of the known columns; every column then has a role: bookkeeping
# (skipped), Arabic script, English gloss, or a Darija variant (everything else).  A table without such a header has
# variants only, its first row included.  Cells are flattened to one line and measured in bytes.
_META_COLS = ("id", "source", "dataset_source", "metadata", "token_count", "word_count", "count", "freq")
_HEADER_NAMES = ("darija", "darija_ar", "eng", "english", "root", "arabic")
_SKIP, _VARIANT, _ARABIC, _ENGLISH = 0, 1, 2, 3
_ASCII_LOWER = str.maketrans("ABCDEFGHIJKLMNOPQRSTUVWXYZ", "abcdefghijklmnopqrstuvwxyz")


def _flat(cell: str) -> str:
    return cell.replace("\n", " ").replace("\r", " ").replace("\t", " ").strip(" \t\r\n")


def _split_row(line: str) -> List[str]:
    """One physical line into cells: commas split, double quotes group, a doubled quote inside quotes is a quote."""
    cells, cur, quoted, i = [], [], False, 0
    while i < len(line):
        c = line[i]
        if quoted:
            if c == '"' and line[i + 1:i + 2] == '"':
                cur.append('"')
                i += 1
            elif c == '"':
                quoted = False
            else:
                cur.append(c)
        elif c == '"':
            quoted = True
        elif c == ",":
            cells.append("".join(cur))
            cur = []
        else:
            cur.append(c)
        i += 1
    cells.append("".join(cur))
    return cells


def _role(name: str) -> int:
    n = name.strip(" \t\r\n").translate(_ASCII_LOWER)
    if n in _META_COLS:
        return _SKIP
    if n in ("arabic", "ar", "darija_ar") or (len(n) > 3 and n.endswith("_ar")):
        return _ARABIC
    if n.startswith("eng"):
        return _ENGLISH
    return _VARIANT


def _table_rows(path: str, min_bytes: int):
    """Yields (variants, arabic cells, english cells, cells in column order as (role, text)) per non-empty row."""
    with open(path, "rb") as f:
        data = f.read()
    if data.startswith(b"\xef\xbb\xbf"):
        data = data[3:]
    lines = [ln[:-1] if ln.endswith("\r") else ln for ln in data.decode("utf-8", "surrogateescape").split("\n")]
    if lines and lines[-1] == "":
        lines.pop()
    if not lines:
        return
    first = [c.strip(" \t\r\n").translate(_ASCII_LOWER) for c in _split_row(lines[0])]
    roles = None
    if any(n in _HEADER_NAMES or n.startswith("n1") for n in first):
        roles = [_role(c) for c in _split_row(lines[0])]
        lines = lines[1:]
    for ln in lines:
        if not ln:
            continue
        ordered = []
        for i, cell in enumerate(_split_row(ln)):
            r = _VARIANT if roles is None or i >= len(roles) else roles[i]
            t = _flat(cell)
            if r != _SKIP and len(t.encode("utf-8", "surrogateescape")) >= min_bytes:
                ordered.append((r, t))
        yield ordered


def _write_text(f, t: str) -> None:
    f.write(t.encode("utf-8", "surrogateescape") + b"\n")


def cmd_csvs(a) -> int:
    """Tables -> corpus lines for the tokenizer trainer: each distinct cell once (English glosses only with
    --with-english), plus one alignment line "variant / [second variant /] arabic" per row that has both."""
    files = _csv_files(a.dir or ".")
    if not files:
        log_error("no .csv files found under: " + (a.dir or "."))
        return 1
    log_info("[csvs] found %d file(s) under %s" % (len(files), a.dir or "."))
    out_path = a.out or "corpus_csv.txt"
    if os.path.dirname(out_path):
        os.makedirs(os.path.dirname(out_path), exist_ok=True)
    seen, kept, aligned, rows_in = set(), 0, 0, 0
    with open(out_path, "wb") as out:
        def emit(t: str) -> bool:
            nonlocal kept
            t = _flat(t)
            if len(t.encode("utf-8", "surrogateescape")) < a.min_chars or t in seen:
                return False
            seen.add(t)
            _write_text(out, t)
            kept += 1
            return True

        for p in files:
            for cells in _table_rows(p, a.min_chars):
                rows_in += 1
                variants = [t for r, t in cells if r == _VARIANT]
                arabic = next((t for r, t in cells if r == _ARABIC), "")
                for r, t in cells:
                    if r != _ENGLISH or a.with_english:
                        emit(t)
                if variants and arabic and variants[0] != arabic:
                    parts = [variants[0]]
                    if len(variants) > 1 and variants[1] not in (variants[0], arabic):
                        parts.append(variants[1])
                    t = _flat(" / ".join(parts + [arabic]))
                    if t not in seen:
                        seen.add(t)
                        _write_text(out, t)
                        kept += 1
                        aligned += 1
    log_info("[csvs] %s rows in, %s corpus lines (alignment lines: %s) -> %s" % (human_count(rows_in), human_count(kept), human_count(aligned), out_path))
    if kept < a.min_keep:
        log_error("only %d lines kept (--min-keep %d)" % (kept, a.min_keep))
        return 1
    return 0


def cmd_csv2json(a) -> int:
    """Tables -> id/question/answer files.  Per row: every variant against the Arabic cell; without Arabic the first
    variant against the English gloss; without either the first variant against each other one.  Pairs with equal
    sides, a side under --min-chars bytes or a question seen before are skipped."""
    files = _csv_files(a.dir or ".")
    if not files:
        log_error("no .csv files found under: " + (a.dir or "."))
        return 1
    if a.docs_per_file <= 0 or a.id_start < 0:
        raise SystemExit("--docs-per-file must be > 0 and --id-start >= 0")
    outdir = a.out or "json_shards"
    os.makedirs(outdir, exist_ok=True)
    seen, pairs, idx, in_file, next_id, rows_in = set(), 0, 0, 0, a.id_start, 0
    skipped = {"same": 0, "empty": 0, "dup": 0}
    jf = None

    def close():
        nonlocal jf
        if jf is not None:
            jf.write(b"\n]\n")
            jf.close()
            jf = None

    def pair(q: str, ans: str) -> None:
        nonlocal jf, idx, in_file, next_id, pairs
        q, ans = _flat(q), _flat(ans)
        if min(len(q.encode("utf-8", "surrogateescape")), len(ans.encode("utf-8", "surrogateescape"))) < a.min_chars:
            skipped["empty"] += 1
        elif q == ans:
            skipped["same"] += 1
        elif q in seen:
            skipped["dup"] += 1
        else:
            seen.add(q)
            if jf is None or in_file >= a.docs_per_file:
                close()
                path = os.path.join(outdir, "train-%05d.json" % idx)
                jf = open(path, "wb")
                jf.write(b"[\n")
                idx, in_file = idx + 1, 0
                log_info("[json] opened " + path)
            # one key per line, no indentation: the layout the reference's own scanner of these files expects
            rec = "{\n\"id\": %d,\n\"question\": %s,\n\"answer\": %s\n}" % (next_id, json.dumps(q, ensure_ascii=False), json.dumps(ans, ensure_ascii=False))
            jf.write((b",\n" if in_file else b"") + rec.encode("utf-8", "surrogateescape"))
            next_id, in_file, pairs = next_id + 1, in_file + 1, pairs + 1

    for p in files:
        for cells in _table_rows(p, a.min_chars):
            rows_in += 1
            variants = [t for r, t in cells if r == _VARIANT]
            arabic = next((t for r, t in cells if r == _ARABIC), "")
            english = next((t for r, t in cells if r == _ENGLISH), "")
            if variants and arabic:
                for v in variants:
                    pair(v, arabic)
            elif variants and english:
                pair(variants[0], english)
            elif len(variants) >= 2:
                for v in variants[1:]:
                    pair(variants[0], v)
            elif variants:
                skipped["empty"] += 1
    close()
    log_info("[json] %s rows in, %s pairs in %d file(s); skipped: %s" % (human_count(rows_in), human_count(pairs), idx,
                                                                       " ".join("%s=%d" % kv for kv in skipped.items())))
    if pairs < a.min_keep:
        log_error("only %d pairs kept (--min-keep %d)" % (pairs, a.min_keep))
        return 1
    return 0


def cmd_jsons(a) -> int:
    """Question/answer files -> corpus lines: each distinct question and answer once, flattened to one line."""
    docs = R.load_qa_dir(a.dir) if os.path.isdir(a.dir or ".") else R.load_qa_json(a.dir)
    out_path = a.out or "corpus_json.txt"
    if os.path.dirname(out_path):
        os.makedirs(os.path.dirname(out_path), exist_ok=True)
    kept, seen = 0, set()
    with open(out_path, "wb") as out:
        for d in docs:
            for v in (d.question, d.answer):
                t = _flat(v)
                if len(t.encode("utf-8", "surrogateescape")) >= a.min_chars and t not in seen:
                    seen.add(t)
                    _write_text(out, t)
                    kept += 1
    log_info("[jsons] %s pairs -> %s lines in %s" % (human_count(len(docs)), human_count(kept), out_path))
    if kept < a.min_keep:
        log_error("only %d lines kept (--min-keep %d)" % (kept, a.min_keep))
        return 1
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = _parser()
    add_common_flags(ap)
    a = ap.parse_args(argv)
    apply_common_flags(a)
    a.n_given, a.seed_given = a.n is not None, a.seed is not None
    a.n = a.n if a.n_given else 50000
    a.seed = a.seed if a.seed_given else 1
    cmd = a.command
    if cmd in ("parquet", "parquet-corpus"):
        try:
            import pyarrow.parquet  # noqa: F401
        except ImportError:
            log_error("parquet support needs pyarrow, which is not importable here")
            return 1
        if a.probe:
            return 0
        lake = a.lake or a.dir or "dataset/parquet/by_domain"
        recs = P.iter_inputs(lake, a.match)
        if a.limit:
            recs = itertools.islice(recs, a.limit)
        if cmd == "parquet-corpus":
            n = 0
            with open(a.out or "corpus.txt", "w", encoding="utf-8") as out:
                for r in recs:
                    for t in ([r.text] if r.messages is None else [m.content for m in r.messages if m.role != "system"]):
                        t = t.replace("\n", " ").strip()
                        if t:
                            out.write(t + "\n")
                            n += 1
            log_info("[parquet] wrote %s lines to %s" % (human_count(n), a.out or "corpus.txt"))
            return 0 if n >= a.min_keep else 1
        mode = a.mode or "auto"
        if mode not in ("qa", "text", "chat", "auto"):
            raise SystemExit("--mode must be qa|text|chat|auto")
        tok = _load_tok(a)
        try:
            rep = P.build_shards(_mode_filter(recs, mode), tok, a.out or "artifacts/shards", _build_cfg(a))
        except ValueError as e:
            log_error(str(e))
            return 1
        log_info("\n" + rep.summary())
        return 0
    if cmd == "build":
        tok = _load_tok(a)
        streams = []
        if a.text:
            streams.append(P.iter_inputs(a.text))
        if a.chat:
            streams.append(P.iter_inputs(a.chat))
        if a.synth:
            gen = S.english_conversations if a.english else S.darija_conversations
            streams.append(r for r in (P._record_from(row, "synth") for row in gen(a.synth, seed=a.seed)) if r is not None)
        if not streams:
            log_error("nothing to build: give --text, --chat and/or --synth")
            return 1
        try:
            rep = P.build_shards(itertools.chain(*streams), tok, a.out or "artifacts/shards", _build_cfg(a))
        except ValueError as e:
            log_error(str(e))
            return 1
        log_info("\n" + rep.summary())
        return 0
    if cmd in ("synth", "synth-en"):
        from ..utils.config import ConfigError
        if cmd == "synth-en" or a.english:
            out = a.out or "data/synth_en.jsonl"
            rows = S.english_conversations(a.n if a.n_given else 20000, seed=a.seed if a.seed_given else 4321)
        else:
            try:
                scfg = S.load_synth_config(a.config, a.section or "synth") if a.config else S.SynthConfig()
            except ConfigError as e:
                log_error(str(e))
                return 1
            if a.n_given or not a.config:
                scfg.num_conversations = a.n
            if a.seed_given:
                scfg.seed = a.seed
            out = a.out or scfg.output_path or "data/synth.jsonl"
            if a.config:
                log_info("[synth] config %s [%s]: %d conversations, seed %d, turns %d-%d" % (
                    a.config, a.section or "synth", scfg.num_conversations, scfg.seed, scfg.min_turns, scfg.max_turns))
            g = S.DarijaSynthGenerator(scfg)
            rows = g.generate_many(scfg.num_conversations)
            log_info("[synth] " + g.stats.summary())
        os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
        n = S.write_jsonl(out, rows)
        log_info("[synth] wrote %s conversations to %s" % (human_count(n), out))
        return 0
    if cmd == "inspect":
        tok = T.Tokenizer.load(a.tokenizer) if a.tokenizer else None
        print(P.inspect_shards(a.shards or "artifacts/shards", tok))
        return 0
    if cmd == "tok-info":
        tok = _load_tok(a)
        n = H.NormalizerConfig.unpack(tok.normalizer_bits)
        print("vocab_size=%d" % tok.vocab_size)          # the line shell scripts of the reference's tool read
        print("vocab        : %d (%d special)" % (tok.vocab_size, T.N_SPECIAL))
        print("fingerprint  : %s" % H.fingerprint_hex(H.fingerprint_file(a.tokenizer)))
        print("normalizer   : " + " ".join(k for k in ("strip_diacritics", "strip_tatweel", "fold_letters", "lowercase_latin",
                                                       "arabic_digits_ascii", "collapse_repeats", "collapse_whitespace") if getattr(n, k)))
        longest = sorted(range(T.N_SPECIAL, tok.vocab_size), key=lambda i: -len(tok.token_bytes(i)))[:10]
        print("longest      : " + " | ".join(tok.token_bytes(i).decode("utf-8", "replace") for i in longest))
        return 0
    if cmd == "csvs":
        return cmd_csvs(a)
    if cmd == "csv2json":
        return cmd_csv2json(a)
    if cmd == "jsons":
        return cmd_jsons(a)
    if cmd in ("json", "json-inspect", "dump-text"):
        src = a.input or (a.rest[0] if a.rest else "")
        if not src:
            raise SystemExit("--input <file> is required")
        n = 0
        cap = (a.limit or None) if cmd == "dump-text" else (a.limit or 20)
        for r in itertools.islice(P.iter_inputs(src), cap):
            n += 1
            if r.messages is None:
                print(r.text if cmd == "dump-text" else "[text] " + r.text[:160])
            elif cmd == "dump-text":
                for m in r.messages:
                    print(m.content.replace("\n", " "))
            else:
                print("[chat] " + " || ".join("%s: %s" % (m.role, m.content[:80]) for m in r.messages))
        if cmd != "dump-text":
            log_info("%d record(s) shown" % n)
        return 0
    if cmd == "retrieve":
        query = a.query or (a.rest[0] if a.rest else "")
        if not a.index or not query:
            raise SystemExit("--index <train-*.json file|dir> and --query <text> are required")
        ix = R.build_index(a.index)
        if len(ix) == 0:
            log_error("no QA pairs loaded from: " + a.index)
            return 1
        log_info("[retrieve] index: %s pairs" % human_count(len(ix)))
        hits = ix.query(query, a.top if a.top > 0 else 3, a.min_score)
        if not hits:
            log_info("[retrieve] no hit above min-score (answer: spontaneous generation)")
            return 0
        for i, (doc, score) in enumerate(hits):
            e = ix.doc(doc)
            print("--- hit %d  id=%d  score=%.3f ---\nQ: %s\nA: %s" % (i + 1, e.id, score, e.question, e.answer))
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
