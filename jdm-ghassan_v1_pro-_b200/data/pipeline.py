"""Dataset construction: readers (text lines, JSON / JSON lines, Parquet), cleaning, quality and style gates,
language tagging, exact + near-duplicate removal with an evaluation blocklist, tokenisation and shard writing
(tools/data_pipeline_cli.cpp, dataset/*.cpp in the reference).

Documents become token windows ``<s> ... </s>`` of at most ``seq_len`` tokens (long documents are split, not cut
off); chat records go through the chat template and carry a loss mask (assistant spans).  Windows are dealt to
``train_[<domain>_]NNNN.gbin`` / ``val_[<domain>_]NNNN.gbin`` shards of ``shard_tokens`` tokens; every
``1/val_ratio``-th window goes to validation.
"""
from __future__ import annotations

import glob
import json
import os
from collections import Counter
from dataclasses import dataclass, field
from typing import Dict, Iterable, Iterator, List, Optional, Tuple

import numpy as np

from .. import _gb200_host as H
from . import tokenizer as T
from ..utils.log import human_count


# ---------------------------------------------------------------------------------------------- readers
@dataclass
class Record:
    text: str = ""
    messages: Optional[List[T.Message]] = None       # chat record when not None
    source: str = ""


def _messages_from(obj) -> Optional[List[T.Message]]:
    """Accepts {"messages": [{role, content}...]}, {"conversations": [{from, value}...]}, question/answer,
    instruction/(input)/output, prompt/response."""
    if not isinstance(obj, dict):
        return None
    roles = {"human": "user", "user": "user", "gpt": "assistant", "assistant": "assistant", "system": "system", "bot": "assistant"}
    for key in ("messages", "conversations", "conversation", "dialog"):
        seq = obj.get(key)
        if isinstance(seq, list) and seq:
            out = []
            for m in seq:
                if not isinstance(m, dict):
                    return None
                role = roles.get(str(m.get("role", m.get("from", ""))).lower())
                content = m.get("content", m.get("value"))
                if role is None or not isinstance(content, str):
                    return None
                out.append(T.Message(role, content))
            return out
    for q, a in (("question", "answer"), ("prompt", "response"), ("instruction", "output"), ("input", "output")):
        if isinstance(obj.get(q), str) and isinstance(obj.get(a), str):
            user = obj[q]
            if q == "instruction" and isinstance(obj.get("input"), str) and obj["input"].strip():
                user = user + "\n" + obj["input"]
            msgs = [T.Message("user", user), T.Message("assistant", obj[a])]
            if isinstance(obj.get("system"), str) and obj["system"].strip():
                msgs.insert(0, T.Message("system", obj["system"]))
            return msgs
    return None


def _record_from(obj, source) -> Optional[Record]:
    msgs = _messages_from(obj)
    if msgs:
        return Record(messages=msgs, source=source)
    if isinstance(obj, dict):
        for key in ("text", "content", "body", "document"):
            if isinstance(obj.get(key), str):
                return Record(text=obj[key], source=source)
    if isinstance(obj, str):
        return Record(text=obj, source=source)
    return None


def read_text_lines(path: str) -> Iterator[Record]:
    with open(path, "rb") as f:
        for raw in f:
            line = raw.rstrip(b"\r\n")
            if line:
                yield Record(text=line.decode("utf-8", errors="surrogateescape"), source=path)


def read_json(path: str) -> Iterator[Record]:
    """A JSON array / object, or one JSON value per line."""
    data = open(path, "rb").read().decode("utf-8", errors="replace")
    try:
        top = json.loads(data)
        rows = top if isinstance(top, list) else (top.get("data") or top.get("rows") or [top])
    except json.JSONDecodeError:
        rows = []
        for line in data.splitlines():
            line = line.strip()
            if line:
                try:
                    rows.append(json.loads(line))
                except json.JSONDecodeError:
                    continue
    for r in rows:
        rec = _record_from(r, path)
        if rec is not None:
            yield rec


def read_parquet(path: str, limit: int = 0) -> Iterator[Record]:
    """Rows of a Parquet file: chat columns (messages / conversations, as lists of structs or JSON strings),
    question/answer style pairs, or a text column."""
    import pyarrow.parquet as pq
    pf = pq.ParquetFile(path)
    n = 0
    for batch in pf.iter_batches(batch_size=2048):
        for row in batch.to_pylist():
            for k, v in list(row.items()):
                if isinstance(v, str) and k in ("messages", "conversations") and v[:1] in "[{":
                    try:
                        row[k] = json.loads(v)
                    except json.JSONDecodeError:
                        pass
            rec = _record_from(row, path)
            if rec is not None:
                yield rec
                n += 1
                if limit and n >= limit:
                    return


def iter_inputs(path: str, match: str = "") -> Iterator[Record]:
    files = [path] if os.path.isfile(path) else sorted(
        p for p in glob.glob(os.path.join(path, "**", "*"), recursive=True) if os.path.isfile(p))
    for p in files:
        if match and match not in os.path.basename(p):
            continue
        ext = os.path.splitext(p)[1].lower()
        if ext == ".parquet":
            yield from read_parquet(p)
        elif ext in (".json", ".jsonl"):
            yield from read_json(p)
        elif ext in (".txt", ".text", ".md", ""):
            yield from read_text_lines(p)


# ---------------------------------------------------------------------------------------------- builder
@dataclass
class BuildConfig:
    seq_len: int = 4096
    shard_tokens: int = 50_000_000
    val_ratio: float = 0.005
    domain: str = ""
    style_mode: str = "darija"          # darija | en | off : which quality / robotic-style gates apply
    keep_robotic: bool = False
    min_keep: int = 1
    dedup: bool = True
    blocklist: List[str] = field(default_factory=list)     # texts (e.g. evaluation prompts) that must not enter training


@dataclass
class BuildReport:
    seen: int = 0
    kept_docs: int = 0
    kept_windows: int = 0
    split_docs: int = 0
    train_windows: int = 0
    train_tokens: int = 0
    val_windows: int = 0
    val_tokens: int = 0
    train_shards: int = 0
    val_shards: int = 0
    dropped: Counter = field(default_factory=Counter)
    languages: Counter = field(default_factory=Counter)
    dedup: Dict[str, int] = field(default_factory=dict)

    def summary(self) -> str:
        lines = ["raw documents      : %d" % self.seen, "passed cleaning    : %d" % self.kept_docs,
                 "split windows      : %d source docs exceeded seq_cap" % self.split_docs,
                 "kept windows        : %d" % self.kept_windows,
                 "train windows/tokens: %d / %d  (%d shards)" % (self.train_windows, self.train_tokens, self.train_shards),
                 "val   windows/tokens: %d / %d  (%d shards)" % (self.val_windows, self.val_tokens, self.val_shards)]
        for k, v in sorted(self.dropped.items()):
            lines.append("dropped %-12s: %d" % (k, v))
        total = sum(self.languages.values()) or 1
        for k, v in self.languages.most_common():
            lines.append("  %-12s %8d  %6.2f%%" % (k, v, 100.0 * v / total))
        if self.dedup:
            lines.append("dedup: " + " ".join("%s=%d" % kv for kv in self.dedup.items()))
        return "\n".join(lines)


class _ShardSink:
    def __init__(self, out_dir, prefix, vocab, with_mask, shard_tokens):
        self.dir, self.prefix, self.vocab, self.with_mask, self.cap = out_dir, prefix, vocab, with_mask, shard_tokens
        self.w, self.n_shards, self.in_shard, self.windows, self.tokens = None, 0, 0, 0, 0

    def add(self, ids: np.ndarray, mask: Optional[np.ndarray]):
        if self.w is None or self.in_shard >= self.cap:
            self.close()
            path = os.path.join(self.dir, "%s%04d.gbin" % (self.prefix, self.n_shards))
            self.w = H.ShardWriter(path, self.vocab, self.with_mask)
            self.n_shards += 1
            self.in_shard = 0
        self.w.add_document(ids, mask if self.with_mask else None)
        self.in_shard += len(ids)
        self.windows += 1
        self.tokens += len(ids)

    def close(self):
        if self.w is not None:
            self.w.close()
            self.w = None


def _windows(ids: np.ndarray, mask: Optional[np.ndarray], seq_len: int):
    """One encoded document as consecutive windows of at most ``seq_len`` tokens (no overlap; every window is kept)."""
    for lo in range(0, len(ids), seq_len):
        yield ids[lo:lo + seq_len], (None if mask is None else mask[lo:lo + seq_len])


def build_shards(records: Iterable[Record], tok: T.Tokenizer, out_dir: str, cfg: BuildConfig) -> BuildReport:
    """The reference builder's procedure (tools/data_pipeline_cli.cpp:1340-1620 there), so that both write the same shards
    from the same input wherever their word lists agree:

    * a text line: cleaned (PII lines dropped, or redacted for English), quality gate (the English limits for style
      ``en``, the default ones otherwise: the gate is on in every style), toxicity, duplicate, then encoded with BOS / EOS
      and supervised everywhere;
    * a conversation: every message cleaned and passed through the quality gate on its own (one failure drops the
      conversation), then toxicity and PII per message and, unless the style is ``off`` or robotic replies are kept, the
      assistant-style check of each reply against the message before it; the duplicate key and the language are taken
      from all messages joined by new lines; encoded with the chat template, assistant tokens supervised;
    * a document goes to validation when the FNV-1a hash of its canonical key, modulo 10000, is below 10000 x
      ``val_ratio``; all windows of a document follow it;
    * shards always carry loss masks; a shard is closed once it holds ``shard_tokens`` tokens.
    """
    os.makedirs(out_dir, exist_ok=True)
    rep = BuildReport()
    english = cfg.style_mode == "en"
    cc = H.CleanConfig()
    cc.drop_pii_lines = not english
    cc.redact_instead_drop = english
    cleaner = H.Cleaner(cc)
    quality = H.quality_check_english if english else H.quality_check
    style_filter = cfg.style_mode != "off" and not cfg.keep_robotic
    dd = H.Deduplicator() if cfg.dedup else None
    if dd is not None:
        for t in cfg.blocklist:
            dd.add_blocklist_text(t)
    st = H.CleanStats()
    dom = (cfg.domain + "_") if cfg.domain else ""
    train = _ShardSink(out_dir, "train_" + dom, tok.vocab_size, True, cfg.shard_tokens)
    val = _ShardSink(out_dir, "val_" + dom, tok.vocab_size, True, cfg.shard_tokens)
    val_cut = int(cfg.val_ratio * 10000.0)

    def clean(text: str) -> Optional[str]:
        return cleaner.clean_line(text.encode("utf-8", errors="surrogateescape"), st)

    def emit(ids: np.ndarray, mask: np.ndarray, key: str, lang: str):
        if len(ids) == 0:
            return
        canon = H.canonical_text(key)
        to_val = (H.fnv1a64((canon or key).encode("utf-8", errors="surrogateescape")) % 10000) < val_cut
        if len(ids) > cfg.seq_len:
            rep.split_docs += 1
        for w_ids, w_mask in _windows(ids, mask, cfg.seq_len):
            (val if to_val else train).add(np.ascontiguousarray(w_ids), np.ascontiguousarray(w_mask))
            rep.kept_windows += 1
            rep.languages[lang] += 1

    for rec in records:
        rep.seen += 1
        if rec.messages is not None:
            if not rec.messages:
                continue
            msgs, bad = [], False
            for m in rec.messages:
                c = clean(m.content)
                if c is None or len(c.encode("utf-8", errors="surrogateescape")) < 2 or not quality(c)[0]:
                    bad = True
                    break
                msgs.append(T.Message(m.role, c))
            if bad:
                rep.dropped["quality"] += 1
                continue
            key = "".join(m.content + "\n" for m in msgs)
            why = None
            for i, m in enumerate(msgs):
                if H.check_toxicity(m.content)["toxic"]:
                    why = "toxicity"
                elif H.scan_pii(m.content)["total"] > 0:
                    why = "pii"
                elif style_filter and m.role == "assistant":
                    if english:
                        robotic = H.has_hard_ai_boilerplate(m.content)
                    else:
                        robotic = H.check_assistant_style(m.content, msgs[i - 1].content if i > 0 else "")["robotic"]
                    if robotic:
                        why = "robotic"
                if why:
                    break
            if why:
                rep.dropped[why] += 1
                continue
            rep.kept_docs += 1
            if dd is not None and not dd.add(key):
                rep.dropped["duplicate"] += 1
                continue
            ids, mask = T.encode_chat(tok, msgs)
            emit(np.asarray(ids, dtype=np.int32), np.asarray(mask, dtype=np.uint8), key, H.classify_language(key)["tag"])
        else:
            body = clean(rec.text)
            if body is None:
                continue
            rep.kept_docs += 1
            if not quality(body)[0]:
                rep.dropped["quality"] += 1
                continue
            if H.check_toxicity(body)["toxic"]:
                rep.dropped["toxicity"] += 1
                continue
            if dd is not None and not dd.add(body):
                rep.dropped["duplicate"] += 1
                continue
            ids = np.asarray(tok.encode(body, add_bos=True, add_eos=True), dtype=np.int32)
            emit(ids, np.ones(len(ids), dtype=np.uint8), body, H.classify_language(body)["tag"])
    if dd is not None:
        rep.dedup = {"seen": dd.seen, "exact_dup": dd.exact_dups, "near_dup": dd.near_dups, "blocked": dd.blocked}
    rep.dropped["pii"] += int(st.dropped_pii)
    rep.dropped["encoding"] += int(st.dropped_encoding)
    train.close()
    val.close()
    rep.train_windows, rep.train_tokens, rep.train_shards = train.windows, train.tokens, train.n_shards
    rep.val_windows, rep.val_tokens, rep.val_shards = val.windows, val.tokens, val.n_shards
    if rep.kept_windows < cfg.min_keep:
        raise ValueError("only %d windows kept (min_keep %d)" % (rep.kept_windows, cfg.min_keep))
    return rep


def inspect_shards(directory: str, tok: Optional[T.Tokenizer] = None, show: int = 2) -> str:
    """One line per shard with its first documents decoded, then per split (train, val) the shard count and the
    token total, as the reference's ``inspect`` sums them (tools/data_pipeline_cli.cpp:1654-1700)."""
    lines = []
    totals = {"train": [0, 0, 0], "val": [0, 0, 0]}
    for p in sorted(glob.glob(os.path.join(directory, "*.gbin"))):
        s = H.ShardFile()
        ok, why = s.open(p)
        if not ok:
            lines.append("%s: INVALID (%s)" % (os.path.basename(p), why))
            continue
        split = "val" if os.path.basename(p).startswith("val") else "train"
        totals[split][0] += 1
        totals[split][1] += s.n_tokens
        totals[split][2] += s.n_docs
        lines.append("%s: %d docs, %d tokens%s" % (os.path.basename(p), s.n_docs, s.n_tokens, ", loss masks" if s.has_mask else ""))
        start = 0
        for d in range(min(show, s.n_docs)):
            end = s.doc_end_after(start)
            ids = np.asarray(s.tokens(start, end - start))
            txt = tok.decode(ids, skip_special=True) if tok is not None else " ".join(map(str, ids[:24]))
            lines.append("    [%d] %s" % (d, txt[:160].replace("\n", " ")))
            start = end
    for split in ("train", "val"):
        n, t, d = totals[split]
        if n:
            lines.append("---- %s: %d shards, %d docs, total: %s tokens ----" % (split, n, d, human_count(t)))
    return "\n".join(lines)


def corpus_stats(records: Iterable[Record], tok: Optional[T.Tokenizer] = None) -> dict:
    """Counts for the ``corpus_stats`` command, by the reference analyser's definitions (dataset/corpus_stats.cpp:10-90):
    a document's script is Arabic or Latin when more than 60 % of its letters are; it is Arabizi above an Arabizi score
    of 0.02 and French-mixed when tagged Darija with a French score above 0.05; lines are newlines + 1; the median is
    the upper middle element and a percentile p the element at floor(p * (n - 1)) of the sorted token counts; the
    byte-fallback share is the part of the distinct tokens used that are raw byte tokens (ids 16..271)."""
    n = chars = words = toks = nbytes = lines = 0
    langs, scripts, style = Counter(), Counter(), Counter()
    lengths, doc_tokens, used = [], [], set()
    for rec in records:
        text = rec.text if rec.messages is None else "\n".join(m.content for m in rec.messages)
        if not text:
            continue
        n += 1
        nbytes += len(text.encode("utf-8", "surrogatepass"))
        lines += 1 + text.count("\n")
        w = len(text.split())
        words += w
        lengths.append(w)
        lang = H.classify_language(text)
        langs[lang["tag"]] += 1
        st = H.script_stats(text)
        chars += st["total"]
        for k in ("arabic", "latin", "digits", "emoji"):
            scripts[k] += st[k]
        letters = st["arabic"] + st["latin"]
        if letters and st["arabic"] / letters > 0.6:
            style["arabic_script"] += 1
        elif letters and st["latin"] / letters > 0.6:
            style["latin_script"] += 1
        style["emoji"] += st["emoji"] > 0
        style["arabizi"] += lang["arabizi_score"] > 0.02
        style["french_mixed"] += lang["french_score"] > 0.05 and lang["tag"] in ("ar-MA-arab", "ar-MA-latn")
        if tok is not None:
            ids = tok.encode(text)
            toks += len(ids)
            doc_tokens.append(len(ids))
            used.update(int(i) for i in ids)
    lengths.sort()
    doc_tokens.sort()
    pct = lambda q: lengths[min(len(lengths) - 1, int(q * len(lengths)))] if lengths else 0
    tq = lambda q: doc_tokens[int(q * (len(doc_tokens) - 1))] if doc_tokens else 0
    out = {"documents": n, "lines": lines, "bytes": nbytes, "characters": chars, "words": words, "tokens": toks,
           "tokens_per_word": (toks / words) if (tok is not None and words) else None,
           "bytes_per_token": (nbytes / toks) if toks else None,
           "avg_chars": chars / n if n else 0.0, "avg_words": words / n if n else 0.0,
           "words_p50": pct(0.5), "words_p90": pct(0.9), "words_p99": pct(0.99),
           "languages": dict(langs.most_common()), "scripts": dict(scripts),
           "style": {k: int(style[k]) for k in ("arabic_script", "latin_script", "arabizi", "french_mixed", "emoji")}}
    if doc_tokens:
        raw = sum(1 for i in used if 16 <= i < 272)
        out.update({"avg_tokens": toks / len(doc_tokens), "median_tokens": doc_tokens[len(doc_tokens) // 2],
                    "tokens_p10": tq(0.10), "tokens_p50": tq(0.50), "tokens_p90": tq(0.90), "tokens_p99": tq(0.99),
                    "vocab_used": len(used), "byte_fallback": raw / len(used) if used else 0.0})
    return out
