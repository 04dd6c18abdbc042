"""Keyword retrieval over question/answer JSON files (dataset/retrieval.cpp:11-576 in the reference): BM25
(k1 1.2, b 0.75) over normalised question words with a fuzzy fallback for unseen words (edit distance 1-2, at 0.75
weight), a character-trigram Dice fallback when no word matches, a bigram bonus (+0.5 each) and an exact-substring
bonus (+5).  Normalisation lowercases ASCII, drops Arabic diacritics, folds the Arabizi digits 3 7 9 5 2 to letters
when the text is Arabic or Arabizi-like, and turns everything else into single spaces."""
from __future__ import annotations

import glob
import json
import math
import os
from collections import Counter
from dataclasses import dataclass
from typing import Dict, List, Tuple

_FOLD = {"3": "a", "7": "h", "9": "q", "5": "k", "2": "a"}
_ARABIZI_DIGITS = set("37952")


def normalize(s: str) -> str:
    raw = s.encode("utf-8", errors="replace")
    has_high = any(b >= 0x80 for b in raw)
    arabizi = False
    for a, b in zip(s, s[1:]):
        a_al, b_al = a.isascii() and a.isalpha(), b.isascii() and b.isalpha()
        if (a_al and b in _ARABIZI_DIGITS) or (a in _ARABIZI_DIGITS and b_al):
            arabizi = True
            break
    fold = has_high or arabizi
    out: List[str] = []
    space = True
    for ch in s:
        o = ord(ch)
        if 0x064B <= o <= 0x0652:                  # harakat
            continue
        if "A" <= ch <= "Z":
            out.append(ch.lower())
            space = False
        elif "a" <= ch <= "z" or o >= 0x80:
            out.append(ch)
            space = False
        elif "0" <= ch <= "9":
            out.append(_FOLD.get(ch, ch) if fold else ch)
            space = False
        else:
            if not space:
                out.append(" ")
            space = True
    return "".join(out).rstrip(" ")


def tokenize(s: str) -> List[str]:
    return [w for w in normalize(s).split(" ") if w]


@dataclass
class QaEntry:
    id: int
    question: str
    answer: str


def load_qa_json(path: str) -> List[QaEntry]:
    """A JSON array (or JSON lines) of objects with ``question`` and ``answer`` (and optionally ``id``)."""
    try:
        text = open(path, encoding="utf-8").read()
    except OSError:
        return []
    rows = None
    try:
        rows = json.loads(text)
    except json.JSONDecodeError:
        rows = []
        for line in text.splitlines():
            line = line.strip()
            if line:
                try:
                    rows.append(json.loads(line))
                except json.JSONDecodeError:
                    pass
    if isinstance(rows, dict):
        rows = rows.get("data") or rows.get("items") or [rows]
    out = []
    for i, r in enumerate(rows or []):
        if isinstance(r, dict) and isinstance(r.get("question"), str) and isinstance(r.get("answer"), str):
            rid = r.get("id", i)
            out.append(QaEntry(int(rid) if isinstance(rid, (int, float)) else i, r["question"], r["answer"]))
    return out


def load_qa_dir(directory: str) -> List[QaEntry]:
    out: List[QaEntry] = []
    for p in sorted(glob.glob(os.path.join(directory, "**", "*.json"), recursive=True)):
        out += load_qa_json(p)
    return out


def _edit_distance(a: str, b: str, maxd: int) -> int:
    n, m = len(a), len(b)
    if abs(n - m) > maxd or n > 15 or m > 15 or n == 0 or m == 0:
        return maxd + 1
    prev = list(range(m + 1))
    for i in range(1, n + 1):
        cur = [i] + [0] * m
        for j in range(1, m + 1):
            cur[j] = min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (a[i - 1] != b[j - 1]))
        prev = cur
    return prev[m]


def _trigrams(s: str) -> Counter:
    t = " " + s + " "
    return Counter(t[i:i + 3] for i in range(len(t) - 2))


class RetrievalIndex:
    K1, B = 1.2, 0.75

    def __init__(self):
        self.docs: List[QaEntry] = []
        self.toks: List[List[str]] = []
        self.norm_q: List[str] = []
        self.idf: Dict[str, float] = {}
        self.inv: Dict[str, List[int]] = {}

    def __len__(self):
        return len(self.docs)

    def build(self, docs: List[QaEntry]) -> None:
        seen = set()
        self.docs = []
        for d in docs:                                   # first occurrence of a normalised question wins
            nq = normalize(d.question)
            if nq and nq not in seen:
                seen.add(nq)
                self.docs.append(d)
        self.toks = [tokenize(d.question) for d in self.docs]
        self.norm_q = [normalize(d.question) for d in self.docs]
        df: Counter = Counter()
        self.inv = {}
        for i, t in enumerate(self.toks):
            for w in dict.fromkeys(t):
                df[w] += 1
                self.inv.setdefault(w, []).append(i)
        n = float(len(self.docs)) if self.docs else 1.0
        self.idf = {w: math.log((n + 1.0) / (c + 1.0)) + 1.0 for w, c in df.items()}

    def query(self, text: str, top_k: int = 3, min_score: float = 0.0) -> List[Tuple[int, float]]:
        if not self.docs or top_k <= 0:
            return []
        qt = tokenize(text)
        if not qt:
            return []
        nq = normalize(text)
        avgdl = max(1.0, sum(len(t) for t in self.toks) / max(1, len(self.toks)))
        acc: Dict[int, float] = {}
        for w, qf in sorted(Counter(qt).items()):
            use, pen = w, 1.0
            if w not in self.idf:
                maxd = 1 if len(w) <= 4 else 2
                best, best_idf = "", 0.0
                for cand, v in sorted(self.idf.items()):
                    if v > best_idf and _edit_distance(w, cand, maxd) <= maxd:
                        best, best_idf = cand, v
                if not best:
                    continue
                use, pen = best, 0.75
            idf = self.idf[use]
            for d in self.inv.get(use, ()):
                tf = self.toks[d].count(use)
                if tf <= 0:
                    continue
                denom = tf + self.K1 * (1.0 - self.B + self.B * len(self.toks[d]) / avgdl)
                acc[d] = acc.get(d, 0.0) + pen * idf * (tf * (self.K1 + 1.0) / denom) * (1.0 + 0.1 * (qf - 1))
        if not acc and nq:
            qg = _trigrams(nq)
            qn = sum(qg.values())
            for d, text_d in enumerate(self.norm_q):
                dg = _trigrams(text_d)
                inter = sum(min(c, dg[g]) for g, c in qg.items() if g in dg)
                if inter:
                    dice = 2.0 * inter / (qn + sum(dg.values()))
                    if dice >= 0.25:
                        acc[d] = dice * 2.0
        hits = []
        for d, s in acc.items():
            td = self.toks[d]
            if len(qt) >= 2 and len(td) >= 2:
                pairs = set(zip(td, td[1:]))
                s += 0.5 * sum(1 for p in zip(qt, qt[1:]) if p in pairs)
            if nq and nq in self.norm_q[d]:
                s += 5.0
            if s >= min_score:
                hits.append((d, s))
        hits.sort(key=lambda h: (-h[1], h[0]))
        return hits[:top_k]

    def doc(self, i: int) -> QaEntry:
        return self.docs[i]


def build_index(path: str) -> RetrievalIndex:
    docs = load_qa_dir(path) if os.path.isdir(path) else (load_qa_json(path) or load_qa_dir(path))
    idx = RetrievalIndex()
    idx.build(docs)
    return idx
