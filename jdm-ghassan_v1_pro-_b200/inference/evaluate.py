"""Perplexity and the heuristic quality benchmark (evaluation/perplexity.cpp:17-58, evaluation/benchmark.cpp:591-790
in the reference).

Benchmark items: {category, id, context (messages), prompt, expect_any, forbid, expect_lang, max_words}.  An item's
score: 0.40 an expected substring appears (or none is required), 0.15 no forbidden substring, 0.10 within the word
limit, 0.10 not robotic, 0.10 not toxic, 0.10 language gate, 0.05 answer discipline (English items) or granted.
"""
from __future__ import annotations

import glob
import json
import os
import re
import time
from collections import Counter
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np

from .. import _gb200_host as H
from ..data import tokenizer as T
from .chat import classify_dialog_act
from .engine import SamplingParams
from .generator import Generator

CATEGORIES = ["basic_conversation", "darija_comprehension", "arabizi_comprehension", "arabic_comprehension", "code_switching",
              "context_retention", "multi_turn", "common_sense", "cultural_context", "instruction_following", "repetition",
              "hallucination", "toxicity", "naturalness"]


# ---------------------------------------------------------------------------------------------- perplexity
def perplexity_text(gen: Generator, text: str) -> dict:
    ids = gen.encode_prompt(text, add_bos=True)
    nll, n = gen.score_tokens(ids)
    return {"tokens": n, "nll": nll / max(1, n), "perplexity": float(np.exp(nll / max(1, n)))}


def perplexity_batches(gen: Generator, directory: str, prefix: str = "val", batch_size: int = 1, seq_len: int = 512,
                       max_batches: int = 20, pack: bool = False, seed: int = 42) -> dict:
    """The reference's held-out measure (evaluation/perplexity.cpp:27-60 there): ``max_batches`` batches of its data
    loader over ``<directory>/<prefix>*.gbin`` (same sampler, same seed, so the same windows), every row scored
    teacher-forced on the supervised positions with its segment mask, z-loss included.  Needs an engine that scores a
    row in one pass (``score_batch``)."""
    from ..data.loader import DataLoader
    dl = DataLoader(batch_size, seq_len, pack, seed, pin=False)
    if not dl.open_glob(directory, prefix):
        raise ValueError("no held-out shards found for perplexity: " + directory)
    total, count, batches = 0.0, 0, 0
    while batches < max_batches:
        b = dl.next()
        if b is None:
            break
        ids, tg, sg = b.ids.numpy(), b.targets.numpy(), b.segments.numpy()
        # one call per batch, as the reference does: the rows of a batch are scored as ONE sequence of B * T positions
        nll, n = gen.engine.score_batch(ids, tg, sg)
        total += nll
        count += n
        batches += 1
    mean = total / max(1, count)
    return {"tokens": count, "nll": mean, "perplexity": float(np.exp(min(20.0, mean))), "batches": batches}


def perplexity_shards(gen: Generator, directory: str, prefix: str = "val_", max_tokens: int = 20000, window: int = 512) -> dict:
    """Token-level NLL over validation shards, document by document, in windows of ``window`` tokens."""
    total, count = 0.0, 0
    for p in sorted(glob.glob(os.path.join(directory, prefix + "*.gbin"))):
        s = H.ShardFile()
        ok, _ = s.open(p)
        if not ok:
            continue
        start = 0
        for _ in range(s.n_docs):
            end = s.doc_end_after(start)
            ids = np.asarray(s.tokens(start, end - start))
            start = end
            for lo in range(0, len(ids) - 1, window):
                nll, n = gen.score_tokens(ids[lo:lo + window + 1])
                total += nll
                count += n
                if count >= max_tokens:
                    break
            if count >= max_tokens:
                break
        if count >= max_tokens:
            break
    return {"tokens": count, "nll": total / max(1, count), "perplexity": float(np.exp(total / max(1, count)))}


# ---------------------------------------------------------------------------------------------- text measures
def _words(text: str) -> List[str]:
    return text.split()


def distinct_n(text: str, n: int) -> float:
    w = _words(text)
    if len(w) < n:
        return 0.0
    grams = [tuple(w[i:i + n]) for i in range(len(w) - n + 1)]
    return len(set(grams)) / len(grams)


def max_ngram_repeat(text: str, n: int) -> int:
    w = _words(text)
    if len(w) < n:
        return 0
    return max(Counter(tuple(w[i:i + n]) for i in range(len(w) - n + 1)).values())


def check_english_reply(user_text: str, reply: str) -> dict:
    """Answer discipline for English items: not empty, no "as an AI" disclosure, a letter answer to a multiple-choice
    prompt, code in the answer to a coding prompt."""
    low = reply.strip().lower()
    act = classify_dialog_act(user_text)
    if len(low) < 2:
        return {"disciplined": False, "reason": "empty", "act": act}
    if any(b in low for b in ("as an ai", "as a language model", "as an ai language model")):
        return {"disciplined": False, "reason": "ai-disclosure", "act": act}
    options = len(re.findall(r"(?<![A-Za-z0-9_])[a-d][.):]", user_text.lower()))
    if options >= 2 and not re.match(r"[a-d][.):]", low):
        return {"disciplined": False, "reason": "bad-mc-format", "act": act}
    if act == "coding" and not any(k in low for k in ("```", "def ", "return ", "function", "{", "print(", "#include", "`")):
        return {"disciplined": False, "reason": "no-code", "act": act}
    return {"disciplined": True, "reason": "", "act": act}


# ---------------------------------------------------------------------------------------------- benchmark
@dataclass
class EvalItem:
    category: str = "basic_conversation"
    id: str = ""
    context: List[T.Message] = field(default_factory=list)
    prompt: str = ""
    expect_any: List[str] = field(default_factory=list)
    forbid: List[str] = field(default_factory=list)
    expect_lang: str = ""
    max_words: int = 0
    note: str = ""


def _items(table) -> List[EvalItem]:
    return [EvalItem(c, i, [T.Message(r, t) for r, t in ctx], p, list(e), list(f), lang, mw)
            for c, i, ctx, p, e, f, lang, mw in table]


def builtin_suite() -> List[EvalItem]:
    """Darija / Arabizi / Arabic items over all fourteen categories (``inference/eval_suites.py``)."""
    from .eval_suites import DARIJA_ITEMS
    return _items(DARIJA_ITEMS)


def builtin_suite_en() -> List[EvalItem]:
    from .eval_suites import ENGLISH_ITEMS
    return _items(ENGLISH_ITEMS)


def load_suite(directory: str) -> List[EvalItem]:
    """Every ``*.jsonl`` file of a directory: one item per line."""
    items: List[EvalItem] = []
    for p in sorted(glob.glob(os.path.join(directory, "*.jsonl"))):
        for line in open(p, encoding="utf-8"):
            line = line.strip()
            if not line:
                continue
            try:
                o = json.loads(line)
            except json.JSONDecodeError:
                continue
            ctx = [T.Message(m.get("role", "user"), m.get("content", "")) for m in o.get("context", []) if isinstance(m, dict)]
            from .eval_suites import category_from_name
            items.append(EvalItem(category_from_name(o.get("category", "")), str(o.get("id", len(items))), ctx, o.get("prompt", ""),
                                  list(o.get("expect_any", [])), list(o.get("forbid", [])), o.get("expect_lang", ""),
                                  int(o.get("max_words", 0)), o.get("note", "")))
    return items


def write_suite(path: str, items: List[EvalItem]) -> None:
    """One compact JSON object per line: the reference reads these files with a scanner that expects no space after
    ``:`` and ``,`` (evaluation/benchmark.cpp:380-470 there)."""
    with open(path, "w", encoding="utf-8") as f:
        for it in items:
            f.write(json.dumps({"category": it.category, "id": it.id, "context": [{"role": m.role, "content": m.content} for m in it.context],
                                "prompt": it.prompt, "expect_any": it.expect_any, "forbid": it.forbid, "expect_lang": it.expect_lang,
                                "max_words": it.max_words, "note": it.note}, ensure_ascii=False, separators=(",", ":")) + "\n")


def score_response(item: EvalItem, response: str, seconds: float = 0.0) -> dict:
    low = response.lower()
    words = len(_words(response))
    matched = not item.expect_any or any(e.lower() in low for e in item.expect_any)
    forbidden = any(b.lower() in low for b in item.forbid)
    length_ok = item.max_words == 0 or words <= item.max_words
    style = H.check_assistant_style(response, item.prompt)
    robotic = bool(style["robotic"])
    toxic = bool(H.check_toxicity(response)["toxic"])
    lang_ok, gated = True, bool(item.expect_lang)
    if gated:
        ls = H.classify_language(response)
        tag = ls["tag"]
        if tag == item.expect_lang:
            lang_ok = True
        elif tag == "mixed" and item.expect_lang in ("ar-MA-arab", "ar-MA-latn", "ar-MSA"):
            lang_ok = True
        elif item.expect_lang == "en" and tag in ("en", "mixed", "other"):
            lang_ok = ls["english_score"] > 0.02
        else:
            lang_ok = False
    disciplined = True
    if item.expect_lang == "en":
        disciplined = check_english_reply(item.prompt, response)["disciplined"]
    s = 0.40 * matched + 0.15 * (not forbidden) + 0.10 * length_ok + 0.10 * (not robotic) + 0.10 * (not toxic) + 0.10 * lang_ok
    s += 0.05 * (disciplined if item.expect_lang == "en" else True)
    return {"id": item.id, "category": item.category, "prompt": item.prompt, "response": response, "matched": matched,
            "forbidden_hit": forbidden, "length_ok": length_ok, "robotic": robotic, "toxic": toxic, "lang_ok": lang_ok,
            "has_lang_gate": gated, "discipline_ok": disciplined, "has_discipline": item.expect_lang == "en",
            "distinct1": distinct_n(response, 1), "distinct2": distinct_n(response, 2),
            "max_ngram_repeat": max_ngram_repeat(response, 3), "msa_ratio": style["msa_ratio"], "words": words,
            "seconds": seconds, "score": float(s), "tokens_per_sec": (words * 1.3 / seconds) if seconds > 0 else 0.0}


def run_benchmark(gen: Generator, items: List[EvalItem], sampling: Optional[SamplingParams] = None, max_new_tokens: int = 128,
                  categories: str = "", max_prompts: int = 0, system: str = "") -> dict:
    want = {c.strip() for c in categories.split(",") if c.strip()}
    results = []
    for it in items:
        if want and it.category not in want:
            continue
        if max_prompts and len(results) >= max_prompts:
            break
        msgs = ([T.Message("system", system)] if system else []) + list(it.context) + [T.Message("user", it.prompt)]
        ids, _ = T.encode_chat(gen.tok, msgs, add_generation_prompt=True)
        t0 = time.perf_counter()
        out = gen.generate([ids], max_new_tokens=max_new_tokens, sampling=sampling or SamplingParams(greedy=True, repetition_penalty=1.1))
        results.append(score_response(it, out.text[0] if out.text else "", time.perf_counter() - t0))
    return summarize(results)


def summarize(results: List[dict]) -> dict:
    by_cat: Dict[str, dict] = {}
    for r in results:
        c = by_cat.setdefault(r["category"], {"items": 0, "score_sum": 0.0, "matched": 0, "robotic": 0, "toxic": 0, "lang_fail": 0,
                                              "length_fail": 0, "discipline_fail": 0})
        c["items"] += 1
        c["score_sum"] += r["score"]
        c["matched"] += r["matched"]
        c["robotic"] += r["robotic"]
        c["toxic"] += r["toxic"]
        c["lang_fail"] += not r["lang_ok"]
        c["length_fail"] += not r["length_ok"]
        c["discipline_fail"] += not r["discipline_ok"]
    n = max(1, len(results))
    gated = [r for r in results if r["has_lang_gate"]]
    disc = [r for r in results if r["has_discipline"]]
    return {"total": len(results), "overall": sum(r["score"] for r in results) / n,
            "robotic_rate": sum(r["robotic"] for r in results) / n, "toxicity_rate": sum(r["toxic"] for r in results) / n,
            "repetition_rate": sum(r["max_ngram_repeat"] > 5 for r in results) / n,
            "lang_ok_rate": (sum(r["lang_ok"] for r in gated) / len(gated)) if gated else 0.0,
            "discipline_rate": (sum(r["discipline_ok"] for r in disc) / len(disc)) if disc else 0.0,
            "avg_distinct1": sum(r["distinct1"] for r in results) / n, "avg_distinct2": sum(r["distinct2"] for r in results) / n,
            "avg_words": sum(r["words"] for r in results) / n, "by_category": {k: dict(v, avg=v["score_sum"] / v["items"]) for k, v in by_cat.items()},
            "results": results}


def report_text(rep: dict) -> str:
    lines = ["items %d | overall %.3f | robotic %.1f%% | toxic %.1f%% | repetition %.1f%% | language ok %.1f%%" % (
        rep["total"], rep["overall"], 100 * rep["robotic_rate"], 100 * rep["toxicity_rate"], 100 * rep["repetition_rate"],
        100 * rep["lang_ok_rate"])]
    for k, v in sorted(rep["by_category"].items()):
        lines.append("  %-24s n=%3d  avg %.3f  matched %d" % (k, v["items"], v["avg"], v["matched"]))
    return "\n".join(lines)
