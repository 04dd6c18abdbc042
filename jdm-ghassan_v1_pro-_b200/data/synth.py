"""Synthetic conversations for bootstrapping and for tests: short Moroccan Darija exchanges (Arabic script and an
Arabizi transliteration with light typing noise) and short English dialogues of several dialog acts.  The role of
the reference's synthesis engines (dataset/darija_synthesis_engine.cpp, english_synthesis_engine.cpp); the templates
and vocabulary here are this project's own and deliberately small.  Output is deterministic for a seed."""
from __future__ import annotations

import json
from typing import Dict, Iterator, List

from .. import _gb200_host as H

# Arabic letter -> Arabizi spelling (digits stand for letters Latin script lacks)
_ARABIZI = {"ا": "a", "أ": "a", "إ": "i", "آ": "a", "ب": "b", "ت": "t", "ث": "t", "ج": "j", "ح": "7", "خ": "kh", "د": "d",
            "ذ": "d", "ر": "r", "ز": "z", "س": "s", "ش": "ch", "ص": "s", "ض": "d", "ط": "t", "ظ": "d", "ع": "3", "غ": "gh",
            "ف": "f", "ق": "9", "ك": "k", "ل": "l", "م": "m", "ن": "n", "ه": "h", "ة": "a", "و": "o", "ي": "i", "ى": "a",
            "ء": "2", "ئ": "2", "ؤ": "2", "گ": "g", "ڤ": "v", "پ": "p", "؟": "?", "،": ","}

_DARIJA = {
    "greeting": [("السلام عليكم، كيداير؟", "وعليكم السلام، لاباس الحمد لله. ونتا كيداير؟"),
                 ("صباح الخير", "صباح النور، كيف صبحتي؟"), ("لاباس عليك؟", "لاباس، كلشي بخير. شنو خبارك نتا؟")],
    "help": [("بغيت نتعلم {topic}، منين نبدا؟", "بدا بالأساسيات ديال {topic} شوية بشوية، وكل نهار دير تمرين صغير."),
             ("واش تقدر تعاوني ف {topic}؟", "واخا، قول ليا شنو بالضبط اللي صعيب عليك ف {topic}.")],
    "daily": [("شنو ندير اليوم؟", "إلا كان الجو مزيان خرج تمشى شوية، وإلا بقى فالدار وقرا شي كتاب."),
              ("فين نمشي نهار الأحد؟", "تقدر تمشي ل{place}، الجو تما زوين وماشي بعيد.")],
    "food": [("شنو نطيب للعشا؟", "دير {dish}، ساهل وكيعجب كلشي."), ("كيفاش كنديرو {dish}؟", "خاصك المقادير ديال {dish} وشوية ديال الصبر، نشرح ليك بالتفصيل إلا بغيتي.")],
}
_FILL = {"topic": ["البرمجة", "الطبخ", "الإنجليزية", "الرياضيات"], "place": ["البحر", "الجبل", "المدينة القديمة"],
         "dish": ["الطاجين", "الكسكس", "الحريرة"]}

_ENGLISH = {
    "greeting": [("Hi there!", "Hello! How can I help you today?"), ("Good morning", "Good morning! What would you like to work on?")],
    "question": [("What is the capital of {country}?", "The capital of {country} is {capital}."),
                 ("How many days are in a leap year?", "A leap year has 366 days; the extra day is February 29.")],
    "instruction": [("Explain what {concept} means in one sentence.", "{concept} is {definition}."),
                    ("List three tips for learning {skill}.", "1. Practise a little every day. 2. Review your mistakes. 3. Teach someone else what you learned about {skill}.")],
    "coding": [("Write a Python function that returns the square of a number.", "```python\ndef square(x):\n    return x * x\n```"),
               ("How do I reverse a list in Python?", "Use slicing: `items[::-1]` returns a reversed copy, and `items.reverse()` reverses in place.")],
    "reasoning": [("If a train travels 60 km in 45 minutes, what is its speed in km/h?", "45 minutes is 0.75 hours, so the speed is 60 / 0.75 = 80 km/h."),
                  ("I have 3 boxes with 4 apples each and eat 2. How many are left?", "3 boxes of 4 apples make 12; after eating 2 there are 10 left.")],
}
_EN_FILL = {"country": ["Morocco", "France", "Japan"], "capital": ["Rabat", "Paris", "Tokyo"],
            "concept": ["Recursion", "Inflation", "Photosynthesis"],
            "definition": ["a function solving a problem by calling itself on smaller inputs", "a general rise in prices over time",
                           "the process plants use to turn light into chemical energy"], "skill": ["a language", "chess", "programming"]}


def to_arabizi(text: str) -> str:
    out = []
    for ch in text:
        out.append(_ARABIZI.get(ch, ch if not ("؀" <= ch <= "ۿ") else ""))
    return "".join(out)


def _noise(rng: "H.Rng", s: str, rate: float) -> str:
    """Typing noise: an occasional doubled letter or a dropped vowel."""
    out = []
    for ch in s:
        r = rng.uniform()
        if ch.isalpha() and r < rate * 0.5:
            out.append(ch + ch)
        elif ch in "aeio" and r < rate:
            continue
        else:
            out.append(ch)
    return "".join(out)


def _fill(rng, template_pair, table) -> List[str]:
    picks: Dict[str, int] = {}
    out = []
    for t in template_pair:
        for key, values in table.items():
            if "{" + key + "}" in t:
                if key in ("capital", "definition"):          # tied to the previous pick
                    idx = picks.get("country" if key == "capital" else "concept", 0)
                else:
                    idx = picks.setdefault(key, int(rng.below(len(values))))
                t = t.replace("{" + key + "}", values[idx])
        out.append(t)
    return out


def darija_conversations(n: int, seed: int = 1, arabizi_ratio: float = 0.4, noise: float = 0.03) -> Iterator[dict]:
    rng = H.Rng(seed)
    cats = sorted(_DARIJA)
    for i in range(n):
        cat = cats[int(rng.below(len(cats)))]
        turns = 1 + int(rng.below(2))
        msgs = []
        latin = rng.uniform() < arabizi_ratio
        for _ in range(turns):
            pair = _DARIJA[cat][int(rng.below(len(_DARIJA[cat])))]
            u, a = _fill(rng, pair, _FILL)
            if latin:
                u, a = _noise(rng, to_arabizi(u), noise), _noise(rng, to_arabizi(a), noise)
            msgs += [{"role": "user", "content": u}, {"role": "assistant", "content": a}]
            cat = cats[int(rng.below(len(cats)))]
        yield {"id": i, "lang": "ar-MA-latn" if latin else "ar-MA-arab", "messages": msgs}


def english_conversations(n: int, seed: int = 1) -> Iterator[dict]:
    rng = H.Rng(seed)
    acts = sorted(_ENGLISH)
    for i in range(n):
        act = acts[int(rng.below(len(acts)))]
        pair = _ENGLISH[act][int(rng.below(len(_ENGLISH[act])))]
        u, a = _fill(rng, pair, _EN_FILL)
        yield {"id": i, "lang": "en", "act": act, "messages": [{"role": "user", "content": u}, {"role": "assistant", "content": a}]}


def write_jsonl(path: str, rows) -> int:
    n = 0
    with open(path, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
            n += 1
    return n
