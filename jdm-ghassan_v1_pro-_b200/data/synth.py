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


# ---------------------------------------------------------------------------------------------- configured generator
from dataclasses import dataclass, fields  # noqa: E402


@dataclass
class SynthConfig:
    """Knobs of the Darija generator; the same keys as the ``synth:`` / ``sft_synth:`` sections of the shipped
    synthesis recipes (tools/data_pipeline_cli.cpp:139-196 in the reference)."""
    seed: int = 1234
    num_conversations: int = 20000
    min_turns: int = 2
    max_turns: int = 10
    p_arabic_script: float = 0.60
    p_latin_script: float = 0.30
    p_msa: float = 0.10
    p_french_switch: float = 0.10
    p_followup: float = 0.40
    p_correction: float = 0.08
    p_misunderstand: float = 0.06
    p_governor: float = 0.0
    p_reasoning: float = 0.0
    include_system: bool = True
    p_system: float = 0.30
    max_template_uses: int = 400
    max_attempts_multiplier: int = 60
    output_path: str = ""
    shards_output: str = ""
    tokenizer_path: str = ""


def load_synth_config(path: str, section: str = "synth") -> SynthConfig:
    """Read one section of a synthesis recipe.  Unknown keys anywhere in the file are an error, not ignored."""
    from ..utils.config import Config, ConfigError
    if section not in ("synth", "sft_synth"):
        raise ConfigError("%s: --section must be 'synth' or 'sft_synth' (got '%s')" % (path, section))
    c = Config.from_file(path)
    names = [f.name for f in fields(SynthConfig)]
    c.check_known([s + "." + n for s in ("synth", "sft_synth") for n in names], [], True)
    out = SynthConfig()
    p = section + "."
    for f in fields(SynthConfig):
        if not c.has(p + f.name):
            continue
        if f.type in ("int", int):
            setattr(out, f.name, c.get_int(p + f.name, getattr(out, f.name)))
        elif f.type in ("float", float):
            setattr(out, f.name, c.get_float(p + f.name, getattr(out, f.name)))
        elif f.type in ("bool", bool):
            setattr(out, f.name, c.get_bool(p + f.name, getattr(out, f.name)))
        else:
            setattr(out, f.name, c.get_str(p + f.name, getattr(out, f.name)))
    if out.min_turns <= 0 or out.max_turns < out.min_turns:
        raise ConfigError("%s: %smin_turns/max_turns invalid (%d/%d)" % (path, p, out.min_turns, out.max_turns))
    if out.num_conversations < 0:
        raise ConfigError("%s: %snum_conversations must be >= 0" % (path, p))
    if out.max_template_uses <= 0:
        raise ConfigError("%s: %smax_template_uses must be > 0" % (path, p))
    return out


_MSA = [("كيف حالك اليوم؟", "أنا بخير، شكراً لك. كيف يمكنني مساعدتك؟"),
        ("ما هي عاصمة المغرب؟", "عاصمة المغرب هي مدينة الرباط."),
        ("هل يمكنك أن تشرح لي هذا الموضوع؟", "بكل سرور، سأشرح لك الموضوع خطوة بخطوة.")]
_FOLLOWUP = [("وشنو آخر؟", "كاين حتى هادي: خود وقتك وما تزربش، وكل مرة زيد شوية."),
             ("عطيني مثال", "مثلا: بدا بحاجة صغيرة اليوم، وغدا زيد عليها شوية.")]
_CORRECTION = [("لا، ماشي هادشي اللي قصدت", "سمح ليا، فهمتك غلط. عاود ليا شنو بغيتي بالضبط ونجاوبك.")]
_CLARIFY = [("هاداك", "ما فهمتش مزيان، واش تقدر توضح ليا شنو كتقصد؟")]
_FRENCH = ["s'il te plaît", "merci", "d'accord", "normalement", "en fait"]
_SYSTEMS = ["نتا مساعد مغربي كتهضر بالدارجة بطريقة طبيعية ومختصرة.", "nta mosa3id maghribi, jaweb b darija b tariqa 9sira."]


class SynthStats:
    def __init__(self):
        self.generated = self.attempts = self.rejected_duplicate = self.rejected_template_cap = 0
        self.by_category: Dict[str, int] = {}
        self.by_script: Dict[str, int] = {}

    def summary(self) -> str:
        return "generated %d in %d attempts (duplicates %d, template cap %d); scripts %s" % (
            self.generated, self.attempts, self.rejected_duplicate, self.rejected_template_cap,
            " ".join("%s=%d" % kv for kv in sorted(self.by_script.items())))


class DarijaSynthGenerator:
    """Multi-turn conversations from the template tables above under the probabilities of a :class:`SynthConfig`:
    script mix (Arabic / Arabizi / MSA), French code-switching, follow-ups, corrections, clarification requests,
    optional system prompt, a cap on how often one template may be used, and exact-duplicate rejection."""

    def __init__(self, cfg: SynthConfig):
        self.cfg, self.rng, self.stats = cfg, H.Rng(cfg.seed), SynthStats()
        self.uses: Dict[tuple, int] = {}
        self.seen = set()

    def _pick(self, table, key):
        i = int(self.rng.below(len(table)))
        k = (key, i)
        if self.uses.get(k, 0) >= self.cfg.max_template_uses:
            return None
        self.uses[k] = self.uses.get(k, 0) + 1
        return table[i]

    def _one(self):
        c, r = self.cfg, self.rng
        u = r.uniform() * max(1e-9, c.p_arabic_script + c.p_latin_script + c.p_msa)
        script = "arab" if u < c.p_arabic_script else ("latn" if u < c.p_arabic_script + c.p_latin_script else "msa")
        n_msgs = c.min_turns + int(r.below(c.max_turns - c.min_turns + 1))
        exchanges = max(1, (n_msgs + 1) // 2)
        cats = sorted(_DARIJA)
        msgs, first_cat = [], None
        while len(msgs) < 2 * exchanges:
            x = r.uniform()
            if msgs and x < c.p_correction:
                pair = self._pick(_CORRECTION, "correction")
            elif msgs and x < c.p_correction + c.p_misunderstand:
                pair = self._pick(_CLARIFY, "clarify")
            elif msgs and x < c.p_correction + c.p_misunderstand + c.p_followup:
                pair = self._pick(_FOLLOWUP, "followup")
            elif script == "msa":
                pair = self._pick(_MSA, "msa")
            else:
                cat = cats[int(r.below(len(cats)))]
                first_cat = first_cat or cat
                pair = self._pick(_DARIJA[cat], cat)
                if pair is not None:
                    pair = tuple(_fill(r, pair, _FILL))
            if pair is None:
                self.stats.rejected_template_cap += 1
                return None
            q, a = pair
            if script != "msa" and r.uniform() < c.p_french_switch:
                q = q + " " + _FRENCH[int(r.below(len(_FRENCH)))]
            if script == "latn":
                q, a = to_arabizi(q), to_arabizi(a)
            msgs += [{"role": "user", "content": q}, {"role": "assistant", "content": a}]
        if c.include_system and r.uniform() < c.p_system:
            msgs.insert(0, {"role": "system", "content": _SYSTEMS[1 if script == "latn" else 0]})
        lang = {"arab": "ar-MA-arab", "latn": "ar-MA-latn", "msa": "ar-MSA"}[script]
        return {"lang": lang, "category": first_cat or script, "messages": msgs}

    def generate_many(self, n: int):
        out = []
        budget = max(1, n) * max(1, self.cfg.max_attempts_multiplier)
        while len(out) < n and self.stats.attempts < budget:
            self.stats.attempts += 1
            conv = self._one()
            if conv is None:
                continue
            key = "\n".join(m["content"] for m in conv["messages"])
            if key in self.seen:
                self.stats.rejected_duplicate += 1
                continue
            self.seen.add(key)
            conv["id"] = len(out)
            out.append(conv)
            self.stats.by_category[conv["category"]] = self.stats.by_category.get(conv["category"], 0) + 1
            self.stats.by_script[conv["lang"]] = self.stats.by_script.get(conv["lang"], 0) + 1
        self.stats.generated = len(out)
        return out


def write_jsonl(path: str, rows) -> int:
    n = 0
    with open(path, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
            n += 1
    return n
