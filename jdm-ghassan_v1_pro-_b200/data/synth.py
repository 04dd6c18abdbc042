"""Synthetic conversations for bootstrapping and for tests: Moroccan Darija exchanges (Arabic script, an Arabizi
transliteration with typing noise, some Modern Standard Arabic, French code-switching) and English dialogues of
several dialog acts.  The generators themselves are native (``csrc/host/synth.cpp``: transliteration rules, template
tables, template-use caps, duplicate / style / entropy rejection), as the reference's are
(dataset/darija_synthesis_engine.cpp, dataset/english_synthesis_engine.cpp); this module adapts them to the recipe
files and to JSONL rows.  Output is deterministic for a seed."""
from __future__ import annotations

import json
from dataclasses import dataclass, fields
from typing import Dict, Iterator, List

from .. import _gb200_host as H

_LANG = {"arab": "ar-MA-arab", "latn": "ar-MA-latn", "msa": "ar-MSA", "en": "en"}


def to_arabizi(text: str, seed: int = 1, heavy_digits: bool = True) -> str:
    """Arabic-script Darija in Latin chat spelling (7 = ح, 3 = ع, 9 = ق ... when ``heavy_digits``)."""
    return H.arabic_to_arabizi(text, seed, heavy_digits)


def _rows(convs, start=0, with_act=False) -> List[dict]:
    out = []
    for i, c in enumerate(convs):
        row = {"id": start + i, "lang": _LANG[c["script"]], "category": c["domain"], "messages": c["messages"]}
        if with_act:
            row["act"] = c["domain"]
        out.append(row)
    return out


def darija_conversations(n: int, seed: int = 1, arabizi_ratio: float = 0.4, noise: float = 0.03) -> Iterator[dict]:
    """``n`` short Darija conversations without system prompt: Arabic script, or Arabizi with probability ``arabizi_ratio``."""
    c = H.SynthConfig()
    c.seed, c.min_turns, c.max_turns = seed, 2, 4
    c.p_arabic_script, c.p_latin_script, c.p_msa = 1.0 - arabizi_ratio, arabizi_ratio, 0.0
    c.p_french_switch, c.include_system, c.noise_rate = 0.0, False, noise
    yield from _rows(H.DarijaSynth(c).generate_many(n))


def english_conversations(n: int, seed: int = 1) -> Iterator[dict]:
    c = H.EnglishSynthConfig()
    c.seed, c.p_system = seed, 0.0
    yield from _rows(H.EnglishSynth(c).generate_many(n), with_act=True)


# ---------------------------------------------------------------------------------------------- configured generator


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


class SynthStats:
    """Counters of one generator run (the native generator's, under the names the log line uses)."""

    def __init__(self, d: dict):
        self.attempts, self.generated = d["attempts"], d["accepted"]
        self.rejected_duplicate, self.rejected_template_cap = d["rejected_duplicate"], d["rejected_template_cap"]
        self.rejected_style, self.rejected_entropy = d["rejected_style"], d["rejected_entropy"]
        self.by_category: Dict[str, int] = dict(d["by_domain"])
        self.by_script: Dict[str, int] = {_LANG[k]: v for k, v in d["by_script"].items()}
        self._summary = d["summary"]

    def summary(self) -> str:
        return self._summary


class DarijaSynthGenerator:
    """Multi-turn conversations under the probabilities of a :class:`SynthConfig`: script mix (Arabic / Arabizi / MSA),
    French code-switching, follow-ups, corrections, clarification requests, boundary-setting and worked-arithmetic
    turns, optional system prompt, a cap on how often one template may open a conversation, and rejection of
    duplicates, boilerplate style and low-information text."""

    def __init__(self, cfg: SynthConfig):
        self.cfg = cfg
        n = H.SynthConfig()
        for f in fields(SynthConfig):
            if hasattr(n, f.name):
                setattr(n, f.name, getattr(cfg, f.name))
        self._g = H.DarijaSynth(n)
        self._made = 0

    @property
    def stats(self) -> SynthStats:
        return SynthStats(self._g.stats())

    def generate_many(self, n: int) -> List[dict]:
        rows = _rows(self._g.generate_many(n), self._made)
        self._made += len(rows)
        return rows

    @staticmethod
    def domains() -> List[str]:
        return list(H.DarijaSynth.domains())


def write_jsonl(path: str, rows) -> int:
    n = 0
    with open(path, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
            n += 1
    return n
