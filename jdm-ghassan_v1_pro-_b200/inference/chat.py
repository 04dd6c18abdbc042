"""Chat session: history with trimming, script policy (Arabic letters vs Arabizi replies), English dialog-act
sampling presets, retrieval (answer directly or as added context), and the interactive loop
(inference/chat.cpp:11-275, dataset/english_style_policy.cpp:38-144 in the reference)."""
from __future__ import annotations

import copy
import math
import re
import sys
from dataclasses import dataclass, field
from typing import List, Optional

from ..data import tokenizer as T
from ..data.retrieval import RetrievalIndex, build_index
from .engine import SamplingParams
from .generator import Generator

_GREET = ("hi", "hello", "hey", "good morning", "good evening", "good afternoon", "how are you", "what's up", "whats up",
          "how is it going", "nice to meet")
_CODE_WORDS = ("python", "javascript", "java", "code", "function", "class", "def", "import", "script", "program", "debug",
               "compile", "algorithm", "plainformat")
_RETURN_CTX = ("value", "statement", "type", "keyword")
_VERBS = ("write", "implement", "create", "develop", "explain", "solve", "convert", "generate", "design", "debug",
          "describe", "summarize", "translate", "classify", "list")
_QWORDS = ("who", "whom", "whose", "what", "when", "where", "why", "how", "which", "whether", "is", "are", "was", "were",
           "do", "does", "did", "can", "could", "would", "should", "will", "have", "has", "had")


def _low(s: str) -> str:
    return "".join(c.lower() if "A" <= c <= "Z" else c for c in s.strip(" \t\n\r"))


def _starts_word(s: str, pre: str) -> bool:
    return s.startswith(pre) and (len(s) == len(pre) or not re.match(r"[A-Za-z0-9_]", s[len(pre)]))


def _has_word(s: str, w: str) -> bool:
    return re.search(r"(?<![A-Za-z0-9_])" + re.escape(w) + r"(?![A-Za-z0-9_])", s) is not None


def classify_dialog_act(text: str) -> str:
    """greeting | coding | instruction | question | reasoning | chitchat | unknown, tested in that order."""
    if not text:
        return "unknown"
    l = _low(text)
    if any(_starts_word(l, g) for g in _GREET):
        return "greeting"
    if "```" in l or "#include" in l or any(_has_word(l, w) for w in _CODE_WORDS) or \
            (_has_word(l, "return") and any(_has_word(l, w) for w in _RETURN_CTX)):
        return "coding"
    if any(_starts_word(l, v) for v in _VERBS):
        return "instruction"
    if text.rstrip(" \t\n\r\"'").endswith("?") or any(_starts_word(l, q) for q in _QWORDS):
        return "question"
    if any(k in l for k in ("how many", "calculate", "prove", "logic", "step")):
        return "reasoning"
    return "chitchat"


def adapt_english_sampling(sp: SamplingParams, max_new: int, user_message: str):
    """Per-turn sampling preset for the English persona; returns (sampling, max_new_tokens)."""
    s = copy.copy(sp)
    act = classify_dialog_act(user_message)
    if act == "greeting":
        max_new = min(max_new, 96)
        s.temperature, s.top_p, s.min_p, s.no_repeat_ngram = min(s.temperature, 0.8), 0.90, 0.02, 0
    elif act == "coding":
        s.temperature, s.top_k, s.top_p, s.min_p, s.no_repeat_ngram = min(s.temperature, 0.4), 40, 1.0, 0.0, 0
    elif act == "reasoning":
        s.temperature, s.top_k, s.top_p, s.min_p, s.no_repeat_ngram = min(s.temperature, 0.6), 40, 0.95, 0.02, 0
    elif act == "instruction":
        s.temperature, s.top_k, s.top_p, s.min_p, s.no_repeat_ngram = min(s.temperature, 0.6), 40, 0.90, 0.05, 0
    elif act == "question":
        s.temperature, s.top_p, s.min_p, s.no_repeat_ngram = min(s.temperature, 0.7), 0.92, 0.05, 0
    return s, max_new


@dataclass
class ChatOptions:
    system: str = ""
    persona: str = "darija"             # darija | en
    max_history_turns: int = 8
    max_new_tokens: int = 256
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stream: bool = True
    show_stats: bool = False
    adaptive_dialog: bool = True
    retrieve_index: str = ""
    retrieve_direct: bool = False
    retrieve_top_k: int = 1
    retrieve_threshold: float = 0.0


class ChatSession:
    def __init__(self, gen: Generator, opts: Optional[ChatOptions] = None, out=None):
        self.gen, self.o, self.out = gen, opts or ChatOptions(), (sys.stdout if out is None else out)
        if self.o.max_history_turns < 0 or self.o.retrieve_top_k < 0 or self.o.max_new_tokens < 0:
            raise ValueError("chat options must be non-negative")
        self.english = self.o.persona in ("en", "english")
        self.custom_system = bool(self.o.system)
        if not self.o.system:
            self.o.system = T.SYSTEM_ENGLISH if self.english else T.SYSTEM_DARIJA_ARABIC
        self.history: List[T.Message] = [T.Message("system", self.o.system)]
        self._index: Optional[RetrievalIndex] = None
        self._index_path = None
        self.last = None

    def clear(self):
        self.history = [T.Message("system", self.history[0].content if self.history else self.o.system)]

    def set_system(self, s: str):
        self.o.system, self.custom_system = s, True
        if self.history and self.history[0].role == "system":
            self.history[0].content = s
        else:
            self.history.insert(0, T.Message("system", s))

    def apply_script_policy(self, user_message: str):
        """Darija persona: answer in the script the user wrote in."""
        if not self.history or self.history[0].role != "system" or self.english:
            return
        script = T.detect_script(user_message)
        if not self.custom_system:
            self.history[0].content = self.o.system = T.system_for_script(script)
        else:
            d = T.script_directive(script)
            if d not in self.history[0].content:
                self.history[0].content += "\n" + d

    def trim_history(self):
        keep = 2 * self.o.max_history_turns
        if len(self.history) <= 1 + keep:
            return
        start = len(self.history) - keep
        while start > 1 and self.history[start].role == "assistant":
            start -= 1                       # never start the window on an answer without its question
        self.history = [self.history[0]] + self.history[start:]

    def _retrieve(self, user_message: str) -> Optional[str]:
        if not self.o.retrieve_index:
            return None
        if self._index_path != self.o.retrieve_index:
            self._index_path = self.o.retrieve_index
            idx = build_index(self.o.retrieve_index)
            self._index = idx if len(idx) else None
        if self._index is None:
            return None
        hits = self._index.query(user_message, self.o.retrieve_top_k or 1, self.o.retrieve_threshold)
        return self._index.doc(hits[0][0]).answer if hits else None

    def send(self, user_message: str) -> str:
        self.apply_script_policy(user_message)
        found = self._retrieve(user_message)
        if self.o.retrieve_direct and found is not None:
            self.history.append(T.Message("user", user_message))
            self.trim_history()
            if self.o.stream:
                print(found, file=self.out, flush=True)
            self.history.append(T.Message("assistant", found))
            return found
        self.history.append(T.Message("user", user_message))
        if found is not None:
            self.history.insert(len(self.history) - 1, T.Message("system", "Context (from dataset): " + found))
        self.trim_history()
        sp, max_new = self.o.sampling, self.o.max_new_tokens
        if self.o.adaptive_dialog and self.english:
            sp, max_new = adapt_english_sampling(sp, max_new, user_message)
        ids, _ = T.encode_chat(self.gen.tok, self.history, add_generation_prompt=True)
        cb = (lambda b, piece: print(piece, end="", file=self.out, flush=True)) if self.o.stream else None
        res = self.gen.generate([ids], max_new_tokens=max_new, sampling=sp, on_text=cb)
        self.last = res
        reply = res.text[0] if res.text else ""
        if self.o.stream:
            print(file=self.out, flush=True)
        self.history.append(T.Message("assistant", reply))
        return reply

    def run_repl(self, inp=None):
        inp = sys.stdin if inp is None else inp          # looked up at call time: callers may have replaced it
        w = lambda s="": print(s, file=self.out, flush=True)
        w("\n  Ghassan AI - chat" + (" (English)" if self.english else ""))
        w("  Type your message. Commands: /help /clear /system <text> /temp <f> /stats /quit" if self.english else
          "  اكتب رسالتك بالدارجة. الأوامر: /help /clear /system <text> /temp <f> /stats /quit")
        w("  ------------------------------------------------------------------\n")
        while True:
            print("\nuser > ", end="", file=self.out, flush=True)
            line = inp.readline()
            if not line:
                break
            line = line.rstrip("\n")
            if not line:
                continue
            if line.startswith("/"):
                cmd, _, arg = line[1:].partition(" ")
                if cmd in ("quit", "exit", "q"):
                    break
                if cmd == "clear":
                    self.clear()
                    w("  [history cleared]")
                elif cmd == "system":
                    if arg:
                        self.set_system(arg)
                        w("  [system prompt updated]")
                    else:
                        w("  system: " + self.o.system)
                elif cmd == "stats":
                    if self.last is not None:
                        w("  prefill %.0f ms, decode %.1f tok/s" % (self.last.prefill_seconds * 1e3,
                                                                    self.last.decode_tokens_per_second))
                    w("  history: %d messages" % len(self.history))
                elif cmd == "temp":
                    try:
                        t = float(arg)
                        t = 0.0 if not math.isfinite(t) else min(5.0, max(0.0, t))
                        self.o.sampling.temperature = t
                        w("  [temperature = %g]" % t)
                    except ValueError:
                        w("  invalid temperature (want 0..5)")
                elif cmd == "help":
                    w("  /clear          reset the conversation\n  /system <text>  set the system prompt\n"
                      "  /temp <f>       set the sampling temperature\n  /stats          show timing and context usage\n"
                      "  /quit           exit")
                else:
                    w("  unknown command: %s (try /help)" % cmd)
                continue
            print("\nghassan > ", end="", file=self.out, flush=True)
            self.send(line)
        w("\n  Goodbye!" if self.english else "\n  بسلامة!")
