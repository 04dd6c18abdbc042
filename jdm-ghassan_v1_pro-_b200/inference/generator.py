"""Text generation on top of :class:`InferenceEngine`: prompt handling, stop tokens and stop strings, streaming
detokenisation, sequence scoring, throughput measurement (inference/generator.cpp:60-420 in the reference).

Two sampling routes.  Settings the device sampler takes run entirely on the GPU: the engine replays one captured
decode step per token and the host looks at the transcript every ``poll`` tokens (for streaming and stop strings).
Other settings (n-gram bans, unbounded top-k) read the logits back each token and use the native host sampler.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from .. import _gb200_host as H
from ..data import tokenizer as T
from .engine import InferenceEngine, SamplingParams


@dataclass
class GenerationResult:
    tokens: List[List[int]]                   # new tokens per sequence (stop token excluded)
    text: List[str] = field(default_factory=list)
    prompt_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    stopped: List[str] = field(default_factory=list)   # "eos" | "stop_string" | "length" per sequence

    @property
    def decode_tokens_per_second(self) -> float:
        n = sum(len(t) for t in self.tokens)
        return n / self.decode_seconds if self.decode_seconds > 0 else 0.0


class Generator:
    def __init__(self, engine: InferenceEngine, tokenizer: Optional[T.Tokenizer] = None):
        self.engine, self.tok = engine, tokenizer
        self.default_stop = [T.EOS, T.END]

    # ------------------------------------------------------------------ helpers
    def encode_prompt(self, prompt, add_bos=True) -> np.ndarray:
        if isinstance(prompt, str):
            if self.tok is None:
                raise ValueError("a text prompt needs a tokenizer")
            return self.tok.encode(prompt, add_bos=add_bos)
        return np.asarray(prompt, dtype=np.int32)

    def _cut_at_stop(self, toks: Sequence[int], stop_ids) -> "tuple[List[int], bool]":
        out = []
        for t in toks:
            if int(t) in stop_ids:
                return out, True
            out.append(int(t))
        return out, False

    # ------------------------------------------------------------------ generation
    def generate(self, prompts, max_new_tokens: int = 256, sampling: Optional[SamplingParams] = None,
                 stop_tokens: Optional[Sequence[int]] = None, stop_strings: Sequence[str] = (),
                 on_text: Optional[Callable[[int, str], None]] = None, poll: int = 16,
                 use_graph: bool = True) -> GenerationResult:
        """``prompts``: one prompt (text or ids) or a list of ``engine.B`` prompts of equal token length."""
        eng = self.engine
        sp = sampling or SamplingParams()
        plist = prompts if (isinstance(prompts, (list, tuple)) and len(prompts) and
                            isinstance(prompts[0], (str, list, tuple, np.ndarray))) else [prompts]
        ids = [self.encode_prompt(p) for p in plist]
        if len(ids) != eng.B:
            raise ValueError(f"engine was built for batch {eng.B}, got {len(ids)} prompts")
        n = len(ids[0])
        if any(len(x) != n for x in ids):
            raise ValueError("prompts of one batch must have the same token length (pad or group them)")
        if n + max_new_tokens > eng.cap and not stop_strings:
            pass        # the ring cache keeps the first 8 and the most recent tokens; generation may run past it
        stop_ids = set(self.default_stop if stop_tokens is None else stop_tokens)
        eng.reset(sp.seed)
        eng.set_stop_tokens(sorted(stop_ids))
        max_new = min(max_new_tokens, eng.tok_log.shape[1])
        t0 = time.perf_counter()
        host_only = getattr(eng, "host_only", False)          # the CPU engine: host sampler, no device to wait for
        eng.prefill(torch.from_numpy(np.stack(ids)).to(torch.int32))
        if not host_only:
            torch.cuda.synchronize()
        t1 = time.perf_counter()
        if sp.device_ok() and not host_only:
            toks, reasons = self._run_device(sp, max_new, stop_ids, stop_strings, on_text, poll, use_graph)
        else:
            toks, reasons = self._run_host(sp, ids, max_new, stop_ids, stop_strings, on_text)
        if not host_only:
            torch.cuda.synchronize()
        t2 = time.perf_counter()
        res = GenerationResult(tokens=toks, prompt_tokens=n, prefill_seconds=t1 - t0, decode_seconds=t2 - t1,
                               stopped=reasons)
        if self.tok is not None:
            res.text = [self.tok.decode(t, skip_special=True) for t in toks]
        return res

    def _run_device(self, sp, max_new, stop_ids, stop_strings, on_text, poll, use_graph):
        eng = self.engine
        B = eng.B
        eng.sample_first(sp)
        produced = 1
        streams = [self.tok.stream() if self.tok is not None else None for _ in range(B)]
        emitted = [0] * B
        text_so_far = [""] * B
        done = [False] * B
        reasons = ["length"] * B
        need_poll = on_text is not None or stop_strings or stop_ids
        while produced < max_new and not all(done):
            n = min(poll if need_poll else max_new, max_new - produced)
            eng.decode_steps(n, sp, use_graph)
            produced += n
            if not need_poll:
                continue
            log = eng.transcript(produced).numpy()
            for b in range(B):
                if done[b]:
                    continue
                row, hit = self._cut_at_stop(log[b], stop_ids)
                if streams[b] is not None and (on_text is not None or stop_strings):
                    for t in row[emitted[b]:]:
                        piece = streams[b].push(int(t)).decode("utf-8", errors="replace")
                        text_so_far[b] += piece
                        if piece and on_text is not None:
                            on_text(b, piece)
                    emitted[b] = len(row)
                if hit:
                    done[b], reasons[b] = True, "eos"
                elif any(s and s in text_so_far[b] for s in stop_strings):
                    done[b], reasons[b] = True, "stop_string"
        log = eng.transcript(produced).numpy()
        out = []
        for b in range(B):
            row, hit = self._cut_at_stop(log[b], stop_ids)
            if hit and reasons[b] == "length":
                reasons[b] = "eos"
            out.append(row)
        return out, reasons

    def _run_host(self, sp, prompt_ids, max_new, stop_ids, stop_strings, on_text):
        eng = self.engine
        B = eng.B
        samplers = []
        for b in range(B):
            c = sp.to_native()
            c.seed = (sp.seed or 1) + b
            samplers.append(H.Sampler(c))
        hist = [list(map(int, p)) for p in prompt_ids]
        out = [[] for _ in range(B)]
        done = [False] * B
        reasons = ["length"] * B
        streams = [self.tok.stream() if self.tok is not None else None for _ in range(B)]
        text_so_far = [""] * B
        for _ in range(max_new):
            logits = eng.logits.cpu().numpy()
            nxt = []
            for b in range(B):
                t = samplers[b].sample(logits[b], hist[b])
                nxt.append(t)
                if done[b]:
                    continue
                if t in stop_ids:
                    done[b], reasons[b] = True, "eos"
                    continue
                out[b].append(t)
                hist[b].append(t)
                if streams[b] is not None:
                    piece = streams[b].push(t).decode("utf-8", errors="replace")
                    text_so_far[b] += piece
                    if piece and on_text is not None:
                        on_text(b, piece)
                    if any(s and s in text_so_far[b] for s in stop_strings):
                        done[b], reasons[b] = True, "stop_string"
            if all(done):
                break
            eng.cur_tok.copy_(torch.tensor(nxt, dtype=torch.int32))
            eng._forward_token()
        return out, reasons

    # ------------------------------------------------------------------ scoring
    def score_tokens(self, ids: Sequence[int]) -> "tuple[float, int]":
        """Sum of negative log-likelihoods of ``ids[1:]`` given their prefixes, and the number of scored tokens.
        Uses the decode path token by token on sequence 0 (exactly what generation would compute)."""
        eng = self.engine
        ids = [int(i) for i in ids]
        if len(ids) < 2:
            return 0.0, 0
        if hasattr(eng, "score_window"):                      # the CPU engine scores a window in one teacher-forced pass
            return eng.score_window(ids)
        eng.reset(1)
        total, count = 0.0, 0
        row = torch.zeros(eng.B, dtype=torch.int32)
        for j in range(len(ids) - 1):
            row.fill_(ids[j])
            eng.cur_tok.copy_(row)
            eng._forward_token()
            lp = torch.log_softmax(eng.logits[0].double(), dim=-1)[ids[j + 1]]
            total -= float(lp)
            count += 1
        return total, count

    def perplexity(self, ids: Sequence[int]) -> float:
        nll, n = self.score_tokens(ids)
        return float(np.exp(nll / max(1, n)))

    # ------------------------------------------------------------------ throughput
    def benchmark(self, prompt_len: int = 1024, new_tokens: int = 512, sampling: Optional[SamplingParams] = None,
                  seed: int = 1234) -> dict:
        """Device-timed decode throughput after a synthetic uniform-random prompt (no host reads while decoding)."""
        eng = self.engine
        if getattr(eng, "host_only", False):
            return self._benchmark_host(prompt_len, new_tokens, sampling, seed)
        if new_tokens < 10:
            raise ValueError("benchmark needs at least 10 new tokens (the first 9 warm the graph up and are not timed)")
        sp = sampling or SamplingParams(temperature=0.8, top_k=40, top_p=0.9, min_p=0.0, seed=seed)
        rng = H.Rng(seed)
        V = eng.cfg.vocab_size
        prompt = np.empty((eng.B, prompt_len), dtype=np.int32)
        for b in range(eng.B):
            rng.fill_uniform_ids(prompt[b], V - 16)
        prompt += 16
        eng.reset(seed)
        eng.set_stop_tokens([])
        e0, e1_pre, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        torch.cuda.synchronize()
        e0.record()
        eng.prefill(torch.from_numpy(prompt))
        e1_pre.record()
        eng.sample_first(sp)
        eng.decode_steps(8, sp)            # capture + warm replays (counted as output, timed separately below)
        torch.cuda.synchronize()
        e1.record()
        eng.decode_steps(new_tokens - 9, sp)
        e2.record()
        torch.cuda.synchronize()
        dec_ms = e1.elapsed_time(e2)
        n_timed = (new_tokens - 9) * eng.B
        toks = eng.transcript(new_tokens)
        return {"batch": eng.B, "prompt_len": prompt_len, "new_tokens": new_tokens, "decode_ms_per_token": dec_ms / (new_tokens - 9),
                "decode_tokens_per_s": n_timed / (dec_ms / 1e3), "stored_weight_bytes": eng.weight_bytes,
                "prefill_ms": e0.elapsed_time(e1_pre), "distinct_tokens": int(len(set(toks.reshape(-1).tolist())))}

    def _benchmark_host(self, prompt_len, new_tokens, sampling, seed) -> dict:
        """The same report for an engine without a device (the CPU engine): wall clock around the host-sampled loop."""
        eng = self.engine
        sp = sampling or SamplingParams(temperature=0.8, top_k=40, top_p=0.9, min_p=0.0, seed=seed)
        rng = H.Rng(seed)
        V = eng.cfg.vocab_size
        prompt = np.empty((eng.B, prompt_len), dtype=np.int32)
        for b in range(eng.B):
            rng.fill_uniform_ids(prompt[b], V - 16)
        prompt += 16
        eng.reset(seed)
        eng.set_stop_tokens([])
        t0 = time.perf_counter()
        eng.prefill(torch.from_numpy(prompt))
        t1 = time.perf_counter()
        toks, _ = self._run_host(sp, [list(map(int, p)) for p in prompt], new_tokens, set(), (), None)
        t2 = time.perf_counter()
        n = sum(len(t) for t in toks)
        return {"batch": eng.B, "prompt_len": prompt_len, "new_tokens": new_tokens,
                "decode_ms_per_token": (t2 - t1) * 1e3 / max(1, new_tokens), "decode_tokens_per_s": n / max(1e-9, t2 - t1),
                "stored_weight_bytes": eng.weight_bytes, "prefill_ms": (t1 - t0) * 1e3,
                "distinct_tokens": int(len({t for row in toks for t in row})), "device": "cpu"}
