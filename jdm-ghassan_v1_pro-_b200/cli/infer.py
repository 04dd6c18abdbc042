"""Inference entry point (the reference's ``ghassan-ai``, tools/inference_cli.cpp:36-860).

    python -m ghassan_b200.cli.infer chat      --model model.gguf
    python -m ghassan_b200.cli.infer generate  --model model.gguf --prompt "شنو هو C++؟"
    python -m ghassan_b200.cli.infer info      --model model.gguf
    python -m ghassan_b200.cli.infer quantize  --model in.gguf --out out.gguf --profile q4_0
    python -m ghassan_b200.cli.infer bench     --model model.gguf [--tokens 128] [--prompt-tokens 32] [--batch 1]
    python -m ghassan_b200.cli.infer tokenize  --model model.gguf --text "شنو خبارك"
    python -m ghassan_b200.cli.infer export    --checkpoint last.ckpt --tokenizer tok.gtok --out model.gguf [--profile fp16|q8_k|q4_0] [--compat native|llama|llama_moe]
    python -m ghassan_b200.cli.infer eval      --model model.gguf [--suite dir] [--persona en]
    python -m ghassan_b200.cli.infer perplexity --model model.gguf (--text "held out" | --shards dir --prefix val)
                                                [--seq-len 512 --batches 20] [--rope-scale s] [--yarn-mscale m]
    python -m ghassan_b200.cli.infer devices
    python -m ghassan_b200.cli.infer logits    --model model.gguf --prompt "salam" [--out logits.f32]

GGUF is the deploy format (weights + tokenizer + configuration in one file); legacy .gai files and training
checkpoints load too.  Generation options: --temp --top-k --top-p --min-p --repeat --no-repeat-ngram --max-tokens
--seed --greedy --system --persona darija|en --no-adaptive --no-stream --retrieve-index <path> --retrieve-direct.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

import numpy as np

from .common import add_common_flags, apply_common_flags


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="ghassan-ai")
    ap.add_argument("command", choices=["chat", "generate", "info", "quantize", "bench", "tokenize", "export", "eval",
                                        "perplexity", "devices", "logits"])
    for name in ("model", "prompt", "out", "profile", "tokenizer", "text", "checkpoint", "suite", "shards", "prefix", "system",
                 "persona", "retrieve-index", "categories", "format", "compat"):
        ap.add_argument("--" + name)
    for name, typ in (("temp", float), ("top-k", int), ("top-p", float), ("min-p", float), ("repeat", float),
                      ("no-repeat-ngram", int), ("max-tokens", int), ("seed", int), ("tokens", int), ("prompt-tokens", int),
                      ("ctx", int), ("batch", int), ("max-prompts", int), ("seq-len", int), ("batches", int),
                      ("batch-size", int), ("rope-scale", float), ("yarn-mscale", float)):
        ap.add_argument("--" + name, type=typ)
    for name in ("greedy", "no-adaptive", "no-stream", "retrieve-direct", "stats", "verbose", "measure", "pack", "raw"):
        ap.add_argument("--" + name, action="store_true")
    add_common_flags(ap)
    return ap


def worst_q4_probe(named, profile: str):
    """``quantize --measure``: how much a 4-bit block format would cost each matrix.  Every non-norm tensor is
    quantised to Q4_0 and expanded again (embeddings and the output head only to fp16, unless the profile's default
    type is 8-bit, when they are probed in 4 bits too: tools/inference_cli.cpp:531-549 in the reference); returns
    (name, relative RMS error) of the worst one."""
    from .. import _gb200_host as H
    worst, worst_name = 0.0, ""
    all_q4 = profile in ("q8_k", "q8_0", "int8")
    for name, w in named.items():
        if "norm" in name:
            continue
        x = np.ascontiguousarray(np.asarray(w, dtype=np.float32)).reshape(-1)
        if x.size == 0:
            continue
        if name in ("tok_embeddings", "lm_head") and not all_q4:
            y = x.astype(np.float16).astype(np.float32)
        elif x.size % 32 == 0:
            y = np.asarray(H.ggml_dequantize(np.asarray(H.ggml_quantize(x, 2)), 2, x.size), dtype=np.float32)
        else:
            continue
        ok = np.isfinite(x) & np.isfinite(y)
        n = max(1, int(ok.sum()))
        rms = float(np.sqrt(np.sum((x[ok].astype(np.float64)) ** 2) / n))
        rel = float(np.sqrt(np.sum((x[ok].astype(np.float64) - y[ok]) ** 2) / n)) / rms if rms > 0 else 0.0
        if rel > worst:
            worst, worst_name = rel, name
    return worst_name, worst


def _sampling(a):
    from ..inference.engine import SamplingParams
    sp = SamplingParams()
    if a.temp is not None:
        sp.temperature = a.temp
    if a.top_k is not None:
        sp.top_k = a.top_k
    if a.top_p is not None:
        sp.top_p = a.top_p
    if a.min_p is not None:
        sp.min_p = a.min_p
    if a.repeat is not None:
        sp.repetition_penalty = a.repeat
    if a.no_repeat_ngram is not None:
        sp.no_repeat_ngram = a.no_repeat_ngram
    if a.seed is not None:
        sp.seed = a.seed
    sp.greedy = bool(a.greedy)
    return sp


def _load(a, batch=1, ctx=0):
    from ..inference import model_io as IO
    from ..inference.generator import Generator
    if not a.model:
        raise SystemExit("--model is required")
    m = IO.load_model(a.model, a.tokenizer or "")
    if a.rope_scale is not None or a.yarn_mscale is not None:      # run-time context extension (perplexity sweeps)
        if a.rope_scale is not None:
            m.cfg.rope_scale = float(a.rope_scale)
        if a.yarn_mscale is not None:
            m.cfg.rope_yarn_mscale = float(a.yarn_mscale)
        m.cfg.validate()
    eng = IO.build_engine(m, batch=batch, max_len=ctx or min(2048, m.cfg.max_seq_len), fmt=a.format or "auto")
    return m, Generator(eng, m.tokenizer)


def main(argv: Optional[List[str]] = None) -> int:
    a = _parser().parse_args(argv)
    apply_common_flags(a)
    cmd = a.command
    if cmd == "devices":
        import torch
        if not torch.cuda.is_available():
            print("  no CUDA device visible")
            return 0
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            print("  cuda:%d  %s  %.1f GiB  sm_%d%d  %d SMs" % (i, p.name, p.total_memory / 2 ** 30, p.major, p.minor, p.multi_processor_count))
        return 0
    if cmd == "info":
        from ..inference import model_io as IO
        kind = IO.sniff(a.model)
        if kind == "gguf":
            from ..formats.gguf import describe
            print(describe(a.model))
        else:
            m = IO.load_model(a.model)
            print("file: %s\nformat: %s\nquant: %s\nconfig: %s\nparameters: %d" % (a.model, kind, IO.quant_name(m), m.cfg.summary(), m.cfg.count_parameters()))
            for k, v in sorted(m.metadata.items()):
                print("  %-20s %s" % (k, v if not isinstance(v, bytes) else v.decode("utf-8", "replace")))
        return 0
    if cmd == "tokenize":
        from ..data.tokenizer import Tokenizer
        from ..inference import model_io as IO
        tok = Tokenizer.load(a.tokenizer) if a.tokenizer else IO.load_model(a.model).tokenizer
        if tok is None:
            raise SystemExit("model has no embedded tokenizer; pass --tokenizer")
        ids = tok.encode(a.text or "")
        print("  input   : %s\n  tokens  : %d\n  pieces  : %s" % (a.text, len(ids), " | ".join(tok.token_bytes(i).decode("utf-8", "replace") for i in ids)))
        print("  ids     : %s" % " ".join(map(str, ids.tolist())))
        words = max(1, len((a.text or "").split()))
        print("  decoded : %s" % tok.decode(ids))
        print("  fertility: %.3f tokens/word, %.2f bytes/token" % (len(ids) / words, len((a.text or "").encode("utf-8")) / max(1, len(ids))))
        return 0
    if cmd == "export":
        from ..formats.gguf import export_gguf
        from ..training import checkpoint as C
        if not (a.checkpoint and a.tokenizer and a.out):
            raise SystemExit("export needs --checkpoint, --tokenizer and --out")
        d = C.read(a.checkpoint, with_optimizer=False)
        cfg = C.config_from_dict(d["config"])
        st = d["state"]
        try:
            info = export_gguf(a.out, cfg, dict(d["params"]), a.tokenizer, a.profile or "fp16", moe_bias=d["moe_bias"],
                               extra_meta={"steps": str(st["step"]), "val_loss": "%.6f" % st["best_val"]},
                               compat=a.compat or "native")
        except ValueError as e:
            raise SystemExit("export: %s" % e)
        print("[gguf] exported %s  profile=%s compat=%s tensors=%d metadata=%d weights=%d bytes" % (
            info["path"], info["profile"], a.compat or "native", info["tensors"], info["metadata"], info["weight_bytes"]))
        return 0
    if cmd == "quantize":
        from ..formats.gguf import export_gguf
        from ..inference import model_io as IO
        import tempfile
        if not (a.model and a.out):
            raise SystemExit("quantize needs --model and --out")
        m = IO.load_model(a.model, a.tokenizer or "")
        if m.tokenizer is None:
            raise SystemExit("the input has no embedded tokenizer; pass --tokenizer")
        with tempfile.NamedTemporaryFile(suffix=".gtok", delete=False) as tf:
            tf.write(m.tokenizer.to_bytes())
            tok_path = tf.name
        if a.measure:
            name, rel = worst_q4_probe(m.named, a.profile or "q8_k")
            print("[quant] worst rel RMSE (Q4 probe): %.4f%% on %s" % (rel * 100.0, name))
        try:
            keep = {k: (v.decode() if isinstance(v, bytes) else str(v)) for k, v in m.metadata.items() if k in ("steps", "val_loss")}
            info = export_gguf(a.out, m.cfg, m.named, tok_path, a.profile or "q8_k", moe_bias=m.moe_bias or None, extra_meta=keep,
                               compat=a.compat or "native")
        except ValueError as e:
            raise SystemExit("quantize: %s" % e)
        finally:
            os.unlink(tok_path)
        print("[quant] %s -> %s   profile=%s compat=%s (%d bytes of weights)" % (
            a.model, a.out, info["profile"], a.compat or "native", info["weight_bytes"]))
        return 0

    # ---- commands that run the model
    if cmd == "bench":
        from ..inference.engine import SamplingParams
        m, gen = _load(a, batch=a.batch or 1, ctx=(a.ctx or ((a.prompt_tokens or 32) + (a.tokens or 64) + 16)))
        r = gen.benchmark(a.prompt_tokens or 32, a.tokens or 64, SamplingParams(greedy=True, repetition_penalty=1.0) if a.greedy else None,
                          seed=a.seed or 1234)
        print(json.dumps(r))
        return 0
    m, gen = _load(a, ctx=a.ctx or 0)
    sp = _sampling(a)
    if cmd == "generate":
        if gen.tok is None:
            raise SystemExit("model has no tokenizer; pass --tokenizer")
        if not a.prompt:
            raise SystemExit("--prompt is required")
        cb = None if a.no_stream else (lambda b, s: print(s, end="", flush=True))
        max_new = a.max_tokens or 256
        prompt = a.prompt
        if not a.raw:
            # one chat turn, as the reference's `generate` does unless --raw (tools/inference_cli.cpp:cmd_generate,
            # inference/generator.cpp:495-512 there): system prompt of the persona (default "en") or the given one plus
            # the script directive, the prompt as the user message, the assistant header; when that does not fit the
            # context next to the new tokens, tokens after the first are dropped from the front
            from ..data import tokenizer as TK
            from ..utils.log import log_warn
            persona = a.persona or "en"
            system = a.system or ""
            if not system:
                system = TK.system_for_persona(persona, TK.detect_script(prompt))
            elif persona not in ("en", "english"):
                system += "\n" + TK.script_directive(TK.detect_script(prompt))
            ids, _ = TK.encode_chat(gen.tok, [TK.Message("system", system), TK.Message("user", prompt)], add_generation_prompt=True)
            ids = [int(i) for i in ids]
            budget = gen.engine.cap - max_new - 4
            if budget > 0 and len(ids) > budget:
                drop = len(ids) - budget
                ids = ids[:1] + ids[1 + drop:]
                log_warn("chat: history truncated by %d tokens" % drop)
            prompt = ids
        res = gen.generate([prompt] if not isinstance(prompt, str) else prompt, max_new_tokens=max_new, sampling=sp, on_text=cb)
        print("" if cb else res.text[0])
        if a.stats:
            print("  [prefill %.0f ms | decode %.1f tok/s | %s]" % (res.prefill_seconds * 1e3, res.decode_tokens_per_second, res.stopped[0]))
        return 0
    if cmd == "chat":
        from ..inference.chat import ChatOptions, ChatSession
        o = ChatOptions(system=a.system or "", persona=a.persona or "darija", max_new_tokens=a.max_tokens or 256, sampling=sp,
                        stream=not a.no_stream, show_stats=a.stats, adaptive_dialog=not a.no_adaptive,
                        retrieve_index=a.retrieve_index or "", retrieve_direct=a.retrieve_direct)
        ChatSession(gen, o).run_repl()
        return 0
    if cmd == "logits":
        ids = gen.encode_prompt(a.prompt or "", add_bos=True)
        import torch
        if hasattr(gen.engine, "all_logits"):
            # the reference's report (tools/inference_cli.cpp:748-812 there): every position's logits to --out as
            # [tokens, vocab] fp32, and per position the arg-max with the five largest
            if len(ids) > 512:
                raise SystemExit("logits prompt too long (more than 512 tokens)")
            print("  tokens: %d  ids: %s" % (len(ids), " ".join(str(int(i)) for i in ids)))
            lg = gen.engine.all_logits(ids)
            if a.out:
                lg.astype(np.float32).tofile(a.out)
            for t in range(lg.shape[0]):
                row = lg[t]
                top = np.argsort(-row, kind="stable")[:5]
                print("  pos %3d argmax=%6d (%.4f) top5:%s" % (t, top[0], row[top[0]], "".join(" %d:%.3f" % (i, row[i]) for i in top)))
            return 0
        gen.engine.reset(1)
        gen.engine.prefill(torch.from_numpy(np.asarray(ids, dtype=np.int32)[None, :]).repeat(gen.engine.B, 1))
        lg = gen.engine.logits[0].float().cpu().numpy()
        if a.out:
            lg.astype(np.float32).tofile(a.out)
        top = np.argsort(-lg)[:10]
        for i in top:
            piece = gen.tok.token_bytes(int(i)).decode("utf-8", "replace") if gen.tok else ""
            print("  %6d  %10.4f  %s" % (i, lg[i], piece))
        return 0
    if cmd == "perplexity":
        from ..inference import evaluate as E
        seq_len, batches, bs = a.seq_len or 512, a.batches or 20, a.batch_size or 1
        if seq_len <= 0 or batches <= 0 or bs <= 0:
            raise SystemExit("perplexity options must be positive")
        if a.text:
            r = E.perplexity_text(gen, a.text)
        elif a.shards and hasattr(gen.engine, "score_batch"):
            # the reference's rule: batches of its data loader, supervised positions, segment masks, z-loss included
            r = E.perplexity_batches(gen, a.shards, a.prefix or "val", bs, seq_len, batches, bool(a.pack), a.seed if a.seed is not None else 42)
        elif a.shards:
            r = E.perplexity_shards(gen, a.shards, a.prefix or "val", max_tokens=batches * bs * seq_len, window=seq_len)
        else:
            raise SystemExit("perplexity requires --text or --shards")
        print("  rope_scale  : %.3f" % m.cfg.rope_scale)
        print("  yarn_mscale : %.3f" % m.cfg.rope_mscale())
        print("  mean_nll    : %.8f" % r["nll"])
        print("  perplexity  : %.6f" % r["perplexity"])
        print("  tokens      : %d" % r["tokens"])
        if "batches" in r:
            print("  batches     : %d" % r["batches"])
        return 0
    if cmd == "eval":
        from ..data.tokenizer import SYSTEM_ENGLISH
        from ..inference import evaluate as E
        english = (a.persona or "") in ("en", "english")
        items = E.load_suite(a.suite) if (a.suite and os.path.isdir(a.suite)) else []
        if not items:
            items = E.builtin_suite_en() if english else E.builtin_suite()
        # the command line's sampling settings as they stand (with --greedy: arg-max under the default repetition penalty),
        # as the reference's eval does
        rep = E.run_benchmark(gen, items, sp, a.max_tokens or 128, a.categories or "", a.max_prompts or 0,
                              SYSTEM_ENGLISH if english else "")
        print(E.report_text(rep))
        if a.out:
            with open(a.out, "w", encoding="utf-8") as f:
                for r in rep["results"]:
                    f.write(json.dumps(r, ensure_ascii=False) + "\n")
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
