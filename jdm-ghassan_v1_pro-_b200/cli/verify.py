"""Acceptance suites run through the package's own command lines, on data the suite generates itself.

    python -m ghassan_b200.cli.verify engine [--device auto|cpu|cuda] [--workdir DIR] [--configs DIR]
    python -m ghassan_b200.cli.verify app    [--device auto|cpu|cuda] [--workdir DIR]

``engine``  the gates of the reference's engine suite (configs/kaggle/verify_engine_suite.sh:118-226): a segmented
            backward pass agrees with the full one (loss after one update, relative 1e-5 in fp32, 5e-3 with 16-bit GEMMs);
            quantised exports stay within the perplexity budget (8-bit at most +15 %, 4-bit at most +60 % and not
            better than fp16); every shipped training recipe passes a strict dry run; a run that is stopped resumes
            from its last checkpoint; and the warnings of all those runs are listed.
``app``     the application chain (configs/kaggle/verify_application_pipeline.sh:27-92): synthesise conversations,
            train a tokenizer, build shards, train a few steps, export fp16 and 4-bit files, describe them, round-trip
            the tokenizer, then generate, chat, measure decode speed and perplexity, re-quantise, dump logits and
            list devices.  The steps that run the model need a CUDA device and are reported as skipped without one.

Each gate prints ``[ok]``, ``[FAIL]`` or ``[skip]``; the exit code is the number of failed gates (0 = pass).
"""
from __future__ import annotations

import argparse
import contextlib
import glob
import io
import json
import os
import re
import sys
import tempfile
from typing import Callable, List, Optional, Tuple

from .common import add_common_flags, apply_common_flags

TINY = ["--vocab", "0", "--layers", "2", "--hidden", "128", "--heads", "4", "--kv-heads", "2"]

RECIPE = """
model:
  vocab_size: {vocab}
  hidden_size: 128
  num_layers: 2
  num_heads: 2
  num_kv_heads: 1
  intermediate_size: 256
  max_seq_len: 128
  use_moe: true
  num_experts: 4
  moe_top_k: 2
  moe_expert_dim: 256
  moe_shared: true
  use_qk_norm: true
  moe_aux_free: true
  moe_aux_scale: 0.0
training:
  optimizer: adamw
  learning_rate: 0.003
  batch_size: 2
  seq_len: 64
  grad_accum: 1
  warmup_steps: 0
  max_steps: 4
  eval_every: 0
  save_every: 0
  log_every: 1
  seed: 21
"""


class Suite:
    def __init__(self, out=None):
        self.failures = 0
        self.lines: List[str] = []
        self.logs: List[str] = []
        self.out = out or sys.stdout

    def say(self, s):
        self.lines.append(s)
        print(s, file=self.out, flush=True)

    def step(self, title):
        self.say("")
        self.say("##### %s #####" % title)

    def ok(self, msg):
        self.say("  [ok] " + msg)

    def bad(self, msg):
        self.failures += 1
        self.say("  [FAIL] " + msg)

    def skip(self, msg):
        self.say("  [skip] " + msg)

    def call(self, fn: Callable[[List[str]], int], argv: List[str]) -> Tuple[int, str]:
        """Run a command-line entry point in-process; returns (exit code, everything it printed)."""
        from ..utils import log as LOG
        buf = io.StringIO()
        rc = 0
        level = LOG.log_level()
        LOG.set_log_level(LOG.INFO)                     # the gates read step lines and resume messages
        with contextlib.redirect_stdout(buf), contextlib.redirect_stderr(buf):
            try:
                rc = fn(argv)
            except SystemExit as e:
                rc = e.code if isinstance(e.code, int) else 1
                if not isinstance(e.code, int) and e.code is not None:
                    print(str(e.code))
            except Exception as e:                                   # a crash is a failed gate, not a crashed suite
                rc = 99
                print("%s: %s" % (type(e).__name__, e))
            finally:
                LOG.set_log_level(level)
        text = buf.getvalue()
        self.logs.append(text)
        return int(rc or 0), text

    def warnings(self):
        self.step("warnings and errors of every run above")
        seen = {}
        for log in self.logs:
            for line in log.splitlines():
                if line.startswith(("[warn", "[error", "[fatal")):
                    seen[line] = seen.get(line, 0) + 1
        if not seen:
            self.say("  (none)")
        for line, n in sorted(seen.items(), key=lambda kv: -kv[1])[:30]:
            self.say("  %4d  %s" % (n, line[:200]))


def _device(name: str) -> str:
    import torch
    if name == "auto":
        return "cuda" if torch.cuda.is_available() else "cpu"
    return name


def make_data(work: str, suite: Suite, n_conv: int = 600, vocab: int = 512) -> Tuple[str, str, str]:
    """Synthetic conversations -> tokenizer -> shards.  Returns (tokenizer, shard directory, recipe file)."""
    from . import data_pipeline as DP
    from . import train_tokenizer as TT
    conv = os.path.join(work, "synth.jsonl")
    rc, out = suite.call(DP.main, ["synth", "--out", conv, "--n", str(n_conv), "--seed", "11"])
    if rc or not os.path.exists(conv):
        suite.bad("synthesis failed: " + out[-300:])
        raise RuntimeError("no data")
    tok = os.path.join(work, "tok.gtok")
    rc, out = suite.call(TT.main, ["--input", conv, "--output", tok, "--vocab", str(vocab)])
    if rc or not os.path.exists(tok):
        suite.bad("tokenizer training failed: " + out[-300:])
        raise RuntimeError("no tokenizer")
    shards = os.path.join(work, "shards")
    rc, out = suite.call(DP.main, ["build", "--tokenizer", tok, "--out", shards, "--chat", conv, "--val-ratio", "0.1",
                                   "--seq-len", "128", "--style-mode", "off", "--no-dedup"])
    if rc or not glob.glob(os.path.join(shards, "train*.gbin")):
        suite.bad("shard build failed: " + out[-300:])
        raise RuntimeError("no shards")
    from ..data.tokenizer import Tokenizer
    recipe = os.path.join(work, "tiny.yaml")
    with open(recipe, "w") as f:
        f.write(RECIPE.format(vocab=Tokenizer.load(tok).vocab_size))
    return tok, shards, recipe


def _step_loss(log: str, step: int) -> Optional[float]:
    m = re.search(r"step +%d \| loss +([0-9.]+)" % step, log)
    return float(m.group(1)) if m else None


def _jsonl_loss(path: str, step: int) -> Optional[float]:
    """Loss of ``step`` at full precision from the per-step JSON log (the step line prints four decimals)."""
    try:
        with open(path) as f:
            for line in f:
                r = json.loads(line)
                if r.get("step") == step:
                    return float(r["loss"])
    except (OSError, ValueError):
        pass
    return None


def _train(suite, recipe, shards, ckpt, dev, extra) -> Tuple[int, str]:
    from . import train as TR
    return suite.call(TR.main, ["--config", recipe, "--data", shards, "--checkpoint-dir", ckpt, "--device", dev,
                                "--resume", "none"] + extra)


def engine_suite(dev: str, work: str, configs_dir: str, suite: Optional[Suite] = None) -> Suite:
    from . import infer as INF
    from . import train as TR
    s = suite or Suite()
    s.step("[1/5] data for the gates (synthetic conversations, tokenizer, shards)")
    try:
        tok, shards, recipe = make_data(work, s)
        s.ok("tokenizer and shards written under " + work)
    except RuntimeError:
        return s

    s.step("[2/5] segmented backward == full backward (same data; the loss after one update)")
    for label, fp16, tol in (("fp32 GEMMs (CPU engine)", "0", 1e-5), ("16-bit GEMMs", "1", 5e-3)):
        if fp16 == "1" and dev != "cuda":
            s.skip(label + ": needs a CUDA device")
            continue
        losses = []
        engaged = False
        for seg in ("2", "1"):
            # one micro-batch per pass, so that segmenting applies; the loss of step 2 depends on step 1's gradients
            jl = os.path.join(work, "seg%s_%s.jsonl" % (seg, fp16))
            old = os.environ.get("GB200_JSONL")
            os.environ["GB200_JSONL"] = jl
            try:
                # fp32 arithmetic is the CPU engine's; the CUDA engine always multiplies 16-bit operands
                rc, log = _train(s, recipe, shards, os.path.join(work, "seg%s_%s" % (seg, fp16)), dev if fp16 == "1" else "cpu",
                                 ["--ckpt-segments", seg, "--gemm-fp16", fp16, "--max-steps", "2", "--set", "b200.fuse_micro_batches", "1"])
            finally:
                if old is None:
                    os.environ.pop("GB200_JSONL", None)
                else:
                    os.environ["GB200_JSONL"] = old
            losses.append(None if rc else _jsonl_loss(jl, 2))
            engaged = engaged or (seg == "2" and "runs as 2 slices" in log)
        a, b = losses
        if a is None or b is None:
            s.bad(label + ": could not read the step-2 loss of both runs")
            continue
        if not engaged:
            s.bad(label + ": segmenting did not engage (batch 2, segments 2 must run as 2 slices)")
            continue
        rel = abs(a - b) / abs(b)
        (s.ok if rel <= tol else s.bad)("%s: step-2 loss with segments=2 -> %.7f, segments=1 -> %.7f (rel %.2e, limit %.0e)" % (label, a, b, rel, tol))

    s.step("[3/5] quantisation accuracy on held-out shards")
    ck = os.path.join(work, "ckpt_q")
    rc, log = _train(s, recipe, shards, ck, dev, ["--max-steps", "30", "--save-every", "30", "--seed", "33"])
    last = os.path.join(ck, "last.ckpt")
    if rc or not os.path.exists(last):
        s.bad("training for the quantisation gate failed: " + log[-300:])
    else:
        files = {}
        for prof in ("fp16", "q8_k", "q4_0"):
            files[prof] = os.path.join(work, "q_%s.gguf" % prof)
            if prof == "q8_k":
                rc, out = s.call(INF.main, ["quantize", "--model", files["fp16"], "--out", files[prof], "--profile", prof])
            else:
                rc, out = s.call(INF.main, ["export", "--checkpoint", last, "--tokenizer", tok, "--out", files[prof], "--profile", prof])
            if rc:
                s.bad("writing the %s file failed: %s" % (prof, out[-200:]))
        if dev != "cuda":
            s.skip("perplexity of the exported files: the inference engine needs a CUDA device")
        elif all(os.path.exists(p) for p in files.values()):
            ppl = {}
            for prof, path in files.items():
                rc, out = s.call(INF.main, ["perplexity", "--model", path, "--shards", shards, "--prefix", "val", "--seq-len", "64",
                                            "--batches", "40"])
                m = re.search(r"perplexity\s*:\s*([0-9.eE+-]+)", out)
                ppl[prof] = float(m.group(1)) if (m and not rc) else 0.0
                s.say("  %s: perplexity = %s" % (prof, ppl[prof] or "?"))
            gate = quant_gate(ppl["fp16"], ppl["q8_k"], ppl["q4_0"])
            (s.ok if gate[0] else s.bad)(gate[1])

    s.step("[4/5] every shipped training recipe under a strict dry run")
    n = 0
    for path in sorted(glob.glob(os.path.join(configs_dir, "*.yaml"))):
        with open(path) as f:
            if not re.search(r"^training:", f.read(), re.M):
                continue                                              # data-pipeline recipes are not training recipes
        rc, out = s.call(TR.main, ["--config", path, "--dry-run", "--strict-config", "--device", "cuda"])
        n += 1
        total = next((ln.strip() for ln in out.splitlines() if "total" in ln and "per GPU" in ln), "")
        (s.ok if rc == 0 else s.bad)("%-36s %s" % (os.path.basename(path), total if rc == 0 else out.strip().splitlines()[-1][:160] if out.strip() else "no output"))
    if n == 0:
        s.bad("no training recipes found under " + configs_dir)

    s.step("[5/5] stop and resume (train 2 steps, then continue to 4 from last.ckpt)")
    ck = os.path.join(work, "ckpt_r")
    rc1, _ = _train(s, recipe, shards, ck, dev, ["--max-steps", "2", "--save-every", "1", "--seed", "77"])
    rc2, log = s.call(TR.main, ["--config", recipe, "--data", shards, "--checkpoint-dir", ck, "--device", dev, "--resume", "auto",
                                "--max-steps", "4", "--save-every", "2", "--seed", "77", "--allow-recipe-drift"])
    if rc1 or rc2:
        s.bad("resume run failed: " + log[-300:])
    elif re.search(r"resumed from .*last\.ckpt", log) and re.search(r"done: 4 steps", log):
        s.ok("resumed from last.ckpt and finished at step 4")
    else:
        s.bad("the second run did not resume from last.ckpt")
    s.warnings()
    return s


def quant_gate(fp16: float, q8: float, q4: float) -> Tuple[bool, str]:
    """The perplexity budget of the quantised exports (configs/kaggle/verify_engine_suite.sh:184-194)."""
    if fp16 <= 0 or q8 <= 0 or q4 <= 0:
        return False, "missing perplexity"
    r8, r4 = (q8 - fp16) / fp16, (q4 - fp16) / fp16
    head = "q8_k drift %+.2f%% | q4_0 drift %+.2f%%: " % (r8 * 100, r4 * 100)
    if -0.5 < r4 < -0.02:
        return False, head + "q4_0 is better than fp16: the perplexity is not measuring anything"
    if r4 > 0.60:
        return False, head + "q4_0 destroys the model (more than +60 %)"
    if r8 > 0.15:
        return False, head + "q8_k drifts more than +15 %"
    return True, head + "within budget"


def app_suite(dev: str, work: str, suite: Optional[Suite] = None) -> Suite:
    from . import infer as INF
    s = suite or Suite()
    s.step("[1/10] synthesise conversations, train a tokenizer, build shards")
    try:
        tok, shards, recipe = make_data(work, s)
        s.ok("data ready")
    except RuntimeError:
        return s

    s.step("[2/10] train 6 steps")
    ck = os.path.join(work, "ckpt")
    rc, log = _train(s, recipe, shards, ck, dev, ["--max-steps", "6", "--save-every", "6"])
    first, last_loss = _step_loss(log, 1), _step_loss(log, 6)
    last = os.path.join(ck, "last.ckpt")
    if rc or first is None or last_loss is None or not os.path.exists(last):
        s.bad("training failed or wrote no last.ckpt: " + log[-300:])
        return s
    s.ok("first loss %.4f, last loss %.4f, last.ckpt written" % (first, last_loss))

    s.step("[3/10] export fp16 and q4_0, describe both")
    f16, q4 = os.path.join(work, "m_fp16.gguf"), os.path.join(work, "m_q4.gguf")
    for path, prof in ((f16, "fp16"), (q4, "q4_0")):
        rc, out = s.call(INF.main, ["export", "--checkpoint", last, "--tokenizer", tok, "--out", path, "--profile", prof])
        rc2, info = s.call(INF.main, ["info", "--model", path])
        (s.ok if (rc == 0 and rc2 == 0 and "ghassan" in info.lower()) else s.bad)("%s: %d bytes" % (prof, os.path.getsize(path) if os.path.exists(path) else 0))
    if os.path.exists(f16) and os.path.exists(q4) and not os.path.getsize(q4) < os.path.getsize(f16):
        s.bad("the 4-bit file is not smaller than the fp16 file")

    s.step("[4/10] tokenizer round trip")
    from ..data.tokenizer import Tokenizer
    t = Tokenizer.load(tok)
    text = "salam, labas 3lik? kifach ndir had l-khedma"
    back = t.decode(t.encode(text), skip_special=True)
    (s.ok if back.replace(" ", "") == text.replace(" ", "").lower() or back.replace(" ", "") == text.replace(" ", "") else s.bad)(
        "'%s' -> %d tokens -> '%s'" % (text, len(t.encode(text)), back))

    runs_model = dev == "cuda"
    s.step("[5/10] generate, [6/10] chat, [7/10] decode speed, [8/10] perplexity")
    if not runs_model:
        s.skip("the inference engine needs a CUDA device")
    else:
        rc, out = s.call(INF.main, ["generate", "--model", f16, "--prompt", "salam", "--max-tokens", "16", "--greedy", "--no-stream"])
        (s.ok if rc == 0 else s.bad)("generate: %s" % out.strip().splitlines()[-1][:80] if out.strip() else "generate: no output")
        old = sys.stdin
        sys.stdin = io.StringIO("salam\n/quit\n")
        try:
            rc, out = s.call(INF.main, ["chat", "--model", f16, "--max-tokens", "12", "--no-stream"])
        finally:
            sys.stdin = old
        (s.ok if rc == 0 else s.bad)("chat session ended cleanly" + ("" if rc == 0 else ": " + out.strip()[-300:]))
        rc, out = s.call(INF.main, ["bench", "--model", f16, "--prompt-tokens", "16", "--tokens", "24", "--greedy"])
        try:
            r = json.loads(out.strip().splitlines()[-1])
            s.ok("bench: %s" % json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in r.items()})[:160])
        except Exception:
            s.bad("bench printed no result: " + out[-200:])
        rc, out = s.call(INF.main, ["perplexity", "--model", f16, "--shards", shards, "--prefix", "val", "--seq-len", "64", "--batches", "10"])
        m = re.search(r"perplexity\s*:\s*([0-9.eE+-]+)", out)
        (s.ok if (rc == 0 and m and float(m.group(1)) > 1.0) else s.bad)("perplexity on held-out shards: %s" % (m.group(1) if m else "?"))

    s.step("[9/10] re-quantise fp16 -> q8_k (with the 4-bit probe), describe")
    q8 = os.path.join(work, "m_q8.gguf")
    rc, out = s.call(INF.main, ["quantize", "--model", f16, "--out", q8, "--profile", "q8_k", "--measure"])
    (s.ok if (rc == 0 and "worst rel RMSE" in out and os.path.exists(q8)) else s.bad)(out.strip().splitlines()[0][:120] if out.strip() else "no output")

    s.step("[10/10] logits dump and device list")
    if runs_model:
        dump = os.path.join(work, "logits.bin")
        rc, out = s.call(INF.main, ["logits", "--model", f16, "--prompt", "salam", "--out", dump])
        want = 4 * t.vocab_size
        (s.ok if (rc == 0 and os.path.exists(dump) and os.path.getsize(dump) == want) else s.bad)("logits: %d bytes (vocabulary x 4 = %d)" % (
            os.path.getsize(dump) if os.path.exists(dump) else 0, want))
    else:
        s.skip("logits: needs a CUDA device")
    rc, out = s.call(INF.main, ["devices"])
    (s.ok if rc == 0 else s.bad)("devices: " + (out.strip().splitlines()[0].strip() if out.strip() else ""))
    s.warnings()
    return s


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="gai_verify")
    ap.add_argument("suite", choices=["engine", "app"])
    ap.add_argument("--device", default="auto")
    ap.add_argument("--workdir", default="")
    ap.add_argument("--configs", default=os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "configs"))
    add_common_flags(ap)
    a = ap.parse_args(argv)
    apply_common_flags(a)
    dev = _device(a.device)
    ctx = tempfile.TemporaryDirectory(prefix="gb200_verify_") if not a.workdir else contextlib.nullcontext(a.workdir)
    with ctx as work:
        os.makedirs(work, exist_ok=True)
        s = engine_suite(dev, work, a.configs) if a.suite == "engine" else app_suite(dev, work)
    print("")
    print("=" * 62)
    print("  %s suite on %s: %s" % (a.suite, dev, "PASS - no gate failed" if s.failures == 0 else "FAIL - %d gate(s) failed (listed above)" % s.failures))
    print("=" * 62)
    return s.failures


if __name__ == "__main__":
    sys.exit(main())
