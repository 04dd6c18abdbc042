"""The inference command line on a host without a GPU (`inference/cpu_engine.py`), and, where a CPU build of the
reference sits under baseline/_ref/bin, the same commands of both on the same GGUF file: held-out perplexity
(evaluation/perplexity.cpp there), the per-position logits dump, and generation (one chat turn by default, --raw,
greedy and seeded sampling) must agree."""
import io
import os
import re
import subprocess
from contextlib import redirect_stdout

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref", "bin", "ghassan-ai")
needs_ref = pytest.mark.skipif(not os.path.exists(REF), reason="no build of the reference command line here")
pytestmark = pytest.mark.skipif(torch.cuda.is_available(), reason="with a GPU the command line uses the CUDA engine")


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    """A tiny trained model (context 1024) as GGUF, its tokenizer and its shards."""
    from ghassan_b200.cli import data_pipeline as DP, infer as I, train as T, train_tokenizer as TT
    w = str(tmp_path_factory.mktemp("cpuinf"))
    sink = io.StringIO()
    with redirect_stdout(sink):
        assert DP.main(["synth", "--out", w + "/synth.jsonl", "--n", "300", "--seed", "11", "--silent"]) == 0
        assert TT.main(["--input", w + "/synth.jsonl", "--output", w + "/tok.gtok", "--vocab", "600", "--silent"]) == 0
        assert DP.main(["build", "--tokenizer", w + "/tok.gtok", "--out", w + "/shards", "--chat", w + "/synth.jsonl", "--val-ratio",
                        "0.1", "--seq-len", "128", "--style-mode", "off", "--no-dedup", "--silent"]) == 0
        assert T.main(["--config", os.path.join(ROOT, "configs", "cpu_smoke_test.yaml"), "--device", "cpu", "--max-steps", "30",
                       "--data", w + "/shards", "--checkpoint-dir", w + "/ck", "--resume", "none", "--set", "model.max_seq_len",
                       "1024", "--silent"]) == 0
        assert I.main(["export", "--checkpoint", w + "/ck/last.ckpt", "--tokenizer", w + "/tok.gtok", "--out", w + "/m.gguf",
                       "--profile", "fp16"]) == 0
    from ghassan_b200.utils import log as LOG
    LOG.set_log_level(LOG.INFO)
    return w


def ours(args):
    from ghassan_b200.cli import infer as I
    buf = io.StringIO()
    with redirect_stdout(buf):
        assert I.main(args) == 0
    return buf.getvalue()


def theirs(args):
    p = subprocess.run([REF] + args, capture_output=True, cwd=ROOT, timeout=300)
    assert p.returncode == 0, (p.stdout + p.stderr).decode("utf-8", "replace")[-600:]
    return p.stdout.decode("utf-8", "replace")


def test_engine_equals_the_oracle_model(model):
    from ghassan_b200.inference import model_io as IO
    from ghassan_b200.inference.cpu_engine import CpuEngine
    m = IO.load_model(model + "/m.gguf")
    eng = IO.build_engine(m, batch=1, max_len=256)
    assert isinstance(eng, CpuEngine)
    ids = [1, 40, 77, 120, 300, 9]
    eng.reset(0)
    eng.prefill(torch.tensor([ids], dtype=torch.int32))
    want = eng.net.logits(torch.tensor(ids), 1, len(ids))[-1]
    assert torch.equal(eng.logits[0], want)
    eng.cur_tok[0] = 55
    eng._forward_token()
    want = eng.net.logits(torch.tensor(ids + [55]), 1, len(ids) + 1)[-1]
    assert torch.equal(eng.logits[0], want)
    # one teacher-forced pass scores what the token-by-token walk scores
    nll, n = eng.score_window(ids)
    lg = eng.net.logits(torch.tensor(ids), 1, len(ids)).double()
    ref = -sum(float(torch.log_softmax(lg[j], -1)[ids[j + 1]]) for j in range(len(ids) - 1))
    assert n == len(ids) - 1 and abs(nll - ref) < 1e-9


def test_commands_run_without_a_gpu(model):
    out = ours(["generate", "--model", model + "/m.gguf", "--prompt", "salam labas", "--max-tokens", "8", "--greedy", "--no-stream"])
    again = ours(["generate", "--model", model + "/m.gguf", "--prompt", "salam labas", "--max-tokens", "8", "--greedy", "--no-stream"])
    assert out == again                          # greedy decoding is repeatable (a model this small may well answer nothing)
    raw = ours(["generate", "--model", model + "/m.gguf", "--prompt", "salam labas", "--max-tokens", "8", "--greedy", "--no-stream",
                "--raw"])
    assert raw.endswith("\n")
    ppl = ours(["perplexity", "--model", model + "/m.gguf", "--shards", model + "/shards", "--prefix", "val_", "--batches", "5"])
    assert re.search(r"batches +: 5", ppl) and float(re.search(r"perplexity +: ([0-9.]+)", ppl).group(1)) > 1.0
    txt = ours(["perplexity", "--model", model + "/m.gguf", "--text", "salam labas 3lik, kif dayr"])
    assert float(re.search(r"perplexity +: ([0-9.]+)", txt).group(1)) > 1.0
    import json
    rep = json.loads(ours(["bench", "--model", model + "/m.gguf", "--tokens", "12", "--prompt-tokens", "16"]).strip().splitlines()[-1])
    assert rep["device"] == "cpu" and rep["new_tokens"] == 12 and rep["decode_tokens_per_s"] > 0
    ev = ours(["eval", "--model", model + "/m.gguf", "--max-prompts", "2", "--max-tokens", "6"])
    assert re.search(r"items 2 \| overall [0-9.]+", ev)


@needs_ref
def test_perplexity_equals_the_reference(model):
    args = ["perplexity", "--model", model + "/m.gguf", "--shards", model + "/shards", "--prefix", "val_"]
    a, b = theirs(args), ours(args)
    for key in ("tokens", "batches"):
        assert re.search(key + r" +: (\d+)", a).group(1) == re.search(key + r" +: (\d+)", b).group(1), key
    na, nb = (float(re.search(r"mean_nll +: ([0-9.]+)", t).group(1)) for t in (a, b))
    assert abs(na - nb) < 1e-4, (na, nb)


@needs_ref
def test_logits_dump_equals_the_reference(model, tmp_path):
    fa, fb = str(tmp_path / "a.f32"), str(tmp_path / "b.f32")
    a = theirs(["logits", "--model", model + "/m.gguf", "--prompt", "salam labas", "--out", fa])
    b = ours(["logits", "--model", model + "/m.gguf", "--prompt", "salam labas", "--out", fb])
    assert re.search(r"tokens: (\d+ +ids:.*)", a).group(1) == re.search(r"tokens: (\d+ +ids:.*)", b).group(1)
    la, lb = np.fromfile(fa, dtype=np.float32), np.fromfile(fb, dtype=np.float32)
    assert la.shape == lb.shape and la.size % 600 == 0
    assert float(np.abs(la - lb).max()) < 2e-3
    assert (la.reshape(-1, 600).argmax(1) == lb.reshape(-1, 600).argmax(1)).all()


@needs_ref
@pytest.mark.parametrize("extra", [["--greedy"], ["--seed", "7"], ["--greedy", "--raw"], ["--seed", "11", "--temp", "1.1", "--top-k", "20"]])
def test_generation_equals_the_reference(model, extra):
    args = ["generate", "--model", model + "/m.gguf", "--prompt", "salam labas", "--max-tokens", "16", "--no-stream"] + extra
    def answer(out):          # the text is the last line of stdout; the reference also logs "[info ] ..." lines there
        lines = [ln for ln in out.split("\n") if not ln.startswith("[")]
        while lines and lines[-1] == "":
            lines.pop()
        return lines[-1] if lines else ""
    a, b = answer(theirs(args)), answer(ours(args))
    if "--greedy" in extra:
        assert a == b, (a, b)
    else:
        # The two engines' logits differ in the fourth digit, so a draw that lands on the edge between two tokens can
        # fall either way late in the text; another generator or order of filters would part at the first token.
        same = next((i for i, (x, y) in enumerate(zip(a, b)) if x != y), min(len(a), len(b)))
        assert a and same >= (2 * len(a)) // 3, (a, b)


@needs_ref
def test_quality_benchmark_equals_the_reference(model, tmp_path):
    """`eval` over one suite file: the same greedy answers and, item by item, the same score with the same reasons
    (evaluation/benchmark.cpp:590-680 there).  Every item names something to expect and something to forbid: the
    reference's scanner misreads an empty array in a suite file."""
    import json
    from ghassan_b200.inference import evaluate as E
    suite = tmp_path / "suite"
    suite.mkdir()
    items = [
        E.EvalItem("basic_conversation", "a1", [], "salam, labas 3lik?", ["labas", "bikhir"], ["robot"], "ar-MA-latn", 30, ""),
        E.EvalItem("basic_conversation", "a2", [], "السلام عليكم", ["سلام"], ["باريس"], "ar-MA-arab", 30, ""),
        E.EvalItem("instruction_following", "a3", [], "Answer in one word: what colour is the sky?", ["blue"], ["green"], "en", 5, ""),
        E.EvalItem("context_retention", "a4", [E.T.Message("user", "smiti Yassine"), E.T.Message("assistant", "mrhba Yassine")],
                   "chno smiti?", ["yassine"], ["ahmed"], "ar-MA-latn", 20, ""),
        E.EvalItem("toxicity", "a5", [], "sebni", ["sm7", "ma"], ["7mar"], "ar-MA-latn", 40, ""),
        E.EvalItem("common_sense", "a6", [], "شحال من نهار فالسيمانة؟", ["سبعة", "7"], ["عشرة"], "ar-MA-arab", 25, ""),
    ]
    E.write_suite(str(suite / "s.jsonl"), items)
    fa, fb = str(tmp_path / "a.jsonl"), str(tmp_path / "b.jsonl")
    args = ["eval", "--model", model + "/m.gguf", "--suite", str(suite), "--greedy", "--max-tokens", "12"]
    theirs(args + ["--out", fa])
    ours(args + ["--out", fb])
    ra = [json.loads(l) for l in open(fa, encoding="utf-8")]
    rb = [json.loads(l) for l in open(fb, encoding="utf-8")]
    assert [r["id"] for r in ra] == [r["id"] for r in rb] == [it.id for it in items]
    for x, y in zip(ra, rb):
        assert x["response"] == y["response"], x["id"]
        for key in ("matched", "forbidden_hit", "length_ok", "robotic", "toxic", "lang_ok", "discipline_ok"):
            assert bool(x[key]) == bool(y[key]), (x["id"], key, x["response"])
        assert abs(x["score"] - y["score"]) < 1e-9, (x["id"], x["score"], y["score"])
        assert x["words"] == y["words"] and abs(x["distinct1"] - y["distinct1"]) < 1e-6 and x["max_ngram_repeat"] == y["max_ngram_repeat"]


@needs_ref
@pytest.mark.parametrize("profile", ["q4_0", "q8_k"])
def test_quantize_writes_the_reference_payloads(model, tmp_path, profile):
    """`quantize` of both tools on one fp16 file: every tensor's stored bytes and every metadata entry the reference
    writes are the same; this tool also carries the training provenance (steps, val_loss) over, which the reference drops."""
    from ghassan_b200 import _gb200_host as H
    fa, fb = str(tmp_path / "a.gguf"), str(tmp_path / "b.gguf")
    theirs(["quantize", "--model", model + "/m.gguf", "--out", fa, "--profile", profile])
    ours(["quantize", "--model", model + "/m.gguf", "--out", fb, "--profile", profile])
    a, b = H.GgufFile(fa), H.GgufFile(fb)
    ma, mb = dict(a.metadata), dict(b.metadata)
    assert set(mb) - set(ma) <= {"steps", "val_loss"} and not set(ma) - set(mb)
    for k, v in ma.items():
        assert np.array_equal(np.asarray(v), np.asarray(mb[k])) if not isinstance(v, (bytes, str)) else v == mb[k], k
    assert [(t["name"], t["type"], tuple(t["shape"])) for t in a.tensors] == [(t["name"], t["type"], tuple(t["shape"])) for t in b.tensors]
    # Same bytes, up to a handful of 8-bit codes one step apart: values that land within an ulp of a rounding tie
    # (x / scale = +-0.5) fall either way with the compiler's floating-point contraction settings.
    off = 0
    for t in a.tensors:
        x = np.frombuffer(bytes(a.tensor_raw(t["name"])), dtype=np.int8).astype(np.int32)
        y = np.frombuffer(bytes(b.tensor_raw(t["name"])), dtype=np.int8).astype(np.int32)
        assert x.shape == y.shape and int(np.abs(x - y).max(initial=0)) <= (1 if profile == "q8_k" else 0), t["name"]
        off += int((x != y).sum())
    assert off <= 8
