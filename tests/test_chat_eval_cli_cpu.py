"""Chat session logic, the heuristic evaluation scorer and the command-line front ends, all on the CPU (the model
is replaced by a canned generator where one is needed)."""
import io
import json
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def tok():
    from ghassan_b200.data.tokenizer import Tokenizer
    return Tokenizer.load(os.path.join(GOLD, "text", "ref_small.gtok"))


class CannedGenerator:
    """Stands in for inference.generator.Generator: records what it was asked and answers from a script."""

    def __init__(self, tok, replies):
        self.tok, self.replies, self.calls = tok, list(replies), []

    def generate(self, prompts, max_new_tokens=256, sampling=None, on_text=None, **kw):
        from ghassan_b200.inference.generator import GenerationResult
        self.calls.append({"ids": np.asarray(prompts[0]).copy(), "max_new": max_new_tokens, "sampling": sampling})
        text = self.replies[(len(self.calls) - 1) % len(self.replies)]
        if on_text is not None:
            on_text(0, text)
        return GenerationResult(tokens=[[5, 6, 7]], text=[text], prompt_tokens=len(prompts[0]), prefill_seconds=0.01,
                                decode_seconds=0.02, stopped=["eos"])


# ------------------------------------------------------------------------------------------ dialog acts
def test_dialog_acts_and_english_presets():
    from ghassan_b200.inference import chat as C
    from ghassan_b200.inference.engine import SamplingParams
    want = {"hi": "greeting", "Hello there!": "greeting", "Write a python function to sort a list": "coding",
            "why is the sky blue?": "question", "Summarize this text": "instruction", "translate hello to french": "instruction",
            "thanks!": "chitchat", "If x + 3 = 7, solve for x step by step": "reasoning"}
    for text, act in want.items():
        assert C.classify_dialog_act(text) == act, text
    base = SamplingParams(temperature=0.9, top_k=80, top_p=0.97, min_p=0.0, no_repeat_ngram=4)
    s, n = C.adapt_english_sampling(base, 256, "hi")
    assert n == 96 and s.temperature == 0.8 and s.no_repeat_ngram == 0
    s, n = C.adapt_english_sampling(base, 256, "Write a python function to sort a list")
    assert n == 256 and s.temperature == 0.4 and s.top_k == 40 and s.top_p == 1.0
    s, n = C.adapt_english_sampling(base, 256, "thanks!")
    assert (s.temperature, s.top_k, s.no_repeat_ngram) == (0.9, 80, 4)         # chit-chat keeps the user's settings
    assert base.temperature == 0.9 and base.top_k == 80                           # the caller's object is never edited


# ------------------------------------------------------------------------------------------ chat session
def test_chat_history_trimming_and_script_policy(tok):
    from ghassan_b200.data import tokenizer as T
    from ghassan_b200.inference import chat as C
    gen = CannedGenerator(tok, ["jawab %d" % i for i in range(10)])
    out = io.StringIO()
    s = C.ChatSession(gen, C.ChatOptions(max_history_turns=2, stream=True), out=out)
    assert s.history[0].role == "system" and s.history[0].content == T.SYSTEM_DARIJA_ARABIC
    s.send("salam, kidayr?")
    assert s.history[0].content == T.system_for_script(T.detect_script("salam, kidayr?"))     # Latin script → Latin persona
    s.send("السلام عليكم")
    assert s.history[0].content == T.system_for_script(T.detect_script("السلام عليكم"))
    for i in range(4):
        s.send("so2al %d" % i)
    roles = [m.role for m in s.history]
    assert roles[0] == "system" and roles[1:] == ["user", "assistant"] * ((len(roles) - 1) // 2)   # whole exchanges only
    assert 5 <= len(s.history) <= 7 and s.history[-1].content == "jawab 5" and s.history[-2].content == "so2al 3"
    assert all(m.content != "salam, kidayr?" for m in s.history)                                  # the oldest turns left
    assert "jawab 5" in out.getvalue()
    # the prompt handed to the model is the chat template of exactly that window plus the generation prompt
    ids, _ = T.encode_chat(tok, s.history[:-1], add_generation_prompt=True)
    assert gen.calls[-1]["ids"].tolist() == ids.tolist()
    s.clear()
    assert len(s.history) == 1
    s.set_system("jawb b ikhtisar")
    s.send("chno smitek?")
    assert s.history[0].content.startswith("jawb b ikhtisar") and T.script_directive(T.detect_script("chno smitek?")) in s.history[0].content
    with pytest.raises(ValueError):
        C.ChatSession(gen, C.ChatOptions(max_history_turns=-1))


def test_chat_english_persona_adapts_sampling(tok):
    from ghassan_b200.data import tokenizer as T
    from ghassan_b200.inference import chat as C
    gen = CannedGenerator(tok, ["ok"])
    s = C.ChatSession(gen, C.ChatOptions(persona="en", stream=False), out=io.StringIO())
    assert s.history[0].content == T.SYSTEM_ENGLISH
    s.send("hi")
    assert gen.calls[-1]["max_new"] == 96
    s.send("write a function in python that adds two numbers")
    assert gen.calls[-1]["sampling"].temperature <= 0.4 and gen.calls[-1]["max_new"] == 256
    assert s.history[0].content == T.SYSTEM_ENGLISH                              # no script switching for this persona
    s2 = C.ChatSession(gen, C.ChatOptions(persona="en", stream=False, adaptive_dialog=False), out=io.StringIO())
    s2.send("hi")
    assert gen.calls[-1]["max_new"] == 256


def test_chat_retrieval_direct_and_context(tok, tmp_path):
    from ghassan_b200.inference import chat as C
    (tmp_path / "qa.json").write_text(json.dumps([{"question": "chno hiya 3asimat lmaghrib", "answer": "Rbat."}]), encoding="utf-8")
    gen = CannedGenerator(tok, ["mn lmodel"])
    s = C.ChatSession(gen, C.ChatOptions(stream=False, retrieve_index=str(tmp_path / "qa.json"), retrieve_direct=True), out=io.StringIO())
    assert s.send("chno hiya 3asimat lmaghrib?") == "Rbat." and not gen.calls           # answered from the index
    assert s.send("xyzzy plugh") == "mn lmodel" and len(gen.calls) == 1                # nothing found → the model answers
    s = C.ChatSession(gen, C.ChatOptions(stream=False, retrieve_index=str(tmp_path / "qa.json")), out=io.StringIO())
    assert s.send("3asimat lmaghrib chno hiya") == "mn lmodel"
    assert any(m.role == "system" and "Rbat." in m.content for m in s.history[1:])       # the hit rides along as context


def test_chat_repl_commands(tok):
    from ghassan_b200.inference import chat as C
    gen = CannedGenerator(tok, ["wakha"])
    out = io.StringIO()
    s = C.ChatSession(gen, C.ChatOptions(stream=True), out=out)
    s.run_repl(io.StringIO("/help\n/temp 0.3\n/temp abc\n/temp 99\nsalam\n/stats\n/system jawb b zerba\n/system\n/bogus\n/clear\n/quit\nnever read\n"))
    text = out.getvalue()
    assert "[temperature = 0.3]" in text and "invalid temperature" in text and "[temperature = 5]" in text
    assert "wakha" in text and "history: 3 messages" in text and "unknown command: bogus" in text
    assert "system: jawb b zerba" in text and "[history cleared]" in text
    assert len(gen.calls) == 1 and len(s.history) == 1


# ------------------------------------------------------------------------------------------ evaluation
def test_score_response_weights():
    from ghassan_b200.inference import evaluate as E
    it = E.EvalItem(category="c", id="x", prompt="شنو هي عاصمة المغرب؟", expect_any=["الرباط"], forbid=["باريس"], expect_lang="ar-MA-arab",
                    max_words=12)
    good = E.score_response(it, "العاصمة ديال المغرب هي الرباط", 1.0)
    assert good["matched"] and good["lang_ok"] and good["score"] == pytest.approx(1.0)
    miss = E.score_response(it, "ما عرفتش والله", 1.0)
    assert not miss["matched"] and miss["score"] == pytest.approx(0.60)
    bad = E.score_response(it, "الرباط ولا باريس", 1.0)
    assert bad["forbidden_hit"] and bad["score"] == pytest.approx(0.85)
    long = E.score_response(it, "الرباط " + "هي " * 20, 1.0)
    assert not long["length_ok"] and long["max_ngram_repeat"] >= 5
    wrong_lang = E.score_response(it, "The capital is الرباط but I will answer in English because I can", 1.0)
    assert not wrong_lang["lang_ok"]
    robot = E.score_response(E.EvalItem(category="c", id="y", prompt="chno ban lik?"), "As an AI language model, I cannot have opinions.")
    assert robot["robotic"] and robot["score"] == pytest.approx(0.90)


def test_english_discipline_and_repetition_metrics():
    from ghassan_b200.inference import evaluate as E
    assert E.distinct_n("a b c a b c", 1) == pytest.approx(0.5) and E.distinct_n("a b c a b c", 2) == pytest.approx(0.6)
    assert E.distinct_n("", 2) == 0.0
    assert E.max_ngram_repeat("a b c a b c a b c", 3) == 3 and E.max_ngram_repeat("one two", 3) == 0
    ok = E.check_english_reply("Write code to add numbers", "Sure:\n```python\nprint(1 + 2)\n```")
    assert ok["disciplined"] and ok["act"] == "coding"
    assert not E.check_english_reply("Write code to add numbers", "Numbers are nice.")["disciplined"]
    assert E.check_english_reply("hi", "As an AI language model I have no name")["reason"] == "ai-disclosure"
    assert E.check_english_reply("hi", " ")["reason"] == "empty"
    mc = "Which is larger? A. 3  B. 7  C. 5"
    assert E.check_english_reply(mc, "B. 7")["disciplined"] and E.check_english_reply(mc, "Seven is larger")["reason"] == "bad-mc-format"


def test_suites_round_trip_and_summary(tok, tmp_path):
    from ghassan_b200.inference import evaluate as E
    items = E.builtin_suite()
    from ghassan_b200.inference import eval_suites as ES
    assert len(items) >= 50 and len({i.id for i in items}) == len(items)
    assert {i.category for i in items} == set(ES.CATEGORIES) and len(ES.CATEGORIES) == 14      # every category has items
    en = E.builtin_suite_en()
    assert len(en) >= 25 and all(i.expect_lang in ("en", "") for i in en) and len({i.category for i in en}) >= 10
    assert ES.category_from_name("Code-Switching") == "code_switching" and ES.category_from_name("nope") == "basic_conversation"
    E.write_suite(str(tmp_path / "suite.jsonl"), items)
    back = E.load_suite(str(tmp_path))
    assert [(i.id, i.prompt, i.expect_any, i.max_words) for i in back] == [(i.id, i.prompt, i.expect_any, i.max_words) for i in items]
    gen = CannedGenerator(tok, ["وعليكم السلام، مرحبا بيك", "As an AI language model, I cannot answer."])
    rep = E.run_benchmark(gen, items, max_new_tokens=32, max_prompts=6)
    assert rep["total"] == 6 and len(gen.calls) == 6 and gen.calls[0]["max_new"] == 32
    assert rep["robotic_rate"] == pytest.approx(0.5) and 0.0 < rep["overall"] < 1.0
    assert sum(c["items"] for c in rep["by_category"].values()) == 6
    only = E.run_benchmark(gen, items, categories=items[-1].category)
    assert set(only["by_category"]) == {items[-1].category}
    text = E.report_text(rep)
    assert "items 6" in text and "robotic 50.0%" in text


# ------------------------------------------------------------------------------------------ command lines
def test_train_cli_dry_run_and_argument_errors(capsys):
    from ghassan_b200.cli import train as TR
    cfgs = os.path.join(os.path.dirname(__file__), "..", "configs")
    rc = TR.main(["--config", os.path.join(cfgs, "pro_1b_2xt4.yaml"), "--dry-run", "--output-budget-mb", "0", "--device", "cuda"])
    out = capsys.readouterr()
    text = out.out + out.err
    assert rc == 0, text
    assert "1.04B" in text and "MoE(ne=8,k=4,E=1280,shared)" in text and "lion" in text and "[dry ]" in text
    rc = TR.main(["--config", os.path.join(cfgs, "pro_1b_2xt4.yaml"), "--dry-run", "--max-vram-mb", "1024", "--output-budget-mb", "0"])
    assert rc != 0 and "1024" in (lambda o: o.out + o.err)(capsys.readouterr())
    assert TR.main(["--config", os.path.join(cfgs, "cpu_smoke_test.yaml"), "--dry-run", "--optimizer", "sgd"]) == 2
    assert TR.main(["--config", os.path.join(cfgs, "cpu_smoke_test.yaml"), "--dry-run", "--resume-mode", "maybe"]) == 2
    assert TR.main(["--config", os.path.join(cfgs, "cpu_smoke_test.yaml"), "--dry-run", "--strict-args", "--batch-size", "4x"]) == 2
    capsys.readouterr()


def test_memory_plan_scales_with_sharding():
    from ghassan_b200.cli.train import memory_plan
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.utils.config import Config
    cfg = Config.from_file(os.path.join(os.path.dirname(__file__), "..", "configs", "pro_1b_2xt4.yaml"))
    m, t = ModelConfig.from_config(cfg), TrainerConfig.from_config(cfg)
    one, eight = memory_plan(m, t, 1, 16), memory_plan(m, t, 8, 16)
    assert one["parameters"] == m.count_parameters() == eight["parameters"]
    # moments live only on the rank that updates their shard (fused exchange); weights and gradients stay whole
    assert eight["optimizer"] == (one["optimizer"] + 7) // 8 and eight["total"] == one["total"] - one["optimizer"] + eight["optimizer"]
    assert eight["checkpoint_bytes"] == one["checkpoint_bytes"]        # a checkpoint still holds all of them
    assert one["optimizer"] == 4 * one["parameters"] and one["weights"] == 6 * one["parameters"]       # lion: one moment
    t2 = TrainerConfig.from_config(cfg)
    t2.optimizer = "muon"                                  # Muon runs whole on every rank: nothing to shard
    assert memory_plan(m, t2, 8, 16)["optimizer"] == memory_plan(m, t2, 1, 16)["optimizer"]
    assert eight["activations"] == one["activations"] and memory_plan(m, t, 1, 1)["activations"] < one["activations"]


def test_infer_cli_export_info_quantize_tokenize(tmp_path, capsys):
    from ghassan_b200.cli import infer as I
    f = os.path.join(GOLD, "formats")
    out = str(tmp_path / "m.gguf")
    assert I.main(["export", "--checkpoint", os.path.join(f, "tiny_ref.ckpt"), "--tokenizer", os.path.join(f, "tiny400.gtok"), "--out", out]) == 0
    assert open(out, "rb").read() == open(os.path.join(f, "tiny_fp16.gguf"), "rb").read()     # the reference exporter's bytes
    capsys.readouterr()
    assert I.main(["info", "--model", out]) == 0
    info = capsys.readouterr().out
    assert "ghassan" in info.lower() and "F16" in info
    q = str(tmp_path / "q.gguf")
    assert I.main(["quantize", "--model", out, "--out", q, "--profile", "q4_0"]) == 0
    assert os.path.getsize(q) < os.path.getsize(out)
    capsys.readouterr()
    assert I.main(["info", "--model", q]) == 0 and "Q4_0" in capsys.readouterr().out
    # --measure: the 4-bit probe names a matrix and a plausible error; --compat writes the llama-style names
    q2 = str(tmp_path / "q2.gguf")
    assert I.main(["quantize", "--model", out, "--out", q2, "--profile", "q8_k", "--measure", "--compat", "native"]) == 0
    msg = capsys.readouterr().out
    assert "worst rel RMSE (Q4 probe):" in msg and "compat=native" in msg
    pct = float(msg.split("worst rel RMSE (Q4 probe):")[1].split("%")[0])
    assert 1.0 < pct < 30.0
    with pytest.raises(SystemExit, match="unknown compat"):
        I.main(["quantize", "--model", out, "--out", q2, "--compat", "nonsense"])
    with pytest.raises(SystemExit, match="refused"):      # this model has a shared expert and QK-norm: no llama.cpp form
        I.main(["quantize", "--model", out, "--out", q2, "--compat", "llama_moe"])
    assert I.main(["tokenize", "--model", out, "--text", "salam"]) == 0
    t = capsys.readouterr().out
    assert "tokens  :" in t and "ids     :" in t
    with pytest.raises(SystemExit):
        I.main(["export", "--checkpoint", os.path.join(f, "tiny_ref.ckpt"), "--out", out])
    assert I.main(["devices"]) == 0
