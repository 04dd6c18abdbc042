"""The acceptance suites (cli/verify.py) on the CPU engine, and the perplexity budget rule on its own."""
import pytest


def test_quant_gate_rule():
    from ghassan_b200.cli.verify import quant_gate
    assert quant_gate(10.0, 10.5, 13.0)[0]
    assert not quant_gate(10.0, 11.6, 13.0)[0]          # 8-bit drifts more than 15 %
    assert not quant_gate(10.0, 10.5, 16.5)[0]          # 4-bit drifts more than 60 %
    assert not quant_gate(10.0, 10.5, 9.0)[0]           # 4-bit better than fp16: the measurement is broken
    assert quant_gate(10.0, 10.0, 9.9)[0]               # within noise of fp16
    assert not quant_gate(10.0, 0.0, 12.0)[0]


def test_app_suite_passes_on_cpu(tmp_path, capsys):
    from ghassan_b200.cli import verify
    assert verify.main(["app", "--device", "cpu", "--workdir", str(tmp_path)]) == 0
    out = capsys.readouterr().out
    assert "PASS" in out and "[FAIL]" not in out
    assert out.count("[ok]") >= 7 and "[skip] the inference engine needs a CUDA device" in out


def test_engine_suite_passes_on_cpu(tmp_path, capsys):
    from ghassan_b200.cli import verify
    assert verify.main(["engine", "--device", "cpu", "--workdir", str(tmp_path)]) == 0
    out = capsys.readouterr().out
    assert "segments=2" in out and "resumed from last.ckpt and finished at step 4" in out
    assert "pro_1b_2xt4.yaml" in out and "[FAIL]" not in out


def test_a_failed_gate_is_counted(tmp_path, capsys, monkeypatch):
    from ghassan_b200.cli import verify
    monkeypatch.setattr(verify, "quant_gate", lambda *a: (False, "forced"))
    s = verify.Suite()
    s.bad("x")
    s.ok("y")
    assert s.failures == 1
    rc, text = s.call(lambda argv: (_ for _ in ()).throw(RuntimeError("boom")), [])
    assert rc == 99 and "boom" in text
    rc, text = s.call(lambda argv: (_ for _ in ()).throw(SystemExit("needs --model")), [])
    assert rc == 1 and "needs --model" in text
