"""The acceptance suites on a CUDA device: the model-running gates (generate, chat, decode speed, perplexity, logits,
16-bit segmented backward, perplexity drift of the quantised files) are live here."""
import pytest

pytestmark = pytest.mark.gpu


def test_app_suite_on_cuda(tmp_path, capsys):
    from ghassan_b200.cli import verify
    rc = verify.main(["app", "--device", "cuda", "--workdir", str(tmp_path)])
    out = capsys.readouterr().out
    assert rc == 0 and "[skip]" not in out, out[-3000:]


def test_engine_suite_on_cuda(tmp_path, capsys):
    from ghassan_b200.cli import verify
    rc = verify.main(["engine", "--device", "cuda", "--workdir", str(tmp_path)])
    out = capsys.readouterr().out
    assert rc == 0 and "16-bit GEMMs: step-2 loss" in out and "within budget" in out, out[-3000:]
