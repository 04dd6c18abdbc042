"""What a dry run prices identically in both engines must agree with the reference trainer on every shipped recipe:
parameter count, fp32 gradient bytes, optimizer-state bytes, tokens per step and the output-budget line.  (Weights and
activations differ by design: this engine keeps a 16-bit shadow of the weights and its own activation arena.)

The expected strings in tests/golden/dry_run_reference.json were printed by the reference's own `gai_train --dry-run
--device cpu` on these recipe files (tools/training_cli.cpp:240-336 there); when a build of it sits under
baseline/_ref/bin the test also runs it live."""
import glob
import json
import os
import re
import subprocess

import pytest

from ghassan_b200.cli import train as T
from ghassan_b200.utils import log as LOG


@pytest.fixture(autouse=True)
def _restore_level():
    before = LOG.log_level()
    yield
    LOG.set_log_level(before)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = json.load(open(os.path.join(ROOT, "tests", "golden", "dry_run_reference.json")))
RECIPES = sorted(k for k, v in GOLDEN.items() if v["rc"] == 0)
REF_BIN = os.path.join(ROOT, "baseline", "_ref", "bin", "gai_train")


def ours(recipe, capsys):
    before = LOG.log_level()
    LOG.set_log_level(LOG.INFO)
    try:
        assert T.main(["--config", os.path.join(ROOT, "configs", recipe), "--dry-run", "--device", "cpu"]) == 0
    finally:
        LOG.set_log_level(before)
    txt = capsys.readouterr().out

    def grab(pat):
        m = re.search(pat, txt)
        return m.group(1).strip() if m else None
    return {"parameters": grab(r"parameters\s+: (\S+)"), "gradients": grab(r"gradients\s+: (.+)"),
            "optimizer_state": grab(r"optimizer\s+: (.+?) \("), "tokens_per_step": grab(r"schedule\s+: (\S+) tokens/step per rank"),
            "output_budget": grab(r"output budget\s+: (.+)")}


def reference_fields(txt):
    def grab(pat):
        m = re.search(pat, txt)
        return m.group(1).strip() if m else None
    return {"parameters": grab(r"parameters\s+: (\S+)"), "gradients": grab(r"gradients \(fp32\)\s+: (.+)"),
            "optimizer_state": grab(r"(?:lion m|adamw m\+v|muon[^:]*)\s+\(fp32\)\s+: (.+)"),
            "tokens_per_step": grab(r"tokens per step\s+: (\S+)"), "output_budget": grab(r"output budget\s+: (.+)")}


def test_every_training_recipe_has_a_recorded_reference_dry_run():
    shipped = {os.path.basename(p) for p in glob.glob(os.path.join(ROOT, "configs", "*.yaml"))}
    assert shipped == set(GOLDEN)
    # the two synthesis recipes are not training recipes: the reference trainer refuses them, and so does this one
    refused = sorted(k for k, v in GOLDEN.items() if v["rc"] != 0)
    assert refused == ["synthesis_billion_scale.yaml", "synthesis_large_200k.yaml"]
    for recipe in refused:          # "no schedule: set training.max_steps (>0) or training.epochs (>0)" from both
        assert T.main(["--config", os.path.join(ROOT, "configs", recipe), "--dry-run", "--device", "cpu", "--silent"]) != 0


@pytest.mark.parametrize("recipe", RECIPES)
def test_dry_run_agrees_with_the_reference(recipe, capsys):
    got = ours(recipe, capsys)
    for key in ("parameters", "gradients", "optimizer_state", "tokens_per_step", "output_budget"):
        assert got[key] == GOLDEN[recipe][key], (recipe, key, got[key], GOLDEN[recipe][key])


@pytest.mark.skipif(not os.path.exists(REF_BIN), reason="no build of the reference trainer here")
def test_recorded_figures_are_what_the_reference_prints_now():
    for recipe in ("pro_1b_2xt4.yaml", "flash_480m_2xt4.yaml", "cpu_smoke_test.yaml"):
        p = subprocess.run([REF_BIN, "--config", os.path.join(ROOT, "configs", recipe), "--dry-run", "--device", "cpu"],
                           capture_output=True, timeout=120)
        live = reference_fields((p.stdout + p.stderr).decode("utf-8", "replace"))
        assert live == {k: GOLDEN[recipe][k] for k in live}, recipe
