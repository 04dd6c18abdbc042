"""Session planner: budget arithmetic, the estimate verdict, and a pilot run of a tiny recipe on the CPU engine."""
import json
import os

import numpy as np
import pytest

VOCAB = 320

RECIPE = """
model:
  vocab_size: %d
  hidden_size: 64
  num_layers: 2
  num_heads: 4
  num_kv_heads: 2
  intermediate_size: 128
  max_seq_len: 32
  use_moe: true
  num_experts: 4
  moe_top_k: 2
  moe_expert_dim: 64
  moe_shared: true
training:
  optimizer: adamw
  learning_rate: 0.003
  batch_size: 2
  seq_len: 32
  grad_accum: 2
  warmup_steps: 2
  epochs: 3
  device: cpu
  data_dir: %s
"""


@pytest.fixture()
def recipe(tmp_path):
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.data.loader import write_shard
    r = H.Rng(1)
    docs = []
    for _ in range(120):
        a = np.empty(20 + int(r.below(80)), dtype=np.int32)
        r.fill_uniform_ids(a, 40)
        docs.append(a + 16)
    d = str(tmp_path / "shards")
    os.makedirs(d)
    write_shard(os.path.join(d, "train_0000.gbin"), docs, VOCAB, None)
    p = str(tmp_path / "recipe.yaml")
    with open(p, "w") as f:
        f.write(RECIPE % (VOCAB, d))
    return p


def test_budget_table_and_estimate_arithmetic():
    from ghassan_b200.cli.plan import budget_table, estimate
    rows = budget_table(32768, 100000.0, corpus_tokens=150_000_000, hours=(2, 10))
    assert rows[0]["steps"] == int(2 * 3600 * 100000.0 / 32768)
    assert rows[1]["tokens"] == rows[1]["steps"] * 32768
    assert abs(rows[1]["epochs"] - rows[1]["tokens"] / 150e6) < 1e-12
    assert budget_table(128, 10.0)[0]["epochs"] is None
    e = estimate(32768, 150e6, 2, 1500.0, 10.0)           # the reference's T4 example: 480M MoE at ~1.5k tokens/s
    assert not e["fits"] and abs(e["hours"] - 300e6 / 1500.0 / 3600.0) < 1e-9 and e["steps"] == int(300e6 / 32768)
    assert estimate(32768, 150e6, 1, 130000.0, 10.0)["fits"]


def test_estimate_command_exit_codes(recipe, capsys):
    from ghassan_b200.cli import plan
    assert plan.main(["estimate", "--config", recipe, "--tps", "50000", "--corpus-tokens", "1e6", "--json"]) == 0
    r = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert r["fits"] and r["epochs"] == 3 and r["tokens_per_step"] == 2 * 32 * 2 and r["total_tokens"] == 3e6
    assert plan.main(["estimate", "--config", recipe, "--tps", "10", "--corpus-gb", "1", "--budget-hours", "1"]) == 3
    assert plan.main(["estimate", "--config", recipe, "--tps", "10"]) == 2              # no corpus size given
    assert plan.main(["estimate", "--config", str(recipe) + ".missing", "--tps", "10", "--corpus-gb", "1"]) == 2


def test_pilot_runs_the_recipe_and_reports_a_rate(recipe, capsys):
    from ghassan_b200.cli import plan
    assert plan.main(["pilot", "--config", recipe, "--steps", "6", "--warm", "2", "--device", "cpu", "--json"]) == 0
    r = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert r["guard"] is None and r["finite"] and r["steps"] == 6
    assert r["tokens_per_step"] == 128 and r["tok_per_s"] > 0 and r["corpus_tokens"] > 1000
    assert [row["hours"] for row in r["table"]] == [2, 4, 6, 8, 10]
    assert r["table"][0]["steps"] == int(2 * 3600 * r["tok_per_s"] / 128)
    assert r["last_loss"] < r["first_loss"] + 0.5
    assert plan.main(["pilot", "--config", recipe, "--steps", "3", "--warm", "5", "--device", "cpu"]) == 2


def test_pilot_reports_a_guard_instead_of_running(recipe, monkeypatch, capsys):
    from ghassan_b200.cli import plan
    from ghassan_b200.training import guards
    real = guards.Probe
    monkeypatch.setattr(guards, "Probe", lambda *a, **k: real(disk_free=lambda p: 1024, **k))
    rc = plan.main(["pilot", "--config", recipe, "--steps", "6", "--warm", "2", "--device", "cpu", "--json"])
    out = capsys.readouterr().out.strip().splitlines()
    assert rc == 1 and "disk guard" in json.loads(out[-1])["guard"]
