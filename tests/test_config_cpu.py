"""Recipe parser (the YAML subset), typed getters, the typo gate, the shipped recipes and model-config validation."""
import glob
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg():
    from ghassan_b200.utils.config import Config, ConfigError
    return Config, ConfigError


def test_nested_maps_lists_quotes_and_comments():
    Config, _ = _cfg()
    c = Config.from_string("""
# leading comment
model:
  hidden_size: 128   # trailing comment
  name: "a # not a comment"
  alt: 'single: quoted'
data:
  sources:
    - first.txt
    - "second file.txt"
  inline: [a, "b c", d]
training:
  mix:
    web: 0.7
    code: 0.3
flag: yes
""")
    assert c.get_int("model.hidden_size") == 128
    assert c.get_str("model.name") == "a # not a comment"
    assert c.get_str("model.alt") == "single: quoted"
    assert c.get_list("data.sources") == ["first.txt", "second file.txt"]
    assert c.get_list("data.inline") == ["a", "b c", "d"]
    assert c.get_float("training.mix.web") == pytest.approx(0.7)
    assert c.get_bool("flag") is True
    assert c.get_int("missing", 7) == 7 and c.get_str("missing", "x") == "x"


@pytest.mark.parametrize("text", [
    "a: &anchor 1", "a: *alias", "a: !!str 1", "a: |", "a: >", "<<: other", "\tkey: 1", "- orphan", "novalue",
    "a: 1\na: 2", ": 3",
])
def test_unsupported_yaml_is_refused(text):
    Config, ConfigError = _cfg()
    with pytest.raises(ConfigError):
        Config.from_string(text)


def test_strict_getters_report_bad_values():
    Config, ConfigError = _cfg()
    c = Config.from_string("a: 12x\nb: 1e\nc: maybe\nd: 5\ne: 0.25\nf: off")
    for call, key in ((c.get_int_strict, "a"), (c.get_float_strict, "b"), (c.get_bool_strict, "c")):
        with pytest.raises(ConfigError):
            call(key)
    assert c.get_int_strict("d") == 5 and c.get_float_strict("e") == 0.25 and c.get_bool_strict("f") is False
    # the lenient getters fall back to the default on a malformed value
    assert c.get_int("a", 3) == 3


def test_typo_gate():
    Config, ConfigError = _cfg()
    c = Config.from_string("model:\n  hidden_size: 8\n  hiden_size: 9\ntraining:\n  lonely:\n")
    assert c.check_known({"model.hidden_size"}, ()) == 2
    with pytest.raises(ConfigError):
        c.check_known({"model.hidden_size"}, (), strict=True)
    assert c.check_known({"model.hidden_size", "model.hiden_size"}, ("training.",)) == 0


TRAIN_RECIPES = sorted(p for p in glob.glob(os.path.join(ROOT, "configs", "*.yaml"))
                       if not os.path.basename(p).startswith("synthesis_"))


@pytest.mark.parametrize("path", TRAIN_RECIPES, ids=[os.path.basename(p) for p in TRAIN_RECIPES])
def test_shipped_recipes_parse_strictly(path):
    Config, _ = _cfg()
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    c = Config.from_file(path)
    m = ModelConfig.from_config(c)
    t = TrainerConfig.from_config(c, strict=True)
    m.validate()
    assert m.count_parameters() == sum(s.numel for s in m.param_specs())
    assert m.active_parameters_per_token() <= m.count_parameters()
    assert t.batch_size > 0 and t.seq_len <= m.max_seq_len
    if os.path.basename(path).startswith("sft_"):
        assert t.stage == "sft"


@pytest.mark.parametrize("name,total", [
    ("cpu_smoke_test", 422656), ("flash_109m_compact_2xt4", 109246464), ("flash_480m_2xt4", 479730688),
    ("pro_1b_2xt4", 1036995840), ("t4_en_120m_fast", 100092672),
])
def test_parameter_counts_of_the_named_models(name, total):
    Config, _ = _cfg()
    from ghassan_b200.models.config import ModelConfig
    m = ModelConfig.from_config(Config.from_file(os.path.join(ROOT, "configs", name + ".yaml")))
    assert m.count_parameters() == total


def _model(**over):
    from ghassan_b200.models.config import ModelConfig
    base = dict(vocab_size=320, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=128,
                max_seq_len=32)
    base.update(over)
    return ModelConfig(**base)


@pytest.mark.parametrize("bad", [
    dict(num_heads=3),                      # hidden not divisible by heads
    dict(num_kv_heads=3),                   # heads not divisible by kv heads
    dict(use_moe=True, num_experts=4, moe_top_k=5, moe_expert_dim=64),
    dict(use_moe=True, num_experts=4, moe_top_k=2, moe_expert_dim=64, moe_aux_free=True, moe_aux_scale=0.01),
    dict(vocab_size=0),
    dict(rope_scale=9.0),
    dict(hidden_size=1028, num_heads=2, num_kv_heads=2),      # head_dim 514 exceeds the attention kernels' limit
])
def test_model_config_validation(bad):
    with pytest.raises(ValueError):
        _model(**bad).validate()


def test_architecture_identity():
    a, b = _model(), _model()
    assert a.arch_identity() == b.arch_identity() and a.same_architecture_as(b)[0]
    for change in (dict(num_layers=3), dict(rope_theta=50000.0), dict(sliding_window=16), dict(use_qk_norm=True)):
        c = _model(**change)
        same, why = a.same_architecture_as(c)
        assert not same and list(change)[0] in why
        assert a.arch_identity() != c.arch_identity()


def test_rope_tables():
    import numpy as np
    m = _model()
    inv = m.rope_inv_freq()
    assert inv.shape == (m.head_dim // 2,) and inv[0] == pytest.approx(1.0)
    assert np.all(np.diff(inv) < 0)
    y = _model(rope_type="yarn", rope_scale=4.0) if hasattr(m, "rope_type") else m
    assert np.all(y.rope_inv_freq() <= inv + 1e-9)        # scaling never raises a frequency
    assert y.rope_mscale() >= 1.0


def test_trainer_config_rules():
    Config, ConfigError = _cfg()
    from ghassan_b200.training.config import TrainerConfig, split_shard_glob
    base = "training:\n  max_steps: 10\n  warmup_steps: 2\n"
    t = TrainerConfig.from_config(Config.from_string(base + "  batch_size: 2\n  seq_len: 16\n  grad_accum: 3\n"))
    assert t.tokens_per_step_local() == 96 and t.tokens_per_step_global(4) == 384
    assert t.epoch_steps(96 * 5 + 1, 1) == 0                      # steps mode: no epochs configured
    e = TrainerConfig.from_config(Config.from_string(
        "training:\n  epochs: 2\n  warmup_steps: 2\n  batch_size: 2\n  seq_len: 16\n  grad_accum: 3\n"))
    assert e.epoch_steps(96 * 5 + 1, 1) == 12 and e.epoch_steps(96 * 5 + 1, 2) == 6
    with pytest.raises(Exception):
        TrainerConfig.from_config(Config.from_string("training:\n  batch_size: 2\n"))      # no schedule
    with pytest.raises(Exception):
        TrainerConfig.from_config(Config.from_string(base + "  optimizer: sgd\n"))
    with pytest.raises(Exception):
        TrainerConfig.from_config(Config.from_string(base + "  bogus_key: 1\n"), strict=True)
    d, p = split_shard_glob("artifacts/shards_en/train_*.gbin")[:2]
    assert d == "artifacts/shards_en" and p.startswith("train")
    lion = TrainerConfig.from_config(Config.from_string(base + "  optimizer: lion\n  learning_rate: 0.001\n"))
    assert lion.effective_peak_lr() == pytest.approx(0.0001)      # Lion runs at a tenth of the recipe rate


# "parameters : <total> (<total minus embedding tables> without embeddings)" as the reference's `gai_train --dry-run`
# prints it for each shipped recipe (recorded from its CPU build)
REFERENCE_DRY_RUN_PARAMETERS = {
    "cpu_smoke_test": ("422.66K", "345.86K"), "flash_109m_compact_2xt4": ("109.25M", "92.86M"),
    "flash_480m_2xt4": ("479.73M", "455.15M"), "flash_480m_ollama_compat": ("433.72M", "409.15M"),
    "flash_480m_single": ("479.73M", "455.15M"), "pilot_moe_smoke": ("479.73M", "455.15M"),
    "pro_1b_2xt4": ("1.04B", "1.01B"), "pro_1b_4xt4_legacy": ("1.04B", "1.01B"),
    "pro_1b_auxfree_research": ("479.73M", "455.15M"), "pro_1b_single": ("1.04B", "1.01B"),
    "sft_flash_109m_compact_2xt4": ("109.25M", "92.86M"), "sft_flash_480m_2xt4": ("479.73M", "455.15M"),
    "sft_flash_480m_4xt4": ("479.73M", "455.15M"), "sft_flash_480m_single": ("479.73M", "455.15M"),
    "sft_pro_1b_2xt4": ("1.04B", "1.01B"), "sft_pro_1b_single": ("1.04B", "1.01B"), "t4_en_120m_fast": ("100.09M", "75.52M"),
}


def test_parameter_totals_match_the_reference_dry_run():
    import os
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.utils.config import Config
    from ghassan_b200.utils.log import human_count
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "configs")
    for name, (total, no_emb) in REFERENCE_DRY_RUN_PARAMETERS.items():
        m = ModelConfig.from_config(Config.from_file(os.path.join(root, name + ".yaml")))
        n = m.count_parameters()
        emb = m.vocab_size * m.hidden_size * (1 if m.tie_embeddings else 2)
        assert human_count(n) == total, (name, human_count(n), total)
        assert human_count(n - emb) == no_emb, (name, human_count(n - emb), no_emb)


def test_every_training_recipe_passes_a_strict_dry_run(capsys):
    import os
    from ghassan_b200.cli import train as TR
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "configs")
    for name in REFERENCE_DRY_RUN_PARAMETERS:
        rc = TR.main(["--config", os.path.join(root, name + ".yaml"), "--dry-run", "--strict-config", "--output-budget-mb", "0"])
        assert rc == 0, (name, capsys.readouterr())
    capsys.readouterr()


def test_every_shipped_recipe_passes_a_strict_dry_run(capsys):
    """`gai_train --config <yaml> --dry-run --strict-config` for every recipe in configs/ (the reference's suite does
    the same: configs/kaggle/verify_engine_suite.sh:196-206): unknown keys, bad ranges and impossible shapes fail here,
    not hours into a run."""
    import glob
    import os
    from ghassan_b200.cli import train as T
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    from ghassan_b200.utils.config import Config
    recipes = sorted(glob.glob(os.path.join(root, "configs", "*.yaml")))
    assert len(recipes) >= 19
    trained = 0
    for path in recipes:
        if not any(k.startswith("training.") for k in Config.from_file(path).kv):
            continue            # synth_*.yaml / synthesis_*.yaml configure data_pipeline, not the trainer
        trained += 1
        assert T.main(["--config", path, "--dry-run", "--strict-config", "--device", "cuda"]) == 0, path
    assert trained >= 15
