"""The flags every command line shares (--quiet, --silent, --verbose, --threads): same meaning as the reference's
apply_common_flags (tools/cli_common.cpp:160-171)."""
import argparse

import pytest

from ghassan_b200.cli import common as C
from ghassan_b200.utils import log as LOG


@pytest.fixture(autouse=True)
def _restore_level():
    before = LOG.log_level()
    yield
    LOG.set_log_level(before)


def _parse(argv, preset=()):
    ap = argparse.ArgumentParser()
    for name in preset:
        ap.add_argument("--" + name, action="store_true")
    C.add_common_flags(ap)
    return ap.parse_args(argv)


@pytest.mark.parametrize("argv,level", [([], None), (["--quiet"], LOG.WARN), (["--silent"], LOG.SILENT),
                                        (["--verbose"], LOG.DEBUG), (["--quiet", "--silent"], LOG.SILENT),
                                        (["--silent", "--verbose"], LOG.DEBUG)])
def test_levels(argv, level):
    LOG.set_log_level(LOG.INFO)
    C.apply_common_flags(_parse(argv))
    assert LOG.log_level() == (LOG.INFO if level is None else level)


def test_flags_are_added_once():
    a = _parse(["--verbose"], preset=("verbose",))      # a parser that already has --verbose keeps its own
    assert a.verbose and not a.quiet


def test_threads():
    import torch
    before = torch.get_num_threads()
    try:
        C.apply_common_flags(_parse(["--threads", "2"]))
        assert torch.get_num_threads() == 2
        C.apply_common_flags(_parse(["--threads", "zero"]))   # not a number: left to the command's own strict parsing
        assert torch.get_num_threads() == 2
    finally:
        torch.set_num_threads(before)


def test_quiet_hides_info_lines_of_a_dry_run(capsys):
    from ghassan_b200.cli import train as T
    tiny = ["--config", "configs/cpu_smoke_test.yaml", "--dry-run"]
    assert T.main(tiny) == 0
    loud = capsys.readouterr().out
    assert "[info ]" in loud
    LOG.set_log_level(LOG.INFO)
    assert T.main(tiny + ["--quiet"]) == 0
    assert "[info ]" not in capsys.readouterr().out


def test_every_command_line_takes_the_flags():
    from ghassan_b200.cli import corpus_stats, data_pipeline, infer, plan, train, train_tokenizer, verify
    for mod in (corpus_stats, data_pipeline, infer, plan, train, train_tokenizer, verify):
        src = open(mod.__file__).read()
        assert "add_common_flags(" in src and "apply_common_flags(" in src, mod.__name__
