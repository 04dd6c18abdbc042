"""Flags that every command line shares: ``--quiet`` (warnings and errors only), ``--silent`` (nothing), ``--verbose``
(debug lines too) and ``--threads N`` (host threads for the CPU parts), with the reference's meaning
(tools/cli_common.cpp:160-171 there: quiet -> Warn, silent -> Silent, verbose -> Debug, threads -> the worker pool)."""
from __future__ import annotations

import argparse

from ..utils import log as LOG


def add_common_flags(ap: argparse.ArgumentParser) -> None:
    """Adds the flags a parser does not have yet (some commands already take ``--verbose`` or ``--threads``)."""
    have = {s for act in ap._actions for s in act.option_strings}
    for name in ("quiet", "silent", "verbose"):
        if "--" + name not in have:
            ap.add_argument("--" + name, action="store_true")
    if "--threads" not in have:
        ap.add_argument("--threads")


def apply_common_flags(args) -> None:
    """Later flags win in the reference's order: quiet, then silent, then verbose."""
    if getattr(args, "quiet", False):
        LOG.set_log_level(LOG.WARN)
    if getattr(args, "silent", False):
        LOG.set_log_level(LOG.SILENT)
    if getattr(args, "verbose", False):
        LOG.set_log_level(LOG.DEBUG)
    raw = getattr(args, "threads", None)
    if raw is None:
        return
    try:
        n = int(raw)
    except (TypeError, ValueError):
        return                      # a command that parses --threads strictly reports it itself
    if n > 0:
        import torch
        torch.set_num_threads(n)
