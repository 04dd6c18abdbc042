"""Pre-flight resource guards of the trainer: device memory (planned and live), host RAM for two checkpoint
snapshots, free disk for a save, and the output quota.  Each guard refuses to start a run that would die hours in
(the reference's Trainer constructor does the same: training/trainer.cpp:672-836; probes in core/device.cpp:65-354).

The measurements come from a :class:`Probe`, so that tests can supply sizes instead of touching the machine.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple

from ..utils.log import human_bytes, log_info, log_warn

MIB = 1 << 20
SKIP_DIRS = ["build", "build_test", "build_cpu", "out", ".git", ".cache", "ccache", "__pycache__"]


class GuardError(RuntimeError):
    """A resource guard refused the run."""


def _native():
    from .. import _gb200_host as H
    return H


def _gpu_total() -> int:
    import torch
    if not torch.cuda.is_available():
        return 0
    return int(torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory)


def _gpu_free_live() -> int:
    import torch
    if not torch.cuda.is_available():
        return 0
    free, _ = torch.cuda.mem_get_info()
    # blocks that PyTorch's allocator holds but has not handed out are available to this process
    return int(free) + int(torch.cuda.memory_reserved() - torch.cuda.memory_allocated())


@dataclass
class Probe:
    """Where the guards get their numbers.  A value of 0 means "unknown": the guard logs that and passes."""
    gpu_total: Callable[[], int] = _gpu_total
    gpu_free_live: Callable[[], int] = _gpu_free_live
    ram_total: Callable[[], int] = field(default=lambda: int(_native().physical_ram_bytes()))
    disk_free: Callable[[str], int] = field(default=lambda path: int(_native().free_disk_bytes(path)))
    tree_size: Callable[[str, List[str]], Tuple[int, int]] = field(
        default=lambda root, skip: tuple(int(x) for x in _native().tree_size_bytes(root, skip)))
    file_size: Callable[[str], int] = field(default=lambda p: os.path.getsize(p) if os.path.isfile(p) else 0)
    same_file: Callable[[str, str], bool] = field(
        default=lambda a, b: os.path.exists(a) and os.path.exists(b) and os.path.samefile(a, b))
    exists: Callable[[str], bool] = os.path.exists


def snapshot_bytes(n_params: int, optimizer: str) -> int:
    """Host bytes of one captured checkpoint: fp32 weights plus the optimizer moments."""
    return n_params * 4 + n_params * 4 * (2 if optimizer == "adamw" else 1)


def check_device_memory(plan_total: int, plan_already_allocated: int, world: int, probe: Probe, on_cuda: bool) -> None:
    """Planned bytes (+ slack) against the device: refuse above 95 %, warn above 85 %; then the part that is not
    allocated yet against what is free right now (another process, or fragmentation, can make the static test lie)."""
    slack = 1024 * MIB + (384 * MIB if world > 1 else 0)        # CUDA context, library workspaces, symmetric control blocks
    need = plan_total + slack
    total = probe.gpu_total() if on_cuda else 0
    if not total:
        log_info("[mem ] est total %s (weights+grads+opt+acts+slack)%s" % (human_bytes(need), " [per GPU]" if world > 1 else ""))
        return
    frac = need / total
    log_info("[mem ] est core %s + slack %s = total %s / GPU %s (%.0f%%)%s" % (
        human_bytes(plan_total), human_bytes(slack), human_bytes(need), human_bytes(total), 100 * frac,
        " [per GPU]" if world > 1 else ""))
    if frac > 0.95:
        raise GuardError("OOM guard: need %s (core %s) but GPU has %s (%.0f%% with slack). Lower batch_size/seq_len or "
                         "b200.fuse_micro_batches, or switch the optimizer to lion before training." % (
                             human_bytes(need), human_bytes(plan_total), human_bytes(total), 100 * frac))
    if frac > 0.85:
        log_warn("[mem ] over 85%% of GPU memory (core %.0f%%): reduce batch/seq_len if unstable" % (100 * plan_total / total))
    free = probe.gpu_free_live()
    still = max(0, plan_total - plan_already_allocated)
    if free > 0 and still > free:
        raise GuardError("OOM guard (live): %s are still to be allocated but only %s are free right now (another "
                         "process on the GPU, or fragmentation). Lower batch_size/seq_len before training." % (
                             human_bytes(still), human_bytes(free)))


def check_host_ram(per_snapshot: int, ram_budget: int, probe: Probe) -> None:
    ram = probe.ram_total()
    if not ram:
        return
    log_info("[mem ] host RAM %s total, checkpoint queue budget %s (%.0f%%), one snapshot %s" % (
        human_bytes(ram), human_bytes(ram_budget), 100.0 * ram_budget / ram, human_bytes(per_snapshot)))
    need = 2 * per_snapshot + 512 * MIB
    if ram < need:
        raise GuardError("host RAM guard: this run needs ~%s (two %s checkpoint snapshots + 512 MB) but the machine has "
                         "only %s. Reduce the model, or free RAM; training here would be OOM-killed mid-save." % (
                             human_bytes(need), human_bytes(per_snapshot), human_bytes(ram)))


def check_disk(checkpoint_dir: str, per_snapshot: int, probe: Probe) -> None:
    free = probe.disk_free(checkpoint_dir)
    if not free:
        log_warn("[disk] could not stat free space for %s: cannot pre-flight the checkpoint budget" % checkpoint_dir)
        return
    best, last = os.path.join(checkpoint_dir, "best.ckpt"), os.path.join(checkpoint_dir, "last.ckpt")
    published = int(probe.exists(best)) + int(probe.exists(last))
    if published == 2 and probe.same_file(best, last):
        published = 1
    need = per_snapshot * (published + 1) + per_snapshot // 4
    log_info("[disk] %s free at %s (%d checkpoint(s) published); a save transiently needs ~%s" % (
        human_bytes(free), checkpoint_dir, published, human_bytes(need)))
    if free < need:
        raise GuardError("disk guard: %s free at %s but a checkpoint save needs ~%s (%d published + one .tmp + 25%% "
                         "margin). Free space or point --checkpoint-dir at a bigger volume; ENOSPC at hour 6 would lose "
                         "the run." % (human_bytes(free), checkpoint_dir, human_bytes(need), published))


def quota_root(checkpoint_dir: str) -> str:
    """The directory whose size counts against the output quota: the nearest ancestor named ``working`` within four
    levels of the checkpoint directory, else the current directory."""
    root = os.path.abspath(checkpoint_dir)
    for _ in range(4):
        if os.path.basename(root) == "working" or os.path.dirname(root) == root:
            break
        root = os.path.dirname(root)
    return root if os.path.basename(root) == "working" else os.path.abspath(".")


def check_output_quota(budget_mb: int, checkpoint_dir: str, per_snapshot: int, n_params: int, probe: Probe,
                       pretrained: str = "") -> None:
    if budget_mb <= 0:
        return
    budget = budget_mb * MIB
    root = quota_root(checkpoint_dir)
    used, files = probe.tree_size(root, SKIP_DIRS)
    freed = 0
    if pretrained:
        sz = probe.file_size(pretrained)
        if 0 < sz <= used:           # loaded into memory at construction, not kept by this run
            freed, used = sz, used - sz
    ckpt_now, _ = probe.tree_size(checkpoint_dir, [])
    transient = 2 * per_snapshot
    gguf = n_params + per_snapshot // 8
    projected = used + transient + gguf
    log_info("[quota] %s budget | %s already in %s (%d files, incl. %s of checkpoints)" % (
        human_bytes(budget), human_bytes(used), root, files, human_bytes(ckpt_now)))
    if freed:
        log_info("[quota] excluding %s of pretrain checkpoint (not kept by this run)" % human_bytes(freed))
    log_info("[quota] projected peak = %s (current %s + save transient %s + gguf %s)" % (
        human_bytes(projected), human_bytes(used), human_bytes(transient), human_bytes(gguf)))
    if projected > budget:
        raise GuardError("output quota guard: this run projects %s of saved output but the budget is %s (over by %s, %s "
                         "of it already-published checkpoints/data). Delete stale checkpoints or shards under %s, or "
                         "lower --output-budget-mb knowingly, or shrink the model." % (
                             human_bytes(projected), human_bytes(budget), human_bytes(projected - budget),
                             human_bytes(used), root))


def preflight(n_params: int, optimizer: str, checkpoint_dir: str, output_budget_mb: int, ram_budget: int,
              plan_total: int = 0, plan_already_allocated: int = 0, world: int = 1, on_cuda: bool = False,
              pretrained: str = "", probe: Optional[Probe] = None, main: bool = True) -> None:
    """All guards in the reference's order.  ``plan_total`` = 0 skips the device-memory guard (CPU engine).  Disk and
    quota are the main rank's business (it alone writes); memory guards run on every rank."""
    probe = probe or Probe()
    per = snapshot_bytes(n_params, optimizer)
    if plan_total > 0:
        check_device_memory(plan_total, plan_already_allocated, world, probe, on_cuda)
    if main:
        check_host_ram(per, ram_budget, probe)
        check_disk(checkpoint_dir, per, probe)
        check_output_quota(output_budget_mb, checkpoint_dir, per, n_params, probe, pretrained)
