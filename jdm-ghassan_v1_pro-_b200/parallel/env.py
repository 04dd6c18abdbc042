"""Rank / world / rendezvous discovery from the process environment.

Order of precedence, as in the reference's DistributedContext (training/distributed.cpp:333-368): explicit
``WORLD_SIZE``/``RANK``/``LOCAL_RANK`` (what this package's launcher and torchrun export), then the SLURM variables
(``SLURM_NTASKS``, ``SLURM_PROCID``, ``SLURM_LOCALID``), else a single process.  ``MASTER_ADDR`` defaults to
127.0.0.1 (a container's host name need not resolve) and ``MASTER_PORT`` to 29500.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Mapping, Optional


class EnvError(ValueError):
    pass


@dataclass
class RankEnv:
    rank: int = 0
    world: int = 1
    local_rank: int = 0
    master_addr: str = "127.0.0.1"
    master_port: int = 29500
    source: str = "single"

    @property
    def distributed(self) -> bool:
        return self.world > 1

    def init_method(self) -> str:
        return "tcp://%s:%d" % (self.master_addr, self.master_port)


def _int(env: Mapping[str, str], key: str) -> Optional[int]:
    v = env.get(key)
    if v is None or v == "":
        return None
    try:
        return int(v)
    except ValueError:
        raise EnvError("%s=%r is not an integer" % (key, v))


def parse_env(env: Optional[Mapping[str, str]] = None) -> RankEnv:
    env = os.environ if env is None else env
    out = RankEnv()
    world, rank, local = _int(env, "WORLD_SIZE"), _int(env, "RANK"), _int(env, "LOCAL_RANK")
    if world is not None:
        out.source = "env"
    else:
        world, rank, local = _int(env, "SLURM_NTASKS"), _int(env, "SLURM_PROCID"), _int(env, "SLURM_LOCALID")
        if world is not None:
            out.source = "slurm"
    if world is not None:
        out.world = world
        out.rank = rank if rank is not None else 0
        out.local_rank = local if local is not None else out.rank
    if out.world < 1 or not (0 <= out.rank < out.world) or out.local_rank < 0:
        raise EnvError("inconsistent rank environment: world=%d rank=%d local_rank=%d" % (out.world, out.rank, out.local_rank))
    out.master_addr = env.get("MASTER_ADDR") or "127.0.0.1"
    port = _int(env, "MASTER_PORT")
    out.master_port = 29500 if port is None else port
    if not (0 < out.master_port < 65536):
        raise EnvError("MASTER_PORT=%d is out of range" % out.master_port)
    return out


def init_process_group(backend: Optional[str] = None, timeout_s: float = 600.0, env: Optional[Mapping[str, str]] = None) -> RankEnv:
    """Join the job's process group (NCCL when CUDA is present, else gloo) and bind this rank's GPU.  The timeout
    bounds every collective: a peer that died surfaces as an error on the survivors instead of a hang
    (the reference exports NCCL_COMM_WATCHDOG_TIMEOUT=600 for the same purpose, configs/kaggle/train_2xt4.sh:118)."""
    import datetime
    import torch
    import torch.distributed as dist
    e = parse_env(env)
    if not e.distributed or dist.is_initialized():
        return e
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(e.local_rank % max(1, torch.cuda.device_count()))
    dist.init_process_group(backend, init_method=e.init_method(), rank=e.rank, world_size=e.world,
                            timeout=datetime.timedelta(seconds=timeout_s))
    return e
