"""Load a model for inference from any of the supported files (GGUF, legacy .gai, training checkpoint) and build an
:class:`InferenceEngine` from it (tools/inference_cli.cpp:120-260 in the reference does the same dispatch)."""
from __future__ import annotations

import os
from typing import Optional

import numpy as np

from ..data.tokenizer import Tokenizer
from ..formats import gai as GAI
from ..formats import gguf as GGUF
from ..formats.gguf import LoadedModel


def sniff(path: str) -> str:
    with open(path, "rb") as f:
        magic = f.read(4)
    return {b"GGUF": "gguf", b"GAI1": "gai", b"GKPT": "ckpt"}.get(magic, "unknown")


def load_model(path: str, tokenizer_path: str = "") -> LoadedModel:
    kind = sniff(path)
    if kind == "gguf":
        m = GGUF.load_gguf(path)
    elif kind == "gai":
        m = GAI.load_gai(path)
    elif kind == "ckpt":
        from ..training import checkpoint as C
        d = C.read(path, with_optimizer=False)
        cfg = C.config_from_dict(d["config"])
        specs = {s.name: s for s in cfg.param_specs()}
        named = {n: np.asarray(a).reshape(specs[n].shape) for n, a in d["params"]}
        m = LoadedModel(cfg, named, [np.asarray(b) for b in d["moe_bias"]], None, {"steps": str(d["state"]["step"])}, {}, None)
    else:
        raise ValueError(f"not a valid model file: {path} (expected .gguf, legacy .gai or a .ckpt)")
    if tokenizer_path:
        m.tokenizer = Tokenizer.load(tokenizer_path)
    return m


def quant_name(m: LoadedModel) -> str:
    md = m.metadata
    for k in ("ghassan.quantization.profile", "quant_profile"):
        v = md.get(k)
        if v:
            return v.decode() if isinstance(v, (bytes, bytearray)) else str(v)
    return "fp32"


def build_engine(m: LoadedModel, batch: int = 1, max_len: int = 2048, fmt: str = "auto", prefill_chunk: int = 1024):
    """Engine whose decode weights keep the file's storage format where the kernels read it directly; on a host without
    a CUDA device the fp32 CPU engine (`cpu_engine.CpuEngine`) over the expanded weights."""
    import torch
    if not torch.cuda.is_available():
        from .cpu_engine import CpuEngine
        return CpuEngine(m.cfg, m.named, batch=batch, max_len=min(max_len, max(64, m.cfg.max_seq_len)), moe_bias=m.moe_bias or None)
    from .engine import InferenceEngine
    raw = m.raw if (m.raw is not None and hasattr(m.raw, "tensor_raw")) else None
    if fmt == "auto" and raw is None:
        fmt = {"int8": "q8_64", "int4": "q4_0"}.get(quant_name(m), "f16")      # .gai block formats
    return InferenceEngine(m.cfg, m.named, fmt=fmt, batch=batch, max_len=min(max_len, max(64, m.cfg.max_seq_len)),
                           prefill_chunk=min(prefill_chunk, max_len), moe_bias=m.moe_bias or None, raw=raw,
                           raw_types=m.tensor_types if raw is not None else None)
