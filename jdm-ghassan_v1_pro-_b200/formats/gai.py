"""Legacy ``.gai`` model files and ``GRAW`` weight dumps (format/legacy_gai_format.cpp:28-162, 405-467 and
model/model.cpp:1696-1798 in the reference): text ``key=value`` header, tensor directory, embedded tokenizer image,
64-byte aligned payloads in the internal block formats.  Reading goes through a read-only memory map."""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np

from .. import _gb200_host as H
from ..data.tokenizer import Tokenizer
from ..models.config import ModelConfig
from .gguf import LoadedModel

PROFILES = {            # name -> (default, embedding, norm)
    "fp32": ("f32", "f32", "f32"),
    "fp16": ("f16", "f16", "f32"),
    "int8": ("q8_0", "q8_0", "f32"),
    "int4": ("q4_0", "q8_0", "f32"),
}


def _f32(x) -> float:
    return float(np.float32(x))


def config_meta(c: ModelConfig) -> Dict[str, str]:
    b = lambda v: "1" if v else "0"
    return {
        "arch": "ghassan", "model_name": "Ghassan v1 Flash",
        "vocab_size": str(c.vocab_size), "hidden_size": str(c.hidden_size), "num_layers": str(c.num_layers),
        "num_heads": str(c.num_heads), "num_kv_heads": str(c.num_kv_heads), "intermediate_size": str(c.intermediate_size),
        "use_moe": b(c.use_moe), "num_experts": str(c.num_experts), "moe_top_k": str(c.moe_top_k),
        "moe_expert_dim": str(c.moe_expert_dim), "moe_shared": b(c.moe_shared),
        "moe_aux_scale": "%.6f" % _f32(c.moe_aux_scale), "moe_jitter": "%.6f" % _f32(c.moe_jitter),
        "max_seq_len": str(c.max_seq_len), "rope_theta": "%.6f" % _f32(c.rope_theta), "rope_scale": "%.6f" % _f32(c.rope_scale),
        "rope_yarn_mscale": "%.6f" % _f32(c.rope_yarn_mscale), "rope_yarn_low": "%.6f" % _f32(c.rope_yarn_low),
        "rope_yarn_high": "%.6f" % _f32(c.rope_yarn_high), "sliding_window": str(c.sliding_window),
        "rope_type": str(c.rope_type), "moe_aux_free": b(c.moe_aux_free), "rms_eps": "%.9f" % _f32(c.rms_eps),
        "use_qk_norm": b(c.use_qk_norm), "z_loss_scale": "%.9f" % _f32(c.z_loss_scale),
        "tie_embeddings": b(c.tie_embeddings), "norm_type": "rmsnorm",
        "ffn_type": "swiglu_moe" if c.use_moe else "swiglu", "pos_type": "rope", "attn_type": "gqa_causal",
    }


def export_gai(path: str, cfg: ModelConfig, named: Dict[str, np.ndarray], tokenizer_path: str = "",
               profile: str = "fp16", extra_meta: Optional[Dict[str, str]] = None) -> dict:
    if profile not in PROFILES:
        raise ValueError(f"unknown quantization profile: {profile} (fp32|fp16|int8|int4)")
    default, emb, norm = PROFILES[profile]
    w = H.GaiWriter()
    for k, v in config_meta(cfg).items():
        w.set_meta(k, v)
    w.set_meta("quant_profile", profile)
    w.set_meta("default_dtype", default)
    w.set_meta("embedding_dtype", emb)
    w.set_meta("norm_dtype", norm)
    w.set_meta("param_count", str(cfg.count_parameters()))
    for k, v in (extra_meta or {}).items():
        w.set_meta(k, v)
    if tokenizer_path:
        w.set_tokenizer_blob(open(tokenizer_path, "rb").read())
    for spec in cfg.param_specs():
        dt = norm if "norm" in spec.name else emb if spec.name in ("tok_embeddings", "lm_head") else default
        w.add_tensor(spec.name, np.ascontiguousarray(np.asarray(named[spec.name], dtype=np.float32).reshape(spec.shape)), dt)
    w.write(path)
    return {"path": path, "profile": profile, "tensors": w.tensor_count}


def config_from_meta(md: Dict[str, str]) -> ModelConfig:
    d = ModelConfig.__dataclass_fields__
    gi = lambda k, dv: int(md.get(k, dv))
    gf = lambda k, dv: float(md.get(k, dv))
    gb = lambda k, dv: int(md.get(k, 1 if dv else 0)) != 0
    c = ModelConfig(
        vocab_size=gi("vocab_size", d["vocab_size"].default), hidden_size=gi("hidden_size", d["hidden_size"].default),
        num_layers=gi("num_layers", d["num_layers"].default), num_heads=gi("num_heads", d["num_heads"].default),
        num_kv_heads=gi("num_kv_heads", d["num_kv_heads"].default),
        intermediate_size=gi("intermediate_size", d["intermediate_size"].default),
        use_moe=gb("use_moe", False), num_experts=gi("num_experts", 0), moe_top_k=gi("moe_top_k", 0),
        moe_expert_dim=gi("moe_expert_dim", 0), moe_shared=gb("moe_shared", False),
        moe_aux_scale=gf("moe_aux_scale", 0.0), moe_jitter=gf("moe_jitter", 0.0),
        max_seq_len=gi("max_seq_len", d["max_seq_len"].default), rope_theta=gf("rope_theta", 10000.0),
        rope_scale=gf("rope_scale", 1.0), rope_yarn_mscale=gf("rope_yarn_mscale", 0.0), rope_yarn_low=gf("rope_yarn_low", 1.0),
        rope_yarn_high=gf("rope_yarn_high", 32.0), sliding_window=gi("sliding_window", 0), rope_type=gi("rope_type", 0),
        moe_aux_free=gb("moe_aux_free", False), rms_eps=gf("rms_eps", 1e-5), use_qk_norm=gb("use_qk_norm", False),
        z_loss_scale=gf("z_loss_scale", 0.0), tie_embeddings=gb("tie_embeddings", True))
    if c.use_moe and c.moe_top_k * 2 > c.num_experts:
        c.moe_allow_dense = True
    c.validate()
    return c


def load_gai(path: str, dequantize: bool = True) -> LoadedModel:
    f = H.GaiFile(path)
    md = dict(f.meta)
    cfg = config_from_meta(md)
    types = {t["name"]: int(t["dtype"]) for t in f.tensors}
    named = {}
    for spec in cfg.param_specs():
        if spec.name not in types:
            raise ValueError(f"model file is missing tensor: {spec.name}")
        if dequantize:
            arr = np.asarray(f.tensor_f32(spec.name))
            if arr.size != spec.numel:
                raise ValueError(f"tensor {spec.name} size mismatch: file {arr.size} vs model {spec.numel}")
            named[spec.name] = arr.reshape(spec.shape)
    blob = bytes(f.tokenizer_blob)
    tok = Tokenizer.from_bytes(blob) if blob else None
    return LoadedModel(cfg, named, [], tok, md, types, f)


def save_raw(path: str, cfg: ModelConfig, named: Dict[str, np.ndarray]) -> None:
    H.write_graw(path, [(s.name, np.ascontiguousarray(np.asarray(named[s.name], dtype=np.float32).reshape(s.shape)))
                        for s in cfg.param_specs()])


def load_raw(path: str, cfg: ModelConfig) -> Dict[str, np.ndarray]:
    got = {n: a for n, a in H.read_graw(path)}
    out = {}
    for s in cfg.param_specs():
        if s.name not in got:
            raise ValueError(f"[raw] missing tensor {s.name}")
        if tuple(got[s.name].shape) != tuple(s.shape):
            raise ValueError(f"[raw] shape mismatch for {s.name}: {tuple(got[s.name].shape)} vs {tuple(s.shape)}")
        out[s.name] = np.asarray(got[s.name])
    return out
