"""Model hyper-parameters, validation, parameter table and initialisation order.

Field names, defaults, accepted ranges, the ``arch_identity`` string and the parameter
names/shapes/order are the reference engine's (model/model.h:12-58, model/model.cpp:280-498,
544-608, 775-833) so recipes, checkpoints and exported files are interchangeable.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, fields
from typing import List, Optional, Tuple

import numpy as np

from ..utils.config import Config

_F32 = np.float32


def _f32(x) -> float:
    return float(np.float32(x))


@dataclass
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    decay: bool          # weight decay applies (2-D matrices except embeddings)
    init: str            # "normal", "normal_res", "router", "ones"

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


@dataclass
class ModelConfig:
    vocab_size: int = 16000
    hidden_size: int = 768
    num_layers: int = 26
    num_heads: int = 12
    num_kv_heads: int = 4
    intermediate_size: int = 2240
    max_seq_len: int = 4096
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5
    tie_embeddings: bool = True
    init_std: float = 0.02
    use_moe: bool = True
    num_experts: int = 8
    moe_top_k: int = 2
    moe_expert_dim: int = 768
    moe_shared: bool = True
    moe_aux_scale: float = 0.01
    moe_jitter: float = 0.0
    moe_allow_dense: bool = False
    use_qk_norm: bool = False
    z_loss_scale: float = 0.0
    rope_scale: float = 1.0
    rope_yarn_mscale: float = 0.0
    moe_aux_free: bool = False
    rope_yarn_low: float = 1.0
    rope_yarn_high: float = 32.0
    sliding_window: int = 0
    rope_type: int = 0

    def __post_init__(self):
        # every float field is a C float in files and identity strings
        for f in fields(self):
            if f.type in ("float", float):
                setattr(self, f.name, _f32(getattr(self, f.name)))

    # ------------------------------------------------------------------ derived sizes
    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    # ------------------------------------------------------------------ validation
    def validate(self) -> None:
        def chk(cond, msg):
            if not cond:
                raise ValueError(msg)

        fin = math.isfinite
        chk(self.vocab_size > 0, "vocab_size must be > 0")
        chk(self.hidden_size > 0, "hidden_size must be > 0")
        chk(self.num_layers > 0, "num_layers must be > 0")
        chk(self.num_heads > 0, "num_heads must be > 0")
        chk(self.num_kv_heads > 0, "num_kv_heads must be > 0")
        chk(self.hidden_size % self.num_heads == 0, "hidden_size must be divisible by num_heads")
        chk(self.num_heads % self.num_kv_heads == 0, "num_heads must be divisible by num_kv_heads")
        chk(self.head_dim % 2 == 0, "head_dim must be even (RoPE pairs)")
        chk(self.intermediate_size > 0, "intermediate_size must be > 0")
        chk(0 < self.max_seq_len <= 65536, "max_seq_len must be in (0, 65536]")
        chk(fin(self.rope_theta) and self.rope_theta > 0, "rope_theta must be finite and > 0")
        chk(fin(self.rms_eps) and _f32(1e-12) <= self.rms_eps <= _f32(1e-2), "rms_eps must be finite and in [1e-12,1e-2]")
        chk(fin(self.init_std) and 0 < self.init_std <= _f32(0.1), "init_std must be finite and in (0,0.1]")
        chk(fin(self.rope_scale) and 1.0 <= self.rope_scale <= 8.0, "rope_scale must be finite and in [1,8]")
        chk(fin(self.z_loss_scale) and 0 <= self.z_loss_scale <= _f32(0.01), "z_loss_scale must be finite and in [0,0.01]")
        chk(fin(self.moe_jitter) and 0 <= self.moe_jitter <= 0.5, "moe_jitter must be finite and in [0,0.5]")
        chk(fin(self.rope_yarn_mscale) and 0 <= self.rope_yarn_mscale <= 2.0, "rope_yarn_mscale must be finite and in [0,2]")
        chk(fin(self.rope_yarn_low) and 1.0 <= self.rope_yarn_low <= 128.0, "rope_yarn_low must be finite and in [1,128]")
        chk(fin(self.rope_yarn_high) and 1.0 <= self.rope_yarn_high <= 128.0, "rope_yarn_high must be finite and in [1,128]")
        chk(self.rope_yarn_high >= self.rope_yarn_low, "rope_yarn_high must be >= rope_yarn_low")
        chk(0 <= self.sliding_window <= 16384, "sliding_window must be in [0,16384]")
        chk(self.rope_type in (0, 1), "rope_type must be 0 (interleaved) or 1 (neox)")
        chk(not (self.moe_aux_free and self.moe_aux_scale != 0.0),
            "moe_aux_free=true requires moe_aux_scale: 0.0 (aux-loss-free has no aux grad)")
        if self.use_moe:
            chk(0 < self.num_experts <= 64, "num_experts must be in [1,64]")
            chk(0 < self.moe_top_k <= self.num_experts, "moe_top_k must be in [1,num_experts]")
            chk(self.moe_top_k <= 8, "moe_top_k must be <= 8 (router kernel limit)")
            chk(self.moe_allow_dense or self.moe_top_k * 2 <= self.num_experts,
                "moe_top_k must be <= num_experts/2 (sparse MoE); set model.moe_allow_dense=true to override")
            chk(self.moe_expert_dim > 0, "moe_expert_dim must be > 0")
            chk(fin(self.moe_aux_scale) and 0 <= self.moe_aux_scale <= 1.0, "moe_aux_scale must be finite and in [0,1]")
        # Attention tiles keep one head row in registers / tensor memory; 256 is the widest head supported.
        chk(self.head_dim <= 256, f"head_dim={self.head_dim} too large for the attention kernels (max 256)")

    @classmethod
    def from_config(cls, c: Config, prefix: str = "model") -> "ModelConfig":
        m = cls()
        key = (lambda k: f"{prefix}.{k}") if prefix else (lambda k: k)

        def pos_int(k, allow_zero=False):
            v = c.get_int(key(k), getattr(m, k))
            lo = 0 if allow_zero else 1
            if not (lo <= v <= 2 ** 31 - 1):
                raise ValueError(f"model.{k} out of int range")
            return int(v)

        for k in ("vocab_size", "hidden_size", "num_layers", "num_heads", "num_kv_heads", "intermediate_size",
                  "max_seq_len", "num_experts", "moe_top_k", "moe_expert_dim"):
            setattr(m, k, pos_int(k))
        for k in ("sliding_window", "rope_type"):
            setattr(m, k, pos_int(k, allow_zero=True))
        for k in ("rope_theta", "rms_eps", "init_std", "moe_aux_scale", "moe_jitter", "rope_yarn_low", "rope_yarn_high",
                  "z_loss_scale", "rope_scale", "rope_yarn_mscale"):
            setattr(m, k, _f32(c.get_float(key(k), getattr(m, k))))
        for k in ("tie_embeddings", "use_moe", "moe_shared", "moe_allow_dense", "moe_aux_free", "use_qk_norm"):
            setattr(m, k, c.get_bool(key(k), getattr(m, k)))
        m.validate()
        return m

    # ------------------------------------------------------------------ RoPE scaling
    def rope_theta_eff(self) -> float:
        """NTK-style base stretch: theta * s^(hd/(hd-2)) when rope_scale > 1 (float32 arithmetic)."""
        if self.rope_scale <= 1.0:
            return self.rope_theta
        hd = _F32(self.head_dim)
        e = hd / (hd - _F32(2.0)) if hd > 2 else _F32(1.0)
        return float(_F32(self.rope_theta) * np.power(_F32(self.rope_scale), e, dtype=_F32))

    def rope_mscale(self) -> float:
        if self.rope_scale <= 1.0:
            return 1.0
        if self.rope_yarn_mscale > 0.0:
            return self.rope_yarn_mscale
        base = _F32(0.1) * np.log(_F32(self.rope_scale)) + _F32(1.0)
        if self.rope_yarn_low <= 1.0 and self.rope_yarn_high >= 32.0:
            return float(base)
        span = _F32(self.rope_yarn_high) - _F32(self.rope_yarn_low)
        ramp = (_F32(32.0) - _F32(self.rope_yarn_low)) / span if span > 0 else _F32(1.0)
        ramp = min(max(float(ramp), 0.0), 1.0)
        return float(_F32(1.0) + (base - _F32(1.0)) * (_F32(0.5) + _F32(0.5) * _F32(ramp)))

    def rope_inv_freq(self) -> np.ndarray:
        """Per-pair rotation frequencies with the YaRN wavelength ramp (model/model.cpp:503-525)."""
        half = self.head_dim // 2
        theta = _F32(self.rope_theta_eff())
        out = np.zeros(half, dtype=_F32)
        for i in range(half):
            base = _F32(1.0) / np.power(theta, _F32(2.0 * i) / _F32(self.head_dim), dtype=_F32)
            if self.rope_scale > 1.0:
                wavelength = _F32(2.0) * _F32(3.14159265358979) / base
                if wavelength > self.rope_yarn_high:
                    base = base / _F32(self.rope_scale)
                elif wavelength > self.rope_yarn_low:
                    span = _F32(self.rope_yarn_high) - _F32(self.rope_yarn_low)
                    t = (wavelength - _F32(self.rope_yarn_low)) / span if span > 0 else _F32(1.0)
                    base = base * (_F32(1.0) - t + t / _F32(self.rope_scale))
            out[i] = base
        return out

    def attn_scale(self) -> float:
        return float(self.head_dim) ** -0.5 * self.rope_mscale()

    # ------------------------------------------------------------------ identity
    def summary(self) -> str:
        s = (f"vocab={self.vocab_size} d={self.hidden_size} L={self.num_layers} H={self.num_heads} "
             f"KV={self.num_kv_heads} hd={self.head_dim} ctx={self.max_seq_len} rope={self.rope_theta:g}")
        if self.rope_scale > 1.0:
            s += "(x%.1f NTK->%.0f)" % (self.rope_scale, self.rope_theta_eff())
        s += " tied" if self.tie_embeddings else " untied"
        if self.use_qk_norm:
            s += " QK-Norm"
        if self.z_loss_scale > 0:
            s += " Z(%.0e)" % self.z_loss_scale
        if self.rope_scale > 1.0:
            s += " YaRN-m%.2f" % self.rope_mscale()
        if self.moe_jitter > 0:
            s += " jit=%.2f" % self.moe_jitter
        if self.use_moe:
            s += (f" MoE(ne={self.num_experts},k={self.moe_top_k},E={self.moe_expert_dim}"
                  f"{',shared' if self.moe_shared else ''}{',aux-free' if self.moe_aux_free else ''}"
                  f"{',dense-ok' if self.moe_allow_dense else ''})")
        else:
            s += f" ffn={self.intermediate_size} (dense)"
        if self.sliding_window > 0:
            s += f" SWA({self.sliding_window})"
        if self.rope_type == 1:
            s += " RoPE-neox"
        return s

    def arch_identity(self) -> str:
        b = lambda v: 1 if v else 0
        return (f"v1|voc={self.vocab_size}|d={self.hidden_size}|L={self.num_layers}|H={self.num_heads}"
                f"|KV={self.num_kv_heads}|ffn={self.intermediate_size}|ctx={self.max_seq_len}"
                f"|theta={self.rope_theta:.6f}|eps={self.rms_eps:.9f}|tie={b(self.tie_embeddings)}"
                f"|moe={b(self.use_moe)}|ne={self.num_experts}|k={self.moe_top_k}|E={self.moe_expert_dim}"
                f"|sh={b(self.moe_shared)}|aux={self.moe_aux_scale:.6f}|auxfree={b(self.moe_aux_free)}"
                f"|denseok={b(self.moe_allow_dense)}|jit={self.moe_jitter:.6f}|qkn={b(self.use_qk_norm)}"
                f"|z={self.z_loss_scale:.7f}|rs={self.rope_scale:.4f}|ym={self.rope_yarn_mscale:.4f}"
                f"|yl={self.rope_yarn_low:.4f}|yh={self.rope_yarn_high:.4f}|swa={self.sliding_window}|rt={self.rope_type}")

    _ARCH_FIELDS = ("vocab_size", "hidden_size", "num_layers", "num_heads", "num_kv_heads", "intermediate_size",
                    "max_seq_len", "rope_theta", "rms_eps", "tie_embeddings", "use_moe", "num_experts", "moe_top_k",
                    "moe_expert_dim", "moe_shared", "moe_aux_scale", "moe_aux_free", "moe_allow_dense", "moe_jitter",
                    "use_qk_norm", "z_loss_scale", "rope_scale", "rope_yarn_mscale", "rope_yarn_low", "rope_yarn_high",
                    "sliding_window", "rope_type")

    def same_architecture_as(self, o: "ModelConfig") -> Tuple[bool, Optional[str]]:
        for k in self._ARCH_FIELDS:
            if getattr(self, k) != getattr(o, k):
                return False, f"arch mismatch: {k}"
        return True, None

    # ------------------------------------------------------------------ parameter table
    def param_specs(self) -> List[ParamSpec]:
        """Parameters in file/table order (model/model.cpp:562-603)."""
        d, V, qd, kvd = self.hidden_size, self.vocab_size, self.q_dim, self.kv_dim
        F, E, ne, hd = self.intermediate_size, self.moe_expert_dim, self.num_experts, self.head_dim
        out = [ParamSpec("tok_embeddings", (V, d), False, "normal")]
        for i in range(self.num_layers):
            p = f"layers.{i}."
            out += [ParamSpec(p + "attn_norm", (d,), False, "ones"),
                    ParamSpec(p + "wq", (qd, d), True, "normal"),
                    ParamSpec(p + "wk", (kvd, d), True, "normal"),
                    ParamSpec(p + "wv", (kvd, d), True, "normal"),
                    ParamSpec(p + "wo", (d, qd), True, "normal_res"),
                    ParamSpec(p + "ffn_norm", (d,), False, "ones")]
            if self.use_qk_norm:
                out += [ParamSpec(p + "qk_qnorm", (hd,), False, "ones"), ParamSpec(p + "qk_knorm", (hd,), False, "ones")]
            if self.use_moe:
                out += [ParamSpec(p + "moe_router", (ne, d), True, "router"),
                        ParamSpec(p + "moe_gate", (ne * E, d), True, "normal"),
                        ParamSpec(p + "moe_up", (ne * E, d), True, "normal"),
                        ParamSpec(p + "moe_down", (ne * d, E), True, "normal_res")]
                if self.moe_shared:
                    out += [ParamSpec(p + "moe_sh_gate", (E, d), True, "normal"),
                            ParamSpec(p + "moe_sh_up", (E, d), True, "normal"),
                            ParamSpec(p + "moe_sh_down", (d, E), True, "normal_res")]
            else:
                out += [ParamSpec(p + "w_gate", (F, d), True, "normal"),
                        ParamSpec(p + "w_up", (F, d), True, "normal"),
                        ParamSpec(p + "w_down", (d, F), True, "normal_res")]
        out.append(ParamSpec("final_norm", (d,), False, "ones"))
        if not self.tie_embeddings:
            out.append(ParamSpec("lm_head", (V, d), True, "normal"))
        return out

    def init_order(self) -> List[str]:
        """Names in the order the initialiser consumes the random stream (model/model.cpp:775-833):
        embeddings, untied head, then per layer the matrices; norm vectors are ones and draw nothing."""
        names = ["tok_embeddings"]
        if not self.tie_embeddings:
            names.append("lm_head")
        for i in range(self.num_layers):
            p = f"layers.{i}."
            names += [p + "wq", p + "wk", p + "wv", p + "wo"]
            if self.use_moe:
                names += [p + "moe_router", p + "moe_gate", p + "moe_up", p + "moe_down"]
                if self.moe_shared:
                    names += [p + "moe_sh_gate", p + "moe_sh_up", p + "moe_sh_down"]
            else:
                names += [p + "w_gate", p + "w_up", p + "w_down"]
        return names

    def count_parameters(self) -> int:
        return sum(p.numel for p in self.param_specs())

    def active_parameters_per_token(self) -> int:
        """Parameters touched by one token (top-k experts + shared expert instead of all experts)."""
        total = 0
        for p in self.param_specs():
            base = p.name.split(".")[-1]
            if base in ("moe_gate", "moe_up", "moe_down"):
                total += p.numel // self.num_experts * self.moe_top_k
            else:
                total += p.numel
        return total


def init_parameters(cfg: ModelConfig, seed: int) -> dict:
    """Bit-exact initial weights as ``{name: float32 ndarray}``.

    One stream seeded with ``seed``; every matrix element is a truncated normal (two sigma, polar
    Box-Muller with the spare variate carried across tensors); residual-output matrices use
    ``std / sqrt(2 L)``, the router ``min(std, 0.01)``; norm weights are ones.
    """
    from .. import _gb200_host as H

    specs = {p.name: p for p in cfg.param_specs()}
    out = {name: None for name in specs}
    rng = H.Rng(seed)
    std = _F32(cfg.init_std)
    std_res = _F32(std / np.sqrt(_F32(2.0) * _F32(cfg.num_layers), dtype=_F32))
    for name in cfg.init_order():
        p = specs[name]
        sd = {"normal": std, "normal_res": std_res, "router": min(std, _F32(0.01))}[p.init]
        flat = np.empty(p.numel, dtype=np.float32)
        rng.fill_truncated_normal(flat, float(sd))
        out[name] = flat.reshape(p.shape)
    for name, p in specs.items():
        if p.init == "ones":
            out[name] = np.ones(p.shape, dtype=np.float32)
    return out
