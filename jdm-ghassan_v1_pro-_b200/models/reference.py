"""Plain-PyTorch fp32 implementation of the model: the CPU path and the oracle for every CUDA kernel.

It restates the reference engine's CPU math (core/ops_cpu_dense.cpp, core/ops_cpu_moe.cpp,
model/model.cpp:1248-1694) with autograd doing the backward pass: sum-of-token losses, z-loss,
router jitter hash, bias-on-selection top-k with lowest-index tie break, renormalised combine weights,
auxiliary balance loss whose gradient flows only through the mean router probabilities, packed
sequences masked by segment id with RoPE positions that are *not* reset per document.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .config import ModelConfig, init_parameters

_M64 = (1 << 64) - 1


def jitter_u(t: np.ndarray, e: np.ndarray, seed: int) -> np.ndarray:
    """Uniform in [-0.5, 0.5) from a 64-bit mix of (row, expert, seed) (core/ops_cpu_moe.cpp:23-33)."""
    with np.errstate(over="ignore"):
        h = t.astype(np.uint64) * np.uint64(0x9E3779B97F4A7C15)
        h ^= e.astype(np.uint64) * np.uint64(0xC2B2AE3D27D4EB4F)
        h ^= np.uint64((seed + 0x9E3779B97F4A7C15) & _M64)
        h ^= h >> np.uint64(33)
        h *= np.uint64(0xFF51AFD7ED558CCD)
        h ^= h >> np.uint64(33)
        h *= np.uint64(0xC4CEB9FE1A85EC53)
        h ^= h >> np.uint64(33)
    return ((h >> np.uint64(40)) & np.uint64(0xFFFFFF)).astype(np.float32) / np.float32(1 << 24) - np.float32(0.5)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    inv = torch.rsqrt(x.double().pow(2).mean(-1, keepdim=True) + eps).to(x.dtype)
    inv = torch.where(torch.isfinite(inv), inv, torch.zeros_like(inv))
    return x * inv * w


def rope(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, rope_type: int) -> torch.Tensor:
    """x: [N, heads, hd]; pos: [N] row positions; type 0 rotates (2i, 2i+1), type 1 rotates (i, i+hd/2)."""
    ang = (pos.double()[:, None] * inv_freq.double()[None, :]).float()
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    if rope_type == 0:
        a, b = x[..., 0::2], x[..., 1::2]
        return torch.stack([a * c - b * s, a * s + b * c], dim=-1).flatten(-2)
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def attention(q, k, v, B, T, scale, window=0, segment_ids=None):
    """q: [B*T, H, hd], k/v: [B*T, KV, hd]; causal with optional sliding window and segment mask."""
    H, KV, hd = q.shape[1], k.shape[1], q.shape[2]
    g = H // KV
    qh = q.view(B, T, H, hd).permute(0, 2, 1, 3)
    kh = k.view(B, T, KV, hd).permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vh = v.view(B, T, KV, hd).permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = (qh @ kh.transpose(-1, -2)) * scale
    i = torch.arange(T, device=q.device)
    keep = i[None, :] <= i[:, None]
    if window and window > 0:
        keep = keep & (i[None, :] > i[:, None] - window)
    keep = keep[None, None]
    if segment_ids is not None:
        seg = segment_ids.view(B, T)
        same = (seg[:, :, None] == seg[:, None, :]) | (seg[:, :, None] < 0)
        keep = keep & same[:, None]
    s = s.masked_fill(~keep, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)  # a row with every key masked produces zeros
    o = p @ vh
    return o.permute(0, 2, 1, 3).reshape(B * T, H * hd)


def swiglu_ffn(x, wg, wu, wd):
    return (torch.nn.functional.silu(x @ wg.t()) * (x @ wu.t())) @ wd.t()


def route(xb, router_w, bias, cfg: ModelConfig, jitter_seed: Optional[int]):
    """Returns (probs [N,ne], idx [N,K] int64, w [N,K]).  ``jitter_seed`` None = evaluation (no jitter)."""
    N, ne, K = xb.shape[0], cfg.num_experts, cfg.moe_top_k
    logits = xb @ router_w.t()
    if cfg.moe_jitter > 0 and jitter_seed is not None:
        tt, ee = np.meshgrid(np.arange(N), np.arange(ne), indexing="ij")
        u = torch.from_numpy(jitter_u(tt, ee, jitter_seed)).to(logits.device)
        logits = logits * (1.0 + 2.0 * cfg.moe_jitter * u)
    probs = torch.softmax(logits, dim=-1)
    sel = probs.detach().clone()
    if bias is not None:
        sel = sel + bias
    idx = []
    for _ in range(K):  # repeated arg-max; argmax returns the lowest index among ties
        j = torch.argmax(sel, dim=-1)
        idx.append(j)
        sel.scatter_(1, j[:, None], float("-inf"))
    idx = torch.stack(idx, dim=1)
    psel = probs.gather(1, idx)
    ssum = psel.sum(-1, keepdim=True)
    w = torch.where(ssum > 1e-8, psel / ssum.clamp_min(1e-30), torch.zeros_like(psel))
    return probs, idx, w


@dataclass
class ForwardResult:
    loss_sum: torch.Tensor          # sum over supervised rows of CE (+ z-loss), unscaled
    ntok: int
    aux_raw: List[torch.Tensor]     # per-layer ne * sum_e m_e f_e (empty without MoE)
    slot_counts: Optional[torch.Tensor]  # [L, ne] routed slots per expert
    logits: Optional[torch.Tensor] = None

    def objective(self, cfg: ModelConfig) -> torch.Tensor:
        """Quantity whose gradient the optimizer consumes (sum form): CE_sum + ntok*aux_scale/L*sum_l raw_l."""
        obj = self.loss_sum
        if cfg.use_moe and cfg.moe_aux_scale > 0 and self.aux_raw:
            obj = obj + self.ntok * cfg.moe_aux_scale / cfg.num_layers * torch.stack(self.aux_raw).sum()
        return obj

    def reported_loss(self, cfg: ModelConfig) -> float:
        if self.ntok == 0:
            return 0.0
        v = float(self.loss_sum.detach()) / self.ntok
        if cfg.use_moe and cfg.moe_aux_scale > 0 and self.aux_raw:
            v += cfg.moe_aux_scale * float(torch.stack(self.aux_raw).sum().detach()) / cfg.num_layers
        return v


class TorchModel:
    """fp32 parameters by reference name + functional forward."""

    def __init__(self, cfg: ModelConfig, device="cpu"):
        cfg.validate()
        self.cfg = cfg
        self.device = torch.device(device)
        self.specs = cfg.param_specs()
        self.params: Dict[str, torch.Tensor] = {
            p.name: torch.zeros(p.shape, dtype=torch.float32, device=self.device) for p in self.specs}
        self.inv_freq = torch.from_numpy(cfg.rope_inv_freq()).to(self.device)
        self.moe_bias: Optional[torch.Tensor] = None
        if cfg.use_moe and cfg.moe_aux_free:
            self.moe_bias = torch.zeros(cfg.num_layers, cfg.num_experts, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ parameters
    def init_weights(self, seed: int) -> None:
        for name, arr in init_parameters(self.cfg, seed).items():
            self.params[name].copy_(torch.from_numpy(arr))
        if self.moe_bias is not None:
            self.moe_bias.zero_()

    def enable_grad(self, on=True):
        for p in self.params.values():
            p.requires_grad_(on)

    def zero_grad(self):
        for p in self.params.values():
            p.grad = None

    def named_parameters(self):
        return [(s.name, self.params[s.name]) for s in self.specs]

    def load_named(self, tensors: Dict[str, np.ndarray]) -> None:
        for name, t in self.params.items():
            if name not in tensors:
                raise KeyError(f"missing parameter '{name}'")
            with torch.no_grad():
                t.copy_(torch.as_tensor(np.asarray(tensors[name], dtype=np.float32)).view_as(t))

    def export_named(self) -> Dict[str, np.ndarray]:
        return {n: p.detach().cpu().numpy() for n, p in self.named_parameters()}

    # ------------------------------------------------------------------ forward
    def hidden_states(self, ids, B, T, segment_ids=None, jitter_seed=None, pos_offset=0, collect=None):
        cfg, P = self.cfg, self.params
        N = B * T
        H, KV, hd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        pos = (torch.arange(T, device=self.device) + pos_offset).repeat(B)
        x = P["tok_embeddings"][ids.view(-1).long()]
        aux_raw, counts = [], []
        scale = cfg.attn_scale()
        for l in range(cfg.num_layers):
            pre = f"layers.{l}."
            xb = rmsnorm(x, P[pre + "attn_norm"], cfg.rms_eps)
            q = (xb @ P[pre + "wq"].t()).view(N, H, hd)
            k = (xb @ P[pre + "wk"].t()).view(N, KV, hd)
            v = (xb @ P[pre + "wv"].t()).view(N, KV, hd)
            if cfg.use_qk_norm:
                q = rmsnorm(q, P[pre + "qk_qnorm"], cfg.rms_eps)
                k = rmsnorm(k, P[pre + "qk_knorm"], cfg.rms_eps)
            q = rope(q, pos, self.inv_freq, cfg.rope_type)
            k = rope(k, pos, self.inv_freq, cfg.rope_type)
            att = attention(q, k, v, B, T, scale, cfg.sliding_window, segment_ids)
            x = x + att @ P[pre + "wo"].t()
            xb2 = rmsnorm(x, P[pre + "ffn_norm"], cfg.rms_eps)
            if cfg.use_moe:
                bias = self.moe_bias[l] if self.moe_bias is not None else None
                probs, idx, w = route(xb2, P[pre + "moe_router"], bias, cfg, jitter_seed)
                ne, K, E, d = cfg.num_experts, cfg.moe_top_k, cfg.moe_expert_dim, cfg.hidden_size
                out = torch.zeros_like(x)
                if cfg.moe_shared:
                    out = out + swiglu_ffn(xb2, P[pre + "moe_sh_gate"], P[pre + "moe_sh_up"], P[pre + "moe_sh_down"])
                gate, up, down = P[pre + "moe_gate"], P[pre + "moe_up"], P[pre + "moe_down"]
                for e in range(ne):
                    hit = (idx == e)
                    rows = hit.any(dim=1).nonzero(as_tuple=True)[0]
                    if rows.numel() == 0:
                        continue
                    we = (w * hit).sum(dim=1)[rows]
                    y = swiglu_ffn(xb2[rows], gate[e * E:(e + 1) * E], up[e * E:(e + 1) * E], down[e * d:(e + 1) * d])
                    out = out.index_add(0, rows, y * we[:, None])
                cnt = torch.bincount(idx.reshape(-1), minlength=ne).float()
                counts.append(cnt)
                f = (cnt / float(N * K)).detach()
                m = probs.mean(dim=0)
                aux_raw.append(ne * (m * f).sum())
                if collect is not None:
                    collect.setdefault("route", []).append((probs.detach(), idx, w.detach()))
                x = x + out
            else:
                x = x + swiglu_ffn(xb2, P[pre + "w_gate"], P[pre + "w_up"], P[pre + "w_down"])
        h = rmsnorm(x, P["final_norm"], cfg.rms_eps)
        return h, aux_raw, (torch.stack(counts) if counts else None)

    def lm_head_weight(self):
        return self.params["tok_embeddings"] if self.cfg.tie_embeddings else self.params["lm_head"]

    def forward(self, ids, targets, B, T, segment_ids=None, jitter_seed=None, return_logits=False) -> ForwardResult:
        """ids/targets/segment_ids: int tensors of B*T elements; targets < 0 are ignored."""
        cfg = self.cfg
        h, aux_raw, counts = self.hidden_states(ids, B, T, segment_ids, jitter_seed)
        logits = h @ self.lm_head_weight().t()
        tgt = targets.view(-1).long()
        sup = tgt >= 0
        ntok = int(sup.sum())
        logz = torch.logsumexp(logits, dim=-1)
        picked = logits.gather(1, tgt.clamp_min(0)[:, None]).squeeze(1)
        per_row = logz - picked + cfg.z_loss_scale * logz * logz
        loss_sum = (per_row * sup).sum()
        return ForwardResult(loss_sum, ntok, aux_raw, counts, logits if return_logits else None)

    @torch.no_grad()
    def logits(self, ids, B, T, segment_ids=None, pos_offset=0):
        h, _, _ = self.hidden_states(ids, B, T, segment_ids, None, pos_offset)
        return h @ self.lm_head_weight().t()
