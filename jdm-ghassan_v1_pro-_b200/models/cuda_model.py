"""The model on a B200: flat parameter storage, pre-allocated activations and the explicit forward/backward
call sequence over the sm_100a kernels (no autograd, no per-step allocation, capturable in a CUDA graph).

What is computed is the reference engine's ``Model::forward_backward`` (model/model.cpp:1248-1669): embedding,
per layer {RMSNorm, fused QKV, QK-norm, RoPE, causal attention, output projection + residual, RMSNorm, MoE or
dense SwiGLU + residual}, final norm, chunked lm-head + cross-entropy with z-loss, and the matching backward
with sum-of-token-loss gradients times the loss scale.  How it is computed differs: 16-bit operands resident
in HBM (shadow weights written by the optimizer, activations produced in 16 bits by the norm kernels), fp32
residual stream and fp32 weight-gradient accumulation inside the GEMM epilogues, experts as one grouped GEMM
per projection with the shared expert as an extra always-routed group, no host synchronisation inside a step.

Internal parameter layout ("compute layout") versus the reference's named tensors:
  wqkv  = rows [wq; wk; wv]                         w_down = rows [moe_down (ne*d); moe_sh_down (d)]
  w_gu  = per expert (shared expert last) gate and up rows interleaved in blocks of 64
The mapping is a pure permutation, applied when weights, gradients or optimizer moments are imported/exported.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from ..ops import gemm as G
from ..ops import kernels as K
from ..utils import canary as CA
from .config import ModelConfig, init_parameters

ALIGN = 64  # elements; keeps every segment 16-byte aligned in both the fp32 and the 16-bit buffer


@dataclass
class Segment:
    key: str
    shape: tuple
    decay: bool
    offset: int = 0

    @property
    def numel(self):
        n = 1
        for s in self.shape:
            n *= s
        return n


class ParamLayout:
    """Flat layout: [no-decay segments | decay segments], each segment aligned to 64 elements."""

    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg
        d, V, qd, kvd, hd = cfg.hidden_size, cfg.vocab_size, cfg.q_dim, cfg.kv_dim, cfg.head_dim
        self.ne1 = (cfg.num_experts + int(cfg.moe_shared)) if cfg.use_moe else 1
        self.Eff = cfg.moe_expert_dim if cfg.use_moe else cfg.intermediate_size
        if self.Eff % 64:
            raise ValueError("expert/FFN hidden size must be a multiple of 64 for the fused SwiGLU layout")
        nd: List[Segment] = [Segment("tok_embeddings", (V, d), False), Segment("final_norm", (d,), False)]
        rt: List[Segment] = []     # routers: weight decay like the matrices, but kernels read them in fp32
        dc: List[Segment] = []
        for i in range(cfg.num_layers):
            p = f"L{i}."
            nd += [Segment(p + "attn_norm", (d,), False), Segment(p + "ffn_norm", (d,), False)]
            if cfg.use_qk_norm:
                nd += [Segment(p + "qk_qnorm", (hd,), False), Segment(p + "qk_knorm", (hd,), False)]
            dc += [Segment(p + "wqkv", (qd + 2 * kvd, d), True), Segment(p + "wo", (d, qd), True)]
            if cfg.use_moe:
                rt.append(Segment(p + "router", (cfg.num_experts, d), True))
            dc += [Segment(p + "w_gu", (self.ne1 * 2 * self.Eff, d), True),
                   Segment(p + "w_down", (self.ne1 * d, self.Eff), True)]
        if not cfg.tie_embeddings:
            dc.append(Segment("lm_head", (V, d), True))
        # [no decay | routers | matrices]: one boundary for weight decay (decay_start) and one for "read in fp32
        # by the kernels" (f32_end), so range-based kernels need no per-tensor table
        off = 0
        self.decay_start = self.f32_end = 0
        for s in nd + rt + dc:
            s.offset = off
            off += (s.numel + ALIGN - 1) // ALIGN * ALIGN
            if s is nd[-1]:
                self.decay_start = self.f32_end = off
            if rt and s is rt[-1]:
                self.f32_end = off
        self.total = off
        self.segments = {s.key: s for s in nd + rt + dc}
        self.order = [s.key for s in nd + rt + dc]

    def view(self, flat: torch.Tensor, key: str) -> torch.Tensor:
        s = self.segments[key]
        return flat[s.offset:s.offset + s.numel].view(s.shape)

    # ------------------------------------------------------------------ reference names <-> compute layout
    def to_internal(self, named: Dict[str, torch.Tensor], flat: torch.Tensor, missing_ok=False) -> List[str]:
        """Scatter reference-named fp32 tensors into ``flat``; returns the names that were absent."""
        cfg = self.cfg
        absent = []

        def get(name):
            if name not in named or named[name] is None:
                absent.append(name)
                return None
            t = named[name]
            t = torch.as_tensor(np.asarray(t)) if not isinstance(t, torch.Tensor) else t
            return t.to(device=flat.device, dtype=torch.float32)

        def put(key, t):
            if t is not None:
                self.view(flat, key).copy_(t.reshape(self.segments[key].shape))

        put("tok_embeddings", get("tok_embeddings"))
        put("final_norm", get("final_norm"))
        if not cfg.tie_embeddings:
            put("lm_head", get("lm_head"))
        E, d, ne = self.Eff, cfg.hidden_size, cfg.num_experts
        for i in range(cfg.num_layers):
            r, p = f"layers.{i}.", f"L{i}."
            put(p + "attn_norm", get(r + "attn_norm"))
            put(p + "ffn_norm", get(r + "ffn_norm"))
            if cfg.use_qk_norm:
                put(p + "qk_qnorm", get(r + "qk_qnorm"))
                put(p + "qk_knorm", get(r + "qk_knorm"))
            q, k, v = get(r + "wq"), get(r + "wk"), get(r + "wv")
            if q is not None and k is not None and v is not None:
                put(p + "wqkv", torch.cat([q, k, v], dim=0))
            put(p + "wo", get(r + "wo"))
            if cfg.use_moe:
                put(p + "router", get(r + "moe_router"))
                g, u, dn = get(r + "moe_gate"), get(r + "moe_up"), get(r + "moe_down")
                if cfg.moe_shared:
                    sg, su, sd = get(r + "moe_sh_gate"), get(r + "moe_sh_up"), get(r + "moe_sh_down")
                    if None not in (g, u, dn, sg, su, sd):
                        g, u, dn = torch.cat([g, sg], 0), torch.cat([u, su], 0), torch.cat([dn, sd], 0)
                    else:
                        g = None
                if g is not None and u is not None and dn is not None:
                    put(p + "w_gu", G.interleave_gate_up(g.view(self.ne1, E, d), u.view(self.ne1, E, d)))
                    put(p + "w_down", dn)
            else:
                g, u, dn = get(r + "w_gate"), get(r + "w_up"), get(r + "w_down")
                if g is not None and u is not None and dn is not None:
                    put(p + "w_gu", G.interleave_gate_up(g.view(1, E, d), u.view(1, E, d)))
                    put(p + "w_down", dn)
        if absent and not missing_ok:
            raise KeyError(f"missing parameter '{absent[0]}'")
        return absent

    def from_internal(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        """Gather a flat buffer back into reference-named tensors (views or small copies on the same device)."""
        cfg = self.cfg
        out: Dict[str, torch.Tensor] = {}
        E, d, ne, qd, kvd = self.Eff, cfg.hidden_size, cfg.num_experts, cfg.q_dim, cfg.kv_dim
        out["tok_embeddings"] = self.view(flat, "tok_embeddings")
        out["final_norm"] = self.view(flat, "final_norm")
        if not cfg.tie_embeddings:
            out["lm_head"] = self.view(flat, "lm_head")
        for i in range(cfg.num_layers):
            r, p = f"layers.{i}.", f"L{i}."
            out[r + "attn_norm"] = self.view(flat, p + "attn_norm")
            out[r + "ffn_norm"] = self.view(flat, p + "ffn_norm")
            if cfg.use_qk_norm:
                out[r + "qk_qnorm"] = self.view(flat, p + "qk_qnorm")
                out[r + "qk_knorm"] = self.view(flat, p + "qk_knorm")
            w = self.view(flat, p + "wqkv")
            out[r + "wq"], out[r + "wk"], out[r + "wv"] = w[:qd], w[qd:qd + kvd], w[qd + kvd:]
            out[r + "wo"] = self.view(flat, p + "wo")
            g, u = G.deinterleave_gate_up(self.view(flat, p + "w_gu").view(self.ne1, 2 * E, d))
            dn = self.view(flat, p + "w_down")
            if cfg.use_moe:
                out[r + "moe_router"] = self.view(flat, p + "router")
                out[r + "moe_gate"] = g[:ne].reshape(ne * E, d)
                out[r + "moe_up"] = u[:ne].reshape(ne * E, d)
                out[r + "moe_down"] = dn[:ne * d]
                if cfg.moe_shared:
                    out[r + "moe_sh_gate"], out[r + "moe_sh_up"] = g[ne].reshape(E, d), u[ne].reshape(E, d)
                    out[r + "moe_sh_down"] = dn[ne * d:]
            else:
                out[r + "w_gate"], out[r + "w_up"], out[r + "w_down"] = g[0], u[0], dn
        return out


class _LayerBuf:
    pass


class CudaModel:
    """Parameters, activations and the forward/backward schedule for a fixed micro-batch shape (B, T)."""

    def __init__(self, cfg: ModelConfig, B: int, T: int, dtype=torch.float16, device=None, ce_chunks: int = 4,
                 use_segments: bool = False, train: bool = True, micro_tokens: int = 0, share_weights=None):
        """``micro_tokens``: when the B x T rows are several of the recipe's micro-batches concatenated, the size of
        one of them; the MoE balance statistics and the router jitter then stay per micro-batch.  ``share_weights``:
        another (inference) model of the same configuration whose parameter buffers this one uses instead of
        allocating its own: a second activation shape over one set of weights."""
        cfg.validate()
        if cfg.head_dim not in (32, 64, 128, 256):
            raise ValueError(f"head_dim {cfg.head_dim} is not supported on the CUDA path (32/64/128/256)")
        if cfg.hidden_size % 8 or cfg.q_dim % 8 or cfg.kv_dim % 8:
            raise ValueError("hidden sizes must be multiples of 8 on the CUDA path")
        self.cfg, self.B, self.T, self.N = cfg, B, T, B * T
        self.micro_tokens = micro_tokens if (cfg.use_moe and 0 < micro_tokens < B * T) else 0
        self.n_seg = (B * T + self.micro_tokens - 1) // self.micro_tokens if self.micro_tokens else 1
        self.dtype = dtype
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.ce_chunks = max(1, min(ce_chunks, self.N))
        self.use_segments = use_segments
        self.layout = ParamLayout(cfg)
        L = self.layout
        f32 = dict(dtype=torch.float32, device=self.dev)
        if share_weights is not None:
            if train or share_weights.layout.total != L.total or share_weights.dtype != dtype:
                raise ValueError("share_weights needs an inference model of the same configuration and dtype")
            self.P, self.W16 = share_weights.P, share_weights.W16
        else:
            self.P = CA.zeros(L.total, **f32)                # fp32 master weights
            self.W16 = CA.zeros(L.total, dtype=dtype, device=self.dev)   # 16-bit shadows (GEMM operands)
        self.Gr = CA.zeros(L.total, **f32) if train else None        # fp32 gradients
        self.moe_bias = None
        self.bias_counts = None
        if share_weights is not None:
            self.moe_bias = share_weights.moe_bias
        elif cfg.use_moe and cfg.moe_aux_free:
            self.moe_bias = CA.zeros(cfg.num_layers, cfg.num_experts, **f32)
        if cfg.use_moe and train:
            # routed slots per (layer, expert) of the current step: balancing input (aux-free) and expert-load report
            self.bias_counts = CA.zeros(cfg.num_layers, cfg.num_experts, **f32)
        self.cos_sin = K.rope_table(torch.from_numpy(cfg.rope_inv_freq()), max(cfg.max_seq_len, T), self.dev)
        self.pos = torch.arange(T, dtype=torch.int32, device=self.dev).repeat(B)
        # per-launch scalars that a captured graph must be able to change
        # [0] CE gradient scale (loss scale); then per micro-batch segment: [2, 2+n) aux coefficient of the backward,
        # [2+n, 2+2n) weight of the segment's balance loss (its supervised tokens)
        self.dyn = CA.zeros(2 + 2 * self.n_seg, **f32)
        self.dyn_aux = self.dyn[2:2 + self.n_seg]
        self.dyn_segw = self.dyn[2 + self.n_seg:2 + 2 * self.n_seg]
        self.seed_dev = CA.zeros(1, dtype=torch.int64, device=self.dev)
        self.ce_acc = CA.zeros(2, dtype=torch.float64, device=self.dev)   # loss sum, supervised rows
        self.aux_acc = CA.zeros(1, **f32)
        self.ids = CA.zeros(self.N, dtype=torch.int32, device=self.dev)
        self.targets = torch.full((self.N,), -100, dtype=torch.int32, device=self.dev)
        self.segs = CA.zeros(self.N, dtype=torch.int32, device=self.dev)
        self.attn_tc = K.attn_tc_supported(cfg.head_dim)
        self.seg_lo = CA.zeros(self.N, dtype=torch.int32, device=self.dev)
        self.ep = None                                      # set by enable_expert_parallel()
        self._alloc_activations(train)

    # ------------------------------------------------------------------ buffers
    def _alloc_activations(self, train: bool):
        cfg, N, dev, dt = self.cfg, self.N, self.dev, self.dtype
        d, qd, kvd, H = cfg.hidden_size, cfg.q_dim, cfg.kv_dim, cfg.num_heads
        E = self.layout.Eff
        f32 = dict(dtype=torch.float32, device=dev)
        c16 = dict(dtype=dt, device=dev)
        nl = cfg.num_layers if train else 1     # evaluation reuses one layer's buffers
        self.x = [CA.empty(N, d, **f32) for _ in range((cfg.num_layers + 1) if train else 2)]
        self.layers: List[_LayerBuf] = []
        for _ in range(nl):
            b = _LayerBuf()
            b.xb, b.rrms1 = CA.empty(N, d, **c16), CA.empty(N, **f32)
            b.qkv, b.qk = CA.empty(N, qd + 2 * kvd, **c16), CA.empty(N, qd + kvd, **c16)
            b.att, b.lse = CA.empty(N, qd, **c16), CA.empty(N, H, **f32)
            b.x_mid = CA.empty(N, d, **f32)
            b.xb2, b.rrms2 = CA.empty(N, d, **c16), CA.empty(N, **f32)
            if cfg.use_moe:
                b.ws = K.MoeWorkspace(N, d, cfg.num_experts, cfg.moe_top_k, cfg.moe_shared, dt, dev,
                                      seg_tokens=self.micro_tokens)
                rows = b.ws.cap
                b.xperm, b.yperm = CA.zeros(rows, d, **c16), CA.zeros(rows, d, **c16)
            else:
                rows = N
            b.gu, b.act = CA.zeros(rows, 2 * E, **c16), CA.zeros(rows, E, **c16)
            self.layers.append(b)
        rows = self.layers[0].ws.cap if cfg.use_moe else N
        self.h16, self.rrms_f = CA.empty(N, d, **c16), CA.empty(N, **f32)
        # ce_chunks bounds the logits buffer (rows x vocab, 16-bit); chunks below 2048 rows only add launches
        self.chunk_rows = max((N + self.ce_chunks - 1) // self.ce_chunks, min(N, 2048))
        self.Vpad = (cfg.vocab_size + 7) // 8 * 8
        self.logits = CA.zeros(self.chunk_rows, self.Vpad, **c16)
        self.row_loss = CA.empty(self.chunk_rows, **f32)
        self.head_splitk = None
        if not train:
            return
        tiles = ((self.chunk_rows + 127) // 128) * ((d + 127) // 128)
        if cfg.vocab_size >= 4096 and tiles < 148:
            splits = max(2, min(32, 296 // tiles, cfg.vocab_size // 512))
            self.head_splitk = G.SplitK(self.chunk_rows, d, cfg.vocab_size, splits, dt, dev)
        t = _LayerBuf()   # backward temporaries shared by all layers
        t.dx, t.dx16 = CA.empty(N, d, **f32), CA.empty(N, d, **c16)
        t.dxb, t.dh16 = CA.empty(N, d, **c16), CA.empty(N, d, **c16)
        t.datt, t.delta = CA.empty(N, qd, **c16), CA.empty(N, H, **f32)
        t.dqkv, t.dqk = CA.zeros(N, qd + 2 * kvd, **c16), CA.empty(N, qd + kvd, **c16)
        t.dgu = CA.zeros(rows, 2 * E, **c16)
        if cfg.use_moe:
            t.dy_perm, t.dxperm = CA.zeros(rows, d, **c16), CA.zeros(rows, d, **c16)
            t.gdot, t.part = CA.empty(N, cfg.moe_top_k, **f32), CA.empty(N, cfg.num_experts, **f32)
            t.part2 = CA.empty(K.ROUTER_WGRAD_CHUNKS * cfg.num_experts * d, **f32)
        else:
            t.dact = CA.empty(N, E, **c16)
        t.norm_part = K.rmsnorm_bwd_scratch(N, d, dev)
        t.qk_part = K.qk_rope_scratch(N, H + cfg.num_kv_heads, cfg.head_dim, dev)
        self.tmp = t

    def enable_expert_parallel(self, buffers=None, capacity: float = 2.0):
        """Divide the routed experts among the ranks of the default process group (all ranks must call this)."""
        from ..parallel.expert_parallel import ExpertParallel
        self.ep = ExpertParallel(self, buffers, capacity, train=hasattr(self, "tmp"))
        return self.ep

    def activation_bytes(self) -> int:
        n = 0
        for obj in [self] + self.layers + ([self.tmp] if hasattr(self, "tmp") else []):
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor):
                    n += v.numel() * v.element_size()
                elif isinstance(v, list):
                    n += sum(t.numel() * t.element_size() for t in v if isinstance(t, torch.Tensor))
        return n

    # ------------------------------------------------------------------ parameters
    def w(self, key):
        return self.layout.view(self.P, key)

    def w16(self, key):
        return self.layout.view(self.W16, key)

    def g(self, key):
        return self.layout.view(self.Gr, key)

    def init_weights(self, seed: int):
        self.load_named(init_parameters(self.cfg, seed))
        if self.moe_bias is not None:
            self.moe_bias.zero_()

    def load_named(self, named, missing_ok=False):
        absent = self.layout.to_internal(named, self.P, missing_ok)
        self.refresh_shadows()
        return absent

    def export_named(self, flat=None) -> Dict[str, np.ndarray]:
        named = self.layout.from_internal(self.P if flat is None else flat)
        return {k: np.ascontiguousarray(v.detach().float().cpu().numpy()) for k, v in named.items()}

    def refresh_shadows(self):
        K.cast_to_16(self.P, self.W16)

    def zero_grad(self):
        self.Gr.zero_()

    # ------------------------------------------------------------------ inputs
    def set_inputs(self, ids, targets, segments):
        """Pinned host tensors -> static device buffers (asynchronous on the current stream)."""
        self.ids.copy_(ids.view(-1), non_blocking=True)
        self.targets.copy_(targets.view(-1), non_blocking=True)
        if self.use_segments and segments is not None:
            self.segs.copy_(segments.view(-1), non_blocking=True)

    # ------------------------------------------------------------------ forward
    def _seg(self):
        return self.segs if self.use_segments else None

    def _layer_forward(self, l: int, x_in, x_out, b: _LayerBuf, train: bool, want_aux: bool):
        cfg = self.cfg
        p = f"L{l}."
        d, qd, kvd, H, KV, hd = cfg.hidden_size, cfg.q_dim, cfg.kv_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        E = self.layout.Eff
        K.rmsnorm_fwd(x_in, self.w(p + "attn_norm"), b.xb, b.rrms1, cfg.rms_eps)
        G.gemm(b.xb, self.w16(p + "wqkv"), out=b.qkv)
        qw = self.w(p + "qk_qnorm") if cfg.use_qk_norm else None
        kw = self.w(p + "qk_knorm") if cfg.use_qk_norm else None
        dec = getattr(self, "decode_engine", None)
        if dec is not None:    # token step of the inference engine (T == 1): this token's k/v go into the cache, the
            #                    query attends over the cache; everything else in this layer is the batched pass
            from ..ops import decode as D
            Lc = dec.layers[l]
            D.qk_rope_append(b.qkv, b.qk, qw, kw, dec.cos_sin, dec.pos, Lc.cK, Lc.cV, dec.slot_pos, dec.state, H, KV, hd,
                             dec.cap, dec.pinned, cfg.rms_eps, cfg.rope_type)
            D.decode_attn(b.qk[:, :qd], Lc.cK, Lc.cV, dec.slot_pos, dec.state, b.att, dec.att_scratch, dec.splits, H, KV, hd,
                          dec.cap, cfg.sliding_window, cfg.attn_scale())
        else:
            self._attention_forward(l, b, qw, kw)
        G.gemm(b.att, self.w16(p + "wo"), out=b.x_mid, addend=x_in)
        K.rmsnorm_fwd(b.x_mid, self.w(p + "ffn_norm"), b.xb2, b.rrms2, cfg.rms_eps)
        self._ffn_forward(l, p, b, x_out, train, want_aux)

    def _attention_forward(self, l: int, b: _LayerBuf, qw, kw):
        cfg = self.cfg
        qd, kvd, H, KV, hd = cfg.q_dim, cfg.kv_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        K.qk_norm_rope_fwd(b.qkv, b.qk, qw, kw, self.cos_sin, self.pos, H, KV, hd, cfg.rms_eps, cfg.rope_type)
        sink = getattr(self, "kv_sink", None)
        if sink is not None:   # prompt pass of the inference engine: keep this layer's keys (after RoPE) and values
            eng, n = sink
            eng.layers[l].cK[:, :n].copy_(b.qk.view(self.B, self.T, -1)[:, :n, qd:])
            eng.layers[l].cV[:, :n].copy_(b.qkv.view(self.B, self.T, -1)[:, :n, qd + kvd:])
        if self.attn_tc:   # tcgen05 path (packed-document segment ids are contiguous runs, as the loader emits them)
            K.attn_tc_fwd(b.qk[:, :qd], b.qk[:, qd:], b.qkv[:, qd + kvd:], b.att, b.lse, None, self.seg_lo,
                          self.B, self.T, H, KV, hd, cfg.sliding_window, cfg.attn_scale(), lo_ready=self.use_segments)
        else:
            K.attn_fwd(b.qk[:, :qd], b.qk[:, qd:], b.qkv[:, qd + kvd:], b.att, b.lse, self._seg(), self.B, self.T, H,
                       KV, hd, cfg.sliding_window, cfg.attn_scale())

    def _ffn_forward(self, l: int, p: str, b: _LayerBuf, x_out, train: bool, want_aux: bool):
        cfg = self.cfg
        d, E = cfg.hidden_size, self.layout.Eff
        if cfg.use_moe and self.ep is not None:     # experts divided among the ranks (parallel/expert_parallel.py)
            self.ep.forward(l, b, x_out, train, want_aux)
        elif cfg.use_moe:
            bias = self.moe_bias[l] if self.moe_bias is not None else None
            counts = self.bias_counts[l] if (train and self.bias_counts is not None) else None
            jit = cfg.moe_jitter if train else 0.0
            K.moe_route_group(b.ws, b.xb2, self.w(p + "router"), bias, b.xperm, counts, jitter=jit,
                              seed_dev=self.seed_dev if jit > 0 else None, want_aux=want_aux,
                              aux_acc=self.aux_acc if want_aux else None, seg_weight=self.dyn_segw if want_aux else None)
            G.gemm_swiglu(b.xperm, self.w16(p + "w_gu"), act_out=b.act, gu_out=b.gu if train else None,
                          tile_expert=b.ws.tile_expert, num_m_tiles=b.ws.num_tiles, group_rows=2 * E)
            G.gemm_grouped_rows(b.act, self.w16(p + "w_down"), b.ws.tile_expert, b.ws.num_tiles, n=d, group_rows=d,
                                out=b.yperm)
            K.moe_combine(b.ws, b.yperm, b.x_mid, x_out)
        else:
            G.gemm_swiglu(b.xb2, self.w16(p + "w_gu"), act_out=b.act, gu_out=b.gu if train else None)
            G.gemm(b.act, self.w16(p + "w_down"), out=x_out, addend=b.x_mid)

    def decode_forward(self, eng):
        """One token per sequence for the inference engine ``eng`` (this model has T == 1 and B == eng.B): embedding of
        ``eng.cur_tok``, all layers with the projections and experts on the tensor cores and the attention over the
        engine's cache, final norm, fp32 logits into ``eng.logits``.  Reads every weight once for the whole batch,
        where the per-sequence GEMV kernels read it once per four sequences."""
        cfg = self.cfg
        assert self.T == 1 and self.B == eng.B
        self.decode_engine = eng
        try:
            K.embed_fwd(eng.cur_tok, self.w("tok_embeddings"), self.x[0])
            for l in range(cfg.num_layers):
                self._layer_forward(l, self.x[l % 2], self.x[(l + 1) % 2], self.layers[0], False, False)
        finally:
            self.decode_engine = None
        K.rmsnorm_fwd(self.x[cfg.num_layers % 2], self.w("final_norm"), self.h16, self.rrms_f, cfg.rms_eps)
        G.gemm(self.h16, self._head_weight16(), out=eng.logits, block_n=256 if cfg.vocab_size >= 4096 else 0)

    def _head_weight16(self):
        return self.w16("tok_embeddings") if self.cfg.tie_embeddings else self.w16("lm_head")

    def _head_grad(self):
        return self.g("tok_embeddings") if self.cfg.tie_embeddings else self.g("lm_head")

    def forward(self, train: bool):
        """Runs on the static input buffers; accumulates (loss sum, rows) into ``ce_acc`` and, in training, leaves
        d(loss)/d(hidden) of the last layer's output in ``tmp.dx`` and the lm-head gradient in ``Gr``."""
        cfg = self.cfg
        want_aux = train and cfg.use_moe and cfg.moe_aux_scale > 0
        K.embed_fwd(self.ids, self.w("tok_embeddings"), self.x[0])
        if self.attn_tc and self.use_segments:
            K.attn_seg_lo(self.segs, self.seg_lo, self.B, self.T)   # once per micro-batch, shared by all layers
        for l in range(cfg.num_layers):
            if train:
                self._layer_forward(l, self.x[l], self.x[l + 1], self.layers[l], True, want_aux)
            else:
                self._layer_forward(l, self.x[l % 2], self.x[(l + 1) % 2], self.layers[0], False, False)
        xf = self.x[cfg.num_layers] if train else self.x[cfg.num_layers % 2]
        K.rmsnorm_fwd(xf, self.w("final_norm"), self.h16, self.rrms_f, cfg.rms_eps)
        V = cfg.vocab_size
        Wh = self._head_weight16()
        for r0 in range(0, self.N, self.chunk_rows):
            r1 = min(self.N, r0 + self.chunk_rows)
            lg = self.logits[:r1 - r0, :V]
            G.gemm(self.h16[r0:r1], Wh, out=lg, block_n=256 if V >= 4096 else 0)
            K.softmax_ce_(lg, self.targets[r0:r1], cfg.z_loss_scale, 1.0, train, self.row_loss, self.ce_acc,
                          grad_scale_dev=self.dyn[0:1] if train else None)
            if train:
                if self.head_splitk is not None:   # long reduction over the vocabulary, few output tiles
                    self.head_splitk.run(lg, Wh, self.tmp.dh16[r0:r1], b_mn=True)
                else:
                    G.gemm(lg, Wh, b_mn=True, out=self.tmp.dh16[r0:r1])
                hg = self._head_grad()
                G.gemm(lg, self.h16[r0:r1], a_mn=True, b_mn=True, out=hg, addend=hg)
        return xf

    # ------------------------------------------------------------------ backward
    def _layer_backward(self, l: int, b: _LayerBuf):
        cfg, t = self.cfg, self.tmp
        p = f"L{l}."
        d, qd, kvd, H, KV, hd = cfg.hidden_size, cfg.q_dim, cfg.kv_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        E, ne1 = self.layout.Eff, self.layout.ne1
        x_in = self.x[l]
        if cfg.use_moe and self.ep is not None:
            self.ep.backward(l, b)
        elif cfg.use_moe:
            ws = b.ws
            K.moe_combine_bwd(ws, t.dx, b.yperm, t.dy_perm, t.gdot)
            G.gemm_swiglu_bwd(t.dy_perm, self.w16(p + "w_down"), b.gu, dgu_out=t.dgu, tile_expert=ws.tile_expert,
                              num_m_tiles=ws.num_tiles, group_rows=d, n=E)
            G.gemm_grouped_reduce(t.dy_perm, b.act, ws.seg_offsets, ne1, self.g(p + "w_down").view(ne1, d, E))
            G.gemm_grouped_rows(t.dgu, self.w16(p + "w_gu"), ws.tile_expert, ws.num_tiles, n=d, b_mn=True,
                                group_rows=2 * E, out=t.dxperm)
            G.gemm_grouped_reduce(t.dgu, b.xperm, ws.seg_offsets, ne1, self.g(p + "w_gu").view(ne1, 2 * E, d))
            want_aux = cfg.moe_aux_scale > 0
            K.moe_router_bwd(ws, b.xb2, self.w(p + "router"), t.gdot, t.dxperm, t.dxb, self.g(p + "router"), t.part,
                             jitter=cfg.moe_jitter, seed_dev=self.seed_dev if cfg.moe_jitter > 0 else None,
                             aux_coef_dev=self.dyn_aux if want_aux else None, part2=t.part2)
        else:
            G.gemm_swiglu_bwd(t.dx16, self.w16(p + "w_down"), b.gu, dgu_out=t.dgu, n=E)
            gd = self.g(p + "w_down")
            G.gemm(t.dx16, b.act, a_mn=True, b_mn=True, out=gd, addend=gd)
            G.gemm(t.dgu, self.w16(p + "w_gu"), b_mn=True, out=t.dxb)
            gg = self.g(p + "w_gu")
            G.gemm(t.dgu, b.xb2, a_mn=True, b_mn=True, out=gg, addend=gg)
        K.rmsnorm_bwd(t.dxb, b.x_mid, self.w(p + "ffn_norm"), b.rrms2, t.dx, t.dx, t.dx16, t.norm_part,
                      self.g(p + "ffn_norm"))
        # attention branch
        G.gemm(t.dx16, self.w16(p + "wo"), b_mn=True, out=t.datt)
        gwo = self.g(p + "wo")
        G.gemm_wgrad(t.dx16, b.att, gwo)
        if self.attn_tc:
            K.attn_tc_bwd(b.qk[:, :qd], b.qk[:, qd:], b.qkv[:, qd + kvd:], b.att, b.lse, None, self.seg_lo, t.datt,
                          t.delta, t.dqk[:, :qd], t.dqk[:, qd:], t.dqkv[:, qd + kvd:], self.B, self.T, H, KV, hd,
                          cfg.sliding_window, cfg.attn_scale(), lo_ready=self.use_segments)
        else:
            K.attn_bwd(b.qk[:, :qd], b.qk[:, qd:], b.qkv[:, qd + kvd:], b.att, b.lse, self._seg(), t.datt, t.delta,
                       t.dqk[:, :qd], t.dqk[:, qd:], t.dqkv[:, qd + kvd:], self.B, self.T, H, KV, hd,
                       cfg.sliding_window, cfg.attn_scale())
        qn = cfg.use_qk_norm
        K.qk_norm_rope_bwd(t.dqk, b.qkv, t.dqkv, self.w(p + "qk_qnorm") if qn else None,
                           self.w(p + "qk_knorm") if qn else None, self.cos_sin, self.pos, t.qk_part,
                           self.g(p + "qk_qnorm") if qn else None, self.g(p + "qk_knorm") if qn else None, H, KV, hd,
                           cfg.rms_eps, cfg.rope_type)
        G.gemm(t.dqkv, self.w16(p + "wqkv"), b_mn=True, out=t.dxb)
        gq = self.g(p + "wqkv")
        G.gemm_wgrad(t.dqkv, b.xb, gq)
        K.rmsnorm_bwd(t.dxb, x_in, self.w(p + "attn_norm"), b.rrms1, t.dx, t.dx, t.dx16, t.norm_part,
                      self.g(p + "attn_norm"))

    def forward_backward(self, freeze_embeddings=False):
        """One micro-batch on the static input buffers; gradients accumulate into ``Gr``."""
        cfg, t = self.cfg, self.tmp
        xf = self.forward(True)
        K.rmsnorm_bwd(t.dh16, xf, self.w("final_norm"), self.rrms_f, None, t.dx, t.dx16, t.norm_part,
                      self.g("final_norm"))
        for l in range(cfg.num_layers - 1, -1, -1):
            self._layer_backward(l, self.layers[l])
        if not freeze_embeddings:
            K.embed_bwd(self.ids, t.dx, self.g("tok_embeddings"))

    def launches_per_micro_batch(self) -> int:
        """Kernel launches issued by one training micro-batch (for the bench report)."""
        cfg = self.cfg
        per_layer_f = 2 + 1 + 1 + 1 + 1 + (2 + 3 + 2 + 1 + (1 if cfg.moe_aux_scale > 0 else 0) if cfg.use_moe else 2)
        per_layer_b = (2 + 4 + 3 if cfg.use_moe else 4) + 2 + 2 + 3 + (3 if cfg.use_qk_norm else 1) + 2 + 2
        chunks = (self.N + self.chunk_rows - 1) // self.chunk_rows
        return 1 + cfg.num_layers * (per_layer_f + per_layer_b) + 1 + chunks * 5 + 2 + 1
