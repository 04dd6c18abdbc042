"""Inference engine for a B200: prompt prefill through the tcgen05 forward pass, token-by-token decode as one
CUDA-graph replay per token.

The reference's generator (inference/generator.cpp:60-420) keeps fp32 activations and an fp32 KV cache, copies
every token id to the device, launches a dozen kernels plus cuBLAS calls per layer and reads logits or top-k
candidates back for every token.  Here:

* weights stay in their storage format (fp16 / bf16 / ggml Q8_0 / Q4_0 / internal Q8_0(64) / Q4_1) and are
  expanded inside the GEMV kernels (``csrc/cuda/decode.cu``); the prompt pass uses 16-bit copies with the GEMM;
* the KV cache is 16-bit ``[batch, capacity, kv_dim]`` per layer with the reference's slot rule: the first 8 tokens
  are pinned, later slots form a ring (inference/kv_cache.h:11-106);
* positions, cache lengths, router choices, sampled tokens, stop flags and the token transcript all live on the
  device, so a decode step has no host dependency and is captured once;
* the sampler is a device kernel fed with uniform numbers drawn from the same generator a host sampler would use.
"""
from __future__ import annotations

import os

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import _gb200_host as H
from ..models.config import ModelConfig
from ..models.cuda_model import CudaModel
from ..ops import decode as D
from ..ops import kernels as K
from ..utils import canary as CA

PINNED_TOKENS = 8


def _lib_status(dev):
    from ..ops import _lib
    return _lib.status_word(dev)


@dataclass
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.92
    min_p: float = 0.05
    repetition_penalty: float = 1.12
    repetition_window: int = 128
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    no_repeat_ngram: int = 0
    greedy: bool = False
    seed: int = 0

    def to_native(self) -> "H.SamplingConfig":
        c = H.SamplingConfig()
        for k, v in self.__dict__.items():
            setattr(c, k, v)
        c.validate()
        return c

    def device_ok(self) -> bool:
        """Settings the device sampler takes; anything else is sampled on the host from the logits."""
        if self.no_repeat_ngram > 0 or self.repetition_window > 1024:
            return False
        return self.greedy or self.temperature <= 0 or 1 <= self.top_k <= 1024


class _Layer:
    pass


class InferenceEngine:
    """Weights in decode formats + KV cache + one captured decode step for ``batch`` sequences."""

    def __init__(self, cfg: ModelConfig, named: Dict[str, np.ndarray], fmt: str = "f16", batch: int = 1,
                 max_len: int = 2048, prefill_chunk: int = 1024, moe_bias: Optional[Sequence] = None, device=None,
                 compute_dtype=torch.float16, keep_f16_embeddings: bool = True, raw=None, raw_types=None,
                 fused_step: bool = True, single_kernel: Optional[bool] = None, gemm_min_batch: Optional[int] = None):
        """``named``: fp32 tensors by parameter name.  ``fmt``: decode weight format, or "auto" with ``raw`` (an object
        with ``tensor_raw(name)``, e.g. a GGUF file) and ``raw_types`` (name -> ggml type) to take the stored bytes.
        ``single_kernel``: run the token step of a batch of one as one cooperative kernel (``csrc/cuda/decode_mega.cu``)
        when the shapes allow it; None takes the default (on; ``GB200_DECODE_MEGA=0`` turns it off).  ``gemm_min_batch``: from this many
        sequences on, the token step runs its projections and experts as tensor-core GEMMs over 16-bit copies of the
        weights (the ones the prompt pass keeps) instead of per-sequence GEMV kernels over the stored bytes; None
        takes ``GB200_DECODE_GEMM_MIN_BATCH`` (default 8), 0 turns it off."""
        cfg.validate()
        if cfg.head_dim not in (32, 64, 128):
            raise ValueError("decode attention supports head_dim 32, 64 and 128")
        self.cfg, self.B, self.cap, self.pinned = cfg, batch, max_len, PINNED_TOKENS
        if gemm_min_batch is None:
            gemm_min_batch = int(os.environ.get("GB200_DECODE_GEMM_MIN_BATCH", "8") or 0)
        self.batched = gemm_min_batch > 0 and batch >= gemm_min_batch
        self._step_model: Optional[CudaModel] = None
        # eight launches per layer instead of eleven (both norms and the cache append folded into their consumers);
        # the separate kernels remain for shapes whose rows do not fit the shared-memory budget
        self.fused = (bool(fused_step) and os.environ.get("GB200_DECODE_UNFUSED", "") != "1"
                      and D.gemv_norm_fits(batch, cfg.hidden_size))
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.dt = compute_dtype
        raw_types = raw_types or {}
        if fmt == "auto":
            kinds = [raw_types.get("layers.0.wq")]
            self.fmt = {1: D.W_F16, 8: D.W_GGML_Q8_0, 2: D.W_Q4_0}.get(kinds[0], D.W_F16)
        else:
            self.fmt = D.FMT_NAMES[fmt] if isinstance(fmt, str) else int(fmt)
        d, qd, kvd, V = cfg.hidden_size, cfg.q_dim, cfg.kv_dim, cfg.vocab_size
        f32 = dict(dtype=torch.float32, device=self.dev)
        c16 = dict(dtype=self.dt, device=self.dev)
        i32 = dict(dtype=torch.int32, device=self.dev)
        t = lambda n: torch.as_tensor(np.asarray(named[n], dtype=np.float32))
        ggml_to_fmt = {1: D.W_F16, 8: D.W_GGML_Q8_0, 2: D.W_Q4_0}

        def q(*names):
            """Rows of the named matrices stacked in one decode-format weight.  With a GGUF source whose stored type
            is one the kernels read directly, the file's bytes are used as they are (no second quantisation)."""
            if raw is not None:
                kinds = {raw_types.get(n) for n in names}
                if len(kinds) == 1 and next(iter(kinds)) in ggml_to_fmt and (fmt == "auto" or ggml_to_fmt[next(iter(kinds))] == self.fmt):
                    f = ggml_to_fmt[next(iter(kinds))]
                    blob = b"".join(bytes(raw.tensor_raw(n)) for n in names)
                    rows = sum(int(np.asarray(named[n]).shape[0]) for n in names)
                    K_ = int(np.asarray(named[names[0]]).shape[1])
                    data = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(self.dev)
                    return D.QWeight(data, f, rows, K_)
            w = torch.cat([t(n) for n in names], 0) if len(names) > 1 else t(names[0])
            return D.QWeight.from_f32(w, self.fmt, self.dev)
        # ---- weights
        self.emb = t("tok_embeddings").to(self.dev)                       # fp32 rows for the embedding lookup
        head = t("tok_embeddings") if cfg.tie_embeddings else t("lm_head")
        # the output projection decides the token: by default it stays 16-bit when the body is quantised
        head_fmt = self.fmt if (self.fmt in (D.W_F16, D.W_BF16) or not keep_f16_embeddings) else D.W_F16
        self.head = D.QWeight.from_f32(head, head_fmt, self.dev)
        self.final_norm = t("final_norm").to(self.dev)
        self.layers: List[_Layer] = []
        E = cfg.moe_expert_dim if cfg.use_moe else cfg.intermediate_size
        self.E = E
        for i in range(cfg.num_layers):
            r = f"layers.{i}."
            L = _Layer()
            L.attn_norm, L.ffn_norm = t(r + "attn_norm").to(self.dev), t(r + "ffn_norm").to(self.dev)
            L.qn = t(r + "qk_qnorm").to(self.dev) if cfg.use_qk_norm else None
            L.kn = t(r + "qk_knorm").to(self.dev) if cfg.use_qk_norm else None
            L.wqkv = q(r + "wq", r + "wk", r + "wv")
            L.wo = q(r + "wo")
            if cfg.use_moe:
                L.router = t(r + "moe_router").to(self.dev)
                sh = cfg.moe_shared
                L.wg = q(*([r + "moe_gate"] + ([r + "moe_sh_gate"] if sh else [])))
                L.wu = q(*([r + "moe_up"] + ([r + "moe_sh_up"] if sh else [])))
                L.wd = q(*([r + "moe_down"] + ([r + "moe_sh_down"] if sh else [])))
                L.bias = (torch.as_tensor(np.asarray(moe_bias[i], dtype=np.float32)).to(self.dev)
                          if (moe_bias is not None and len(moe_bias) > i) else None)
                L.ws = K.MoeWorkspace(batch, d, cfg.num_experts, cfg.moe_top_k, cfg.moe_shared, self.dt, self.dev)
            else:
                L.wg, L.wu, L.wd = q(r + "w_gate"), q(r + "w_up"), q(r + "w_down")
            L.cK = CA.zeros(batch, max_len, kvd, **c16)
            L.cV = CA.zeros(batch, max_len, kvd, **c16)
            self.layers.append(L)
        self.weight_bytes = sum(w.nbytes for L in self.layers for w in (L.wqkv, L.wo, L.wg, L.wu, L.wd)) + self.head.nbytes
        # ---- decode state and buffers (all static: one graph serves every step)
        B = batch
        self.state = CA.zeros(B, D.STATE_INTS, **i32)
        self.slot_pos = CA.zeros(B, max_len, **i32)
        self.pos = CA.zeros(B, **i32)
        self.cur_tok = CA.zeros(B, **i32)
        self.x = [CA.zeros(B, d, **f32) for _ in range(2)]
        self.x_mid = CA.zeros(B, d, **f32)
        self.xb = CA.zeros(B, d, **c16)
        self.rr = CA.zeros(B, **f32)
        self.qkv = CA.zeros(B, qd + 2 * kvd, **c16)
        self.qk = CA.zeros(B, qd + kvd, **c16)
        self.att = CA.zeros(B, qd, **c16)
        slots = (cfg.moe_top_k + int(cfg.moe_shared)) if cfg.use_moe else 1
        self.slots = slots
        self.act = CA.zeros(B, slots, E, **c16)
        self.r_idx = CA.zeros(B, max(1, cfg.moe_top_k), **i32)      # router output of the current layer
        self.r_w = CA.zeros(B, max(1, cfg.moe_top_k), **f32)
        self.dense_idx = CA.zeros(B, 1, **i32)          # dense FFN = one "expert" with weight 1
        self.dense_w = torch.ones(B, 1, **f32)
        self.logits = CA.zeros(B, V, **f32)
        # split-KV: enough (sequence, kv head, split) blocks to cover the GPU; a warp walks its slots one by one,
        # so at batch 1 the cache is cut fine (a few slots per warp) and the partial results merged afterwards
        self.splits = int(min(64, max(8, 512 // (B * cfg.num_kv_heads))))
        self.att_scratch = CA.zeros(B * cfg.num_heads * self.splits * (cfg.head_dim + 2), **f32)
        self.att_ticket = CA.zeros(B * cfg.num_kv_heads, **i32)
        self.cos_sin = K.rope_table(torch.from_numpy(cfg.rope_inv_freq()), max(cfg.max_seq_len, max_len) + 1, self.dev)
        self.hist_cap = max_len + 8
        self.history = CA.zeros(B, self.hist_cap, **i32)
        self.hist_len = CA.zeros(B, **i32)
        self.uniforms = CA.zeros(max_len, B, **f32)      # one row of draws per sampling step
        self.tok_log = CA.zeros(B, max_len, **i32)
        self.step = CA.zeros(1, **i32)
        self.stop = CA.zeros(8, **i32)
        self.n_stop = 0
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._graph_key = None
        self.mega: Optional[D.MegaArgs] = None
        if single_kernel is None:
            single_kernel = os.environ.get("GB200_DECODE_MEGA", "1") != "0"
        if single_kernel and batch == 1:
            self._build_mega()
        self.prefill_chunk = min(prefill_chunk, max_len)
        self._prefill_model: Optional[CudaModel] = None
        self._named = named
        self.rng = H.Rng(1)
        self._uni_host = torch.zeros(max_len, B, dtype=torch.float32).pin_memory()
        self._host_step = 0

    # ------------------------------------------------------------------ single-kernel step
    def _build_mega(self):
        """Argument block of the one-kernel token step; leaves ``self.mega`` None when the kernel does not cover the
        model (row lengths that are not whole 256-value units, head sizes, expert counts: ``gb_decode_mega_ok``)."""
        cfg = self.cfg
        p = lambda t: None if t is None else t.data_ptr()
        rows = []
        for L in self.layers:
            m = D.MegaLayer()
            m.attn_norm, m.ffn_norm, m.q_norm, m.k_norm = p(L.attn_norm), p(L.ffn_norm), p(L.qn), p(L.kn)
            m.wqkv, m.wo = L.wqkv.data.data_ptr(), L.wo.data.data_ptr()
            m.router = p(L.router) if cfg.use_moe else None
            m.bias = p(L.bias) if cfg.use_moe else None
            m.wg, m.wu, m.wd = L.wg.data.data_ptr(), L.wu.data.data_ptr(), L.wd.data.data_ptr()
            m.cache_k, m.cache_v = L.cK.data_ptr(), L.cV.data_ptr()
            rows.append(m)
        self._mega_layers = D.mega_layer_table(rows, self.dev)
        grid = D.mega_grid()
        a = D.MegaArgs()
        a.layers = self._mega_layers.data_ptr()
        a.n_layers, a.d, a.H, a.KV, a.hd = cfg.num_layers, cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        a.ne = cfg.num_experts if cfg.use_moe else 0
        a.top_k = cfg.moe_top_k if cfg.use_moe else 1
        a.shared = int(bool(cfg.use_moe and cfg.moe_shared))
        a.E, a.V = self.E, cfg.vocab_size
        a.fmt, a.head_fmt, a.is_bf16, a.rope_type = self.fmt, self.head.fmt, int(self.dt == torch.bfloat16), cfg.rope_type
        a.eps, a.scale = cfg.rms_eps, cfg.attn_scale()
        a.emb, a.cur_tok = self.emb.data_ptr(), self.cur_tok.data_ptr()
        a.final_norm, a.head, a.logits = self.final_norm.data_ptr(), self.head.data.data_ptr(), self.logits.data_ptr()
        a.cos_sin, a.pos = self.cos_sin.data_ptr(), self.pos.data_ptr()
        a.state, a.slot_pos = self.state.data_ptr(), self.slot_pos.data_ptr()
        a.cap, a.pinned, a.window = self.cap, PINNED_TOKENS, cfg.sliding_window
        self._mega_x = torch.zeros(2 * cfg.hidden_size, dtype=torch.float32, device=self.dev)
        a.xbuf, a.qkv = self._mega_x.data_ptr(), self.qkv.data_ptr()
        a.max_splits = max(1, min(64, grid // max(1, cfg.num_kv_heads)))
        self._mega_scratch = torch.zeros(cfg.num_heads * a.max_splits * (cfg.head_dim + 2), dtype=torch.float32, device=self.dev)
        a.att_scratch, a.act = self._mega_scratch.data_ptr(), self.act.data_ptr()
        a.r_idx, a.r_w = self.r_idx.data_ptr(), self.r_w.data_ptr()
        self._mega_sync = torch.zeros(4, dtype=torch.int32, device=self.dev)
        a.sync, a.status = self._mega_sync.data_ptr(), _lib_status(self.dev).data_ptr()
        if grid > 0 and D.mega_ok(a) == 0:
            self.mega = a

    def trace_phases(self, n_tokens: int = 16) -> Dict[str, float]:
        """Mean microseconds that CTA 0 of the one-kernel step spends in each phase of a layer and at the barrier
        behind it, over ``n_tokens`` eager steps from the current state (the marks come from the device's global
        timer).  Keys: A (norm + QKV), B (attention: ``B_rope``, ``B_walk``, ``B_merge``), C (``C_factors``, ``C_sum``,
        ``C_proj``), D (``D_norm``, ``D_route``, ``D_experts``), E (down projection), ``wait_X`` for the barrier after
        phase X, ``head`` and ``step``."""
        assert self.mega is not None, "the one-kernel token step is not in use"
        nl, M = self.cfg.num_layers, 16
        buf = torch.zeros(M * nl + 2, dtype=torch.int64, device=self.dev)
        self.mega.prof = buf.data_ptr()
        acc = np.zeros(M * nl + 1)
        try:
            for _ in range(n_tokens):
                self._forward_token()
                torch.cuda.synchronize()
                acc += np.diff(buf.cpu().numpy().astype(np.float64))
        finally:
            self.mega.prof = None
        acc /= n_tokens * 1e3
        per = acc[:M * nl].reshape(nl, M)
        names = ["A", "wait_A", "B_rope", "B_walk", "B_merge", "wait_B", "C_factors", "C_sum", "C_proj", "wait_C", "D_norm",
                 "D_route", "D_experts", "wait_D", "E", "wait_E"]
        out = {k: float(per[:, i].mean()) for i, k in enumerate(names)}
        for ph in "BCD":
            out[ph] = sum(v for k, v in out.items() if k.startswith(ph + "_"))
        out["layer"] = float(per.sum(1).mean())
        out["head"] = float(acc[M * nl])
        out["step"] = float(acc.sum())
        return out

    # ------------------------------------------------------------------ one decode step (captured)
    def _layer_step(self, L: _Layer, x_in, x_out):
        cfg = self.cfg
        d, qd, kvd, Hh, KV, hd = cfg.hidden_size, cfg.q_dim, cfg.kv_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        bf = self.dt == torch.bfloat16
        if self.fused:
            D.gemv_norm(L.wqkv, x_in, L.attn_norm, cfg.rms_eps, self.qkv, bf)
            D.qk_rope_append(self.qkv, self.qk, L.qn, L.kn, self.cos_sin, self.pos, L.cK, L.cV, self.slot_pos, self.state,
                             Hh, KV, hd, self.cap, PINNED_TOKENS, cfg.rms_eps, cfg.rope_type)
            D.decode_attn(self.qk[:, :qd], L.cK, L.cV, self.slot_pos, self.state, self.att, self.att_scratch, self.splits,
                          Hh, KV, hd, self.cap, cfg.sliding_window, cfg.attn_scale())
            D.gemv(L.wo, self.att, self.x_mid, addend=x_in)
            if cfg.use_moe:
                D.route_norm(self.x_mid, L.ffn_norm, cfg.rms_eps, L.router, L.bias, cfg.moe_top_k, self.r_idx, self.r_w, bf)
                D.swiglu_norm(L.wg, L.wu, cfg.num_experts, self.E, d, self.x_mid, L.ffn_norm, cfg.rms_eps, self.r_idx,
                              cfg.moe_top_k, cfg.moe_shared, self.act)
                D.expert_down(L.wd, cfg.num_experts, d, self.E, self.act, self.r_idx, self.r_w, cfg.moe_top_k, cfg.moe_shared,
                              self.x_mid, x_out)
            else:
                D.swiglu_norm(L.wg, L.wu, 0, self.E, d, self.x_mid, L.ffn_norm, cfg.rms_eps, None, 1, False, self.act)
                D.expert_down(L.wd, 0, d, self.E, self.act, self.dense_idx, self.dense_w, 1, False, self.x_mid, x_out)
            return
        K.rmsnorm_fwd(x_in, L.attn_norm, self.xb, self.rr, cfg.rms_eps)
        D.gemv(L.wqkv, self.xb, self.qkv)
        K.qk_norm_rope_fwd(self.qkv, self.qk, L.qn, L.kn, self.cos_sin, self.pos, Hh, KV, hd, cfg.rms_eps, cfg.rope_type)
        D.kv_append(self.qk[:, qd:], self.qkv[:, qd + kvd:], L.cK, L.cV, self.slot_pos, self.state, self.cap, PINNED_TOKENS)
        D.decode_attn(self.qk[:, :qd], L.cK, L.cV, self.slot_pos, self.state, self.att, self.att_scratch, self.splits,
                      Hh, KV, hd, self.cap, cfg.sliding_window, cfg.attn_scale())
        D.gemv(L.wo, self.att, self.x_mid, addend=x_in)
        K.rmsnorm_fwd(self.x_mid, L.ffn_norm, self.xb, self.rr, cfg.rms_eps)
        if cfg.use_moe:
            D.decode_route(self.xb, L.router, L.bias, cfg.moe_top_k, self.r_idx, self.r_w)
            D.expert_swiglu(L.wg, L.wu, cfg.num_experts, self.E, d, self.xb, self.r_idx, cfg.moe_top_k, cfg.moe_shared, self.act)
            D.expert_down(L.wd, cfg.num_experts, d, self.E, self.act, self.r_idx, self.r_w, cfg.moe_top_k, cfg.moe_shared,
                          self.x_mid, x_out)
        else:
            D.expert_swiglu(L.wg, L.wu, 0, self.E, d, self.xb, self.dense_idx, 1, False, self.act)
            D.expert_down(L.wd, 0, d, self.E, self.act, self.dense_idx, self.dense_w, 1, False, self.x_mid, x_out)

    def _sample_args(self, sp: SamplingParams) -> D.SampleArgs:
        a = D.SampleArgs()
        a.logits, a.ld, a.B, a.V = self.logits.data_ptr(), self.logits.stride(0), self.B, self.cfg.vocab_size
        n = sp.to_native()
        a.temperature, a.top_k, a.top_p, a.min_p = n.temperature, n.top_k, n.top_p, n.min_p
        a.rep_penalty, a.freq_penalty, a.presence_penalty = n.repetition_penalty, n.frequency_penalty, n.presence_penalty
        a.rep_window, a.greedy = n.repetition_window, int(n.greedy)
        a.history, a.hist_cap, a.hist_len = self.history.data_ptr(), self.hist_cap, self.hist_len.data_ptr()
        a.uniforms, a.out_tok, a.state = self.uniforms.data_ptr(), self.cur_tok.data_ptr(), self.state.data_ptr()
        a.stop, a.n_stop = self.stop.data_ptr(), self.n_stop
        a.tok_log, a.log_cap, a.step = self.tok_log.data_ptr(), self.tok_log.shape[1], self.step.data_ptr()
        return a

    def _forward_token(self):
        """Embedding of ``cur_tok`` through all layers to fp32 logits; advances the per-sequence state."""
        cfg = self.cfg
        if self.mega is not None:
            try:
                D.decode_mega(self.mega)
                return
            except RuntimeError as e:      # the launch itself was refused (e.g. no cooperative launch): use the kernel chain
                from ..utils.log import log_warn
                log_warn("[decode] one-kernel token step not available (%s); using the kernel chain" % e)
                self.mega = None
        if self.batched:
            self._step_net().decode_forward(self)
            D.decode_advance(self.state, self.pos, self.cap, PINNED_TOKENS)
            return
        K.embed_fwd(self.cur_tok, self.emb, self.x[0])
        for i, L in enumerate(self.layers):
            self._layer_step(L, self.x[i % 2], self.x[(i + 1) % 2])
        xf = self.x[cfg.num_layers % 2]
        if self.fused:
            D.gemv_norm(self.head, xf, self.final_norm, cfg.rms_eps, self.logits, self.dt == torch.bfloat16)
        else:
            K.rmsnorm_fwd(xf, self.final_norm, self.xb, self.rr, cfg.rms_eps)
            D.gemv(self.head, self.xb, self.logits)
        D.decode_advance(self.state, self.pos, self.cap, PINNED_TOKENS)

    def _step_eager(self, sp: Optional[SamplingParams]):
        self._forward_token()
        if sp is not None:
            D.sample(self._sample_args(sp))

    def decode_steps(self, n: int, sp: SamplingParams, use_graph: bool = True):
        """Run ``n`` decode steps (forward of ``cur_tok`` + sampling of the next token) without host reads."""
        if not sp.device_ok():
            raise ValueError("these sampling settings need the host sampler: use Generator.generate")
        key = (sp.temperature, sp.top_k, sp.top_p, sp.min_p, sp.repetition_penalty, sp.repetition_window,
               sp.frequency_penalty, sp.presence_penalty, sp.greedy, self.n_stop)
        self._draw_uniforms(n)
        if use_graph and (self.graph is None or self._graph_key != key):
            self._step_eager(sp)          # a real step, run eagerly: first-use set-up must happen outside capture
            n -= 1
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):   # other threads (prefetch, checkpoint writer) may call CUDA
                self._step_eager(sp)
            self.graph, self._graph_key = g, key
        for _ in range(max(0, n)):
            if use_graph:
                self.graph.replay()
            else:
                self._step_eager(sp)

    def _draw_uniforms(self, n: int):
        """Draws for the next ``n`` sampling steps: rows [done, done + n) of the device table the sampler indexes with
        its own step counter.  Each row is written once per generation, so the asynchronous copy never races with
        the host filling later rows."""
        lo = self._host_step
        hi = min(lo + n, self._uni_host.shape[0])
        for s in range(lo, hi):
            for b in range(self.B):
                self._uni_host[s, b] = self.rng.uniform()
        if hi > lo:
            self.uniforms[lo:hi].copy_(self._uni_host[lo:hi], non_blocking=True)
        self._host_step = lo + n

    # ------------------------------------------------------------------ prompt
    def reset(self, seed: int = 0):
        self.state.zero_()
        self.pos.zero_()
        self.hist_len.zero_()
        self.step.zero_()
        self._host_step = 0
        self.rng.reseed(seed if seed else 1)

    def set_stop_tokens(self, ids: Sequence[int]):
        ids = list(ids)[:8]
        self.n_stop = len(ids)
        if ids:
            self.stop[:len(ids)].copy_(torch.tensor(ids, dtype=torch.int32))

    def _prefill_net(self) -> CudaModel:
        if self._prefill_model is None:
            m = CudaModel(self.cfg, self.B, self.prefill_chunk, self.dt, self.dev, ce_chunks=1, use_segments=False, train=False)
            m.load_named(self._named)
            if m.moe_bias is not None:                     # selection bias of aux-free balancing, as the token step uses it
                for i, L in enumerate(self.layers):
                    if getattr(L, "bias", None) is not None:
                        m.moe_bias[i].copy_(L.bias)
            self._prefill_model = m
        return self._prefill_model

    def _step_net(self) -> CudaModel:
        """Activation buffers for one token per sequence over the prompt model's weights (tensor-core token step)."""
        if self._step_model is None:
            self._step_model = CudaModel(self.cfg, self.B, 1, self.dt, self.dev, ce_chunks=1, use_segments=False, train=False,
                                         share_weights=self._prefill_net())
        return self._step_model

    def prefill(self, prompts: torch.Tensor):
        """``prompts``: int32 [B, n] (same length for every sequence).  The first ``prefill_chunk`` tokens go through
        the batched forward pass, whose K/V land in the cache; the rest (and the last prompt token, which produces
        the first logits) go through the decode step."""
        B, n = prompts.shape
        if B != self.B or n < 1:
            raise ValueError("prefill needs [%d, n >= 1] token ids, got %s" % (self.B, tuple(prompts.shape)))
        prompts = prompts.to(self.dev, dtype=torch.int32)
        keep = min(n, self.hist_cap)                       # the penalty window looks at the most recent tokens only
        self.history[:, :keep].copy_(prompts[:, n - keep:])
        self.hist_len.fill_(keep)
        # A prompt longer than the cache goes token by token: the ring keeps the first tokens and the most recent ones
        # (inference/kv_cache.h:11-106 in the reference), which the batched pass cannot express.
        head = min(n - 1, self.prefill_chunk) if (n - 1 >= 64 and n <= self.cap) else 0
        if head > 0:
            m = self._prefill_net()
            T = self.prefill_chunk
            ids = torch.zeros(B, T, dtype=torch.int32, device=self.dev)
            ids[:, :head] = prompts[:, :head]
            m.ids.copy_(ids.view(-1))
            m.targets.fill_(-100)
            m.kv_sink = (self, head)
            m.forward(False)
            m.kv_sink = None
            self.state[:, 0] = head
            self.state[:, 1] = head
            self.pos.fill_(head)
            ar = torch.arange(head, dtype=torch.int32, device=self.dev)
            self.slot_pos[:, :head] = ar
        for j in range(head, n):
            self.cur_tok.copy_(prompts[:, j])
            self._forward_token()
        # logits of the last prompt token are in self.logits; cur_tok is set by the first sample call

    def sample_first(self, sp: SamplingParams):
        self._draw_uniforms(1)
        D.sample(self._sample_args(sp))

    def transcript(self, n_new: int) -> torch.Tensor:
        """Tokens sampled so far, [B, n_new] on the host (one device->host copy)."""
        return self.tok_log[:, :n_new].cpu()
