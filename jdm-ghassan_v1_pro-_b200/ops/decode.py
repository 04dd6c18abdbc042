"""Launchers for the decode-time kernels (``csrc/cuda/decode.cu``, ``sample.cu``; contract in ``gb_decode.h``)."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib

c_int, c_ll, c_vp, c_float = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_float

W_F16, W_BF16, W_GGML_Q8_0, W_Q4_0, W_Q8_64, W_Q4_1 = range(6)
FMT_NAMES = {"f16": W_F16, "bf16": W_BF16, "q8_0": W_GGML_Q8_0, "q4_0": W_Q4_0, "q8_64": W_Q8_64, "q4_1": W_Q4_1}
STATE_INTS = 4   # gb_seq_state: abs_pos, cache_len, ring_start, done


class SampleArgs(ctypes.Structure):
    _fields_ = [
        ("logits", c_vp), ("ld", c_ll), ("B", c_int), ("V", c_int),
        ("temperature", c_float), ("top_k", c_int), ("top_p", c_float), ("min_p", c_float),
        ("rep_penalty", c_float), ("freq_penalty", c_float), ("presence_penalty", c_float), ("rep_window", c_int),
        ("greedy", c_int),
        ("history", c_vp), ("hist_cap", c_int), ("hist_len", c_vp),
        ("uniforms", c_vp), ("out_tok", c_vp), ("state", c_vp),
        ("stop", c_vp), ("n_stop", c_int),
        ("tok_log", c_vp), ("log_cap", c_int), ("step", c_vp),
    ]


def row_bytes(fmt: int, K: int) -> int:
    lib = _lib.lib()
    lib.gb_wfmt_row_bytes.restype = c_ll
    n = lib.gb_wfmt_row_bytes(c_int(fmt), c_int(K))
    if n < 0:
        raise ValueError(f"row length {K} does not fit the block size of weight format {fmt}")
    return int(n)


class QWeight:
    """A [N, K] matrix stored row by row in one of the decode formats (device uint8 buffer)."""

    def __init__(self, data: torch.Tensor, fmt: int, N: int, K: int):
        self.data, self.fmt, self.N, self.K = data, fmt, N, K
        self.row_bytes = row_bytes(fmt, K)
        assert data.numel() == N * self.row_bytes, (data.numel(), N, self.row_bytes)

    @classmethod
    def from_f32(cls, w: torch.Tensor, fmt: int, device) -> "QWeight":
        """Quantise / cast fp32 ``w`` ([N, K]) with the host codecs (byte-exact with the file formats)."""
        from .. import _gb200_host as H
        N, K = w.shape
        row_bytes(fmt, K)
        w32 = np.ascontiguousarray(w.detach().float().cpu().numpy())
        if fmt == W_F16:
            raw = torch.from_numpy(w32).to(torch.float16).contiguous().view(torch.uint8)
        elif fmt == W_BF16:
            raw = torch.from_numpy(w32).to(torch.bfloat16).contiguous().view(torch.uint8)
        # K is a multiple of the block size (checked by row_bytes), so blocks never straddle rows and quantising
        # the flat array equals quantising row by row
        elif fmt == W_GGML_Q8_0:
            raw = torch.from_numpy(np.asarray(H.ggml_quantize(w32.reshape(-1), 8)))
        elif fmt == W_Q4_0:
            raw = torch.from_numpy(np.asarray(H.ggml_quantize(w32.reshape(-1), 2)))
        elif fmt == W_Q8_64:
            raw = torch.from_numpy(np.asarray(H.quantize(w32.reshape(-1), "q8_0")))
        elif fmt == W_Q4_1:
            raw = torch.from_numpy(np.asarray(H.quantize(w32.reshape(-1), "q4_1")))
        else:
            raise ValueError(f"unknown weight format {fmt}")
        return cls(raw.reshape(-1).to(device), fmt, N, K)

    def dequantize(self) -> torch.Tensor:
        """fp32 [N, K] on the host (oracle for tests and source of the prefill operands)."""
        from .. import _gb200_host as H
        raw = self.data.cpu().numpy().reshape(self.N, self.row_bytes)
        if self.fmt == W_F16:
            return torch.from_numpy(raw.copy()).view(torch.float16).float().reshape(self.N, self.K)
        if self.fmt == W_BF16:
            return torch.from_numpy(raw.copy()).view(torch.bfloat16).float().reshape(self.N, self.K)
        flat, n = raw.reshape(-1), self.N * self.K
        if self.fmt in (W_GGML_Q8_0, W_Q4_0):
            out = H.ggml_dequantize(flat, 8 if self.fmt == W_GGML_Q8_0 else 2, n)
        else:
            out = H.dequantize(flat, "q8_0" if self.fmt == W_Q8_64 else "q4_1", n)
        return torch.from_numpy(np.asarray(out)).reshape(self.N, self.K)

    @property
    def nbytes(self):
        return self.data.numel()


def _bf(t):
    return int(t.dtype == torch.bfloat16)


def gemv(w: QWeight, x16, out, addend=None):
    """``out[b, :] = W @ x16[b, :] (+ addend[b, :])``; ``out`` is 16-bit or fp32."""
    B = x16.shape[0]
    rc = _lib.lib().gb_gemv(c_vp(w.data.data_ptr()), c_int(w.fmt), c_int(w.N), c_int(w.K), c_vp(x16.data_ptr()),
                            c_int(x16.stride(0)), c_int(B), c_vp(out.data_ptr()), c_int(out.stride(0)),
                            c_int(int(out.dtype == torch.float32)), _lib.ptr(addend),
                            c_int(addend.stride(0) if addend is not None else 0), c_int(_bf(x16)), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_gemv")
    return out


def expert_swiglu(wg: QWeight, wu: QWeight, ne, E, d, x16, idx, top_k, shared, act):
    rc = _lib.lib().gb_gemv_expert_swiglu(c_vp(wg.data.data_ptr()), c_vp(wu.data.data_ptr()), c_int(wg.fmt), c_int(ne),
                                          c_int(E), c_int(d), c_vp(x16.data_ptr()), c_int(x16.shape[0]),
                                          c_vp(idx.data_ptr()), c_int(top_k), c_int(int(shared)), c_vp(act.data_ptr()),
                                          c_int(_bf(x16)), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_gemv_expert_swiglu")


def expert_down(wd: QWeight, ne, d, E, act, idx, w, top_k, shared, resid, out):
    rc = _lib.lib().gb_gemv_expert_down(c_vp(wd.data.data_ptr()), c_int(wd.fmt), c_int(ne), c_int(d), c_int(E),
                                        c_vp(act.data_ptr()), c_int(resid.shape[0]), c_vp(idx.data_ptr()),
                                        c_vp(w.data_ptr()), c_int(top_k), c_int(int(shared)), c_vp(resid.data_ptr()),
                                        c_vp(out.data_ptr()), c_int(_bf(act)), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_gemv_expert_down")


def decode_route(x16, router_w, bias, top_k, idx, w):
    """Router for the ``B`` rows of ``x16``: ``idx[b, k]`` experts and ``w[b, k]`` renormalised probabilities."""
    B, d = x16.shape
    rc = _lib.lib().gb_decode_route(c_vp(x16.data_ptr()), c_vp(router_w.data_ptr()), _lib.ptr(bias), c_int(B), c_int(d),
                                    c_int(router_w.shape[0]), c_int(top_k), c_vp(idx.data_ptr()), c_vp(w.data_ptr()),
                                    c_int(_bf(x16)), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_decode_route")


def kv_append(k16, v16, cacheK, cacheV, slot_pos, state, cap, pinned):
    B, kv_dim = k16.shape[0], k16.shape[1]
    rc = _lib.lib().gb_kv_append(c_vp(k16.data_ptr()), c_ll(k16.stride(0)), c_vp(v16.data_ptr()), c_ll(v16.stride(0)),
                                 c_vp(cacheK.data_ptr()), c_vp(cacheV.data_ptr()), c_vp(slot_pos.data_ptr()),
                                 c_vp(state.data_ptr()), c_int(B), c_int(cap), c_int(pinned), c_int(kv_dim),
                                 _lib.stream_ptr())
    _lib.check_rc(rc, "gb_kv_append")


def decode_attn(q16, cacheK, cacheV, slot_pos, state, out16, scratch, splits, H, KV, hd, cap, window, scale):
    B = q16.shape[0]
    rc = _lib.lib().gb_decode_attn(c_vp(q16.data_ptr()), c_ll(q16.stride(0)), c_vp(cacheK.data_ptr()),
                                   c_vp(cacheV.data_ptr()), c_vp(slot_pos.data_ptr()), c_vp(state.data_ptr()),
                                   c_vp(out16.data_ptr()), c_ll(out16.stride(0)), c_vp(scratch.data_ptr()), c_int(splits),
                                   c_int(B), c_int(H), c_int(KV), c_int(hd), c_int(cap), c_int(window), c_float(scale),
                                   c_int(_bf(q16)), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_decode_attn")


# ---------------------------------------------------------------------------------------------- fused token step
def gemv_norm_fits(B: int, K: int) -> bool:
    return B * K * 2 <= 40 * 1024


def gemv_norm(w: QWeight, x32, norm_w, eps, out, is_bf16=False):
    """``out[b, :] = W @ rmsnorm(x32[b, :]) `` with the normalisation done inside the GEMV (one launch)."""
    B = x32.shape[0]
    rc = _lib.lib().gb_gemv_norm(c_vp(w.data.data_ptr()), c_int(w.fmt), c_int(w.N), c_int(w.K), c_vp(x32.data_ptr()),
                                 c_int(x32.stride(0)), c_vp(norm_w.data_ptr()), c_float(eps), c_int(B), c_vp(out.data_ptr()),
                                 c_int(out.stride(0)), c_int(int(out.dtype == torch.float32)), c_int(int(is_bf16)),
                                 _lib.stream_ptr())
    _lib.check_rc(rc, "gb_gemv_norm")
    return out


def route_norm(x32, norm_w, eps, router_w, bias, top_k, idx, w, is_bf16=False):
    """Router of ``rmsnorm(x32)``: one launch, one block per row."""
    B, d = x32.shape
    rc = _lib.lib().gb_route_norm(c_vp(x32.data_ptr()), c_vp(norm_w.data_ptr()), c_float(eps), c_vp(router_w.data_ptr()),
                                  _lib.ptr(bias), c_int(B), c_int(d), c_int(router_w.shape[0]), c_int(top_k),
                                  c_vp(idx.data_ptr()), c_vp(w.data_ptr()), c_int(int(is_bf16)), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_route_norm")


def swiglu_norm(wg: QWeight, wu: QWeight, ne, E, d, x32, norm_w, eps, idx, top_k, shared, act):
    """RMSNorm + gate/up of the experts in ``idx`` (``None``: dense block) in one launch."""
    rc = _lib.lib().gb_swiglu_norm(c_vp(wg.data.data_ptr()), c_vp(wu.data.data_ptr()), c_int(wg.fmt), c_int(ne), c_int(E),
                                   c_int(d), c_vp(x32.data_ptr()), c_vp(norm_w.data_ptr()), c_float(eps), _lib.ptr(idx),
                                   c_int(x32.shape[0]), c_int(top_k), c_int(int(shared)), c_vp(act.data_ptr()),
                                   c_int(_bf(act)), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_swiglu_norm")


def qk_rope_append(qkv, q_out, qw, kw, cos_sin, pos, cacheK, cacheV, slot_pos, state, H, KV, hd, cap, pinned, eps, rope_type):
    B = qkv.shape[0]
    rc = _lib.lib().gb_qk_rope_append(c_vp(qkv.data_ptr()), c_ll(qkv.stride(0)), c_vp(q_out.data_ptr()), c_ll(q_out.stride(0)),
                                      _lib.ptr(qw), _lib.ptr(kw), c_vp(cos_sin.data_ptr()), c_vp(pos.data_ptr()),
                                      c_vp(cacheK.data_ptr()), c_vp(cacheV.data_ptr()), c_vp(slot_pos.data_ptr()),
                                      c_vp(state.data_ptr()), c_int(B), c_int(H), c_int(KV), c_int(hd), c_int(cap),
                                      c_int(pinned), c_float(eps), c_int(rope_type), c_int(_bf(qkv)), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_qk_rope_append")


def decode_attn_fused(q16, cacheK, cacheV, slot_pos, state, out16, scratch, ticket, splits, H, KV, hd, cap, window, scale):
    B = q16.shape[0]
    rc = _lib.lib().gb_decode_attn_fused(c_vp(q16.data_ptr()), c_ll(q16.stride(0)), c_vp(cacheK.data_ptr()),
                                         c_vp(cacheV.data_ptr()), c_vp(slot_pos.data_ptr()), c_vp(state.data_ptr()),
                                         c_vp(out16.data_ptr()), c_ll(out16.stride(0)), c_vp(scratch.data_ptr()), c_int(splits),
                                         c_int(B), c_int(H), c_int(KV), c_int(hd), c_int(cap), c_int(window), c_float(scale),
                                         c_int(_bf(q16)), c_vp(ticket.data_ptr()), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_decode_attn_fused")


def decode_advance(state, pos_out, cap, pinned):
    rc = _lib.lib().gb_decode_advance(c_vp(state.data_ptr()), c_vp(pos_out.data_ptr()), c_int(state.shape[0]), c_int(cap),
                                      c_int(pinned), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_decode_advance")


def sample(args: SampleArgs):
    rc = _lib.lib().gb_sample(ctypes.byref(args), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_sample")


# ------------------------------------------------------------------------------ single-kernel token step
class MegaLayer(ctypes.Structure):
    _fields_ = [(n, c_vp) for n in ("attn_norm", "ffn_norm", "q_norm", "k_norm", "wqkv", "wo", "router", "bias",
                                    "wg", "wu", "wd", "cache_k", "cache_v")]


class MegaArgs(ctypes.Structure):
    _fields_ = [
        ("layers", c_vp),
        ("n_layers", c_int), ("d", c_int), ("H", c_int), ("KV", c_int), ("hd", c_int), ("ne", c_int), ("top_k", c_int),
        ("shared", c_int), ("E", c_int), ("V", c_int),
        ("fmt", c_int), ("head_fmt", c_int), ("is_bf16", c_int), ("rope_type", c_int),
        ("eps", c_float), ("scale", c_float),
        ("emb", c_vp), ("cur_tok", c_vp),
        ("final_norm", c_vp), ("head", c_vp), ("logits", c_vp),
        ("cos_sin", c_vp), ("pos", c_vp),
        ("state", c_vp), ("slot_pos", c_vp),
        ("cap", c_int), ("pinned", c_int), ("window", c_int),
        ("xbuf", c_vp), ("qkv", c_vp),
        ("att_scratch", c_vp), ("max_splits", c_int),
        ("act", c_vp),
        ("r_idx", c_vp), ("r_w", c_vp),
        ("sync", c_vp), ("status", c_vp), ("prof", c_vp), ("stage_bytes", c_int),
    ]


def mega_layer_table(layers, device) -> torch.Tensor:
    """Device copy of a list of :class:`MegaLayer` (the kernel indexes it by layer)."""
    arr = (MegaLayer * len(layers))(*layers)
    raw = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
    return raw.to(device)


def mega_grid() -> int:
    return int(_lib.lib().gb_decode_mega_grid())


def mega_ok(a: MegaArgs) -> int:
    """0 when the single-kernel step covers these shapes and formats, else the negative code that says why not."""
    return int(_lib.lib().gb_decode_mega_ok(ctypes.byref(a)))


def decode_mega(a: MegaArgs):
    rc = _lib.lib().gb_decode_mega(ctypes.byref(a), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_decode_mega")
