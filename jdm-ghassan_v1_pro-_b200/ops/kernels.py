"""Python launchers for the non-GEMM sm_100a kernels (elementwise, attention, MoE, CE, optimizer).

Thin wrappers: they validate shapes, fill the C argument structs of ``csrc/cuda/gb_api.h`` and launch on the
current CUDA stream.  Nothing here synchronises with the host or allocates behind the caller's back except
where an ``out=None`` convenience is documented.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from ..utils import canary as CA

from . import _lib
from ._lib import check_rc, lib, stream_ptr

c_ll = c_longlong


def _p(t):
    return None if t is None else t.data_ptr()


def _bf(dt) -> int:
    return int(dt == torch.bfloat16)


class AttnArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("ld_q", c_ll), ("k", c_void_p), ("ld_k", c_ll), ("v", c_void_p), ("ld_v", c_ll),
                ("o", c_void_p), ("ld_o", c_ll), ("lse", c_void_p), ("seg", c_void_p),
                ("B", c_int), ("T", c_int), ("H", c_int), ("KV", c_int), ("hd", c_int), ("window", c_int),
                ("is_bf16", c_int), ("scale", c_float),
                ("d_o", c_void_p), ("ld_do", c_ll), ("delta", c_void_p),
                ("dq", c_void_p), ("ld_dq", c_ll), ("dk", c_void_p), ("ld_dk", c_ll), ("dv", c_void_p), ("ld_dv", c_ll)]


class MoeArgs(ctypes.Structure):
    _fields_ = [("n_tok", c_int), ("d", c_int), ("ne", c_int), ("top_k", c_int), ("shared", c_int), ("is_bf16", c_int),
                ("x16", c_void_p), ("router_w", c_void_p), ("bias", c_void_p),
                ("jitter", c_float), ("jitter_seed", c_ulonglong), ("use_jitter", c_int),
                ("probs", c_void_p), ("idx", c_void_p), ("w", c_void_p), ("block_hist", c_void_p),
                ("seg_offsets", c_void_p), ("tile_expert", c_void_p), ("num_tiles", c_void_p), ("block_base", c_void_p),
                ("slot_pos", c_void_p), ("counts", c_void_p), ("x_perm", c_void_p), ("cap", c_int),
                ("y_perm", c_void_p), ("resid", c_void_p), ("out", c_void_p),
                ("dout", c_void_p), ("dy_perm", c_void_p), ("gdot", c_void_p), ("dx_perm", c_void_p),
                ("aux_coef", c_float), ("f_frac", c_void_p), ("d_router_w", c_void_p), ("dx16", c_void_p),
                ("aux_m", c_void_p), ("part", c_void_p), ("aux_acc", c_void_p), ("dyn_seed", c_void_p),
                ("dyn_aux_coef", c_void_p), ("part2", c_void_p), ("seg_tokens", c_int), ("seg_weight", c_void_p),
                ("status", c_void_p)]

ROUTER_WGRAD_CHUNKS = 256


class OptArgs(ctypes.Structure):
    _fields_ = [("w", c_void_p), ("g", c_void_p), ("m", c_void_p), ("v", c_void_p), ("w16", c_void_p), ("n", c_ll),
                ("kind", c_int), ("beta1", c_float), ("beta2", c_float), ("eps", c_float), ("wd", c_float),
                ("hyper", c_void_p), ("scale_dev", c_void_p), ("is_bf16", c_int)]


_proto_done = False


def _protos():
    global _proto_done
    if _proto_done:
        return lib()
    L = lib()
    L.gb_softmax_ce.argtypes = [c_void_p, c_ll, c_void_p, c_int, c_int, c_float, c_float, c_void_p, c_int, c_void_p,
                                c_void_p, c_int, c_void_p]
    L.gb_embed_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    L.gb_embed_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    L.gb_embed_bwd_sorted.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    L.gb_rmsnorm_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]
    L.gb_rmsnorm_bwd.argtypes = [c_void_p] * 9 + [c_int, c_int, c_int, c_void_p]
    L.gb_qk_norm_rope_fwd.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    L.gb_qk_norm_rope_bwd.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                      c_int, c_int, c_void_p]
    L.gb_cast_f32_to_16.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_void_p]
    L.gb_sqnorm_blocks.argtypes = [c_ll]
    L.gb_sqnorm_partial.argtypes = [c_void_p, c_ll, c_void_p, c_void_p]
    L.gb_finish_norm.argtypes = [c_void_p, c_int, c_void_p, c_float, c_float, c_void_p, c_void_p]
    L.gb_fill_f32.argtypes = [c_void_p, c_float, c_ll, c_void_p]
    _proto_done = True
    return L


# ------------------------------------------------------------------------------------------ elementwise
def embed_fwd(ids, table, out):
    n, d = out.shape
    check_rc(_protos().gb_embed_fwd(_p(ids), _p(table), _p(out), n, d, table.shape[0], stream_ptr()), "embed_fwd")
    return out


def embed_bwd(ids, dx, dtable, presorted: bool = True):
    """dtable[id] += the rows of dx whose token has that id, added in token order (bit-reproducible).

    `presorted` (default): the ids go through a stable sort first (torch.sort on n int32 values: a library radix sort,
    not a hot op) and the kernel adds each run of equal ids from its first position: linear in n.  Without it the
    kernel finds the later occurrences of an id by walking the id list: no scratch memory, quadratic in n."""
    n, d = dx.shape
    if presorted and n > 1:
        sid, order = torch.sort(ids, stable=True)
        check_rc(_protos().gb_embed_bwd_sorted(_p(sid), _p(order), _p(dx), _p(dtable), n, d, dtable.shape[0],
                                               stream_ptr()), "embed_bwd_sorted")
        return
    check_rc(_protos().gb_embed_bwd(_p(ids), _p(dx), _p(dtable), n, d, dtable.shape[0], stream_ptr()), "embed_bwd")


def rmsnorm_fwd(x, w, y16, rrms, eps):
    rows, d = x.shape
    check_rc(_protos().gb_rmsnorm_fwd(_p(x), _p(w), _p(y16), _p(rrms), rows, d, eps, _bf(y16.dtype), stream_ptr()),
             "rmsnorm_fwd")
    return y16


def rmsnorm_bwd_scratch(rows, d, device):
    return torch.empty(_protos().gb_rmsnorm_bwd_blocks(rows) * d, dtype=torch.float32, device=device)


def rmsnorm_bwd(g16, x, w, rrms, dres, dx_out, dx16, part, dw):
    """dx_out = dres + d(norm); dw += column sums; dres may alias dx_out; dx16 optional 16-bit copy of dx_out."""
    rows, d = x.shape
    check_rc(_protos().gb_rmsnorm_bwd(_p(g16), _p(x), _p(w), _p(rrms), _p(dres), _p(dx_out), _p(dx16), _p(part), _p(dw),
                                      rows, d, _bf(g16.dtype), stream_ptr()), "rmsnorm_bwd")


def qk_rope_scratch(n_tok, heads, hd, device):
    return torch.empty(2 * _protos().gb_qk_rope_blocks(n_tok * heads) * hd, dtype=torch.float32, device=device)


def qk_norm_rope_fwd(qkv, out, qw, kw, cos_sin, pos, H, KV, hd, eps, rope_type):
    n = qkv.shape[0]
    check_rc(_protos().gb_qk_norm_rope_fwd(_p(qkv), qkv.stride(0), _p(out), out.stride(0), _p(qw), _p(kw), _p(cos_sin),
                                           _p(pos), n, H, KV, hd, eps, rope_type, _bf(qkv.dtype), stream_ptr()),
             "qk_norm_rope_fwd")
    return out


def qk_norm_rope_bwd(dout, qkv, dqkv, qw, kw, cos_sin, pos, part, dqw, dkw, H, KV, hd, eps, rope_type):
    n = qkv.shape[0]
    check_rc(_protos().gb_qk_norm_rope_bwd(_p(dout), dout.stride(0), _p(qkv), qkv.stride(0), _p(dqkv), dqkv.stride(0),
                                           _p(qw), _p(kw), _p(cos_sin), _p(pos), _p(part), _p(dqw), _p(dkw), n, H, KV,
                                           hd, eps, rope_type, _bf(qkv.dtype), stream_ptr()), "qk_norm_rope_bwd")


def cast_to_16(src, dst):
    check_rc(_protos().gb_cast_f32_to_16(_p(src), _p(dst), src.numel(), _bf(dst.dtype), stream_ptr()), "cast")
    return dst


def fill_(t, v: float):
    check_rc(_protos().gb_fill_f32(_p(t), float(v), t.numel(), stream_ptr()), "fill")
    return t


def rope_table(inv_freq: torch.Tensor, max_pos: int, device) -> torch.Tensor:
    """[max_pos, hd] fp32: first half cos(pos * f_i), second half sin; angle rounded to fp32 from a double product."""
    pos = torch.arange(max_pos, dtype=torch.float64)
    ang = (pos[:, None] * inv_freq.double().cpu()[None, :]).float().double()
    return torch.cat([torch.cos(ang), torch.sin(ang)], dim=1).float().contiguous().to(device)


# ------------------------------------------------------------------------------------------ attention
def _attn_args(q, k, v, o, lse, seg, B, T, H, KV, hd, window, scale):
    a = AttnArgs()
    a.q, a.ld_q, a.k, a.ld_k, a.v, a.ld_v = _p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0)
    a.o, a.ld_o, a.lse, a.seg = _p(o), o.stride(0), _p(lse), _p(seg)
    a.B, a.T, a.H, a.KV, a.hd, a.window, a.is_bf16, a.scale = B, T, H, KV, hd, window, _bf(q.dtype), scale
    return a


def attn_fwd(q, k, v, o, lse, seg, B, T, H, KV, hd, window, scale):
    """q/k/v/o: 2-D views [B*T, *] whose column h*hd starts head h; lse fp32 [B*T, H]."""
    a = _attn_args(q, k, v, o, lse, seg, B, T, H, KV, hd, window, scale)
    check_rc(lib().gb_attn_fwd(ctypes.byref(a), stream_ptr()), "attn_fwd")
    return o


def attn_bwd(q, k, v, o, lse, seg, d_o, delta, dq, dk, dv, B, T, H, KV, hd, window, scale):
    a = _attn_args(q, k, v, o, lse, seg, B, T, H, KV, hd, window, scale)
    a.d_o, a.ld_do, a.delta = _p(d_o), d_o.stride(0), _p(delta)
    a.dq, a.ld_dq, a.dk, a.ld_dk, a.dv, a.ld_dv = _p(dq), dq.stride(0), _p(dk), dk.stride(0), _p(dv), dv.stride(0)
    check_rc(lib().gb_attn_bwd(ctypes.byref(a), stream_ptr()), "attn_bwd")


def attn_tc_supported(hd: int) -> bool:
    """Head sizes served by the tcgen05 attention kernels (others use the CUDA-core kernels)."""
    return hd in (64, 128)


def attn_seg_lo(seg, lo, B, T):
    """``lo[i]`` = start of the run of equal segment ids containing position i (per sequence)."""
    check_rc(lib().gb_attn_seg_lo(c_void_p(_p(seg)), c_void_p(_p(lo)), c_int(B), c_int(T), stream_ptr()), "attn_seg_lo")
    return lo


def attn_tc_fwd(q, k, v, o, lse, seg, lo_scratch, B, T, H, KV, hd, window, scale, lo_ready=False):
    """Tensor-core forward; ``seg`` ids must form contiguous runs per sequence, ``lo_scratch`` int32 [B*T].
    With ``lo_ready`` the scratch already holds :func:`attn_seg_lo` output and ``seg`` is not read."""
    a = _attn_args(q, k, v, o, lse, seg, B, T, H, KV, hd, window, scale)
    check_rc(lib().gb_attn_tc_fwd(ctypes.byref(a), c_void_p(_p(lo_scratch)), c_int(int(lo_ready)),
                                  c_void_p(_lib.status_word(q.device).data_ptr()), stream_ptr()), "attn_tc_fwd")
    return o


def attn_tc_bwd(q, k, v, o, lse, seg, lo_scratch, d_o, delta, dq, dk, dv, B, T, H, KV, hd, window, scale, lo_ready=False):
    a = _attn_args(q, k, v, o, lse, seg, B, T, H, KV, hd, window, scale)
    a.d_o, a.ld_do, a.delta = _p(d_o), d_o.stride(0), _p(delta)
    a.dq, a.ld_dq, a.dk, a.ld_dk, a.dv, a.ld_dv = _p(dq), dq.stride(0), _p(dk), dk.stride(0), _p(dv), dv.stride(0)
    check_rc(lib().gb_attn_tc_bwd(ctypes.byref(a), c_void_p(_p(lo_scratch)), c_int(int(lo_ready)),
                                  c_void_p(_lib.status_word(q.device).data_ptr()), stream_ptr()), "attn_tc_bwd")


# ------------------------------------------------------------------------------------------ MoE
def moe_num_blocks(n_tok):
    return lib().gb_moe_num_blocks(n_tok)


def moe_capacity(n_tok, ne, top_k, shared):
    return lib().gb_moe_capacity(n_tok, ne, top_k, int(shared))


class MoeWorkspace:
    """Routing buffers of one MoE layer invocation (sizes depend on n_tok only)."""

    def __init__(self, n_tok, d, ne, top_k, shared, dtype, device, seg_tokens=0):
        """``seg_tokens``: size of the micro-batches that the pass concatenates (0 = the pass is one micro-batch); the
        balance statistics and the jitter token index are then kept per micro-batch."""
        self.n_tok, self.d, self.ne, self.K, self.shared = n_tok, d, ne, top_k, bool(shared)
        self.dtype = dtype
        if seg_tokens and not lib().gb_moe_seg_ok(n_tok, seg_tokens):
            raise ValueError(f"micro-batches of {seg_tokens} tokens do not line up with the routing blocks of a "
                             f"{n_tok}-token pass")
        self.seg_tokens = seg_tokens if 0 < seg_tokens < n_tok else 0
        self.n_seg = (n_tok + self.seg_tokens - 1) // self.seg_tokens if self.seg_tokens else 1
        nb = moe_num_blocks(n_tok)
        S = top_k + int(self.shared)
        i32 = dict(dtype=torch.int32, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.cap = moe_capacity(n_tok, ne, top_k, shared)
        self.probs = CA.empty(n_tok, ne, **f32)
        self.idx = CA.empty(n_tok, top_k, **i32)
        self.w = CA.empty(n_tok, top_k, **f32)
        self.block_hist = CA.empty(nb, ne + 1, **i32)
        self.block_base = CA.empty(nb + 1, ne + 1, **i32)
        self.seg_offsets = CA.zeros(ne + 2, **i32)
        self.tile_expert = CA.zeros(self.cap // 128, **i32)
        self.num_tiles = CA.zeros(1, **i32)
        self.slot_pos = CA.empty(n_tok, S, **i32)
        self.aux_m = CA.zeros(self.n_seg, ne, **f32)
        self.f_frac = CA.zeros(self.n_seg, ne, **f32)

    def args(self) -> MoeArgs:
        a = MoeArgs()
        a.n_tok, a.d, a.ne, a.top_k, a.shared, a.is_bf16 = self.n_tok, self.d, self.ne, self.K, int(self.shared), _bf(self.dtype)
        a.probs, a.idx, a.w = _p(self.probs), _p(self.idx), _p(self.w)
        a.block_hist, a.block_base = _p(self.block_hist), _p(self.block_base)
        a.seg_offsets, a.tile_expert, a.num_tiles = _p(self.seg_offsets), _p(self.tile_expert), _p(self.num_tiles)
        a.slot_pos, a.cap = _p(self.slot_pos), self.cap
        a.aux_m, a.f_frac = _p(self.aux_m), _p(self.f_frac)
        a.seg_tokens = self.seg_tokens
        a.status = _p(_lib.status_word(self.probs.device))
        return a


def moe_route_group(ws: MoeWorkspace, x16, router_w, bias, x_perm, counts=None, jitter=0.0, jitter_seed=None,
                    want_aux=False, aux_acc=None, seed_dev=None, seg_weight=None):
    """``jitter_seed`` (host int) or ``seed_dev`` (uint64 device tensor, read at run time) enables the jitter.
    ``seg_weight`` (fp32 device [ws.n_seg]): weight of each micro-batch's balance loss in ``aux_acc`` (default 1)."""
    a = ws.args()
    a.x16, a.router_w, a.bias = _p(x16), _p(router_w), _p(bias)
    a.jitter = float(jitter)
    a.use_jitter = int(jitter > 0 and (jitter_seed is not None or seed_dev is not None))
    a.jitter_seed = int(jitter_seed or 0)
    a.dyn_seed = _p(seed_dev)
    a.x_perm, a.counts = _p(x_perm), _p(counts)
    a.aux_acc = _p(aux_acc)
    a.seg_weight = _p(seg_weight)
    if not want_aux:
        a.aux_m = None
        a.f_frac = None
    check_rc(lib().gb_moe_route(ctypes.byref(a), stream_ptr()), "moe_route")
    check_rc(lib().gb_moe_group(ctypes.byref(a), stream_ptr()), "moe_group")


def moe_route_only(ws: MoeWorkspace, x16, router_w, bias):
    """Router without grouping (decode): fills ``ws.probs``, ``ws.idx`` and ``ws.w``; no jitter, no statistics."""
    a = ws.args()
    a.x16, a.router_w, a.bias = _p(x16), _p(router_w), _p(bias)
    a.jitter, a.use_jitter = 0.0, 0
    a.aux_m = None
    a.f_frac = None
    check_rc(lib().gb_moe_route(ctypes.byref(a), stream_ptr()), "moe_route")


def moe_combine(ws: MoeWorkspace, y_perm, resid, out):
    a = ws.args()
    a.y_perm, a.resid, a.out = _p(y_perm), _p(resid), _p(out)
    check_rc(lib().gb_moe_combine(ctypes.byref(a), stream_ptr()), "moe_combine")
    return out


def moe_combine_bwd(ws: MoeWorkspace, dout, y_perm, dy_perm, gdot):
    a = ws.args()
    a.dout, a.y_perm, a.dy_perm, a.gdot = _p(dout), _p(y_perm), _p(dy_perm), _p(gdot)
    check_rc(lib().gb_moe_combine_bwd(ctypes.byref(a), stream_ptr()), "moe_combine_bwd")


def moe_router_bwd(ws: MoeWorkspace, x16, router_w, gdot, dx_perm, dx16, d_router_w, part, aux_coef=0.0, jitter=0.0,
                   jitter_seed=None, seed_dev=None, aux_coef_dev=None, part2=None):
    """``part2`` (fp32 [ROUTER_WGRAD_CHUNKS * ne * d]) lets the router weight gradient run on many blocks."""
    a = ws.args()
    a.part2 = _p(part2)
    a.x16, a.router_w, a.gdot, a.dx_perm, a.dx16 = _p(x16), _p(router_w), _p(gdot), _p(dx_perm), _p(dx16)
    a.d_router_w, a.part, a.aux_coef = _p(d_router_w), _p(part), float(aux_coef)
    a.jitter = float(jitter)
    a.use_jitter = int(jitter > 0 and (jitter_seed is not None or seed_dev is not None))
    a.jitter_seed = int(jitter_seed or 0)
    a.dyn_seed, a.dyn_aux_coef = _p(seed_dev), _p(aux_coef_dev)
    if aux_coef == 0.0 and aux_coef_dev is None:
        a.f_frac = None
    check_rc(lib().gb_moe_router_bwd(ctypes.byref(a), stream_ptr()), "moe_router_bwd")


# ------------------------------------------------------------------------------------------ CE / optimizer
def softmax_ce_(logits16, targets, z_loss, grad_scale, write_grad, row_loss, acc, grad_scale_dev=None):
    """In place on a [rows, V] 16-bit chunk; ``acc`` (float64[2]) accumulates (loss sum, supervised rows).
    ``grad_scale_dev`` (fp32 device scalar) overrides ``grad_scale`` when given."""
    rows, V = logits16.shape
    check_rc(_protos().gb_softmax_ce(_p(logits16), logits16.stride(0), _p(targets), rows, V, float(z_loss),
                                     float(grad_scale), _p(grad_scale_dev), int(write_grad), _p(row_loss), _p(acc),
                                     _bf(logits16.dtype), stream_ptr()), "softmax_ce")


def sqnorm_blocks(n):
    return _protos().gb_sqnorm_blocks(n)


def sqnorm_partial(g, partial):
    check_rc(_protos().gb_sqnorm_partial(_p(g), g.numel(), _p(partial), stream_ptr()), "sqnorm")


def finish_norm(partial, n_partial, grad_scale_dev, grad_scale, clip, out):
    check_rc(_protos().gb_finish_norm(_p(partial), n_partial, _p(grad_scale_dev), float(grad_scale), float(clip), _p(out),
                                      stream_ptr()), "finish_norm")


def optimizer_step(kind, w, g, m, v, w16, hyper_dev, scale_dev, beta1, beta2, eps, wd):
    a = OptArgs()
    a.w, a.g, a.m, a.v, a.w16, a.n = _p(w), _p(g), _p(m), _p(v), _p(w16), w.numel()
    a.kind = {"adamw": 0, "lion": 1}[kind]
    a.beta1, a.beta2, a.eps, a.wd = beta1, beta2, eps, wd
    a.hyper, a.scale_dev = _p(hyper_dev), _p(scale_dev)
    a.is_bf16 = _bf(w16.dtype) if w16 is not None else 0
    check_rc(lib().gb_optimizer_step(ctypes.byref(a), stream_ptr()), "optimizer_step")
