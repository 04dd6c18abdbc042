"""Python launchers for the tcgen05 GEMM (``csrc/cuda/gemm_sm100.cu``).

Conventions: ``a`` holds the A operand either as ``[M, K]`` (K contiguous, ``a_mn=False``) or as
``[K, M]`` (``a_mn=True``); ``b`` holds B either as ``[N, K]`` (the ``[out, in]`` weight layout of the
reference, core/ops_cpu_dense.cpp:199-201) or as ``[K, N]`` (``b_mn=True``).  Operands are fp16 or
bf16, accumulation is fp32, the output dtype is chosen by the caller.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

EPI_STORE, EPI_SWIGLU_FWD, EPI_SWIGLU_BWD = 0, 1, 2

# Two-CTA 256 x 256 tiles (csrc/cuda/gemm_pair_sm100.cu) are taken when the problem has at least this many of them
# (74 CTA pairs on a B200); GB200_GEMM_PAIR=0 keeps every product on the one-CTA kernel.
PAIR_ENABLED = os.environ.get("GB200_GEMM_PAIR", "1") != "0"
PAIR_MIN_TILES = int(os.environ.get("GB200_GEMM_PAIR_MIN_TILES", "60"))


def pair_tiles(M, N, groups=1):
    return ((M + 255) // 256) * ((N + 255) // 256) * groups


def pair_ok(M, N, out, groups=1, extra=()):
    """True when the two-CTA kernel can and should run this product: enough 256 x 256 tiles, and every matrix that
    its epilogue moves with TMA (the output, saved gate/up) 16-byte aligned with a 16-byte row pitch."""
    if not PAIR_ENABLED or pair_tiles(M, N, groups) < PAIR_MIN_TILES:
        return False
    for t in (out,) + tuple(extra):
        if t is not None and (t.data_ptr() % 16 or (t.stride(-2) * t.element_size()) % 16):
            return False
    return True


def _check_operand(t, name):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit inner stride")
    if t.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"{name} must be fp16 or bf16")
    if t.data_ptr() % 16 or (t.stride(0) * 2) % 16:
        raise ValueError(f"{name} must be 16-byte aligned with a row pitch that is a multiple of 16 bytes")


def _launch(args: _lib.GemmArgs):
    rc = _lib.lib().gb_gemm(ctypes.byref(args), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_gemm")


def _base_args(a, b, M, N, K, a_mn, b_mn, out, block_n):
    _check_operand(a, "a")
    _check_operand(b, "b")
    if a.dtype != b.dtype:
        raise ValueError("operand dtypes differ")
    g = _lib.GemmArgs()
    g.A, g.B = a.data_ptr(), b.data_ptr()
    g.M, g.N, g.K = M, N, K
    g.a_rows, g.a_cols, g.lda = a.shape[0], a.shape[1], a.stride(0)
    g.b_rows, g.b_cols, g.ldb = b.shape[0], b.shape[1], b.stride(0)
    g.a_mn_major, g.b_mn_major = int(a_mn), int(b_mn)
    g.is_bf16 = int(a.dtype == torch.bfloat16)
    g.out_dtype = _lib.DT_CODE[out.dtype]
    g.block_n = block_n
    g.out = out.data_ptr()
    g.ldo = out.stride(-2)
    g.status = _lib.status_word(a.device).data_ptr()
    return g


def pick_block_n(M, N, mn_major=False):
    """Tile width.  A 128 x 256 tile reads 1.5 operand bytes per MMA where 128 x 128 reads 2, and one CTA's
    tcgen05 pipe at 128 x 128 is bound by shared-memory bandwidth: measured 1.5x faster at 256 once there are tiles
    for every SM.  Narrow tiles only when the problem would otherwise leave most of the 148 SMs idle; operands that
    are both stored MN-major (weight gradients) want one and a half waves of 256-wide tiles before they gain."""
    tiles_m = (M + 127) // 128
    if N % 256 == 0 and tiles_m * (N // 256) >= (222 if mn_major else 120):
        return 256
    tiles128 = tiles_m * ((N + 127) // 128)
    if tiles128 < 100 and N % 64 == 0:
        return 64
    return 128


def gemm(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=None, addend=None, block_n=0, pair=None):
    """``out = A @ B^T (+ addend)``; ``addend`` is fp32 and may alias an fp32 ``out`` (accumulate).
    ``pair``: force (True) or forbid (False) the two-CTA kernel; None picks by size."""
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"reduction dims differ: {K} vs {Kb}")
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    if pair is None:
        pair = (block_n in (0, 256) and (addend is None or out.dtype == torch.float32) and pair_ok(M, N, out))
    if not block_n:
        block_n = pick_block_n(M, N, mn_major=a_mn and b_mn)
    g = _base_args(a, b, M, N, K, a_mn, b_mn, out, block_n)
    g.epilogue = EPI_STORE
    g.pair = int(bool(pair))
    if addend is not None:
        if addend.dtype != torch.float32:
            raise ValueError("addend must be fp32")
        g.addend, g.ld_add = addend.data_ptr(), addend.stride(0)
    _launch(g)
    return out


def gemm_swiglu(a, w_gu, *, act_out=None, gu_out=None, tile_expert=None, num_m_tiles=None, group_rows=0, pair=None):
    """Fused ``[gate|up]`` projection + SwiGLU.

    ``w_gu`` stores gate and up rows interleaved in blocks of 64 (``g0..g63,u0..u63,g64..``) so that one
    128-column accumulator tile holds matching gate/up columns; ``gu_out`` (optional, same interleaved
    column order) keeps the pre-activations for backward, ``act_out[m, j] = silu(g_j) * u_j``.
    With ``tile_expert``/``num_m_tiles`` the rows are expert-sorted and ``w_gu`` stacks ``group_rows`` rows per expert.
    """
    M, K = a.shape
    N = group_rows if group_rows else w_gu.shape[0]
    if N % 128:
        raise ValueError("2*E must be a multiple of 128")
    if act_out is None:
        act_out = torch.empty(M, N // 2, dtype=a.dtype, device=a.device)
    g = _base_args(a, w_gu, M, N, K, False, False, act_out, 256 if (N % 256 == 0 and M >= 4096) else 128)
    g.epilogue = EPI_SWIGLU_FWD
    g.pair = int(pair_ok(M, N, act_out, extra=(gu_out,)) if pair is None else bool(pair))
    if gu_out is not None:
        g.aux_out, g.ld_aux = gu_out.data_ptr(), gu_out.stride(0)
    if tile_expert is not None:
        g.mode = 1
        g.tile_expert, g.num_m_tiles = tile_expert.data_ptr(), num_m_tiles.data_ptr()
        g.b_group_rows = group_rows
    _launch(g)
    return act_out


def gemm_swiglu_bwd(dy, w_down, gu, *, dgu_out=None, b_mn=True, tile_expert=None, num_m_tiles=None, group_rows=0,
                    n=None, pair=None):
    """``d_act = dy @ W_down`` fused with the SwiGLU derivative: writes interleaved ``(dg, du)``.

    ``w_down`` is the stored ``[d, E]`` matrix (``[ne*d, E]`` when grouped), i.e. B in ``[K, N]`` layout.
    """
    M, K = dy.shape
    N = n if n is not None else (w_down.shape[1] if b_mn else w_down.shape[0])
    if dgu_out is None:
        dgu_out = torch.empty(M, 2 * N, dtype=dy.dtype, device=dy.device)
    g = _base_args(dy, w_down, M, N, K, False, b_mn, dgu_out,
                   256 if (N % 256 == 0 and M >= 4096) else (128 if N % 128 == 0 else 64))
    g.epilogue = EPI_SWIGLU_BWD
    g.pair = int((N % 64 == 0 and pair_ok(M, N, dgu_out, extra=(gu,))) if pair is None else bool(pair))
    g.aux_in, g.ld_aux = gu.data_ptr(), gu.stride(0)
    if tile_expert is not None:
        g.mode = 1
        g.tile_expert, g.num_m_tiles = tile_expert.data_ptr(), num_m_tiles.data_ptr()
        g.b_group_rows = group_rows
    _launch(g)
    return dgu_out


def gemm_grouped_rows(a, b, tile_expert, num_m_tiles, *, n, b_mn=False, group_rows, out=None, out_dtype=None,
                      block_n=0, tile_out=None, ldo=None, pair=None, addend=None):
    """Expert-sorted rows: every 128-row tile of ``a`` multiplies the weight block of ``tile_expert[tile]``.
    The two-CTA kernel (``pair``) needs tiles ``2i`` and ``2i+1`` to belong to one expert: segments padded to 256 rows.

    ``b`` stacks the per-expert matrices along its rows: ``group_rows`` stored rows per expert.
    ``tile_out`` (device int64 table, one entry per 128-row tile) redirects each tile's rows to the given address,
    row pitch ``ldo`` elements; the destinations may be buffers of other GPUs mapped into this process.
    ``addend`` (fp32 ``[M, n]``, fp32 ``out`` only, not with ``tile_out``): ``out = product + addend``.
    """
    M, K = a.shape
    if out is None:
        out = torch.empty((M, n) if tile_out is None else (1, n), dtype=out_dtype or a.dtype, device=a.device)
    if not block_n:
        block_n = 256 if (n % 256 == 0 and M >= 4096) else 128
    if addend is not None and (addend.dtype != torch.float32 or out.dtype != torch.float32 or tile_out is not None):
        raise ValueError("addend needs fp32 addend and output and no tile_out")
    if pair is None:
        pair = tile_out is None and pair_ok(M, n, out)
    g = _base_args(a, b, M, n, K, False, b_mn, out, block_n)
    g.epilogue = EPI_STORE
    g.mode = 1
    g.pair = int(bool(pair))
    if addend is not None:
        g.addend, g.ld_add = addend.data_ptr(), addend.stride(0)
    g.tile_expert, g.num_m_tiles = tile_expert.data_ptr(), num_m_tiles.data_ptr()
    g.b_group_rows = group_rows
    if tile_out is not None:
        if tile_out.dtype != torch.int64:
            raise ValueError("tile_out must be int64 addresses")
        g.tile_out = tile_out.data_ptr()
        g.ldo = int(ldo if ldo is not None else n)
    _launch(g)
    return out


def gemm_grouped_reduce(a, b, seg_offsets, groups, out, *, accumulate=True, block_n=0, pair=None):
    """Per-expert weight gradient: ``out[g] (+)= a[rows_g]^T @ b[rows_g]`` with ``rows_g`` given by the padded
    offsets ``seg_offsets[g] .. seg_offsets[g+1]`` (device int32, multiples of 128; pad rows must be zero).
    ``a`` is ``[rows, M]``, ``b`` is ``[rows, N]``, ``out`` is fp32 ``[groups, M, N]``.
    """
    M, N = a.shape[1], b.shape[1]
    if out.dtype != torch.float32 or out.shape != (groups, M, N) or not out.is_contiguous():
        raise ValueError("out must be contiguous fp32 [groups, M, N]")
    if not block_n:    # 256-wide tiles measured 1.47x faster once the groups supply tiles for every SM
        block_n = 256 if (N % 256 == 0 and groups * ((M + 127) // 128) * (N // 256) >= 222) else 128
    if pair is None:
        pair = pair_ok(M, N, out, groups=groups)
    g = _base_args(a, b, M, N, 0, True, True, out, block_n)
    g.epilogue = EPI_STORE
    g.mode = 2
    g.pair = int(bool(pair))
    g.seg_offsets = seg_offsets.data_ptr()
    g.groups = groups
    g.out_group_stride = M * N
    g.ldo = N
    if accumulate:
        g.addend, g.ld_add = out.data_ptr(), N
    _launch(g)
    return out


class SplitK:
    """Split-K plan for a product with a long reduction and few output tiles (e.g. d(hidden) = d(logits) @ W over
    the vocabulary): ``splits`` CTAs per output tile each reduce a K range into an fp32 partial, a second kernel
    adds the partials in a fixed order and casts.  Buffers are created once and reused."""

    def __init__(self, M, N, K, splits, dtype, device):
        kc = (K + splits - 1) // splits
        kc = (kc + 63) // 64 * 64
        offs = [min(K, i * kc) for i in range(splits + 1)]
        self.splits, self.M, self.N, self.K = splits, M, N, K
        self.offsets = torch.tensor(offs, dtype=torch.int32, device=device)
        self.partial = torch.empty(splits, M, N, dtype=torch.float32, device=device)
        self.dtype = dtype

    def run(self, a, b, out16, *, a_mn=False, b_mn=False, block_n=0):
        """``out16[:M] = A @ B^T`` for the first ``a`` rows given (M may be smaller than planned)."""
        M = a.shape[1] if a_mn else a.shape[0]
        N = self.N
        part = self.partial[:, :M, :] if M == self.M else self.partial.view(-1)[:self.splits * M * N].view(self.splits, M, N)
        g = _base_args(a, b, M, N, 0, a_mn, b_mn, part, block_n or (64 if N % 128 else 128))
        g.epilogue = EPI_STORE
        g.mode = 2
        g.seg_offsets = self.offsets.data_ptr()
        g.groups = self.splits
        g.out_group_stride = M * N
        g.ldo = N
        _launch(g)
        rc = _lib.lib().gb_splitk_reduce(ctypes.c_void_p(part.data_ptr()), ctypes.c_int(self.splits),
                                         ctypes.c_longlong(M * N), ctypes.c_void_p(out16.data_ptr()),
                                         ctypes.c_int(int(out16.dtype == torch.bfloat16)), _lib.stream_ptr())
        _lib.check_rc(rc, "gb_splitk_reduce")
        return out16


_WGRAD_PLANS = {}


def gemm_wgrad(a, b, grad):
    """``grad += a^T @ b`` for a weight gradient: ``a`` is ``[tokens, M]``, ``b`` is ``[tokens, N]``, ``grad`` is
    contiguous fp32 ``[M, N]``.  A product with few output tiles and a long token dimension (the attention
    projections: 36-60 tiles for 148 SMs) is split over the tokens: ``splits`` CTAs per tile write fp32 partials and
    a second kernel adds them to ``grad`` in a fixed order (measured 60 us -> 23-36 us on the pro_1b shapes).
    Everything else takes the plain accumulate path."""
    Kt, M = a.shape
    N = b.shape[1]
    splittable = not (Kt % 64 or not grad.is_contiguous() or grad.shape != (M, N) or (M * N) % 4)
    use_pair = False
    if PAIR_ENABLED and splittable and pair_tiles(M, N) < PAIR_MIN_TILES:
        # two-CTA tiles: the split count that best fills the 74 CTA pairs (at most 8 partials, 1024 tokens or more each)
        t, best = pair_tiles(M, N), (0.0, 1)
        for sp in range(1, 9):
            if sp > 1 and Kt // sp < 1024:
                break
            eff = t * sp / (-(-t * sp // 74) * 74.0)
            if eff > best[0] + 0.04:
                best = (eff, sp)
        if best[1] >= 2 and t * best[1] >= 30:
            use_pair, splits = True, best[1]
    if not use_pair:
        tiles = ((M + 127) // 128) * ((N + 127) // 128)
        splits = min(8, 148 // max(1, tiles), Kt // 1024)
        if splits < 2 or not splittable:
            return gemm(a, b, a_mn=True, b_mn=True, out=grad, addend=grad)
    key = (M, N, Kt, splits, a.device.index)
    plan = _WGRAD_PLANS.get(key)
    if plan is None:
        kc = (Kt // splits + 63) // 64 * 64
        offs = [min(Kt, i * kc) for i in range(splits)] + [Kt]
        plan = (torch.tensor(offs, dtype=torch.int32, device=a.device),
                torch.empty(splits, M, N, dtype=torch.float32, device=a.device))
        _WGRAD_PLANS[key] = plan
    offsets, part = plan
    g = _base_args(a, b, M, N, 0, True, True, part, 128)
    g.epilogue = EPI_STORE
    g.mode = 2
    g.pair = int(use_pair)
    g.seg_offsets = offsets.data_ptr()
    g.groups = splits
    g.out_group_stride = M * N
    g.ldo = N
    _launch(g)
    rc = _lib.lib().gb_splitk_accumulate(ctypes.c_void_p(part.data_ptr()), ctypes.c_int(splits), ctypes.c_longlong(M * N),
                                         ctypes.c_void_p(grad.data_ptr()), _lib.stream_ptr())
    _lib.check_rc(rc, "gb_splitk_accumulate")
    return grad


def interleave_gate_up(gate, up, block=64):
    """``[.., E, d]`` gate and up -> ``[.., 2E, d]`` with rows interleaved in blocks of ``block``."""
    *lead, E, d = gate.shape
    g = gate.reshape(*lead, E // block, 1, block, d)
    u = up.reshape(*lead, E // block, 1, block, d)
    return torch.cat([g, u], dim=-3).reshape(*lead, 2 * E, d)


def deinterleave_gate_up(gu, block=64):
    """Inverse of :func:`interleave_gate_up` along the second-to-last dim."""
    *lead, E2, d = gu.shape
    v = gu.reshape(*lead, E2 // (2 * block), 2, block, d)
    return v[..., 0, :, :].reshape(*lead, E2 // 2, d), v[..., 1, :, :].reshape(*lead, E2 // 2, d)


def interleave_cols(g, u, block=64):
    """Column version for activations: ``[M, E]`` x2 -> ``[M, 2E]`` interleaved in blocks of 64."""
    M, E = g.shape
    return torch.stack([g.reshape(M, E // block, block), u.reshape(M, E // block, block)], dim=2).reshape(M, 2 * E)


def deinterleave_cols(gu, block=64):
    M, E2 = gu.shape
    v = gu.reshape(M, E2 // (2 * block), 2, block)
    return v[:, :, 0, :].reshape(M, E2 // 2), v[:, :, 1, :].reshape(M, E2 // 2)
