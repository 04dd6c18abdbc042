#!/usr/bin/env python
"""GEMM shapes of one pro_1b training pass (32,768 tokens: 64 micro-batches of 512), timed one by one.

    python bench_gemm.py [--tokens 32768] [--iters 20] [--json out.json]

For every product of a layer's forward and backward (and the lm-head) it prints the time and TFLOP/s of
this framework's default path (``ops/gemm.py`` picks the two-CTA 256 x 256 kernel or the one-CTA kernel), of the
one-CTA kernel alone, and of the library product of the same size (``torch.matmul`` / ``torch.bmm``: cuBLAS, the
yardstick; it has no fused epilogue, so on the SwiGLU rows it does less work).  Timing: CUDA events around ``iters``
launches after 3 warm-up launches; operands rotate through enough copies that consecutive launches never find their
inputs in the 126 MB L2.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def timed(fns, iters):
    """Mean milliseconds per launch of the callables in ``fns`` used in rotation."""
    n = len(fns)
    for i in range(3):
        fns[i % n]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fns[i % n]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default="")
    ap.add_argument("--only", default="", help="comma-separated row names")
    args = ap.parse_args()
    from ghassan_b200.ops import gemm as G, _lib

    dev = "cuda"
    T = args.tokens
    d, qkv, E, V, ne1, topk1 = 768, 1280, 1280, 32000, 9, 5     # pro_1b: 8 experts top-4 + the always-on expert
    per = (T * topk1 // ne1 + 255) // 256 * 256                 # equal expert segments, padded like the router does
    R = per * ne1
    CH = max(2048, T // 4)                                       # lm-head chunk rows (ce_chunks 4)
    h = torch.float16
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, dtype=h, scale=0.05):
        return (torch.randn(*shape, device=dev, generator=g) * scale).to(dtype)

    tile_expert = torch.arange(ne1, device=dev, dtype=torch.int32).repeat_interleave(per // 128).contiguous()
    ntiles = torch.tensor([R // 128], dtype=torch.int32, device=dev)
    seg = (torch.arange(ne1 + 1, device=dev, dtype=torch.int32) * per).contiguous()

    def copies(nbytes):
        return max(2, min(8, int(400e6 // max(1, nbytes)) + 1))

    rows = []

    def add(name, flops, make, lib_make, note=""):
        if args.only and name not in args.only.split(","):
            return
        n = make(None)
        ours = [make(i) for i in range(n)]
        t_auto = timed([f[0] for f in ours], args.iters)
        t_one = timed([f[1] for f in ours], args.iters) if ours[0][1] is not None else None
        del ours
        libs = [lib_make(i) for i in range(n)]
        t_lib = timed(libs, args.iters)
        del libs
        torch.cuda.empty_cache()
        _lib.check_status(what=name)
        tf = lambda ms: flops / ms / 1e9 if ms else None
        rows.append(dict(name=name, gflop=flops / 1e9, ms=t_auto, tflops=tf(t_auto), ms_one_cta=t_one,
                         tflops_one_cta=tf(t_one), ms_cublas=t_lib, tflops_cublas=tf(t_lib),
                         ratio=t_lib / t_auto, note=note))
        r = rows[-1]
        print("%-16s %8.1f GF | ours %7.1f us %6.0f TF/s | one-CTA %s | cuBLAS %7.1f us %6.0f TF/s | ours/cuBLAS %.2f %s"
              % (name, r["gflop"], 1e3 * t_auto, r["tflops"],
                 ("%7.1f us %6.0f TF/s" % (1e3 * t_one, r["tflops_one_cta"])) if t_one else "      -            ",
                 1e3 * t_lib, r["tflops_cublas"], r["ratio"], note), flush=True)

    # ---- dense K-major / MN-major products
    def dense(name, M, N, K, a_mn=False, b_mn=False, out_dtype=h, addend=None, note=""):
        nb = (M * K + N * K) * 2 + M * N * (4 if out_dtype == torch.float32 else 2)

        def make(i):
            if i is None:
                return copies(nb)
            a = rnd(K, M) if a_mn else rnd(M, K)
            b = rnd(K, N) if b_mn else rnd(N, K)
            out = torch.zeros(M, N, device=dev, dtype=out_dtype)
            add_t = out if addend == "self" else (rnd(M, N, dtype=torch.float32) if addend == "other" else None)
            return (lambda: G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, addend=add_t),
                    lambda: G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, addend=add_t, pair=False))

        def lib(i):
            a = rnd(K, M).t() if a_mn else rnd(M, K)
            b = rnd(K, N) if b_mn else rnd(N, K).t()
            out = torch.empty(M, N, device=dev, dtype=h)
            return lambda: torch.matmul(a, b, out=out)

        add(name, 2.0 * M * N * K, make, lib, note)

    dense("qkv", T, qkv, d)
    dense("wo+res", T, d, d, out_dtype=torch.float32, addend="other")
    dense("dgrad wo", T, d, d, b_mn=True)
    dense("dgrad qkv", T, d, qkv, b_mn=True)
    dense("logits", CH, V, d)
    dense("dlogits->dh", CH, d, V, b_mn=True)
    dense("wgrad head", V, d, CH, a_mn=True, b_mn=True, out_dtype=torch.float32, addend="self")

    # ---- attention weight gradients (split over the tokens)
    def wgrad(name, M, N):
        def make(i):
            if i is None:
                return copies((M + N) * T * 2)
            a, b = rnd(T, M), rnd(T, N)
            grad = torch.zeros(M, N, device=dev)
            saved = (G.PAIR_ENABLED,)

            def one():
                G.PAIR_ENABLED = False
                try:
                    G.gemm_wgrad(a, b, grad)
                finally:
                    G.PAIR_ENABLED = saved[0]
            return (lambda: G.gemm_wgrad(a, b, grad), one)

        def lib(i):
            a, b = rnd(T, M), rnd(T, N)
            out = torch.empty(M, N, device=dev, dtype=h)
            return lambda: torch.matmul(a.t(), b, out=out)

        add(name, 2.0 * M * N * T, make, lib)

    wgrad("wgrad wo", d, d)
    wgrad("wgrad qkv", qkv, d)

    # ---- expert products over expert-sorted rows
    def grouped_lib(M_, N_, K_):
        def lib(i):
            a = rnd(ne1, M_, K_)
            b = rnd(ne1, K_, N_)
            out = torch.empty(ne1, M_, N_, device=dev, dtype=h)
            return lambda: torch.bmm(a, b, out=out)
        return lib

    def gate_up(i):
        if i is None:
            return copies(R * d * 2 + R * 3 * E * 2)
        x, w = rnd(R, d), rnd(ne1 * 2 * E, d)
        act, gu = torch.empty(R, E, device=dev, dtype=h), torch.empty(R, 2 * E, device=dev, dtype=h)
        kw = dict(act_out=act, gu_out=gu, tile_expert=tile_expert, num_m_tiles=ntiles, group_rows=2 * E)
        return (lambda: G.gemm_swiglu(x, w, **kw), lambda: G.gemm_swiglu(x, w, pair=False, **kw))

    add("gate-up+swiglu", 2.0 * R * 2 * E * d, gate_up, grouped_lib(per, 2 * E, d), "(library: no SwiGLU)")

    def down(i):
        if i is None:
            return copies(R * (E + d) * 2)
        a, w = rnd(R, E), rnd(ne1 * d, E)
        out = torch.empty(R, d, device=dev, dtype=h)
        kw = dict(n=d, group_rows=d, out=out)
        return (lambda: G.gemm_grouped_rows(a, w, tile_expert, ntiles, **kw),
                lambda: G.gemm_grouped_rows(a, w, tile_expert, ntiles, pair=False, **kw))

    add("down", 2.0 * R * d * E, down, grouped_lib(per, d, E))

    def dact(i):
        if i is None:
            return copies(R * d * 2 + R * 4 * E * 2)
        dy, w, gu = rnd(R, d), rnd(ne1 * d, E), rnd(R, 2 * E, scale=1.0)
        dgu = torch.empty(R, 2 * E, device=dev, dtype=h)
        kw = dict(dgu_out=dgu, tile_expert=tile_expert, num_m_tiles=ntiles, group_rows=d, n=E)
        return (lambda: G.gemm_swiglu_bwd(dy, w, gu, **kw), lambda: G.gemm_swiglu_bwd(dy, w, gu, pair=False, **kw))

    add("dact+swiglu'", 2.0 * R * E * d, dact, grouped_lib(per, E, d), "(library: no SwiGLU')")

    def dgrad_gu(i):
        if i is None:
            return copies(R * (2 * E + d) * 2)
        a, w = rnd(R, 2 * E), rnd(ne1 * 2 * E, d)
        out = torch.empty(R, d, device=dev, dtype=h)
        kw = dict(n=d, b_mn=True, group_rows=2 * E, out=out)
        return (lambda: G.gemm_grouped_rows(a, w, tile_expert, ntiles, **kw),
                lambda: G.gemm_grouped_rows(a, w, tile_expert, ntiles, pair=False, **kw))

    add("dgrad gate-up", 2.0 * R * d * 2 * E, dgrad_gu, grouped_lib(per, d, 2 * E))

    def grouped_wgrad(name, M_, N_):
        def make(i):
            if i is None:
                return copies(R * (M_ + N_) * 2)
            a, b = rnd(R, M_), rnd(R, N_)
            out = torch.zeros(ne1, M_, N_, device=dev)
            return (lambda: G.gemm_grouped_reduce(a, b, seg, ne1, out),
                    lambda: G.gemm_grouped_reduce(a, b, seg, ne1, out, pair=False))

        def lib(i):
            a, b = rnd(ne1, per, M_), rnd(ne1, per, N_)
            out = torch.empty(ne1, M_, N_, device=dev, dtype=h)
            return lambda: torch.bmm(a.transpose(1, 2), b, out=out)

        add(name, 2.0 * R * M_ * N_, make, lib)

    grouped_wgrad("wgrad gate-up", 2 * E, d)
    grouped_wgrad("wgrad down", d, E)

    tot = sum(r["ms"] for r in rows)
    tot_lib = sum(r["ms_cublas"] for r in rows)
    print("sum of rows: ours %.2f ms, cuBLAS %.2f ms" % (tot, tot_lib))
    if args.json:
        os.makedirs(os.path.dirname(os.path.abspath(args.json)), exist_ok=True)
        with open(args.json, "w") as f:
            json.dump(dict(tokens=T, iters=args.iters, rows=rows, device=torch.cuda.get_device_name(0)), f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
