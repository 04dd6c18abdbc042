"""Fused gradient exchange kernels (reduce-scatter + norm + optimizer + all-gather) against plain PyTorch fp32.

On one GPU the ranks are emulated: every "rank" has its own buffers on the same device and the per-rank kernels run
back to back (all reduces first, then all updates), so no launch ever waits for another one.  With two or more GPUs
``test_two_gpu_*`` runs the real thing as one process per GPU.
"""
import math
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _emulated_exchange(W, total, kind, dtype, seed, inf_at=None, clip=1.0, ntok=(37, 41, 11, 5), pull=False):
    from ghassan_b200.ops import _lib, comm as C
    dev = torch.device("cuda")
    g = torch.Generator(device="cuda").manual_seed(seed)
    shard = ((total + W - 1) // W + 63) // 64 * 64
    pad = shard * W
    decay_start, f32_end = 128, 256
    P0 = torch.randn(pad, device=dev, generator=g) * 0.05
    grads = [torch.randn(pad, device=dev, generator=g) * 3.0 for _ in range(W)]
    if inf_at is not None:
        grads[1 % W][inf_at] = float("inf")
    m0 = torch.randn(pad, device=dev, generator=g) * 0.01
    v0 = torch.rand(pad, device=dev, generator=g) * 0.01
    ranks = []
    for r in range(W):
        ranks.append(dict(P=P0.clone(), W16=P0.to(dtype), Gr=grads[r].clone(), m=m0.clone(), v=v0.clone(),
                          ctl=torch.zeros(C.CTL_WORDS, dtype=torch.int32, device=dev),
                          partial=torch.zeros(C.SYNC_BLOCKS, dtype=torch.float64, device=dev),
                          ticket=torch.zeros(1, dtype=torch.int32, device=dev), out=torch.zeros(4, device=dev)))
    tab = lambda k: C.pointer_table([x[k].data_ptr() for x in ranks], dev)
    t_grad, t_master, t_w16, t_ctl = tab("Gr"), tab("P"), tab("W16"), tab("ctl")
    lr, b1, b2, eps, wd, loss_scale = 1e-2, 0.9, 0.95, 1e-8, 0.1, 64.0
    bc1, bc2 = 1 - b1, 1 - b2
    hyper = torch.tensor([lr, bc1, bc2], device=dev)
    args = []
    for r in range(W):
        a = C.SyncArgs()
        a.rank, a.world, a.shard, a.total = r, W, shard, total
        a.decay_start, a.f32_end = decay_start, f32_end
        a.peer_grad, a.peer_master, a.peer_w16, a.peer_ctl = (t_grad.data_ptr(), t_master.data_ptr(), t_w16.data_ptr(),
                                                              t_ctl.data_ptr())
        a.m, a.v = ranks[r]["m"].data_ptr(), ranks[r]["v"].data_ptr()
        a.kind, a.beta1, a.beta2, a.eps, a.wd = {"adamw": 0, "lion": 1, "none": 2}[kind], b1, b2, eps, wd
        a.local_only = int(pull)
        a.hyper = hyper.data_ptr()
        a.loss_scale, a.clip, a.ntok_local, a.epoch = loss_scale, clip, float(ntok[r]), 7
        a.partial, a.ticket, a.out = ranks[r]["partial"].data_ptr(), ranks[r]["ticket"].data_ptr(), ranks[r]["out"].data_ptr()
        a.status = _lib.status_word(dev).data_ptr()
        a.is_bf16, a.no_wait = int(dtype == torch.bfloat16), 1
        args.append(a)
    for a in args:
        C.reduce(a)
    for a in args:
        C.update(a)
    if pull:          # every rank fetches the other ranks' shards: 16-bit weights everywhere, fp32 below f32_end
        for r in range(W):
            C.gather(t_w16, ranks[r]["W16"], shard, total, r, W)
            C.gather(t_master, ranks[r]["P"], shard, f32_end, r, W)
    if kind == "none":  # the optimizer runs elsewhere: every rank fetches the reduced gradient shards instead
        for r in range(W):
            C.gather(t_grad, ranks[r]["Gr"], shard, total, r, W)
    torch.cuda.synchronize()
    _lib.check_status(dev, "emulated exchange")
    # ---- plain PyTorch reference
    gsum = torch.zeros(pad, device=dev)
    for r in range(W):
        gsum += grads[r]
    gsum[total:] = 0
    nt = float(sum(ntok[:W]))
    gs = 1.0 / (nt * loss_scale)
    gnorm = float(gsum[:total].double().pow(2).sum().sqrt()) * gs
    cs = clip / (gnorm + 1e-6) if (clip > 0 and gnorm > clip) else 1.0
    scale = gs * cs if math.isfinite(gnorm) else 0.0
    ref = dict(P=P0.clone(), m=m0.clone(), v=v0.clone())
    if scale != 0.0:
        gi = gsum * scale
        wdv = torch.zeros(pad, device=dev)
        wdv[decay_start:] = wd
        if kind == "adamw":
            ref["m"] = b1 * m0 + (1 - b1) * gi
            ref["v"] = b2 * v0 + (1 - b2) * gi * gi
            upd = (ref["m"] / bc1) / ((ref["v"] / bc2).sqrt() + eps) + wdv * P0
        else:
            c = b1 * m0 + (1 - b1) * gi
            upd = torch.sign(c) + wdv * P0
            ref["m"] = b2 * m0 + (1 - b2) * gi
        ref["P"] = P0 - lr * upd
    return ranks, ref, dict(shard=shard, total=total, f32_end=f32_end, gnorm=gnorm, scale=scale, nt=nt, P0=P0, W=W)


@pytest.mark.parametrize("pull", [False, True])
@pytest.mark.parametrize("W", [1, 2, 4])
@pytest.mark.parametrize("kind", ["adamw", "lion"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_emulated_ranks_match_reference(W, kind, dtype, pull):
    total = 64 * 37 + 8 * 3          # not a multiple of the shard size: the last shard is short
    ranks, ref, info = _emulated_exchange(W, total, kind, dtype, seed=W * 10 + (kind == "lion"), pull=pull)
    T, S = info["total"], info["shard"]
    for r, x in enumerate(ranks):
        assert float(x["out"][1]) == pytest.approx(info["gnorm"], rel=1e-5)
        assert float(x["out"][0]) == pytest.approx(info["scale"], rel=1e-5)
        assert float(x["out"][2]) == info["nt"]
        lo, hi = r * S, min(T, (r + 1) * S)
        # every rank holds the same 16-bit weights everywhere
        assert torch.equal(x["W16"][:T], ranks[0]["W16"][:T])
        assert torch.allclose(x["W16"][:T].float(), ref["P"][:T].to(dtype).float(), rtol=2e-2 if kind == "lion" else 1e-2,
                              atol=2e-3)
        # master: own shard and the fp32-consumed prefix are current
        own = slice(lo, hi)
        assert torch.allclose(x["P"][own], ref["P"][own], rtol=1e-5, atol=1e-6) or kind == "lion"
        assert torch.allclose(x["P"][:info["f32_end"]], ranks[0]["P"][:info["f32_end"]])
        assert torch.allclose(x["m"][own], ref["m"][own], rtol=1e-4, atol=1e-6)
        # outside the own shard and the fp32 prefix the master copy is untouched
        if hi < T and r + 1 < W:
            other = slice(max(hi, info["f32_end"]), T)
            if other.start < other.stop and other.start >= (r + 1) * S:
                assert torch.equal(x["P"][other], info["P0"][other])
    if kind == "lion":
        # sign updates: compare where the sign argument is not within rounding distance of zero
        x = ranks[0]
        diff = (torch.cat([ranks[r]["P"][r * S:min(T, (r + 1) * S)] for r in range(W)]) - ref["P"][:T]).abs()
        assert float((diff > 1e-6).float().mean()) < 1e-3


def test_reduction_is_reproducible_and_identical_across_ranks():
    a, _, _ = _emulated_exchange(4, 64 * 50, "adamw", torch.float16, seed=3)
    b, _, _ = _emulated_exchange(4, 64 * 50, "adamw", torch.float16, seed=3)
    for x, y in zip(a, b):
        assert torch.equal(x["W16"], y["W16"]) and torch.equal(x["out"], y["out"]) and torch.equal(x["m"], y["m"])
    assert all(torch.equal(a[0]["out"], x["out"]) for x in a)       # same norm, clip and skip decision on every rank


def test_overflow_skips_on_every_rank():
    ranks, ref, info = _emulated_exchange(2, 64 * 20, "adamw", torch.float16, seed=5, inf_at=700)
    for x in ranks:
        assert float(x["out"][0]) == 0.0 and not math.isfinite(float(x["out"][1]))
        assert torch.equal(x["P"], info["P0"]) and torch.equal(x["W16"], info["P0"].to(torch.float16))


@pytest.mark.parametrize("W", [1, 2, 4])
def test_norm_only_exchange_gathers_the_reduced_gradient(W):
    """The form Muon uses: reduce-scatter + norm, no update, then every rank pulls the other ranks' reduced shards."""
    total = 64 * 41 + 16
    ranks, ref, info = _emulated_exchange(W, total, "none", torch.float16, seed=21 + W)
    gsum = None
    for x in ranks:
        assert float(x["out"][1]) == pytest.approx(info["gnorm"], rel=1e-5)
        assert float(x["out"][0]) == pytest.approx(info["scale"], rel=1e-5)
        assert torch.equal(x["P"], info["P0"])                       # nothing was updated
        gsum = x["Gr"][:total] if gsum is None else gsum
        assert torch.equal(x["Gr"][:total], gsum)                    # the same complete sum on every rank
    assert float(gsum.double().pow(2).sum().sqrt()) / (info["nt"] * 64.0) == pytest.approx(info["gnorm"], rel=1e-6)


def test_small_allreduce():
    from ghassan_b200.ops import comm as C
    src = [torch.arange(100, device="cuda", dtype=torch.float32) * (r + 1) for r in range(3)]
    dst = torch.zeros(100, device="cuda")
    C.small_allreduce(C.pointer_table([s.data_ptr() for s in src], src[0].device), dst, 100, 3)
    torch.cuda.synchronize()
    assert torch.equal(dst, torch.arange(100, device="cuda", dtype=torch.float32) * 6)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_gpu_fused_equals_nccl(tmp_path, world):
    """The peer-memory exchange (AdamW, Lion, and the gather form that Muon uses) against the NCCL all-reduce path of
    the same engine, one process per GPU."""
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "multi_gpu_worker.py"), "parity",
           str(tmp_path)]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    said = "\n".join(l for l in p.stdout.splitlines() if any(k in l for k in ("mismatch", "differ", "disagree", "moments",
                                                                             "losses", "PARITY", "Error")))
    assert p.returncode == 0, said[-3000:] + "\n" + p.stdout[-1500:]
    assert "PARITY OK" in p.stdout, said[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_expert_parallel_equals_replicated(tmp_path):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "multi_gpu_worker.py"), "ep_parity",
           str(tmp_path)]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-3000:]
    assert "EP PARITY OK" in p.stdout, p.stdout[-3000:]


@pytest.mark.parametrize("world", [2, 8])
def test_multi_gpu_exchange_through_nvswitch_multicast(tmp_path, world):
    """`b200.grad_sync_nvls`: the reduce-scatter as multimem.ld_reduce and the distribution of the new weights as
    multimem.st, against the NCCL path.  All ranks stay for the whole test."""
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "multi_gpu_worker.py"), "nvls_parity",
           str(tmp_path)]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-3000:]
    assert "NVLS PARITY OK" in p.stdout, p.stdout[-3000:]
