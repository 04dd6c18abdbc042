"""Expert parallelism: the planning / dispatch / per-tile-destination kernels with several ranks emulated on one GPU
(phase by phase, so no kernel ever waits for another), and the model-level path on a single rank."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from ghassan_b200.ops import _lib, comm as C, ep as EP, gemm as G, kernels as K
    return _lib, C, EP, G, K


def _rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).cuda()


@pytest.mark.parametrize("W,shared", [(2, True), (4, True), (2, False), (1, True)])
def test_emulated_ranks_equal_local_experts(W, shared):
    L, C, EP, G, K = _ops()
    ne, top_k, d, E, N = 4, 2, 128, 64, 200
    ne1 = ne + int(shared)
    dev = torch.device("cuda")
    router = _rand(ne, d, seed=1, scale=0.5)
    w_gu = (_rand(ne1 * 2 * E, d, seed=2, scale=0.2)).half()
    w_down = (_rand(ne1 * d, E, seed=3, scale=0.2)).half()
    ws, xperm, y_ref, y_ep = [], [], [], []
    for r in range(W):
        x = _rand(N, d, seed=10 + r).half()
        w = K.MoeWorkspace(N, d, ne, top_k, shared, torch.float16, dev)
        xp = torch.zeros(w.cap, d, dtype=torch.float16, device=dev)
        K.moe_route_group(w, x, router, None, xp)
        act = torch.zeros(w.cap, E, dtype=torch.float16, device=dev)
        G.gemm_swiglu(xp, w_gu, act_out=act, tile_expert=w.tile_expert, num_m_tiles=w.num_tiles, group_rows=2 * E)
        y = torch.zeros(w.cap, d, dtype=torch.float16, device=dev)
        G.gemm_grouped_rows(act, w_down, w.tile_expert, w.num_tiles, n=d, group_rows=d, out=y)
        ws.append(w); xperm.append(xp); y_ref.append(y)
        y_ep.append(torch.full((w.cap, d), 7.0, dtype=torch.float16, device=dev))
    L.check_status(dev, "local experts")
    t_seg = C.pointer_table([w.seg_offsets.data_ptr() for w in ws], dev)
    t_x = C.pointer_table([x.data_ptr() for x in xperm], dev)
    base_y = C.pointer_table([y.data_ptr() for y in y_ep], dev)
    cap = (W * N * top_k + N + 256 * (ne + 1) + 255) // 256 * 256
    routed = 0
    for r in range(W):                                    # the owner's phase of every emulated rank, one after another
        plan = EP.Plan(ne1, cap, dev)
        EP.plan(plan, r, W, ne, shared, t_seg, base_y, base_y, d * 2, d * 2)
        xrecv = torch.zeros(cap, d, dtype=torch.float16, device=dev)
        EP.pull(t_x, xrecv, plan)
        act = torch.zeros(cap, E, dtype=torch.float16, device=dev)
        G.gemm_swiglu(xrecv, w_gu, act_out=act, tile_expert=plan.tile_expert, num_m_tiles=plan.num_tiles, group_rows=2 * E)
        G.gemm_grouped_rows(act, w_down, plan.tile_expert, plan.num_tiles, n=d, group_rows=d, tile_out=plan.tile_out_a, ldo=d)
        L.check_status(dev, "emulated rank %d" % r)
        seg = plan.recv_seg.cpu().tolist()
        nt, nd = int(plan.num_tiles), int(plan.num_desc)
        assert seg[-1] == nt * 128 and seg == sorted(seg)
        per = ne // W
        for e in range(ne):                               # only the own experts (and the shared one) have rows here
            rows = seg[e + 1] - seg[e]
            want = sum(int(w.seg_offsets[e + 1] - w.seg_offsets[e]) for w in ws) if e // per == r else 0
            assert rows == want, (r, e, rows, want)
        if shared:
            assert seg[ne + 1] - seg[ne] == int(ws[r].seg_offsets[ne + 1] - ws[r].seg_offsets[ne])
        assert nd <= per * W + 1
        te = plan.tile_expert.cpu().tolist()[:nt]
        assert te == sorted(te) and all(e // per == r or e == ne for e in te)
        routed += seg[ne] - seg[0]
    assert routed == sum(int(w.seg_offsets[ne]) for w in ws)           # every routed row was served exactly once
    for r in range(W):
        live = int(ws[r].seg_offsets[ne1])
        assert torch.equal(y_ep[r][:live], y_ref[r][:live]), r          # same kernel, same rows: bit-identical
        assert bool((y_ep[r][live:] == 7.0).all())                       # nothing was written past the live rows


def test_plan_reports_overflow_and_stays_consistent():
    L, C, EP, G, K = _ops()
    dev = torch.device("cuda")
    ne, N, d = 4, 300, 64
    ws = K.MoeWorkspace(N, d, ne, 2, True, torch.float16, dev)
    xp = torch.zeros(ws.cap, d, dtype=torch.float16, device=dev)
    K.moe_route_group(ws, _rand(N, d, seed=3).half(), _rand(ne, d, seed=4), None, xp)
    t_seg = C.pointer_table([ws.seg_offsets.data_ptr()], dev)
    base = C.pointer_table([xp.data_ptr()], dev)
    plan = EP.Plan(ne + 1, 256, dev)                       # far too small for 300 tokens x (2 + shared)
    EP.plan(plan, 0, 1, ne, True, t_seg, base, base, d * 2, d * 2)
    with pytest.raises(RuntimeError, match="302"):
        L.check_status(dev, "plan")
    assert int(plan.num_tiles) == 0 and int(plan.num_desc) == 0 and plan.recv_seg.cpu().tolist() == [0] * (ne + 2)
    L.check_status(dev, "after reset")                     # the status word was cleared by the report


def test_graph_replayable_barrier_single_rank():
    L, C, EP, G, K = _ops()
    dev = torch.device("cuda")
    ctl = torch.zeros(C.CTL_WORDS, dtype=torch.int32, device=dev)
    table = C.pointer_table([ctl.data_ptr()], dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    for _ in range(3):
        EP.barrier_auto(table, 0, 1, counter)
    L.check_status(dev, "barrier")
    assert int(counter) == 3 and int(ctl[0]) == 3
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            EP.barrier_auto(table, 0, 1, counter)
    for _ in range(4):
        g.replay()
    torch.cuda.synchronize()
    L.check_status(dev, "barrier in a graph")
    assert int(counter) == 7 and int(ctl[0]) == 7          # the epoch lives on the device: replays advance it


def _tiny_cfg():
    from ghassan_b200.models.config import ModelConfig
    c = ModelConfig(vocab_size=608, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=256,
                    max_seq_len=64, use_moe=True, num_experts=4, moe_top_k=2, moe_expert_dim=64, moe_shared=True,
                    use_qk_norm=True, moe_aux_scale=0.01)
    c.validate()
    return c


def test_model_with_one_rank_group_equals_plain_model():
    from ghassan_b200.models.cuda_model import CudaModel
    from ghassan_b200.ops import _lib
    cfg = _tiny_cfg()
    B, T = 2, 64
    ids = torch.randint(16, 608, (B, T), generator=torch.Generator().manual_seed(5), dtype=torch.int32)
    tgt = torch.roll(ids, -1, 1)
    out = []
    for use_ep in (False, True):
        m = CudaModel(cfg, B, T, torch.float16, None, 2, False, True)
        m.init_weights(7)
        if use_ep:
            m.enable_expert_parallel()
        m.zero_grad()
        m.ce_acc.zero_()
        m.dyn[0] = 64.0
        m.set_inputs(ids, tgt, None)
        m.forward_backward()
        torch.cuda.synchronize()
        _lib.check_status(m.dev, "forward/backward")
        out.append((m.ce_acc.cpu().clone(), m.Gr.cpu().clone()))
    (la, ga), (lb, gb) = out
    assert torch.equal(la, lb)                              # forward: bit-identical
    denom = float(ga.abs().max())
    assert float((ga - gb).abs().max()) <= 2e-3 * denom, float((ga - gb).abs().max()) / denom
