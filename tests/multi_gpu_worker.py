"""One process per GPU (launched by torchrun): ``multi_gpu_worker.py <mode> <work_dir>``.

parity      train a small MoE model for a few steps twice, once with the fused peer-memory gradient exchange and
            once with the NCCL all-reduce path, from the same seed and data; weights must agree.
ep_parity   the same model trained with the routed experts divided among the ranks (peer-memory dispatch, combine in
            the GEMM epilogue) and with replicated experts: same losses, same weights.
bench_sync  time the exchange alone on buffers of the pro_1b size (device time, max over ranks) against one NCCL
            all-reduce of the same gradient buffer.
"""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

RECIPE = """
model:
  vocab_size: 608
  hidden_size: 128
  num_layers: 2
  num_heads: 4
  num_kv_heads: 2
  intermediate_size: 256
  max_seq_len: 64
  use_moe: true
  num_experts: 4
  moe_top_k: 2
  moe_expert_dim: 64
  moe_shared: true
  use_qk_norm: true
  moe_aux_free: true
  moe_aux_scale: 0.0
training:
  optimizer: adamw
  learning_rate: 0.002
  batch_size: 2
  seq_len: 64
  grad_accum: 2
  warmup_steps: 1
  max_steps: 8
  save_every: 1000
  eval_every: 0
  log_every: 100
  loss_scale_init: 256
  loss_scale_max: 256
  pack_sequences: true
  resume: none
  ddp: true
"""


def make_shards(d, vocab):
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.data.loader import write_shard
    r = H.Rng(11)
    docs = []
    for _ in range(300):
        a = np.empty(30 + int(r.below(150)), dtype=np.int32)
        r.fill_uniform_ids(a, vocab - 16)
        docs.append(a + 16)
    write_shard(os.path.join(d, "train_0000.gbin"), docs, vocab, None)


def run_engine(work, sync, steps=5, opt="adamw", extra=None):
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer
    from ghassan_b200.utils import log as L
    from ghassan_b200.utils.config import Config
    L.set_log_level(L.WARN)
    c = Config.from_string(RECIPE)
    c.set("training.data_dir", work)
    c.set("training.checkpoint_dir", os.path.join(work, "ck_" + sync))
    c.set("training.optimizer", opt)
    c.set("b200.grad_sync", sync)
    for k, v in (extra or {}).items():
        c.set(k, v)
    tr = Trainer(ModelConfig.from_config(c), TrainerConfig.from_config(c), device="cuda")
    tr.prepare()
    out = []
    for _ in range(steps):
        res, _, _ = tr.train_step()
        out.append((res.loss, res.gnorm, res.ntok_global, res.applied))
    tr.engine.prepare_export()
    named = dict(tr.engine.export_weights())
    bias = tr.engine.export_moe_bias()
    tr.prefetch.stop()
    return out, named, bias, tr


def parity(work):
    rank = dist.get_rank()
    if rank == 0:
        os.makedirs(work, exist_ok=True)
        make_shards(work, 608)
    dist.barrier()
    ok = True
    for opt in ("adamw", "lion"):
        # AdamW turns a last-bit difference of one update into a different top-k choice for a token near a routing tie,
        # and from there the two runs drift (measured: identical after 1 step, 2e-2 after 5); two steps compare the
        # arithmetic, not the chaos.  Lion's sign update hides last-bit differences, so it gets the longer run.
        steps = 2 if opt == "adamw" else 5
        a, wa, ba, tra = run_engine(work, "fused", steps=steps, opt=opt)
        assert tra.engine.grad_sync is not None, "fused path not taken"
        b, wb, bb, _ = run_engine(work, "nccl", steps=steps, opt=opt)
        for (la, ga, na, apa), (lb, gb_, nb, apb) in zip(a, b):
            if na != nb or apa != apb or abs(la - lb) > 2e-3 * max(1.0, abs(lb)) or abs(ga - gb_) > 2e-2 * max(1e-3, abs(gb_)):
                print(rank, opt, "step mismatch", (la, ga, na, apa), (lb, gb_, nb, apb), flush=True)
                ok = False
        worst = 0.0
        for n in wb:
            d = float(np.abs(wa[n] - wb[n]).max()) / (float(np.abs(wb[n]).max()) + 1e-9)
            worst = max(worst, d)
        tol = 2e-2 if opt == "lion" else 2e-3      # sign updates amplify last-bit differences of the reduced gradient
        if worst > tol:
            print(rank, opt, "weights differ", worst, flush=True)
            ok = False
        for x, y in zip(ba, bb):
            if np.abs(x - y).max() > 1e-6:
                ok = False
        # every rank must hold the same exported state
        digest = torch.tensor([float(np.float64(sum(float(np.asarray(v, dtype=np.float64).sum()) for v in wa.values())))],
                              dtype=torch.float64, device="cuda")
        both = [torch.zeros_like(digest) for _ in range(dist.get_world_size())]
        dist.all_gather(both, digest)
        if any(float(x) != float(both[0]) for x in both):
            print(rank, opt, "ranks disagree", [float(x) for x in both], flush=True)
            ok = False
        print(rank, opt, "losses", [round(x[0], 4) for x in a], "worst rel weight diff", worst, flush=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("PARITY OK" if int(flag) else "PARITY FAILED", flush=True)
    return 0 if int(flag) else 1


def ep_parity(work):
    rank, world = dist.get_rank(), dist.get_world_size()
    if rank == 0:
        os.makedirs(work, exist_ok=True)
        make_shards(work, 608)
    dist.barrier()
    ok = True
    # Lion for the long runs and AdamW for two steps only, for the reason given in parity()
    for graphs, opt, steps in (("false", "lion", 5), ("true", "lion", 5), ("true", "adamw", 2)):
        a, wa, _, tra = run_engine(work, "fused", steps=steps, opt=opt,
                                   extra={"b200.ep_size": str(world), "b200.cuda_graphs": graphs,
                                          "training.checkpoint_dir": os.path.join(work, "ck_ep" + graphs + opt)})
        assert tra.engine.expert_parallel is not None, "expert-parallel path not taken"
        tra.engine.expert_parallel.check("expert parallel run")
        b, wb, _, _ = run_engine(work, "fused", steps=steps, opt=opt, extra={"b200.cuda_graphs": graphs})
        for (la, ga, na, apa), (lb, gb_, nb, apb) in zip(a, b):
            if na != nb or apa != apb or abs(la - lb) > 1e-3 * max(1.0, abs(lb)) or abs(ga - gb_) > 2e-2 * max(1e-3, abs(gb_)):
                print(rank, "step mismatch", (la, ga, na, apa), (lb, gb_, nb, apb), flush=True)
                ok = False
        if a[0][0] != b[0][0]:                       # the first forward pass sees identical weights: bit-equal loss
            print(rank, "first loss differs", a[0][0], b[0][0], flush=True)
            ok = False
        worst = max(float(np.abs(wa[n] - wb[n]).max()) / (float(np.abs(wb[n]).max()) + 1e-9) for n in wb)
        # Lion's weights come out identical; AdamW divides by sqrt(v), which turns the reassociated sums of the
        # owner-side weight gradients into visible differences on near-zero elements already at the second step
        if worst > 2e-2:
            print(rank, "weights differ", worst, flush=True)
            ok = False
        print(rank, "graphs", graphs, opt, "losses", [round(x[0], 4) for x in a], "vs", [round(x[0], 4) for x in b],
              "worst rel weight diff", worst, flush=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EP PARITY OK" if int(flag) else "EP PARITY FAILED", flush=True)
    return 0 if int(flag) else 1


def bench_sync(work, total=1_036_995_840):
    from ghassan_b200.ops import _lib, comm as C
    from ghassan_b200.parallel.grad_sync import SymmetricBuffers
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    total = (total + 63) // 64 * 64
    buf = SymmetricBuffers()
    shard = ((total + world - 1) // world + 63) // 64 * 64
    pad = shard * world
    P, tP = buf.alloc(pad, torch.float32)
    W16, tW = buf.alloc(pad, torch.float16)
    Gr, tG = buf.alloc(pad, torch.float32)
    ctl, tC = buf.alloc(C.CTL_WORDS, torch.int32)
    Gr.normal_()
    m = torch.zeros(pad, device=dev)
    partial = torch.zeros(C.SYNC_BLOCKS, dtype=torch.float64, device=dev)
    ticket = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(4, device=dev)
    hyper = torch.tensor([1e-5, 0.1, 0.01], device=dev)
    a = C.SyncArgs()
    a.rank, a.world, a.shard, a.total = rank, world, shard, total
    a.decay_start, a.f32_end = 25_000_000 // 64 * 64, 25_400_000 // 64 * 64
    a.peer_grad, a.peer_master, a.peer_w16, a.peer_ctl = tG.data_ptr(), tP.data_ptr(), tW.data_ptr(), tC.data_ptr()
    a.m, a.v, a.kind = m.data_ptr(), None, 1
    a.beta1, a.beta2, a.eps, a.wd = 0.9, 0.99, 1e-8, 0.1
    a.hyper, a.loss_scale, a.clip, a.ntok_local = hyper.data_ptr(), 1024.0, 1.0, 32768.0
    a.partial, a.ticket, a.out = partial.data_ptr(), ticket.data_ptr(), out.data_ptr()
    a.status = _lib.status_word(dev).data_ptr()
    a.is_bf16, a.no_wait = 0, 0
    be = 0

    def exchange(epoch):
        nonlocal be
        a.epoch = epoch
        be += 1
        C.barrier(tC, rank, world, be)
        C.reduce(a)
        C.update(a)
        be += 1
        C.barrier(tC, rank, world, be)

    torch.cuda.synchronize()
    dist.barrier()
    for e in range(1, 4):
        exchange(e)
    torch.cuda.synchronize()
    _lib.check_status(dev, "bench exchange")
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = 5
    e0.record()
    for e in range(4, 4 + iters):
        exchange(e)
    e1.record()
    torch.cuda.synchronize()
    fused_ms = e0.elapsed_time(e1) / iters
    # the two phases on their own (events around each kernel of one more run of exchanges)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(iters)]
    for k, e in enumerate(range(4 + iters, 4 + 2 * iters)):
        a.epoch = e
        be += 1
        C.barrier(tC, rank, world, be)
        ev[k][0].record()
        C.reduce(a)
        ev[k][1].record()
        C.update(a)
        ev[k][2].record()
        be += 1
        C.barrier(tC, rank, world, be)
        ev[k][3].record()
    torch.cuda.synchronize()
    reduce_ms = sum(x[0].elapsed_time(x[1]) for x in ev) / iters
    update_ms = sum(x[1].elapsed_time(x[2]) for x in ev) / iters
    g2 = torch.randn(total, device=dev)
    for _ in range(2):
        dist.all_reduce(g2)
    torch.cuda.synchronize()
    dist.barrier()
    e0.record()
    for _ in range(iters):
        dist.all_reduce(g2)
    e1.record()
    torch.cuda.synchronize()
    nccl_ms = e0.elapsed_time(e1) / iters
    t = torch.tensor([fused_ms, nccl_ms, reduce_ms, update_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    fused_ms, nccl_ms, reduce_ms, update_ms = (float(x) for x in t)
    # bytes that must cross NVLink per rank: read (W-1) peers' shard as fp32, write the shard as 16-bit to (W-1) peers
    nv_in = (world - 1) * shard * 4
    nv_out = (world - 1) * (shard * 2 + min(shard, a.f32_end) * 4 / world)
    link = 770e9
    roof_ms = max(nv_in, nv_out) / link * 1e3
    if rank == 0:
        print(json.dumps({"bench": "fused_grad_sync", "world": world, "elements": total, "fused_ms": fused_ms,
                          "nccl_allreduce_only_ms": nccl_ms, "reduce_scatter_phase_ms": reduce_ms,
                          "update_allgather_phase_ms": update_ms, "nvlink_in_bytes_per_rank": nv_in,
                          "nvlink_out_bytes_per_rank": nv_out, "roofline_ms_at_770GBs": roof_ms,
                          "fraction_of_roofline": roof_ms / fused_ms,
                          "note": "fused = barrier + reduce-scatter + norm + mailbox + Lion update + 16-bit all-gather + "
                                  "barrier; the NCCL figure is the all-reduce alone (no norm, no optimizer)"}), flush=True)
    return 0


def main():
    mode, work = sys.argv[1], sys.argv[2]
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rc = {"parity": parity, "ep_parity": ep_parity, "bench_sync": bench_sync}[mode](work)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(rc)


if __name__ == "__main__":
    main()
