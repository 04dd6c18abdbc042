"""Child process of the gloo data-parallel tests: ``python ddp_worker.py <out_dir> <data_dir> <steps>``.

Rank, world size and rendezvous come from the environment (RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT).  Each rank
trains the tiny recipe below for ``steps`` optimizer steps and writes its final weights to ``<out_dir>/rank<r>.npz``.
"""
import datetime
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

RECIPE = """
model:
  vocab_size: 320
  hidden_size: 64
  num_layers: 2
  num_heads: 4
  num_kv_heads: 2
  intermediate_size: 128
  max_seq_len: 32
  use_moe: true
  num_experts: 4
  moe_top_k: 2
  moe_expert_dim: 64
  moe_shared: true
  moe_aux_free: true
  moe_aux_scale: 0.0
training:
  optimizer: adamw
  learning_rate: 0.003
  batch_size: 2
  seq_len: 32
  grad_accum: 2
  warmup_steps: 1
  max_steps: 6
  save_every: 3
  eval_every: 0
  log_every: 100
  pack_sequences: true
  resume: none
  resume_mode: exact
"""


def build(data_dir, ckpt_dir, ddp, **over):
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.trainer import Trainer
    from ghassan_b200.utils import log as L
    from ghassan_b200.utils.config import Config
    L.set_log_level(L.WARN)
    c = Config.from_string(RECIPE)
    c.set("training.data_dir", data_dir)
    c.set("training.checkpoint_dir", ckpt_dir)
    c.set("training.ddp", "true" if ddp else "false")
    for k, v in over.items():
        c.set("training." + k, v)
    return Trainer(ModelConfig.from_config(c), TrainerConfig.from_config(c), device="cpu")


def main():
    out, data, steps = sys.argv[1], sys.argv[2], int(sys.argv[3])
    mode = sys.argv[4] if len(sys.argv) > 4 else "train"
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=float(os.environ.get("PG_TIMEOUT_S", "60"))))
    over = {"resume": os.path.join(out, "ckpt", "last.ckpt")} if mode == "resume" else {}
    tr = build(data, os.path.join(out, "ckpt"), True, **over)
    if mode == "absent":
        dist.barrier()
        if rank == 1:
            # a rank that stops between steps with nothing in flight; the others must see an error, not a hang
            tr.prefetch.stop()
            os._exit(0)
        try:
            tr.prepare()
            for _ in range(steps):
                tr.train_step()
            code = 0
        except Exception as e:                      # the collective's timeout surfaces as an exception
            open(os.path.join(out, "rank%d.err" % rank), "w").write(type(e).__name__ + ": " + str(e)[:200])
            code = 17
        tr.prefetch.stop()
        os._exit(code)
    if mode == "peer_raises":
        # rank 1 fails at the start of its third step (nothing of its own in flight); rank 0 dawdles after its second
        # step, so its next look at the heartbeat store finds the failure before it launches another collective
        import time
        from ghassan_b200.training.trainer import TrainerError
        orig = tr.train_step
        calls = [0]

        def step():
            calls[0] += 1
            if rank == 1 and calls[0] == 3:
                raise RuntimeError("injected: device lost on rank 1")
            r = orig()
            if rank == 0 and calls[0] == 2:
                time.sleep(1.5)
            return r
        tr.train_step = step
        code = 0
        try:
            tr.run()
        except TrainerError as e:
            open(os.path.join(out, "rank%d.err" % rank), "w").write("TrainerError: " + str(e)[:300])
            code = 22
        except RuntimeError as e:
            open(os.path.join(out, "rank%d.err" % rank), "w").write("RuntimeError: " + str(e)[:300])
            code = 21
        os._exit(code)
    if mode == "resume":
        tr.run()
    else:
        tr.prepare()
        tr.writer.start()
        for i in range(steps):
            tr.train_step()
            if i + 1 == 3:
                tr.save("last.ckpt")
                tr.writer.wait()
        tr.prefetch.stop()
        tr.writer.stop()
    np.savez(os.path.join(out, "rank%d_%s.npz" % (rank, mode)),
             **{n: p.detach().numpy() for n, p in tr.engine.model.named_parameters()},
             moe_bias=tr.engine.model.moe_bias.numpy(), tokens=np.array([tr.state.tokens_seen]))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
