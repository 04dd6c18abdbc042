"""Closed-form device memory of the CUDA engine for a recipe: what ``--dry-run`` prints, what the trainer's memory
guard compares with the device, and what picks the number of micro-batches per pass.  Nothing is allocated.
Plays the role of the reference's ``Model::plan_memory`` / ``workspace_plan`` (model/model.cpp:919-1238) for this
engine's buffers (``models/cuda_model.py``), which are not the reference's arenas."""
from __future__ import annotations

from ..models.config import ModelConfig
from .config import TrainerConfig


def memory_plan(m: ModelConfig, t: TrainerConfig, world: int = 1, fuse: int = 1) -> dict:
    """Closed-form device memory of the CUDA engine for this recipe (nothing is allocated)."""
    n = m.count_parameters()
    d, qd, kvd, H = m.hidden_size, m.q_dim, m.kv_dim, m.num_heads
    N = t.batch_size * fuse * t.seq_len
    E = m.moe_expert_dim if m.use_moe else m.intermediate_size
    rows = N * (m.moe_top_k + int(m.moe_shared)) + 256 * (m.num_experts + 1) if m.use_moe else N   # segments padded to 256 rows
    weights = n * 4 + n * 2                       # fp32 master + 16-bit shadow
    grads = n * 4
    moments_full = n * 4 * (2 if t.optimizer == "adamw" else 1)
    # With the fused gradient exchange a rank keeps only the moments of the shard it updates (AdamW / Lion; Muon runs
    # whole on every rank).  Rank 0 gathers them for the moment a checkpoint snapshot is taken.
    sharded = world > 1 and getattr(t, "grad_sync", "fused") == "fused" and t.optimizer != "muon"
    moments = (moments_full + world - 1) // world if sharded else moments_full
    per_layer = (N * d * 4 * 2                    # residual stream in and mid (fp32)
                 + N * d * 2 * 2                  # normalised activations (16-bit)
                 + N * (qd + 2 * kvd) * 2 + N * (qd + kvd) * 2 + N * qd * 2 + N * H * 4
                 + (rows * d * 2 * 2 if m.use_moe else 0) + rows * 2 * E * 2 + rows * E * 2
                 + (N * m.num_experts * 4 + N * m.moe_top_k * 8 if m.use_moe else 0))
    chunk = max((N + max(1, t.ce_chunks) - 1) // max(1, t.ce_chunks), min(N, 2048))
    head = chunk * ((m.vocab_size + 7) // 8 * 8) * 2 + N * d * 2
    temps = N * d * (4 + 2 * 3) + N * (2 * qd + 2 * kvd + qd + kvd) * 2 + rows * (2 * E + 2 * d) * 2
    acts = per_layer * m.num_layers + head + temps
    ckpt = n * 4 + moments_full + 4096
    return {"parameters": n, "active_per_token": m.active_parameters_per_token(), "tokens_per_pass": N,
            "weights": weights, "gradients": grads, "optimizer": moments, "activations": acts,
            "total": weights + grads + moments + acts, "checkpoint_bytes": ckpt}
