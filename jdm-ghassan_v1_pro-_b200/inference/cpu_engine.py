"""Inference without a GPU: the fp32 oracle model behind the engine interface the generator drives.

The reference's inference command line runs on a CPU as well as on CUDA (tools/inference_cli.cpp:120-260 there picks the
device); this engine gives the same reach to `ghassan_b200.cli.infer` on a host without a device.  It is the portable
path, not a fast one: weights are expanded to fp32 (block-quantised files are dequantised once at load, which is what the
reference's CPU kernels compute with), a token step re-runs the model over the tokens it keeps (no KV cache), sampling is
the host sampler, and scoring a window is one teacher-forced pass.  Beyond `max_len` tokens it keeps the first
`PINNED` and the most recent ones and re-encodes them at contiguous positions (the CUDA engine's ring cache keeps the
same tokens but their original rotary positions).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.reference import TorchModel

PINNED = 8


class CpuEngine:
    host_only = True                    # the generator samples on the host and never asks for CUDA events

    def __init__(self, cfg: ModelConfig, named: Dict[str, np.ndarray], batch: int = 1, max_len: int = 2048,
                 moe_bias: Optional[Sequence[np.ndarray]] = None):
        self.cfg = cfg
        self.B = int(batch)
        self.cap = int(max_len)
        self.net = TorchModel(cfg, device="cpu")
        self.net.load_named({k: np.asarray(v, dtype=np.float32) for k, v in named.items()})
        if moe_bias and cfg.use_moe and cfg.moe_aux_free:
            self.net.moe_bias = [torch.as_tensor(np.asarray(b, dtype=np.float32)) for b in moe_bias]
        self.weight_bytes = int(sum(int(np.asarray(v).size) for v in named.values()) * 4)
        self.cur_tok = torch.zeros(self.B, dtype=torch.int32)
        self.logits = torch.zeros(self.B, cfg.vocab_size)
        self.tok_log = torch.zeros(self.B, max(16, self.cap), dtype=torch.int32)
        self.hist = [[] for _ in range(self.B)]
        self.stop = []

    # ------------------------------------------------------------------ state
    def reset(self, seed: int = 0):
        self.hist = [[] for _ in range(self.B)]
        self.logits.zero_()

    def set_stop_tokens(self, ids: Sequence[int]):
        self.stop = list(ids)

    def _kept(self, h):
        if len(h) <= self.cap:
            return h
        return h[:PINNED] + h[len(h) - (self.cap - PINNED):]

    @torch.no_grad()
    def _last_logits(self):
        rows = [self._kept(h) for h in self.hist]
        T = len(rows[0])
        if T == 0 or any(len(r) != T for r in rows):
            raise ValueError("sequences of one batch advance together")
        ids = torch.tensor(rows, dtype=torch.int64).view(-1)
        lg = self.net.logits(ids, self.B, T)
        self.logits.copy_(lg.view(self.B, T, -1)[:, -1, :])

    # ------------------------------------------------------------------ the calls the generator makes
    def prefill(self, prompts: torch.Tensor):
        p = prompts.to(torch.int64)
        if p.dim() != 2 or p.shape[0] != self.B:
            raise ValueError("prefill expects [batch, tokens] ids")
        for b in range(self.B):
            self.hist[b].extend(int(t) for t in p[b].tolist())
        self._last_logits()

    def _forward_token(self):
        for b in range(self.B):
            self.hist[b].append(int(self.cur_tok[b]))
        self._last_logits()

    # ------------------------------------------------------------------ scoring in one pass
    @torch.no_grad()
    def score_window(self, ids: Sequence[int]) -> "tuple[float, int]":
        """Sum of -log p(ids[j + 1] | ids[:j + 1]) over the window, teacher-forced in one pass (sequence 0)."""
        ids = [int(i) for i in ids]
        if len(ids) < 2:
            return 0.0, 0
        if len(ids) > self.cap:
            raise ValueError("window longer than the engine's context")
        x = torch.tensor(ids, dtype=torch.int64)
        lg = self.net.logits(x, 1, len(ids)).double()
        lp = torch.log_softmax(lg[:-1], dim=-1)
        nll = -lp.gather(1, x[1:, None]).sum()
        return float(nll), len(ids) - 1

    @torch.no_grad()
    def score_batch(self, ids: Sequence[int], targets: Sequence[int], segment_ids: Optional[Sequence[int]] = None
                    ) -> "tuple[float, int]":
        """Sum over the supervised positions of CE + z-loss, and their number, for one row of a data-loader batch
        (``targets[i]`` is the token after ``ids[i]`` or negative), with the reference scorer's windowing
        (inference/generator.cpp:514-590 there): the row is cut to the model's context, then scored in independent
        chunks of 512 positions, each at its rotary offset."""
        cfg = self.cfg
        T = min(len(ids), cfg.max_seq_len)
        if T < 2:
            return 0.0, 0
        x = torch.as_tensor(np.asarray(ids[:T], dtype=np.int64))
        tg = torch.as_tensor(np.asarray(targets[:T], dtype=np.int64))
        sg = None if segment_ids is None else torch.as_tensor(np.asarray(segment_ids[:T], dtype=np.int32))
        W = self.net.lm_head_weight()
        total, count = 0.0, 0
        for off in range(0, T, 512):
            end = min(T, off + 512 + 1)
            n = end - off
            if n < 2:
                break
            tt = tg[off:end].clone()
            tt[n - 1] = -100                                   # the last position of a chunk predicts nothing in it
            h, _, _ = self.net.hidden_states(x[off:end], 1, n, None if sg is None else sg[off:end], None, pos_offset=off)
            logits = h @ W.t()
            sup = tt >= 0
            logz = torch.logsumexp(logits, dim=-1)
            picked = logits.gather(1, tt.clamp_min(0)[:, None]).squeeze(1)
            per_row = logz - picked + cfg.z_loss_scale * logz * logz
            total += float((per_row * sup).double().sum())
            count += int(sup.sum())
        return total, count

    @torch.no_grad()
    def all_logits(self, ids: Sequence[int]) -> np.ndarray:
        """Logits of every position of one prompt, [tokens, vocab] fp32 (what the reference's `logits` command dumps)."""
        x = torch.as_tensor(np.asarray(ids, dtype=np.int64))
        return self.net.logits(x, 1, len(ids)).float().numpy()
