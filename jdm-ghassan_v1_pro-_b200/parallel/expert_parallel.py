"""Expert parallelism for the MoE feed-forward block, over NVSwitch peer memory.

The reference keeps every expert on every GPU and loops over them (cuda/moe.cu:734-751); data parallelism is its only
strategy.  Here the routed experts are divided among the ranks of a group (expert e belongs to rank
``e // (num_experts // world)``); the shared expert and everything outside the MoE block stay data parallel.

Per layer, forward:
  route locally -> barrier -> plan + pull the rows of the own experts from every rank (peer loads) ->
  gate/up GEMM + SwiGLU -> down GEMM whose epilogue stores each 128-row tile into the *source* rank's buffer
  (peer stores from the tcgen05 epilogue) -> barrier -> combine locally.
Backward mirrors it: the gradient rows are pulled, the weight gradients of the own experts are formed from *all*
ranks' rows, and the input-gradient GEMM's epilogue stores into the source ranks' buffers.

Weights stay replicated, so the data-parallel gradient exchange is unchanged: an expert's gradient is complete on
its owner and zero elsewhere, and the cross-rank sum gives what data parallelism gives (up to fp32 reassociation).
The forward result is bit-identical to the replicated computation: a GEMM row does not depend on its neighbours.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import comm as C
from ..ops import ep as EP
from ..ops import gemm as G
from ..ops import kernels as K
from .grad_sync import LocalBuffers, SymmetricBuffers

BARRIER_SPINS = 20 * 1000 * 1000         # polls of roughly half a microsecond each: about ten seconds; ranks may drift by a
                                         # data-loader stall, not by more


class ExpertParallel:
    def __init__(self, model, buffers=None, capacity: float = 2.0, train: bool = True):
        cfg = model.cfg
        if not cfg.use_moe:
            raise ValueError("expert parallelism needs a mixture-of-experts model")
        if buffers is None:
            buffers = SymmetricBuffers() if (dist.is_available() and dist.is_initialized() and
                                             dist.get_world_size() > 1) else LocalBuffers()
        self.buf, self.model = buffers, model
        self.rank, self.world = buffers.rank, buffers.world
        ne = cfg.num_experts
        if ne % self.world or ne > EP.MAX_EXPERTS or (ne // self.world) * self.world + 1 > EP.MAX_DESC:
            raise ValueError(f"{ne} experts cannot be divided among {self.world} ranks")
        self.ne, self.ne1, self.shared = ne, model.layout.ne1, bool(cfg.moe_shared)
        d, E, N, dt, dev = cfg.hidden_size, model.layout.Eff, model.N, model.dtype, model.dev
        self.d, self.E = d, E
        cap_local = model.layers[0].ws.cap                                  # rows of one rank's grouped layout
        routed_all = self.world * (N * cfg.moe_top_k)
        want = int(min(self.world, max(1.0, capacity)) * N * cfg.moe_top_k) + (N if self.shared else 0)
        want = min(want, routed_all + N) + 256 * ((ne // self.world) * self.world + 1)   # segments are padded to 256 rows
        self.cap = (want + 255) // 256 * 256
        nl = len(model.layers)
        esz = torch.empty(0, dtype=dt).element_size()
        # ---- symmetric: what peers read (grouped rows, their offsets) and what peers write (results)
        flat, self.t_xperm = buffers.alloc(cap_local * d, dt)
        self.xperm = flat.view(cap_local, d)
        flat, t_y = buffers.alloc(nl * cap_local * d, dt)
        self.yperm = flat.view(nl, cap_local, d)
        y_bases = t_y.cpu().tolist()
        self.base_y = [torch.tensor([b + l * cap_local * d * esz for b in y_bases], dtype=torch.int64, device=dev) for l in range(nl)]
        seg, self.t_seg = buffers.alloc(64 * ((self.ne1 + 2 + 63) // 64), torch.int32)
        self.seg = seg
        ctl, self.t_ctl = buffers.alloc(C.CTL_WORDS, torch.int32)
        self.ctl = ctl
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        c16 = dict(dtype=dt, device=dev)
        self.plans = [EP.Plan(self.ne1, self.cap, dev) for _ in range(nl)]
        self.xrecv = [torch.zeros(self.cap, d, **c16) for _ in range(nl)]
        self.act = [torch.zeros(self.cap, E, **c16) for _ in range(nl)]
        self.gu = [torch.zeros(self.cap, 2 * E, **c16) for _ in range(nl)] if train else None
        if train:
            flat, self.t_dyperm = buffers.alloc(cap_local * d, dt)
            self.dy_perm = flat.view(cap_local, d)
            flat, self.t_dxperm = buffers.alloc(cap_local * d, dt)
            self.dxperm = flat.view(cap_local, d)
            self.base_dx = self.t_dxperm
            self.dyrecv = torch.zeros(self.cap, d, **c16)
            self.dgu = torch.zeros(self.cap, 2 * E, **c16)
        else:
            self.base_dx = self.base_y[0]              # never written in evaluation: the backward tables are unused
        # the model's own per-layer buffers that this scheme replaces
        for l, b in enumerate(model.layers):
            b.yperm = self.yperm[l]
            b.xperm = self.xperm
            b.gu = self.gu[l] if train else None
            b.act = self.act[l]
        if train and hasattr(model, "tmp"):
            model.tmp.dy_perm, model.tmp.dxperm, model.tmp.dgu = self.dy_perm, self.dxperm, self.dgu
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()

    # ------------------------------------------------------------------ pieces
    def _barrier(self):
        if self.world > 1:
            EP.barrier_auto(self.t_ctl, self.rank, self.world, self.counter, BARRIER_SPINS)

    def owner(self, expert: int) -> int:
        return expert // (self.ne // self.world)

    # ------------------------------------------------------------------ forward of layer l (called by CudaModel)
    def forward(self, l: int, b, x_out, train: bool, want_aux: bool):
        m, cfg = self.model, self.model.cfg
        p = f"L{l}."
        li = min(l, len(self.plans) - 1)            # a model built for evaluation only keeps one layer's buffers
        plan = self.plans[li]
        bias = m.moe_bias[l] if m.moe_bias is not None else None
        counts = m.bias_counts[l] if (train and m.bias_counts is not None) else None
        jit = cfg.moe_jitter if train else 0.0
        K.moe_route_group(b.ws, b.xb2, m.w(p + "router"), bias, self.xperm, counts, jitter=jit,
                          seed_dev=m.seed_dev if jit > 0 else None, want_aux=want_aux,
                          aux_acc=m.aux_acc if want_aux else None, seg_weight=m.dyn_segw if want_aux else None)
        self.seg[:self.ne1 + 1].copy_(b.ws.seg_offsets[:self.ne1 + 1])
        self._barrier()                                    # every rank's rows and offsets are in place
        EP.plan(plan, self.rank, self.world, self.ne, self.shared, self.t_seg, self.base_y[li], self.base_dx,
                self.d * self.xperm.element_size(), self.d * self.xperm.element_size())
        EP.pull(self.t_xperm, self.xrecv[li], plan)
        G.gemm_swiglu(self.xrecv[li], m.w16(p + "w_gu"), act_out=self.act[li], gu_out=self.gu[li] if train else None,
                      tile_expert=plan.tile_expert, num_m_tiles=plan.num_tiles, group_rows=2 * self.E)
        G.gemm_grouped_rows(self.act[li], m.w16(p + "w_down"), plan.tile_expert, plan.num_tiles, n=self.d,
                            group_rows=self.d, tile_out=plan.tile_out_a, ldo=self.d, out=self.yperm[li])
        self._barrier()                                    # every expert output has landed in its source rank
        K.moe_combine(b.ws, self.yperm[li], b.x_mid, x_out)

    # ------------------------------------------------------------------ backward of layer l
    def backward(self, l: int, b):
        m, cfg, t = self.model, self.model.cfg, self.model.tmp
        p = f"L{l}."
        plan, ws = self.plans[l], b.ws
        K.moe_combine_bwd(ws, t.dx, self.yperm[l], self.dy_perm, t.gdot)
        self._barrier()
        EP.pull(self.t_dyperm, self.dyrecv, plan)
        G.gemm_swiglu_bwd(self.dyrecv, m.w16(p + "w_down"), self.gu[l], dgu_out=self.dgu, tile_expert=plan.tile_expert,
                          num_m_tiles=plan.num_tiles, group_rows=self.d, n=self.E)
        G.gemm_grouped_reduce(self.dyrecv, self.act[l], plan.recv_seg, self.ne1, m.g(p + "w_down").view(self.ne1, self.d, self.E))
        G.gemm_grouped_rows(self.dgu, m.w16(p + "w_gu"), plan.tile_expert, plan.num_tiles, n=self.d, b_mn=True,
                            group_rows=2 * self.E, tile_out=plan.tile_out_b, ldo=self.d, out=self.dxperm)
        G.gemm_grouped_reduce(self.dgu, self.xrecv[l], plan.recv_seg, self.ne1, m.g(p + "w_gu").view(self.ne1, 2 * self.E, self.d))
        self._barrier()
        want_aux = cfg.moe_aux_scale > 0
        K.moe_router_bwd(ws, b.xb2, m.w(p + "router"), t.gdot, self.dxperm, t.dxb, m.g(p + "router"), t.part,
                         jitter=cfg.moe_jitter, seed_dev=m.seed_dev if cfg.moe_jitter > 0 else None,
                         aux_coef_dev=m.dyn_aux if want_aux else None, part2=t.part2)

    def check(self, what="expert parallel"):
        _lib.check_status(self.model.dev, what)
