"""Muon on the GPU (training/muon_cuda.py + csrc/cuda/muon.cu + the tcgen05 GEMM) against the fp32 reference
implementation of the same rule (training/optim.py, which restates training/optimizer.cpp:385-455)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(min_ns_dim=0, d=128, E=64, ne=4, layers=2, tie=True):
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.models.cuda_model import CudaModel
    from ghassan_b200.training.config import TrainerConfig
    from ghassan_b200.training.muon_cuda import MuonCuda
    cfg = ModelConfig(vocab_size=608, hidden_size=d, num_layers=layers, num_heads=4, num_kv_heads=2, max_seq_len=64,
                      use_moe=True, num_experts=ne, moe_top_k=2, moe_expert_dim=E, moe_shared=True, use_qk_norm=True,
                      tie_embeddings=tie)
    t = TrainerConfig()
    t.optimizer, t.learning_rate, t.weight_decay, t.muon_min_ns_dim, t.muon_ns_steps = "muon", 0.02, 0.1, min_ns_dim, 5
    model = CudaModel(cfg, 2, 64, torch.float16, "cuda", train=True)
    model.init_weights(7)
    opt = MuonCuda(model, cfg, t)
    return cfg, t, model, opt


def _oracle(cfg, t, named_w, named_g, steps_scale):
    """The CPU rule on copies of the same weights / gradients; returns the optimizer after the given steps."""
    from ghassan_b200.training import optim as O
    specs = list(cfg.param_specs())
    params = [O.OptParam(s.name, named_w[s.name].clone().float().cpu(), s.decay) for s in specs]
    opt = O.Muon(params, t.learning_rate, t.muon_vec_ratio, t.beta1, t.beta2, t.eps, t.weight_decay, t.grad_clip,
                 t.muon_ns_steps, t.muon_min_ns_dim)
    for scale in steps_scale:
        for p in params:
            p.w.grad = named_g[p.name].clone().float().cpu()
        opt.grad_clip = 0.0                       # the clip factor is part of `scale` here
        opt.step(t.learning_rate, scale)
    return opt, {p.name: p.w for p in params}


@pytest.mark.parametrize("min_ns_dim", [0, 100])
def test_muon_step_matches_the_fp32_rule(min_ns_dim):
    cfg, t, model, opt = _setup(min_ns_dim)
    g = torch.Generator(device="cuda").manual_seed(3)
    model.Gr.copy_(torch.randn(model.layout.total, device="cuda", generator=g) * 0.3)
    named_w0 = {k: v.clone() for k, v in model.layout.from_internal(model.P).items()}
    named_g = {k: v.clone() for k, v in model.layout.from_internal(model.Gr).items()}
    scale = torch.tensor([0.5], device="cuda")
    for _ in range(2):                             # second step exercises the momentum carried over
        opt.launch(t.learning_rate, scale)
        opt.t += 1
    from ghassan_b200.ops import _lib
    _lib.check_status(what="muon")
    ref_opt, ref_w = _oracle(cfg, t, named_w0, named_g, [0.5, 0.5])
    got_w = model.layout.from_internal(model.P)
    n_ns = 0
    for s in cfg.param_specs():
        w0, wr, wg = named_w0[s.name].float().cpu(), ref_w[s.name], got_w[s.name].float().cpu()
        d_ref, d_got = wr - w0, wg - w0
        rel = float((d_got - d_ref).norm() / (d_ref.norm() + 1e-12))
        if opt.rule[s.name] == "ns":
            n_ns += 1
            assert rel < 2e-2, (s.name, rel)      # bf16 GEMM operands inside Newton-Schulz, fp32 everything else
        else:
            assert rel < 1e-4, (s.name, opt.rule[s.name], rel)
    assert n_ns > 0
    # the 16-bit shadow follows the master weights
    assert torch.equal(model.W16, model.P.to(model.W16.dtype))
    # state: reference layout, momentum of NS matrices equals the rule's, second moments only for vectors
    blob = opt.export_state()
    specs = list(cfg.param_specs())
    assert blob["kind"] == "muon" and blob["t"] == 2 and len(blob["m"]) == len(specs)
    for i, s in enumerate(specs):
        assert np.allclose(blob["m"][i], ref_opt.m[i].numpy().reshape(-1), rtol=1e-4, atol=1e-6), s.name
        assert (blob["v"][i] is not None) == (len(s.shape) == 1), s.name
        if blob["v"][i] is not None:
            assert np.allclose(blob["v"][i], ref_opt.v[i].numpy().reshape(-1), rtol=1e-4, atol=1e-9), s.name


def test_rejected_step_changes_nothing_and_state_round_trips():
    cfg, t, model, opt = _setup()
    model.Gr.normal_()
    opt.launch(t.learning_rate, torch.tensor([1.0], device="cuda"))
    opt.t += 1
    w, blob = model.P.clone(), opt.export_state()
    opt.launch(t.learning_rate, torch.zeros(1, device="cuda"))          # scale 0 = overflow / nothing supervised
    assert torch.equal(model.P, w)
    again = opt.export_state()
    for a, b in zip(blob["m"], again["m"]):
        assert np.array_equal(a, b)
    cfg2, t2, model2, opt2 = _setup()
    assert opt2.import_state(blob) and opt2.t == 1
    back = opt2.export_state()
    for a, b in zip(blob["m"], back["m"]):
        assert np.array_equal(a, b)
    for a, b in zip(blob["v"], back["v"]):
        assert (a is None and b is None) or np.array_equal(a, b)
    assert not opt2.import_state({"kind": "lion", "m": []})
