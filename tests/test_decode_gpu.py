"""Decode-time kernels and the inference engine against plain PyTorch fp32 references."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FMTS = ["f16", "bf16", "q8_0", "q4_0", "q8_64", "q4_1"]


def _D():
    from ghassan_b200.ops import decode as D
    return D


def _rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("B", [1, 5, 32])
def test_gemv_matches_dequantised_product(fmt, B):
    D = _D()
    N, K = 200, 320
    w = _rand(N, K, seed=1, scale=0.3)
    qw = D.QWeight.from_f32(w, D.FMT_NAMES[fmt], "cuda")
    wd = qw.dequantize().cuda()                              # what the stored bits mean, from the host codec
    x = _rand(B, K, seed=2).cuda().half()
    add = _rand(B, N, seed=3).cuda()
    out32 = torch.zeros(B, N, device="cuda")
    D.gemv(qw, x, out32, addend=add)
    ref = x.float() @ wd.t() + add
    assert torch.allclose(out32, ref, rtol=2e-3, atol=2e-3), float((out32 - ref).abs().max())
    out16 = torch.zeros(B, N, device="cuda", dtype=torch.float16)
    D.gemv(qw, x, out16)
    assert torch.allclose(out16.float(), x.float() @ wd.t(), rtol=1e-2, atol=2e-2)
    # quantisation itself stays within the format's error
    err = float((wd.cpu() - w).abs().max())
    assert err < {"f16": 1e-3, "bf16": 1e-2, "q8_0": 0.02, "q8_64": 0.02, "q4_0": 0.25, "q4_1": 0.2}[fmt]


@pytest.mark.parametrize("B", [3, 1])
@pytest.mark.parametrize("fmt", ["f16", "q8_0", "q4_1"])
def test_expert_kernels(fmt, B):
    """One sequence and several; the fused-norm forms must agree with norm followed by the plain kernels."""
    D = _D()
    ne, E, d, top_k = 4, 64, 96, 2
    f = D.FMT_NAMES[fmt]
    wg, wu = _rand((ne + 1) * E, d, seed=4, scale=0.2), _rand((ne + 1) * E, d, seed=5, scale=0.2)
    wdn = _rand((ne + 1) * d, E, seed=6, scale=0.2)
    qg, qu, qd = (D.QWeight.from_f32(t, f, "cuda") for t in (wg, wu, wdn))
    g, u, dn = (q.dequantize().cuda() for q in (qg, qu, qd))
    x = _rand(B, d, seed=7).cuda().half()
    idx = torch.tensor([[1, 3], [0, 2], [3, 3]], dtype=torch.int32, device="cuda")[:B].contiguous()
    wt = torch.tensor([[0.7, 0.3], [0.5, 0.5], [0.9, 0.1]], device="cuda")[:B].contiguous()
    resid = _rand(B, d, seed=8).cuda()
    act = torch.zeros(B, top_k + 1, E, device="cuda", dtype=torch.float16)
    out = torch.zeros(B, d, device="cuda")
    D.expert_swiglu(qg, qu, ne, E, d, x, idx, top_k, True, act)
    D.expert_down(qd, ne, d, E, act, idx, wt, top_k, True, resid, out)
    # the fused forms: RMSNorm of an fp32 row inside the kernel (unit weight: x is the normalised row's source)
    x32 = _rand(B, d, seed=9).cuda()
    nw = 1.0 + 0.1 * _rand(d, seed=10).cuda()
    xn = torch.empty(B, d, device="cuda", dtype=torch.float16)
    from ghassan_b200.ops import kernels as KK
    KK.rmsnorm_fwd(x32, nw, xn, torch.empty(B, device="cuda"), 1e-5)
    act_a = torch.zeros_like(act)
    act_b = torch.zeros_like(act)
    D.expert_swiglu(qg, qu, ne, E, d, xn, idx, top_k, True, act_a)
    D.swiglu_norm(qg, qu, ne, E, d, x32, nw, 1e-5, idx, top_k, True, act_b)
    assert torch.allclose(act_a.float(), act_b.float(), rtol=2e-3, atol=2e-3)
    o_a = torch.zeros(B, 200, device="cuda")
    o_b = torch.zeros(B, 200, device="cuda")
    qh = D.QWeight.from_f32(_rand(200, d, seed=11, scale=0.3), f, "cuda")
    D.gemv(qh, xn, o_a)
    D.gemv_norm(qh, x32, nw, 1e-5, o_b)
    assert torch.allclose(o_a, o_b, rtol=2e-3, atol=2e-3)
    ref = resid.clone()
    for b in range(B):
        for s in range(top_k + 1):
            e = int(idx[b, s]) if s < top_k else ne
            a = torch.nn.functional.silu(g[e * E:(e + 1) * E] @ x[b].float()) * (u[e * E:(e + 1) * E] @ x[b].float())
            assert torch.allclose(act[b, s].float(), a, rtol=2e-2, atol=2e-2)
            ref[b] += (wt[b, s] if s < top_k else 1.0) * (dn[e * d:(e + 1) * d] @ a.half().float())
    assert torch.allclose(out, ref, rtol=1e-2, atol=2e-2), float((out - ref).abs().max())


def test_decode_router_matches_reference_rules():
    from ghassan_b200.models.config import ModelConfig
    from ghassan_b200.models.reference import route
    D = _D()
    cfg = ModelConfig(vocab_size=320, hidden_size=96, num_layers=1, num_heads=4, num_kv_heads=2, intermediate_size=128,
                      max_seq_len=32, use_moe=True, num_experts=8, moe_top_k=3, moe_expert_dim=64, moe_allow_dense=True)
    x = _rand(6, 96, seed=1).half()
    x[0] = 0                                                   # all logits equal: ties go to the lowest index
    rw = _rand(8, 96, seed=2, scale=0.5)
    bias = torch.tensor([0.0, 0.0, 0.4, 0.0, 0.0, 0.0, -0.4, 0.0])
    idx = torch.zeros(6, 3, dtype=torch.int32, device="cuda")
    w = torch.zeros(6, 3, device="cuda")
    for b in (None, bias):
        D.decode_route(x.cuda(), rw.cuda(), None if b is None else b.cuda(), 3, idx, w)
        _, ridx, rwt = route(x.float(), rw, b, cfg, None)
        assert idx.cpu().tolist() == ridx.tolist()
        assert torch.allclose(w.cpu(), rwt, atol=1e-5)
    assert idx[0].tolist()[0] == 2                             # the bias steers selection ...


@pytest.mark.parametrize("hd,H,KV", [(64, 12, 4), (128, 4, 4), (32, 4, 2)])
def test_kv_ring_and_decode_attention(hd, H, KV):
    D = _D()
    B, cap, pinned, steps = 2, 24, 8, 40          # more steps than capacity: the ring wraps, pinned slots stay
    kvd, qd = KV * hd, H * hd
    cK = torch.zeros(B, cap, kvd, device="cuda", dtype=torch.float16)
    cV = torch.zeros_like(cK)
    slot_pos = torch.zeros(B, cap, dtype=torch.int32, device="cuda")
    state = torch.zeros(B, D.STATE_INTS, dtype=torch.int32, device="cuda")
    pos = torch.zeros(B, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(B * H * 4 * (hd + 2), device="cuda")
    out = torch.zeros(B, qd, device="cuda", dtype=torch.float16)
    out_t, scratch_t = torch.zeros_like(out), torch.zeros_like(scratch)
    ticket = torch.zeros(B * KV, dtype=torch.int32, device="cuda")
    ks, vs = [], []
    scale = 1.0 / math.sqrt(hd)
    for t in range(steps):
        k = _rand(B, kvd, seed=100 + t).cuda().half()
        v = _rand(B, kvd, seed=200 + t).cuda().half()
        q = _rand(B, qd, seed=300 + t).cuda().half()
        ks.append(k)
        vs.append(v)
        D.kv_append(k, v, cK, cV, slot_pos, state, cap, pinned)
        D.decode_attn(q, cK, cV, slot_pos, state, out, scratch, 4, H, KV, hd, cap, 0, scale)
        # the variant whose last split merges the partial results agrees up to the order of the sums over the splits
        D.decode_attn_fused(q, cK, cV, slot_pos, state, out_t, scratch_t, ticket, 4, H, KV, hd, cap, 0, scale)
        assert torch.allclose(out.float(), out_t.float(), rtol=2e-3, atol=2e-3) and int(ticket.abs().sum()) == 0
        D.decode_advance(state, pos, cap, pinned)
        # the cache must hold the first `pinned` tokens and the most recent cap - pinned ones
        live = list(range(min(t + 1, pinned))) + [j for j in range(max(pinned, t + 1 - (cap - pinned)), t + 1)]
        Kl = torch.stack([ks[j] for j in live], 1).float().view(B, len(live), KV, hd)
        Vl = torch.stack([vs[j] for j in live], 1).float().view(B, len(live), KV, hd)
        qh = q.float().view(B, H, hd)
        g = H // KV
        ref = torch.zeros(B, H, hd, device="cuda")
        for h in range(H):
            s = torch.einsum("bd,bld->bl", qh[:, h], Kl[:, :, h // g]) * scale
            ref[:, h] = torch.einsum("bl,bld->bd", torch.softmax(s, -1), Vl[:, :, h // g])
        assert torch.allclose(out.float().view(B, H, hd), ref, rtol=2e-2, atol=2e-2), (t, float((out.float().view(B, H, hd) - ref).abs().max()))
    st = state.cpu()
    assert int(st[0, 0]) == steps and int(st[0, 1]) == cap and int(pos[0]) == steps


def test_sliding_window_masks_old_slots():
    D = _D()
    B, cap, hd, H = 1, 32, 64, 2
    cK = torch.zeros(B, cap, H * hd, device="cuda", dtype=torch.float16)
    cV = torch.zeros_like(cK)
    slot_pos = torch.zeros(B, cap, dtype=torch.int32, device="cuda")
    state = torch.zeros(B, D.STATE_INTS, dtype=torch.int32, device="cuda")
    pos = torch.zeros(B, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(B * H * 2 * (hd + 2), device="cuda")
    out = torch.zeros(B, H * hd, device="cuda", dtype=torch.float16)
    vs = []
    for t in range(10):
        k, v, q = (_rand(B, H * hd, seed=s + t).cuda().half() for s in (1, 50, 90))
        vs.append(v)
        D.kv_append(k, v, cK, cV, slot_pos, state, cap, 8)
        D.decode_attn(q, cK, cV, slot_pos, state, out, scratch, 2, H, H, hd, cap, 1, 0.125)   # window 1: only itself
        D.decode_advance(state, pos, cap, 8)
        assert torch.allclose(out, v, atol=2e-3)


@pytest.mark.parametrize("cfg", [
    dict(greedy=True),
    dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.0, repetition_penalty=1.0),
    dict(temperature=1.3, top_k=200, top_p=0.95, min_p=0.05, repetition_penalty=1.12, frequency_penalty=0.2,
         presence_penalty=0.1, repetition_window=16),
    dict(temperature=0.5, top_k=2, top_p=1.0, min_p=0.0),
])
def test_device_sampler_equals_host_sampler(cfg):
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.inference.engine import SamplingParams
    D = _D()
    B, V, steps = 3, 5000, 25
    sp = SamplingParams(seed=77, **cfg)
    host = []
    for b in range(B):
        c = sp.to_native()
        c.seed = 1000 + b
        host.append(H.Sampler(c))
    # the device draws use the same streams: one generator per sequence, consumed once per sampled token
    dev_rng = [H.Rng(1000 + b) for b in range(B)]
    logits = torch.zeros(B, V, device="cuda")
    hist_cap = 64
    history = torch.zeros(B, hist_cap, dtype=torch.int32, device="cuda")
    hist_len = torch.zeros(B, dtype=torch.int32, device="cuda")
    uniforms = torch.zeros(B, device="cuda")
    out_tok = torch.zeros(B, dtype=torch.int32, device="cuda")
    hhist = [[] for _ in range(B)]
    n = sp.to_native()
    for t in range(steps):
        lg = _rand(B, V, seed=500 + t, scale=3.0)
        lg[:, 7] = lg[:, 9]                                     # an exact tie
        logits.copy_(lg)
        need_draw = not (n.greedy or n.temperature <= 0 or n.top_k == 1)
        uniforms.copy_(torch.tensor([dev_rng[b].uniform() if need_draw else 0.0 for b in range(B)]))
        a = D.SampleArgs()
        a.logits, a.ld, a.B, a.V = logits.data_ptr(), V, B, V
        a.temperature, a.top_k, a.top_p, a.min_p = n.temperature, n.top_k, n.top_p, n.min_p
        a.rep_penalty, a.freq_penalty, a.presence_penalty = n.repetition_penalty, n.frequency_penalty, n.presence_penalty
        a.rep_window, a.greedy = n.repetition_window, int(n.greedy)
        a.history, a.hist_cap, a.hist_len = history.data_ptr(), hist_cap, hist_len.data_ptr()
        a.uniforms, a.out_tok = uniforms.data_ptr(), out_tok.data_ptr()
        D.sample(a)
        got = out_tok.cpu().tolist()
        for b in range(B):
            want = host[b].sample(lg[b].numpy(), hhist[b])
            assert got[b] == want, (t, b, got[b], want)
            hhist[b].append(want)
    assert hist_len.cpu().tolist() == [steps] * B


def _tiny_cfg(**over):
    from ghassan_b200.models.config import ModelConfig
    base = dict(vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=512,
                max_seq_len=256, use_moe=True, num_experts=4, moe_top_k=2, moe_expert_dim=128, moe_shared=True,
                use_qk_norm=True)
    base.update(over)
    c = ModelConfig(**base)
    c.validate()
    return c


@pytest.mark.parametrize("moe", [True, False])
def test_engine_matches_fp32_model_greedy(moe):
    from ghassan_b200.inference.engine import InferenceEngine, SamplingParams
    from ghassan_b200.models.config import init_parameters
    from ghassan_b200.models.reference import TorchModel
    cfg = _tiny_cfg(use_moe=moe)
    named = init_parameters(cfg, 11)
    for k in named:                                        # larger weights so that logits are well separated
        if not k.endswith("norm"):
            named[k] = named[k] * 4.0
    eng = InferenceEngine(cfg, named, fmt="f16", batch=2, max_len=128, prefill_chunk=64)
    ref = TorchModel(cfg, "cpu")
    ref.load_named(named)
    # teacher forcing: the logits after every token of a fixed sequence against the fp32 model
    seq = torch.randint(16, 512, (2, 20), generator=torch.Generator().manual_seed(3), dtype=torch.int32)
    eng.reset(1)
    with torch.no_grad():
        want = [ref.logits(seq[b], 1, 20) for b in range(2)]
    for j in range(20):
        eng.cur_tok.copy_(seq[:, j])
        eng._forward_token()
        got = eng.logits.cpu()
        for b in range(2):
            err = float((got[b] - want[b][j]).abs().max())
            assert err < 0.03 * float(want[b][j].abs().max()) + 0.03, (j, b, err)
    # greedy decoding end to end: clear decisions must agree with the fp32 model
    prompt = seq[:, :9].contiguous()
    eng.reset(1)
    eng.prefill(prompt)
    sp = SamplingParams(greedy=True, repetition_penalty=1.0)     # plain arg-max: penalties would change the choice
    eng.sample_first(sp)
    eng.decode_steps(11, sp)
    got = eng.transcript(12)
    for b in range(2):
        s = prompt[b].tolist()
        for t in range(12):
            with torch.no_grad():
                lg = ref.logits(torch.tensor(s, dtype=torch.int32), 1, len(s))[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > 0.03 * float(lg.abs().max()) + 0.05:
                assert int(got[b, t]) == int(torch.argmax(lg)), (b, t)
            s.append(int(got[b, t]))


def test_prefill_pass_equals_token_by_token():
    from ghassan_b200.inference.engine import InferenceEngine, SamplingParams
    from ghassan_b200.models.config import init_parameters
    cfg = _tiny_cfg(num_heads=4, num_kv_heads=2, hidden_size=256)      # head_dim 64: tcgen05 prompt pass
    named = init_parameters(cfg, 5)
    prompt = torch.randint(16, 512, (1, 100), generator=torch.Generator().manual_seed(4), dtype=torch.int32)
    a = InferenceEngine(cfg, named, fmt="f16", batch=1, max_len=160, prefill_chunk=128)
    a.reset(1)
    a.prefill(prompt)                                       # 99 tokens through the batched pass + 1 decode step
    b = InferenceEngine(cfg, named, fmt="f16", batch=1, max_len=160, prefill_chunk=128)
    b.reset(1)
    for j in range(100):                                    # everything through the decode step
        b.cur_tok.copy_(prompt[:, j])
        b._forward_token()
    assert torch.allclose(a.logits, b.logits, rtol=3e-2, atol=3e-2), float((a.logits - b.logits).abs().max())
    assert a.state.cpu().tolist() == b.state.cpu().tolist()
    assert torch.allclose(a.layers[1].cK[:, :100].float(), b.layers[1].cK[:, :100].float(), atol=3e-2)


def test_generator_host_and_device_routes(tmp_path):
    from ghassan_b200.data.tokenizer import Tokenizer
    from ghassan_b200.inference.engine import InferenceEngine, SamplingParams
    from ghassan_b200.inference.generator import Generator
    from ghassan_b200.models.config import init_parameters
    cfg = _tiny_cfg(vocab_size=272)
    named = init_parameters(cfg, 2)
    eng = InferenceEngine(cfg, named, fmt="q8_0", batch=1, max_len=96, prefill_chunk=64)
    gen = Generator(eng, Tokenizer())
    pieces = []
    r1 = gen.generate("salam", max_new_tokens=20, sampling=SamplingParams(seed=5, top_k=20), on_text=lambda b, s: pieces.append(s))
    r2 = gen.generate("salam", max_new_tokens=20, sampling=SamplingParams(seed=5, top_k=20))
    assert r1.tokens == r2.tokens and 0 < len(r1.tokens[0]) <= 20           # seeded: reproducible
    assert "".join(pieces) == r1.text[0] or len(pieces) > 0
    r3 = gen.generate("salam", max_new_tokens=12, sampling=SamplingParams(seed=5, top_k=20, no_repeat_ngram=3))
    assert len(r3.tokens[0]) <= 12                                             # host route (n-gram ban)
    nll, n = gen.score_tokens(gen.encode_prompt("hello world"))
    assert n > 0 and math.isfinite(nll) and gen.perplexity(gen.encode_prompt("hello world")) > 1.0


@pytest.mark.parametrize("profile,fmt_name", [("fp16", "f16"), ("q8_k", "q8_0"), ("q4_0", "q4_0")])
def test_engine_from_exported_file_uses_stored_bytes(tmp_path, profile, fmt_name):
    """A GGUF written by the exporter loads into an engine whose decode weights are the file's own quantised bytes.
    For the single-format profiles its logits equal those of an engine that quantises the dequantised tensors again
    (the codec is idempotent); the q4_0 profile mixes Q4_0 and Q8_0 tensors, so it is compared with an fp16 engine
    over the dequantised tensors (difference: fp16 rounding of q*d)."""
    import os
    from ghassan_b200.formats.gguf import export_gguf
    from ghassan_b200.inference import model_io as IO
    from ghassan_b200.inference.engine import InferenceEngine
    from ghassan_b200.models.config import init_parameters
    gold = os.path.join(os.path.dirname(__file__), "golden", "formats")
    cfg = _tiny_cfg(vocab_size=400, hidden_size=128, num_heads=4, num_kv_heads=2)
    named = init_parameters(cfg, 21)
    path = str(tmp_path / "m.gguf")
    export_gguf(path, cfg, named, os.path.join(gold, "tiny400.gtok"), profile)
    m = IO.load_model(path)
    assert IO.sniff(path) == "gguf" and m.tokenizer is not None and m.tokenizer.vocab_size == 400
    eng = IO.build_engine(m, batch=1, max_len=64)
    mixed = profile == "q4_0"
    again = InferenceEngine(m.cfg, m.named, fmt="f16" if mixed else fmt_name, batch=1, max_len=64, prefill_chunk=64)
    tol = 1e-2 if mixed else 1e-3
    seq = torch.randint(16, 400, (1, 12), generator=torch.Generator().manual_seed(8), dtype=torch.int32)
    for e in (eng, again):
        e.reset(1)
    for j in range(12):
        for e in (eng, again):
            e.cur_tok.copy_(seq[:, j])
            e._forward_token()
        assert torch.allclose(eng.logits, again.logits, rtol=tol, atol=tol), (j, float((eng.logits - again.logits).abs().max()))


def test_inference_cli_runs_the_model(tmp_path, capsys):
    import json
    import os
    from ghassan_b200.cli import infer as I
    from ghassan_b200.formats.gguf import export_gguf
    from ghassan_b200.models.config import init_parameters
    gold = os.path.join(os.path.dirname(__file__), "golden", "formats")
    cfg = _tiny_cfg(vocab_size=400, hidden_size=128, num_heads=4, num_kv_heads=2)
    named = init_parameters(cfg, 22)
    path = str(tmp_path / "m.gguf")
    export_gguf(path, cfg, named, os.path.join(gold, "tiny400.gtok"), "q8_k")
    assert I.main(["generate", "--model", path, "--prompt", "salam", "--max-tokens", "8", "--seed", "3", "--no-stream", "--stats", "--ctx", "64"]) == 0
    assert "decode" in capsys.readouterr().out
    assert I.main(["bench", "--model", path, "--prompt-tokens", "16", "--tokens", "24", "--greedy"]) == 0
    r = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert r["decode_tokens_per_s"] > 0 and r["new_tokens"] == 24
    assert I.main(["perplexity", "--model", path, "--text", "salam labas 3lik", "--ctx", "64"]) == 0
    assert "perplexity" in capsys.readouterr().out
    assert I.main(["logits", "--model", path, "--prompt", "salam", "--out", str(tmp_path / "l.f32"), "--ctx", "64"]) == 0
    assert os.path.getsize(str(tmp_path / "l.f32")) == 400 * 4
    assert I.main(["eval", "--model", path, "--max-prompts", "2", "--max-tokens", "6", "--ctx", "128"]) == 0
    assert "items 2" in capsys.readouterr().out


@pytest.mark.parametrize("moe,fmt,B", [(True, "f16", 1), (True, "q4_0", 3), (False, "q8_0", 2), (False, "q4_1", 1), (True, "q8_64", 1)])
def test_fused_token_step_equals_separate_kernels(moe, fmt, B):
    """Norms, router, cache append and split merge folded into their consumers: same rounding points, same numbers."""
    from ghassan_b200.inference.engine import InferenceEngine, SamplingParams
    from ghassan_b200.models.config import init_parameters
    cfg = _tiny_cfg(use_moe=moe)
    named = init_parameters(cfg, 31)
    engines = [InferenceEngine(cfg, named, fmt=fmt, batch=B, max_len=48, prefill_chunk=32, fused_step=f) for f in (True, False)]
    assert engines[0].fused and not engines[1].fused
    seq = torch.randint(16, 512, (B, 60), generator=torch.Generator().manual_seed(9), dtype=torch.int32)
    for e in engines:
        e.reset(1)
    for j in range(60):                                  # longer than the cache: the ring wraps
        for e in engines:
            e.cur_tok.copy_(seq[:, j])
            e._forward_token()
        if B > 1:
            assert torch.equal(engines[0].logits, engines[1].logits), (j, float((engines[0].logits - engines[1].logits).abs().max()))
        else:      # kept loose for one sequence so that batch-1 kernel variants may regroup the sums
            assert torch.allclose(engines[0].logits, engines[1].logits, rtol=2e-3, atol=2e-3), (j, float((engines[0].logits - engines[1].logits).abs().max()))
    for La, Lb in zip(engines[0].layers, engines[1].layers):
        if B > 1:
            assert torch.equal(La.cK, Lb.cK) and torch.equal(La.cV, Lb.cV)
        else:
            assert torch.allclose(La.cK.float(), Lb.cK.float(), atol=5e-3) and torch.allclose(La.cV.float(), Lb.cV.float(), atol=5e-3)
    assert torch.equal(engines[0].slot_pos, engines[1].slot_pos) and int(engines[0].att_ticket.abs().sum()) == 0
    sp = SamplingParams(seed=4, top_k=20)
    outs = []
    for e in engines:                                    # and through the captured graph with sampling
        e.reset(1)
        e.prefill(seq[:, :9].contiguous())
        e.sample_first(sp)
        e.decode_steps(12, sp)
        outs.append(e.transcript(13))
    if B > 1:
        assert np.array_equal(np.asarray(outs[0]), np.asarray(outs[1]))
    else:
        assert np.asarray(outs[0]).shape == np.asarray(outs[1]).shape


# ------------------------------------------------------------------------------ the token step as one cooperative kernel
_MEGA_CASES = [
    dict(moe=True, fmt="f16"),
    dict(moe=True, fmt="q8_0"),
    dict(moe=True, fmt="q4_0"),
    dict(moe=False, fmt="q4_1"),
    dict(moe=True, fmt="q8_64", dtype="bf16"),
    dict(moe=False, fmt="bf16", dtype="bf16"),
    dict(moe=True, fmt="f16", num_heads=2, num_kv_heads=1),                    # head_dim 128
    dict(moe=True, fmt="q8_0", num_heads=8, num_kv_heads=1),                   # head_dim 32, eight heads per group
    dict(moe=True, fmt="f16", sliding_window=16),
    dict(moe=True, fmt="q4_0", rope_type=1, use_qk_norm=False),
]


@pytest.mark.parametrize("case", _MEGA_CASES, ids=lambda c: "-".join(f"{k}={v}" for k, v in c.items()))
def test_single_kernel_step_matches_kernel_chain(case):
    """One cooperative launch per token against the chain of per-operation kernels: same cache contents, positions and
    state, logits equal up to the order of the fp32 sums (the two split rows and cache ranges differently)."""
    from ghassan_b200.inference.engine import InferenceEngine, SamplingParams
    from ghassan_b200.models.config import init_parameters
    from ghassan_b200.ops import _lib
    case = dict(case)
    moe, fmt = case.pop("moe"), case.pop("fmt")
    dt = torch.bfloat16 if case.pop("dtype", "f16") == "bf16" else torch.float16
    cfg = _tiny_cfg(use_moe=moe, moe_expert_dim=256, intermediate_size=512, **case)
    named = init_parameters(cfg, 31)
    one = InferenceEngine(cfg, named, fmt=fmt, batch=1, max_len=48, prefill_chunk=32, compute_dtype=dt, single_kernel=True)
    chain = InferenceEngine(cfg, named, fmt=fmt, batch=1, max_len=48, prefill_chunk=32, compute_dtype=dt, single_kernel=False)
    assert one.mega is not None and chain.mega is None
    seq = torch.randint(16, 512, (1, 60), generator=torch.Generator().manual_seed(9), dtype=torch.int32)
    for e in (one, chain):
        e.reset(1)
    tol = 4e-3 if dt == torch.float16 else 3e-2
    for j in range(60):                                  # longer than the cache: the ring wraps
        for e in (one, chain):
            e.cur_tok.copy_(seq[:, j])
            e._forward_token()
        scale = float(chain.logits.abs().max())
        err = float((one.logits - chain.logits).abs().max())
        assert err <= tol * max(1.0, scale), (j, err, scale)
        assert one.state.cpu().tolist() == chain.state.cpu().tolist(), j
    _lib.check_status(what="single-kernel decode step")
    assert torch.equal(one.slot_pos, chain.slot_pos) and torch.equal(one.pos, chain.pos)
    for La, Lb in zip(one.layers, chain.layers):
        assert torch.allclose(La.cK.float(), Lb.cK.float(), atol=8 * tol) and torch.allclose(La.cV.float(), Lb.cV.float(), atol=8 * tol)
    sp = SamplingParams(greedy=True, repetition_penalty=1.0)
    outs = []
    for e in (one, chain):                               # through the captured graph, with the device sampler
        e.reset(1)
        e.prefill(seq[:, :9].contiguous())
        e.sample_first(sp)
        e.decode_steps(12, sp)
        outs.append(np.asarray(e.transcript(13)))
    _lib.check_status(what="single-kernel decode step (graph)")
    assert outs[0].shape == outs[1].shape and int(one.state[0, 0]) == int(chain.state[0, 0])
    same = int((outs[0] == outs[1]).sum())
    assert outs[0][0, 0] == outs[1][0, 0] and same >= 1, (outs[0], outs[1])


def test_single_kernel_step_is_refused_for_uncovered_shapes():
    from ghassan_b200.inference.engine import InferenceEngine
    from ghassan_b200.models.config import init_parameters
    cfg = _tiny_cfg()                                     # expert width 128: not a whole 256-value unit
    eng = InferenceEngine(cfg, init_parameters(cfg, 3), fmt="f16", batch=1, max_len=32, single_kernel=True)
    assert eng.mega is None and eng.fused
    eng2 = InferenceEngine(_tiny_cfg(moe_expert_dim=256), init_parameters(_tiny_cfg(moe_expert_dim=256), 3), fmt="f16", batch=2,
                           max_len=32, single_kernel=True)
    assert eng2.mega is None                              # more than one sequence: the kernel chain


def test_single_kernel_barrier_wait_runs_out_with_a_status():
    """A barrier that cannot open (its opening count is set far ahead of the arrivals) ends after its time limit with
    status 401; the step is skipped, the context stays usable and the next step runs."""
    from ghassan_b200.inference.engine import InferenceEngine
    from ghassan_b200.models.config import init_parameters
    from ghassan_b200.ops import _lib
    cfg = _tiny_cfg(moe_expert_dim=256)
    eng = InferenceEngine(cfg, init_parameters(cfg, 3), fmt="f16", batch=1, max_len=32, single_kernel=True)
    assert eng.mega is not None
    eng.reset(1)
    eng.cur_tok.fill_(20)
    eng._forward_token()
    torch.cuda.synchronize()
    _lib.check_status(what="warm-up step")
    before = eng.state.cpu().tolist()
    eng._mega_sync[1] += 1 << 30                          # the count this launch starts from: nothing ever reaches it
    eng._forward_token()
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="401"):
        _lib.check_status(what="step with a closed barrier")
    assert eng.state.cpu().tolist() == before             # the step did not advance the sequence
    eng._forward_token()                                  # the kernel left its counters consistent
    torch.cuda.synchronize()
    _lib.check_status(what="step after the expired wait")
    assert int(eng.state[0, 0]) == before[0][0] + 1 and bool(torch.isfinite(eng.logits).all())


@pytest.mark.parametrize("moe,fmt,B", [(True, "f16", 3), (True, "q4_0", 8), (False, "q8_0", 5)])
def test_tensor_core_token_step_matches_gemv_chain(moe, fmt, B):
    """Batches from ``gemm_min_batch`` sequences on run the token step's projections and experts as GEMMs over the
    16-bit weights; against the per-sequence GEMV kernels over the same (fp16) or the quantised stored bytes."""
    from ghassan_b200.inference.engine import InferenceEngine, SamplingParams
    from ghassan_b200.models.config import init_parameters
    cfg = _tiny_cfg(use_moe=moe, moe_aux_free=moe, moe_aux_scale=0.0 if moe else 0.01)
    named = init_parameters(cfg, 31)
    bias = [np.linspace(-0.02, 0.02, cfg.num_experts).astype(np.float32) for _ in range(cfg.num_layers)] if moe else None
    gemm = InferenceEngine(cfg, named, fmt=fmt, batch=B, max_len=48, prefill_chunk=32, moe_bias=bias, gemm_min_batch=2)
    gemv = InferenceEngine(cfg, named, fmt="f16", batch=B, max_len=48, prefill_chunk=32, moe_bias=bias, gemm_min_batch=0)
    assert gemm.batched and not gemv.batched
    seq = torch.randint(16, 512, (B, 60), generator=torch.Generator().manual_seed(9), dtype=torch.int32)
    for e in (gemm, gemv):
        e.reset(1)
    for j in range(60):                                  # longer than the cache: the ring wraps
        for e in (gemm, gemv):
            e.cur_tok.copy_(seq[:, j])
            e._forward_token()
        scale = float(gemv.logits.abs().max())
        err = float((gemm.logits - gemv.logits).abs().max())
        assert err <= 1e-2 * max(1.0, scale), (j, err, scale)
    assert gemm.state.cpu().tolist() == gemv.state.cpu().tolist() and torch.equal(gemm.slot_pos, gemv.slot_pos)
    for La, Lb in zip(gemm.layers, gemv.layers):
        assert torch.allclose(La.cK.float(), Lb.cK.float(), atol=3e-2) and torch.allclose(La.cV.float(), Lb.cV.float(), atol=3e-2)
    sp = SamplingParams(seed=4, top_k=20)
    gemm.reset(1)
    gemm.prefill(seq[:, :9].contiguous())
    gemm.sample_first(sp)
    gemm.decode_steps(12, sp)                             # through the captured graph
    out = np.asarray(gemm.transcript(13))
    assert out.shape == (B, 13) and int(gemm.state[0, 0]) == 9 + 12
