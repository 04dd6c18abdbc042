"""File formats against files written by the reference's own tools (``tests/golden/formats``):

* ``tiny_ref.ckpt``   checkpoint (v12, AdamW moments) left by its trainer after 3 steps of a tiny MoE model;
* ``tiny400.gtok``    the tokenizer its ``train_tokenizer --vocab 400`` learned from ``golden/text/corpus_small.txt``;
* ``tiny_*.gguf``     its ``ghassan-ai export`` of that checkpoint with profiles fp16, q8_k and q4_0.
"""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "formats")


def H():
    from ghassan_b200 import _gb200_host as h
    return h


@pytest.fixture(scope="module")
def ckpt():
    return H().read_checkpoint(os.path.join(GOLD, "tiny_ref.ckpt"), False, True)


def test_reference_checkpoint_reads_and_rewrites_identically(ckpt, tmp_path):
    h = H()
    assert ckpt["version"] == 12 and ckpt["state"]["step"] == 3 and ckpt["payload_finite"]
    assert ckpt["has_optimizer"] and ckpt["optimizer"]["kind"] == "adamw" and ckpt["optimizer"]["t"] == 3
    assert ckpt["trailing_bytes"] == 0 and len(ckpt["moe_bias"]) == 1
    from ghassan_b200.training import checkpoint as C
    cfg = C.config_from_dict(ckpt["config"])
    assert [n for n, _ in ckpt["params"]] == [s.name for s in cfg.param_specs()]
    out = str(tmp_path / "again.ckpt")
    h.write_checkpoint(out, ckpt["config"], ckpt["state"], ckpt["moe_bias"], ckpt["params"], ckpt["optimizer"])
    assert open(out, "rb").read() == open(os.path.join(GOLD, "tiny_ref.ckpt"), "rb").read()
    head = h.read_checkpoint(os.path.join(GOLD, "tiny_ref.ckpt"), True, False)       # header only
    assert head["state"]["step"] == 3


def test_checkpoint_damage_is_detected(ckpt, tmp_path):
    h = H()
    blob = open(os.path.join(GOLD, "tiny_ref.ckpt"), "rb").read()
    p = str(tmp_path / "bad.ckpt")
    open(p, "wb").write(b"XXXX" + blob[4:])
    with pytest.raises(Exception):
        h.read_checkpoint(p, False, True)
    open(p, "wb").write(blob[:len(blob) // 3])
    with pytest.raises(Exception):
        h.read_checkpoint(p, False, True)
    open(p, "wb").write(blob + b"\0\0\0")
    assert h.read_checkpoint(p, False, True)["trailing_bytes"] == 3


@pytest.mark.parametrize("profile", ["fp16", "q8_k", "q4_0"])
def test_gguf_export_is_byte_identical(ckpt, tmp_path, profile):
    from ghassan_b200.formats import gguf as G
    from ghassan_b200.training import checkpoint as C
    cfg = C.config_from_dict(ckpt["config"])
    st = ckpt["state"]
    out = str(tmp_path / "m.gguf")
    info = G.export_gguf(out, cfg, dict(ckpt["params"]), os.path.join(GOLD, "tiny400.gtok"), profile,
                         moe_bias=ckpt["moe_bias"], extra_meta={"steps": str(st["step"]), "val_loss": "%.6f" % st["best_val"]})
    assert info["tensors"] == len(cfg.param_specs()) + 1          # + one balancing-bias row
    assert open(out, "rb").read() == open(os.path.join(GOLD, "tiny_%s.gguf" % profile), "rb").read()


@pytest.mark.parametrize("profile,tol", [("fp16", 1e-3), ("q8_k", 0.02), ("q4_0", 0.2)])
def test_gguf_import(ckpt, profile, tol):
    from ghassan_b200.formats import gguf as G
    from ghassan_b200.training import checkpoint as C
    m = G.load_gguf(os.path.join(GOLD, "tiny_%s.gguf" % profile))
    cfg = C.config_from_dict(ckpt["config"])
    assert m.cfg.same_architecture_as(cfg)[0]
    assert m.tokenizer is not None and m.tokenizer.to_bytes() == open(os.path.join(GOLD, "tiny400.gtok"), "rb").read()
    src = dict(ckpt["params"])
    for name, arr in m.named.items():
        ref = np.asarray(src[name]).reshape(arr.shape)
        scale = np.abs(ref).max() + 1e-9
        assert np.abs(arr - ref).max() <= tol * scale, name
        if "norm" in name:
            assert np.array_equal(arr, ref)                         # norm gains are stored in fp32 in every profile
    assert len(m.moe_bias) == 1 and np.allclose(m.moe_bias[0], np.asarray(ckpt["moe_bias"][0]))
    assert "Q4_0" in G.describe(os.path.join(GOLD, "tiny_q4_0.gguf"))


def test_tokenizer_rebuilds_from_token_and_merge_arrays():
    from ghassan_b200.formats import gguf as G
    f = H().GgufFile(os.path.join(GOLD, "tiny_fp16.gguf"))
    md = dict(f.metadata)
    full = G.tokenizer_from_metadata(md)
    md.pop("ghassan.tokenizer.gtok")
    rebuilt = G.tokenizer_from_metadata(md)                         # llama.cpp-style arrays only
    for text in ("salam 3lik, kidayr?", "The quick brown fox", "السلام عليكم ١٢٣"):
        assert rebuilt.encode(text).tolist() == full.encode(text).tolist()


def test_gguf_reader_refuses_garbage(tmp_path):
    h = H()
    blob = open(os.path.join(GOLD, "tiny_fp16.gguf"), "rb").read()
    for bad in (b"NOPE" + blob[4:], blob[:200], blob[:len(blob) - 64]):
        p = str(tmp_path / "bad.gguf")
        open(p, "wb").write(bad)
        with pytest.raises(Exception):
            h.GgufFile(p)


@pytest.mark.parametrize("name,block,nbytes", [("q8_0", 64, 68), ("q4_0", 32, 18), ("q4_1", 32, 20)])
def test_internal_quantisers(name, block, nbytes):
    h = H()
    rs = np.random.RandomState(0)
    x = (rs.randn(block * 7 + 5) * 0.3).astype(np.float32)            # ragged tail
    q = np.asarray(h.quantize(x, name))
    assert q.size == 8 * nbytes
    y = np.asarray(h.dequantize(q, name, x.size))
    err = h.quant_error(x, y)
    assert err["cosine"] > (0.999 if name == "q8_0" else 0.98)
    x[3] = np.inf                                                      # a block with a non-finite value is zeroed
    z = np.asarray(h.dequantize(np.asarray(h.quantize(x, name)), name, x.size))
    assert np.all(z[:block] == 0) and np.allclose(z[block:], y[block:])


def test_ggml_block_layouts():
    h = H()
    x = np.linspace(-1, 1, 64).astype(np.float32)
    q8 = np.asarray(h.ggml_quantize(x, 8))
    assert q8.size == 2 * 34
    scale = np.frombuffer(q8[:2].tobytes(), dtype=np.float16)[0]
    assert float(scale) == pytest.approx(np.abs(x[:32]).max() / 127, rel=1e-3)
    assert np.frombuffer(q8[2:34].tobytes(), dtype=np.int8)[0] == -127
    q4 = np.asarray(h.ggml_quantize(x, 2))
    assert q4.size == 2 * 18
    byte0 = int(q4[2])
    lo, hi = byte0 & 15, byte0 >> 4                                    # adjacent values share a byte, first one low
    d = float(np.frombuffer(q4[:2].tobytes(), dtype=np.float16)[0])
    assert (lo - 8) * d == pytest.approx(x[0], abs=d) and (hi - 8) * d == pytest.approx(x[1], abs=d)


@pytest.mark.parametrize("profile,tol", [("fp32", 0.0), ("fp16", 1e-3), ("int8", 0.02), ("int4", 0.2)])
def test_gai_round_trip(ckpt, tmp_path, profile, tol):
    """The reference's tools read files written here (checked by hand with its ``info`` and ``quantize`` commands);
    this test pins the layout and the round trip."""
    import struct
    from ghassan_b200.formats import gai as GA
    from ghassan_b200.training import checkpoint as C
    cfg = C.config_from_dict(ckpt["config"])
    named = dict(ckpt["params"])
    p = str(tmp_path / "m.gai")
    GA.export_gai(p, cfg, named, os.path.join(GOLD, "tiny400.gtok"), profile, {"steps": "3"})
    blob = open(p, "rb").read()
    magic, version, hb = struct.unpack_from("<III", blob, 0)
    assert magic == 0x31494147 and version == 1
    header = blob[12:12 + hb].decode()
    keys = [l.split("=")[0] for l in header.splitlines()]
    assert keys == sorted(keys) and "rms_eps=0.000010000" in header and "quant_profile=" + profile in header
    m = GA.load_gai(p)
    assert m.cfg.same_architecture_as(cfg)[0] and m.tokenizer.vocab_size == 400
    for t in m.raw.tensors:
        assert t["offset"] % 64 == 0
    for name, arr in m.named.items():
        ref = np.asarray(named[name]).reshape(arr.shape)
        assert np.abs(arr - ref).max() <= tol * (np.abs(ref).max() + 1e-9), name
    view = m.raw.tensor_view("final_norm")                       # zero-copy bytes out of the mapping
    assert np.array_equal(np.frombuffer(view, dtype=np.float32), np.asarray(named["final_norm"]).ravel())


def test_graw_round_trip(ckpt, tmp_path):
    from ghassan_b200.formats import gai as GA
    from ghassan_b200.training import checkpoint as C
    cfg = C.config_from_dict(ckpt["config"])
    named = dict(ckpt["params"])
    p = str(tmp_path / "m.graw")
    GA.save_raw(p, cfg, named)
    back = GA.load_raw(p, cfg)
    for s in cfg.param_specs():
        assert np.array_equal(back[s.name], np.asarray(named[s.name]).reshape(s.shape))
    open(p, "r+b").write(b"XXXX")
    with pytest.raises(Exception):
        GA.load_raw(p, cfg)


@pytest.mark.parametrize("ckpt,golden,profile,compat", [("dense_ref.ckpt", "dense_llama_fp16.gguf", "fp16", "llama"),
                                                        ("dense_ref.ckpt", "dense_llama_q8.gguf", "q8_k", "llama"),
                                                        ("moe_noshared_ref.ckpt", "moens_llamamoe_fp16.gguf", "fp16", "llama_moe")])
def test_llama_compat_export_is_byte_identical_to_the_reference(tmp_path, ckpt, golden, profile, compat):
    """Golden files: the reference's ``ghassan-ai export --compat llama|llama_moe`` on checkpoints its trainer wrote."""
    from ghassan_b200.cli import infer as I
    out = str(tmp_path / "m.gguf")
    assert I.main(["export", "--checkpoint", os.path.join(GOLD, ckpt), "--tokenizer", os.path.join(GOLD, "tiny400.gtok"), "--out", out,
                   "--profile", profile, "--compat", compat]) == 0
    assert open(out, "rb").read() == open(os.path.join(GOLD, golden), "rb").read()


def test_llama_compat_refusals_and_names(tmp_path):
    from ghassan_b200.cli import infer as I
    from ghassan_b200.formats import gguf as G
    tok = os.path.join(GOLD, "tiny400.gtok")
    for ckpt, compat in (("tiny_ref.ckpt", "llama"), ("tiny_ref.ckpt", "llama_moe"), ("dense_ref.ckpt", "llama_moe")):
        with pytest.raises(SystemExit, match="refused"):            # MoE as dense, shared expert / QK-norm, dense as MoE
            I.main(["export", "--checkpoint", os.path.join(GOLD, ckpt), "--tokenizer", tok, "--out", str(tmp_path / "x.gguf"), "--compat", compat])
    with pytest.raises(SystemExit, match="unknown compat"):
        I.main(["export", "--checkpoint", os.path.join(GOLD, "dense_ref.ckpt"), "--tokenizer", tok, "--out", str(tmp_path / "x.gguf"), "--compat", "gpt2"])
    assert G.llama_tensor_name("layers.3.wq") == "blk.3.attn_q.weight" and G.llama_tensor_name("layers.0.w_down") == "blk.0.ffn_down.weight"
    assert G.llama_tensor_name("layers.2.moe_gate", moe=True) == "blk.2.ffn_gate_exps.weight"
    assert G.llama_tensor_name("layers.2.moe_sh_gate", moe=True) == "" and G.llama_tensor_name("layers.2.qk_qnorm") == ""
