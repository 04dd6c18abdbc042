"""GGUF export and import of a model (weights + embedded tokenizer + configuration).

The metadata keys, their value types and the tensor order reproduce the reference exporter
(format/gguf_codec.cpp:1186-1437) so that a file written here is byte-identical to the reference's for the same
checkpoint and tokenizer: ``<arch>.*`` hyper-parameters, the llama.cpp-style ``tokenizer.ggml.*`` arrays, the
authoritative ``.gtok`` image under ``ghassan.tokenizer.gtok``, tensors in parameter-table order (dims fastest
first), per-layer balancing biases as ``layers.N.moe_bias``.

Profiles: fp32, fp16 (norms fp32), q8_k = ggml Q8_0 body and embeddings, q4_0 = ggml Q4_0 body with Q8_0
embeddings; norm gains always fp32.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from .. import _gb200_host as H
from ..data.tokenizer import N_SPECIAL, UNK, Tokenizer
from ..models.config import ModelConfig

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0 = 0, 1, 2, 8
GGML_NAMES = {GGML_F32: "F32", GGML_F16: "F16", GGML_Q4_0: "Q4_0", GGML_Q8_0: "Q8_0"}

CHAT_TEMPLATE = (
    "{%- for message in messages %}"
    "{%- if message['role'] == 'system' %}"
    "{{- '<s><|system|>' + message['content'] + '<|end|>' }}"
    "{%- elif message['role'] == 'user' %}"
    "{{- '<|user|>' + message['content'] + '<|end|>' }}"
    "{%- elif message['role'] == 'assistant' %}"
    "{{- '<|assistant|>' + message['content'] + '<|end|>' }}"
    "{%- endif %}{%- endfor %}"
    "{%- if add_generation_prompt %}{{- '<|assistant|>' }}{%- endif %}")


@dataclass
class Profile:
    name: str
    default: int
    embedding: int
    norm: int


def profile_for(name: str) -> Profile:
    if name == "fp32":
        return Profile("fp32", GGML_F32, GGML_F32, GGML_F32)
    if name == "fp16":
        return Profile("fp16", GGML_F16, GGML_F16, GGML_F32)
    if name in ("q8_k", "int8", "q6_k", "q5_k_m", "q5_k_s"):
        return Profile("q8_k", GGML_Q8_0, GGML_Q8_0, GGML_F32)
    if name in ("q4_0", "int4", "q4_k_m", "q4_k_s", "q4_k"):
        return Profile("q4_0", GGML_Q4_0, GGML_Q8_0, GGML_F32)
    raise ValueError(f"unknown export profile: {name} (fp32|fp16|q8_k|q4_0|q4_k_m|q6_k)")


def size_label(n_params: int) -> str:
    return "%.1fB" % (n_params / 1e9) if n_params >= 1_000_000_000 else "%dM" % ((n_params + 500_000) // 1_000_000)


def _escape_merge_piece(b: bytes) -> bytes:
    return b.replace(b"\\", b"\\\\").replace(b" ", b"\\x20")


def _unescape_merge_piece(b: bytes) -> bytes:
    out, i = bytearray(), 0
    while i < len(b):
        if b[i:i + 2] == b"\\\\":
            out += b"\\"
            i += 2
        elif b[i:i + 4] == b"\\x20":
            out += b" "
            i += 4
        else:
            out.append(b[i])
            i += 1
    return bytes(out)


def llama_compat_refusal(cfg: ModelConfig, compat: str) -> str:
    """Why ``cfg`` cannot be written under a llama.cpp architecture name ("" = it can); the rules of the reference's
    exporter (format/gguf_codec.cpp:966-997)."""
    if compat == "llama":
        if cfg.use_moe:
            return ("MoE has no llama.cpp dense equivalent; export native GGUF for ghassan-ai, --compat llama_moe for MoE "
                    "Ollama (needs moe_shared=false), or train a dense (use_moe=false) variant for ollama")
    else:
        if not cfg.use_moe:
            return "llama_moe needs use_moe=true (use --compat llama for dense)"
        if cfg.moe_shared:
            return ("llama_moe has no shared-expert equivalent in llama.cpp; train with moe_shared=false for Ollama, or use "
                    "native GGUF (full quality)")
    if cfg.use_qk_norm:
        return "use_qk_norm has no llama-arch equivalent; disable it for --compat " + compat
    if cfg.rope_scale != 1.0:
        return "rope_scale YaRN has no exact llama mapping here; use rope_scale=1"
    if cfg.moe_aux_free:
        return "moe_aux_free has no llama mapping; use native GGUF"
    if cfg.sliding_window != 0:
        return "sliding_window has no llama mapping here; use 0"
    if cfg.rope_type != 0:
        return "rope_type=neox mismatches the interleaved rotation of this export; use 0"
    return ""


def llama_tensor_name(internal: str, moe: bool = False) -> str:
    """llama.cpp tensor name of a parameter ("" = none), format/gguf_codec.cpp:929-951 and :999-1024."""
    top = {"tok_embeddings": "token_embd.weight", "final_norm": "output_norm.weight", "lm_head": "output.weight"}
    if internal in top:
        return top[internal]
    if not internal.startswith("layers.") or internal.count(".") < 2:
        return ""
    _, layer, rest = internal.split(".", 2)
    names = {"attn_norm": "attn_norm.weight", "wq": "attn_q.weight", "wk": "attn_k.weight", "wv": "attn_v.weight",
             "wo": "attn_output.weight", "ffn_norm": "ffn_norm.weight"}
    names.update({"moe_router": "ffn_gate_inp.weight", "moe_gate": "ffn_gate_exps.weight", "moe_up": "ffn_up_exps.weight",
                  "moe_down": "ffn_down_exps.weight"} if moe else
                 {"w_gate": "ffn_gate.weight", "w_up": "ffn_up.weight", "w_down": "ffn_down.weight"})
    return ("blk.%s.%s" % (layer, names[rest])) if rest in names else ""


def export_gguf(path: str, cfg: ModelConfig, named: Dict[str, np.ndarray], tokenizer_path: str, profile: str = "fp16",
                moe_bias: Optional[Sequence[np.ndarray]] = None, extra_meta: Optional[Dict[str, str]] = None,
                compat: str = "native") -> dict:
    """Write a self-contained GGUF file; returns a small summary.  ``compat``: "native" (architecture "ghassan", what
    this framework loads), "llama" (dense models under llama.cpp names) or "llama_moe" (Mixtral-style names;
    experimental in the reference too).  The compat forms are write-only: they drop what llama.cpp cannot express."""
    if compat not in ("native", "llama", "llama_moe"):
        raise ValueError(f"unknown compat '{compat}' (native|llama|llama_moe)")
    want_llama, want_moe = compat == "llama", compat == "llama_moe"
    if compat != "native":
        why = llama_compat_refusal(cfg, compat)
        if why:
            raise ValueError(f"--compat {compat} refused: {why}")
    prof = profile_for(profile)
    tok = Tokenizer.load(tokenizer_path)
    if tok.vocab_size != cfg.vocab_size:
        raise ValueError(f"tokenizer/model vocab mismatch: {tok.vocab_size} vs {cfg.vocab_size}")
    gtok_blob = open(tokenizer_path, "rb").read()
    extra_meta = dict(extra_meta or {})
    n_params = cfg.count_parameters()
    w = H.GgufWriter()
    s = lambda k, v: w.set_str(k, v.encode("utf-8") if isinstance(v, str) else v)
    arch = "ghassan" if compat == "native" else "llama"
    a = lambda k: arch + "." + k
    s("general.architecture", arch)
    net = "MoE-%d" % cfg.num_experts if cfg.use_moe else "dense"
    s("general.name", extra_meta.get("model_name") or "Ghassan %s %s L%d" % (size_label(n_params), net, cfg.num_layers))
    s("general.description", "Ghassan MoE language model for Moroccan Darija")
    s("general.type", "model")
    s("general.size_label", size_label(n_params))
    w.set_u64("general.parameter_count", n_params)
    w.set_u64(a("vocab_size"), cfg.vocab_size)
    w.set_u64(a("embedding_length"), cfg.hidden_size)
    w.set_u64(a("block_count"), cfg.num_layers)
    w.set_u64(a("feed_forward_length"), cfg.moe_expert_dim if want_moe else cfg.intermediate_size)
    w.set_u64(a("attention.head_count"), cfg.num_heads)
    w.set_u64(a("attention.head_count_kv"), cfg.num_kv_heads)
    w.set_f32(a("attention.layer_norm_rms_epsilon"), cfg.rms_eps)
    w.set_u64(a("rope.dimension_count"), cfg.head_dim)
    w.set_f32(a("rope.freq_base"), cfg.rope_theta)
    w.set_u64(a("context_length"), cfg.max_seq_len)
    w.set_bool(a("tie_word_embeddings"), cfg.tie_embeddings)
    if want_moe:
        w.set_u64(a("expert_count"), cfg.num_experts)
        w.set_u64(a("expert_used_count"), cfg.moe_top_k)
        w.set_u64(a("expert_feed_forward_length"), cfg.moe_expert_dim)
    if compat == "native":
        w.set_bool(a("use_moe"), cfg.use_moe)
        w.set_u64(a("moe.expert_count"), cfg.num_experts)
        w.set_u64(a("moe.experts_used_count"), cfg.moe_top_k)
        w.set_u64(a("moe.expert_feed_forward_length"), cfg.moe_expert_dim)
        w.set_bool(a("moe.shared_expert"), cfg.moe_shared)
        w.set_f32(a("rope.scale"), cfg.rope_scale)
        w.set_f32(a("rope.yarn_mscale"), cfg.rope_yarn_mscale)
        w.set_f32(a("rope.yarn_low"), cfg.rope_yarn_low)
        w.set_f32(a("rope.yarn_high"), cfg.rope_yarn_high)
        w.set_u64(a("sliding_window"), cfg.sliding_window)
        w.set_u64(a("rope.type"), cfg.rope_type)
        w.set_bool(a("moe.aux_free"), cfg.moe_aux_free)
        w.set_f32(a("moe.aux_scale"), cfg.moe_aux_scale)
        w.set_f32(a("moe.jitter"), cfg.moe_jitter)
        w.set_f32(a("z_loss_scale"), cfg.z_loss_scale)
        w.set_bool(a("use_qk_norm"), cfg.use_qk_norm)
        s(a("norm_type"), "rmsnorm")
        s(a("ffn_type"), "swiglu_moe" if cfg.use_moe else "swiglu")
        s(a("attention.type"), "gqa_causal")
    # ---- tokenizer, llama.cpp style + the authoritative .gtok image
    s("tokenizer.ggml.model", "gpt2")
    s("tokenizer.ggml.pre", "gpt-2")
    vocab = tok.t.vocab_bytes()
    w.set_str_array("tokenizer.ggml.tokens", vocab)
    w.set_f32_array("tokenizer.ggml.scores", np.zeros(len(vocab), dtype=np.float32))
    types = np.zeros(len(vocab), dtype=np.int32)      # 0 normal, 1 unknown, 2 control, 5 byte
    types[:N_SPECIAL] = 2
    types[UNK] = 1
    types[N_SPECIAL:N_SPECIAL + 256] = 5
    w.set_i32_array("tokenizer.ggml.token_type", types)
    w.set_str_array("tokenizer.ggml.merges", [_escape_merge_piece(l) + b" " + _escape_merge_piece(r) for l, r in tok.t.merges()])
    w.set_u32("tokenizer.ggml.bos_token_id", 1)
    w.set_u32("tokenizer.ggml.eos_token_id", 2)
    w.set_u32("tokenizer.ggml.unknown_token_id", 3)
    w.set_u32("tokenizer.ggml.padding_token_id", 0)
    w.set_bool("tokenizer.ggml.add_bos_token", True)
    w.set_bool("tokenizer.ggml.add_eos_token", False)
    s("tokenizer.chat_template", CHAT_TEMPLATE)
    w.set_u8_array("ghassan.tokenizer.gtok", gtok_blob)
    w.set_u32("ghassan.normalizer.config", tok.normalizer_bits)
    s("ghassan.tokenizer.pre_tokenizer", "darija_byte_bpe_v1:leading-space-glue,nl-separator,byte-fallback")
    s("ghassan.tokenizer.canonical", "gtok-blob:tokenizer.ggml.tokens+merges reconstruct; authoritative=ghassan.gtok_blob")
    w.set_u64("ghassan.tokenizer.specials", N_SPECIAL)
    w.set_u32("general.quantization_version", 2)
    s("ghassan.quantization.profile", prof.name)
    w.set_u32("general.file_type", {GGML_Q8_0: 7, GGML_Q4_0: 2}.get(prof.default, 1))
    for k, v in extra_meta.items():
        if k != "model_name":
            s(k, v)
    # ---- tensors in parameter-table order
    total = 0
    for spec in cfg.param_specs():
        is_norm = "norm" in spec.name
        is_emb = spec.name in ("tok_embeddings", "lm_head")
        t = prof.norm if is_norm else prof.embedding if is_emb else prof.default
        arr = np.ascontiguousarray(np.asarray(named[spec.name], dtype=np.float32).reshape(spec.shape))
        name = spec.name
        if compat != "native":
            name = llama_tensor_name(spec.name, moe=want_moe)
            if not name:
                raise ValueError(f"no llama.cpp name for tensor {spec.name} (use native GGUF)")
            if want_moe and spec.name.endswith("moe_down"):          # [ne*d, E] -> [ne, E, d]
                arr = np.ascontiguousarray(arr.reshape(cfg.num_experts, cfg.hidden_size, cfg.moe_expert_dim).transpose(0, 2, 1))
        w.add_tensor(name, arr, t)
        total += H.ggml_tensor_nbytes(t, arr.size)
        if compat != "native" and spec.name == "tok_embeddings" and cfg.tie_embeddings:
            w.add_tensor("output.weight", arr, t)                     # llama.cpp wants the head by name
            total += H.ggml_tensor_nbytes(t, arr.size)
    if compat == "native" and cfg.moe_aux_free and moe_bias is not None:
        for l, b in enumerate(moe_bias):
            b = np.asarray(b, dtype=np.float32).reshape(-1)
            if l < cfg.num_layers and b.size == cfg.num_experts:
                w.add_tensor("layers.%d.moe_bias" % l, b, GGML_F32)
    w.write(path)
    return {"path": path, "profile": prof.name, "tensors": w.tensor_count, "metadata": w.metadata_count, "weight_bytes": total}


@dataclass
class LoadedModel:
    cfg: ModelConfig
    named: Dict[str, np.ndarray]          # fp32 tensors by parameter name
    moe_bias: List[np.ndarray]
    tokenizer: Optional[Tokenizer]
    metadata: dict
    tensor_types: Dict[str, int]
    raw: Optional["H.GgufFile"] = None


def _meta_str(md, key, default=""):
    v = md.get(key)
    return v.decode("utf-8", "replace") if isinstance(v, (bytes, bytearray)) else (default if v is None else str(v))


def config_from_metadata(md: dict) -> ModelConfig:
    arch = _meta_str(md, "general.architecture", "ghassan")
    if arch != "ghassan":
        raise ValueError(f"GGUF architecture '{arch}' is not a native ghassan export")
    g = lambda k, d=None: md.get(arch + "." + k, d)
    cfg = ModelConfig(
        vocab_size=int(g("vocab_size")), hidden_size=int(g("embedding_length")), num_layers=int(g("block_count")),
        num_heads=int(g("attention.head_count")), num_kv_heads=int(g("attention.head_count_kv")),
        intermediate_size=int(g("feed_forward_length")), max_seq_len=int(g("context_length")),
        rope_theta=float(g("rope.freq_base", 10000.0)), rms_eps=float(g("attention.layer_norm_rms_epsilon", 1e-5)),
        tie_embeddings=bool(g("tie_word_embeddings", True)), use_moe=bool(g("use_moe", False)),
        num_experts=int(g("moe.expert_count", 0)), moe_top_k=int(g("moe.experts_used_count", 0)),
        moe_expert_dim=int(g("moe.expert_feed_forward_length", 0)), moe_shared=bool(g("moe.shared_expert", False)),
        moe_aux_scale=float(g("moe.aux_scale", 0.0)), moe_aux_free=bool(g("moe.aux_free", False)),
        moe_jitter=float(g("moe.jitter", 0.0)), use_qk_norm=bool(g("use_qk_norm", False)),
        z_loss_scale=float(g("z_loss_scale", 0.0)), rope_scale=float(g("rope.scale", 1.0)),
        rope_yarn_mscale=float(g("rope.yarn_mscale", 0.0)), rope_yarn_low=float(g("rope.yarn_low", 1.0)),
        rope_yarn_high=float(g("rope.yarn_high", 32.0)), sliding_window=int(g("sliding_window", 0)),
        rope_type=int(g("rope.type", 0)))
    if cfg.use_moe and cfg.moe_top_k * 2 > cfg.num_experts:
        cfg.moe_allow_dense = True
    cfg.validate()
    return cfg


def tokenizer_from_metadata(md: dict) -> Optional[Tokenizer]:
    blob = md.get("ghassan.tokenizer.gtok")
    if isinstance(blob, (bytes, bytearray)) and len(blob) > 0:
        return Tokenizer.from_bytes(bytes(blob))
    toks, merges = md.get("tokenizer.ggml.tokens"), md.get("tokenizer.ggml.merges")
    if toks is None:
        return None
    pairs = []
    for m in merges or []:
        l, _, r = bytes(m).partition(b" ")
        pairs.append((_unescape_merge_piece(l), _unescape_merge_piece(r)))
    t = H.Tokenizer()
    t.build([bytes(x) for x in toks], pairs, int(md.get("ghassan.normalizer.config", 0)) or None)
    return Tokenizer(t)


def load_gguf(path: str, dequantize: bool = True) -> LoadedModel:
    f = H.GgufFile(path)
    md = dict(f.metadata)
    cfg = config_from_metadata(md)
    types = {t["name"]: int(t["type"]) for t in f.tensors}
    named, bias = {}, [None] * cfg.num_layers
    for spec in cfg.param_specs():
        if spec.name not in types:
            raise ValueError(f"GGUF file lacks tensor '{spec.name}'")
        if dequantize:
            named[spec.name] = np.asarray(f.tensor_f32(spec.name)).reshape(spec.shape)
    for l in range(cfg.num_layers):
        n = "layers.%d.moe_bias" % l
        if n in types:
            bias[l] = np.asarray(f.tensor_f32(n))
    if any(b is None for b in bias):
        bias = []
    return LoadedModel(cfg, named, bias, tokenizer_from_metadata(md), md, types, f)


def describe(path: str) -> str:
    """Human-readable summary (the ``info`` command)."""
    f = H.GgufFile(path)
    md = dict(f.metadata)
    cfg = config_from_metadata(md)
    by_type: Dict[int, list] = {}
    for t in f.tensors:
        by_type.setdefault(int(t["type"]), []).append(int(t["nbytes"]))
    lines = ["file: %s" % path, "format: GGUF v%d" % f.version, "arch: %s" % _meta_str(md, "general.architecture"),
             "name: %s" % _meta_str(md, "general.name"), "quant: %s" % _meta_str(md, "ghassan.quantization.profile", "?"),
             "tokenizer: %s" % ("embedded" if md.get("ghassan.tokenizer.gtok") else "tokens+merges"),
             "config: " + cfg.summary(), "tensors: %d" % len(f.tensors)]
    for t, sizes in sorted(by_type.items()):
        lines.append("  %-5s %4d tensors %12d bytes" % (GGML_NAMES.get(t, str(t)), len(sizes), sum(sizes)))
    n = cfg.count_parameters()
    wbytes = sum(sum(v) for v in by_type.values())
    lines.append("size: %d bytes" % os.path.getsize(path))
    lines.append("parameters: %d (%.2f M)" % (n, n / 1e6))
    lines.append("weight bytes: %d (%.2f bits/param)" % (wbytes, 8.0 * wbytes / max(1, n)))
    return "\n".join(lines)
