"""Text stack: normaliser, pre-tokeniser, tokenizer (.gtok), streaming detokeniser, BPE trainer, chat template.

``tests/golden/text`` holds files written by the reference's own tools: ``ref_small.gtok`` is what its
``train_tokenizer --vocab 800 --min-freq 2`` learned from ``corpus_small.txt``; ``probe_train_0000.gbin`` is the shard
its ``data_pipeline build --text probe.txt`` produced with that tokenizer (token ids of 59 cleaned documents).
"""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "text")


def H():
    from ghassan_b200 import _gb200_host as h
    return h


def T():
    from ghassan_b200.data import tokenizer as t
    return t


@pytest.fixture(scope="module")
def ref_tok():
    return T().Tokenizer.load(os.path.join(GOLD, "ref_small.gtok"))


# ---------------------------------------------------------------------------------------------- normaliser
def test_normalizer_flag_packing():
    h = H()
    c = h.NormalizerConfig()
    assert c.pack() == 0x305EF                      # defaults: everything on except letter folding and repeat collapsing
    c.lowercase_latin = False
    c.collapse_repeats = True
    c.max_repeat = 2
    d = h.NormalizerConfig.unpack(c.pack())
    assert (d.lowercase_latin, d.collapse_repeats, d.max_repeat) == (False, True, 2)
    assert h.NormalizerConfig.unpack(0).max_repeat == 3


@pytest.mark.parametrize("raw,want", [
    ("  Hello   WORLD \n", "hello world"),
    ("a \n b", "a\nb"),                                                # a blank run containing a newline becomes a newline
    ("كِتَابٌ", "كتاب"),                                                  # diacritics
    ("كتـــاب", "كتاب"),                                                # tatweel
    ("١٢٣ ۴۵", "123 45"),                                              # Arabic-Indic and Persian digits
    ("ﻻ", "لا"),                                                        # lam-alef ligature expands
    ("ﻣﺮﺣﺒﺎ", "مرحبا"),                                                 # presentation forms fold to base letters
    ("ＦＵＬＬ　ｗｉｄｔｈ", "full width"),
    ("a​b‏c", "abc"),                                         # zero-width characters
    ("مي‌خواهم", "مي‌خواهم"),                                 # ... except a ZWNJ between Arabic letters
    ("x\x00y\x7fz", "xyz"),                                             # controls
    ("ÀÉ", "àé"),
])
def test_normalize_defaults(raw, want):
    assert H().normalize(raw) == want


def test_normalize_options():
    h = H()
    c = h.NormalizerConfig()
    c.fold_letters = True
    assert h.normalize("أإآ ى ة ؤ", c) == "ااا ي ه ء"
    c = h.NormalizerConfig()
    c.collapse_repeats = True
    c.max_repeat = 2
    assert h.normalize("waaaaaw!!!!", c) == "waaw!!"
    c = h.NormalizerConfig()
    c.lowercase_latin = False
    assert h.normalize("Keep CASE", c) == "Keep CASE"
    assert h.canonical_text("هههههه  أحمد") == "ههه احمد"


def test_pre_tokenize_rules():
    h = H()
    A, L, N, P, S, E, O = range(7)
    chunks = lambda s: [(t, k) for t, k in h.pre_tokenize(s)]
    assert chunks("salam 3lik m3a sa7bi") == [("salam", L), (" 3lik", L), (" m3a", L), (" sa7bi", L)]
    assert chunks("don't stop") == [("don't", L), (" stop", L)]
    assert chunks("pi 3.14 1,000 x2") == [("pi", L), (" 3.14", N), (" 1,000", N), (" x2", L)]
    assert chunks("wow!!! ok?") == [("wow", L), ("!!!", P), (" ok", L), ("?", P)]
    assert chunks("a  b") == [("a", L), ("  ", S), ("b", L)]            # two blanks do not glue
    assert chunks("a\nb") == [("a", L), ("\n", S), ("b", L)]
    assert chunks("مرحبا بيك") == [("مرحبا", A), (" بيك", A)]
    assert chunks("hi 😀😀") == [("hi", L), (" 😀😀", E)]
    assert chunks("x ") == [("x", L), (" ", S)]
    assert chunks("§") == [("§", P)] or chunks("§") == [("§", O)]


# ---------------------------------------------------------------------------------------------- tokenizer
def test_empty_tokenizer_is_byte_level(tmp_path):
    tk = T().Tokenizer()
    assert tk.vocab_size == 16 + 256
    ids = tk.encode("hé")
    assert ids.tolist() == [16 + b for b in "hé".encode()]
    assert tk.decode(ids) == "hé"
    assert tk.encode("x", add_bos=True, add_eos=True).tolist() == [1, 16 + ord("x"), 2]
    p = str(tmp_path / "e.gtok")
    tk.save(p)
    assert T().Tokenizer.load(p).to_bytes() == tk.to_bytes()


def test_gtok_byte_round_trip_and_refusals(ref_tok, tmp_path):
    t = T()
    blob = open(os.path.join(GOLD, "ref_small.gtok"), "rb").read()
    assert ref_tok.to_bytes() == blob and ref_tok.vocab_size == 800
    for bad in (blob[:100], b"XXXX" + blob[4:], blob[:4] + b"\x02\0\0\0" + blob[8:], b""):
        with pytest.raises(t.TokenizerError):
            t.Tokenizer.from_bytes(bad)
    swapped = bytearray(blob)
    swapped[16 + 4] ^= 1                       # first special token string no longer "<pad>"
    with pytest.raises(t.TokenizerError):
        t.Tokenizer.from_bytes(bytes(swapped))
    with pytest.raises(t.TokenizerError):
        t.Tokenizer.load(str(tmp_path / "missing.gtok"))


def test_encode_matches_reference_shard(ref_tok):
    h = H()
    s = h.ShardFile()
    ok, why = s.open(os.path.join(GOLD, "probe_train_0000.gbin"))
    assert ok, why
    toks = np.asarray(s.tokens(0, s.n_tokens))
    start, checked = 0, 0
    for _ in range(s.n_docs):
        end = s.doc_end_after(start)
        ids = toks[start:end].tolist()
        start = end
        assert ids[0] == 1 and ids[-1] == 2                     # <s> ... </s>
        body = ids[1:-1]
        text = ref_tok.decode(body)
        assert ref_tok.encode(text).tolist() == body, text
        checked += len(body)
    assert checked > 700


def test_trainer_reproduces_the_reference_file(ref_tok):
    t = T()
    mine = t.train_bpe([os.path.join(GOLD, "corpus_small.txt")], vocab_size=800, min_frequency=2,
                       normalizer_bits=ref_tok.normalizer_bits)
    assert mine.to_bytes() == ref_tok.to_bytes()
    # the corpus runs out of pairs before 800: the rest are placeholder slots that never encode
    assert mine.token_bytes(799).startswith(b"<|unused")
    assert mine.token_to_id(mine.token_bytes(799)) == -1
    assert 3 not in mine.encode("<|unused5|>").tolist()


def test_long_piece_path_equals_short_piece_path(ref_tok):
    # pieces longer than 24 bytes go through the heap-based merger; compare with merging the parts by hand
    word = "lmochkil" * 5
    ids = ref_tok.encode(word).tolist()
    assert ref_tok.decode(ids) == word
    assert len(ids) < len(word)
    again = ref_tok.encode(word).tolist()                        # second time from the memo
    assert again == ids


def test_specials_and_batch(ref_tok):
    txt = "<|user|>salam<|end|><|assistant|>labas 3lik<|end|>"
    ids = ref_tok.encode_with_specials(txt).tolist()
    assert ids[0] == 5 and 7 in ids and 6 in ids
    assert ref_tok.decode(ids, skip_special=True) == "salamlabas 3lik"
    plain = ref_tok.encode(txt).tolist()
    assert all(i >= 16 for i in plain)                           # plain encode never produces special ids
    lines = open(os.path.join(GOLD, "probe.txt"), encoding="utf-8").read().splitlines()
    one = [ref_tok.encode(l, True, True).tolist() for l in lines]
    many = [a.tolist() for a in ref_tok.encode_batch(lines, True, True, threads=4)]
    assert one == many


def test_stream_holds_back_split_characters(ref_tok):
    tk = T().Tokenizer()                                          # byte-level: every character is split
    st = tk.stream()
    out = [st.push(i) for i in tk.encode("aé😀").tolist()]
    assert out[0] == b"a" and out[1] == b"" and out[2] == "é".encode()
    assert b"".join(out) + st.flush() == "aé😀".encode()
    st = tk.stream()
    st.push(16 + 0xE2)                                            # a lone lead byte at the end
    assert st.flush() == "�".encode()
    assert st.flush() == b""


# ---------------------------------------------------------------------------------------------- chat template
def test_chat_encoding_and_loss_mask(ref_tok):
    t = T()
    msgs = [("system", "be brief"), ("user", "salam"), ("assistant", "labas"), ("user", "chno"), ("assistant", "walo")]
    ids, mask = t.encode_chat(ref_tok, msgs)
    assert ids[0] == t.BOS and mask[0] == 0 and len(ids) == len(mask)
    pos = 1
    for role, content in msgs:
        body = ref_tok.encode(content).tolist()
        assert ids[pos] == t.ROLE_TOKEN[role] and mask[pos] == 0
        seg = slice(pos + 1, pos + 1 + len(body))
        assert ids[seg].tolist() == body
        want = 1 if role == "assistant" else 0
        assert set(mask[seg].tolist()) <= {want}
        assert ids[seg.stop] == t.END and mask[seg.stop] == want   # the closing token of an assistant turn is supervised
        pos = seg.stop + 1
    assert pos == len(ids)
    ids2, mask2 = t.encode_chat(ref_tok, msgs[:2], add_generation_prompt=True)
    assert ids2[-1] == t.ASSISTANT and mask2[-1] == 0 and mask2.sum() == 0
    assert t.render_chat(msgs[:2], True) == "<s><|system|>be brief<|end|><|user|>salam<|end|><|assistant|>"
    assert ref_tok.encode_with_specials(t.render_chat(msgs)).tolist() == ids.tolist()


def test_script_policy():
    t = T()
    assert t.detect_script("شنو خبارك") == "arabic"
    assert t.detect_script("chno khbarek") == "latin"
    assert t.detect_script("123 !!") == "arabic"
    assert t.system_for_persona("en", "arabic") == t.SYSTEM_ENGLISH
    assert t.system_for_persona("darija", "latin") == t.SYSTEM_DARIJA_LATIN
    assert t.script_directive("latin").startswith("Reply ONLY")
