"""Text pipeline on the CPU: cleaning primitives, language id, dedup, shard building (against a shard the reference's
``data_pipeline build`` wrote from the same probe file with the same tokenizer), synthesis, retrieval."""
import io
import json
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden", "text")


def H():
    import ghassan_b200
    from ghassan_b200 import _gb200_host as h
    return h


@pytest.fixture(scope="module")
def tok():
    from ghassan_b200.data.tokenizer import Tokenizer
    return Tokenizer.load(os.path.join(GOLD, "ref_small.gtok"))


def _docs(path):
    h = H()
    s = h.ShardFile()
    ok, why = s.open(path)
    assert ok, why
    t = np.asarray(s.tokens(0, s.n_tokens))
    out, st = [], 0
    for _ in range(s.n_docs):
        e = s.doc_end_after(st)
        out.append(tuple(t[st:e].tolist()))
        st = e
    return out, s


# ------------------------------------------------------------------------------------------ primitives
def test_pii_scan_and_redaction():
    h = H()
    text = "ping me at someone@example.com or +212 661-234567, server 192.168.10.44, https://bob:hunter2@host.tld/x"
    rep = h.scan_pii(text)
    assert rep["emails"] == 1 and rep["phones"] >= 1 and rep["ips"] == 1 and rep["urls_with_creds"] == 1
    red, rep2 = h.redact_pii(text)
    assert "someone@example.com" not in red and "hunter2" not in red and "192.168.10.44" not in red
    assert rep2["total"] == rep["total"]
    assert h.scan_pii("كيداير اليوم؟ كلشي بخير الحمد لله")["total"] == 0


def test_html_and_mojibake():
    h = H()
    assert h.strip_html_tags("<p>salam <b>sahbi</b></p>&amp; more").replace("  ", " ").strip().startswith("salam sahbi")
    broken = "café".encode("utf-8").decode("latin-1")
    assert h.fix_mojibake(broken) == "café"
    assert h.fix_mojibake("plain ascii") == "plain ascii"


def test_cleaner_drops_and_counts():
    h = H()
    c, st = h.Cleaner(), h.CleanStats()
    assert c.clean_line("   ".encode(), st) is None
    assert c.clean_line("mail me: x.y@z.org please, this line is long enough".encode(), st) is None
    out = c.clean_line("<i>واش نتا بخير؟</i> kolchi mzyan had nhar".encode(), st)
    assert out is not None and "<i>" not in out
    assert st.lines_in == 3 and st.lines_out == 1 and st.dropped_pii == 1 and st.dropped_empty == 1
    cfg = h.CleanConfig()
    cfg.redact_instead_drop = True
    out = h.Cleaner(cfg).clean_line("mail me: x.y@z.org please, this line is long enough".encode(), h.CleanStats())
    assert out is not None and "x.y@z.org" not in out


def test_quality_and_toxicity_gates():
    h = H()
    ok, _ = h.quality_check("واش كاين شي حد هنا باش يعاوني ف هاد المشكل ديال الخدمة؟")
    assert ok
    ok, why = h.quality_check("$$$ ### @@@ !!! %%% ^^^ &&& *** ((( )))")
    assert not ok and why
    ok, why = h.quality_check("spam spam spam spam spam spam spam spam spam spam spam spam")
    assert not ok and why == "word repetition"
    ok, why = h.quality_check("wach nta bikhir a sahbi wach nta mzyan lyoum wla la")          # 2 of 11 words: above the 15 % limit
    assert not ok and why == "word repetition"
    ok, why = h.quality_check_english("wach nta bikhir a sahbi wach nta mzyan lyoum wla la")  # the English limit is 40 %
    assert ok
    ok, why = h.quality_check("As an AI language model, I cannot help with that request at all.")
    assert not ok and why == "ai_disclaimer"
    ok, why = h.quality_check_english("As an AI language model, I cannot help with that request at all.")
    assert not ok and why == "ai_disclosure_hard"
    ok, why = h.quality_check("ok")
    assert not ok and why == "too few words"
    assert h.quality_check_english("ok")[0]
    ok, why = h.quality_check("\n".join(["nfs ster kol mera"] * 4 + ["ster akhor mkhtalf 3la lokhrin"]))
    assert not ok and why in ("word repetition", "duplicated lines")
    assert not h.check_toxicity("nhar zwin had lyoum, nmchiw l b7ar")["toxic"]


def test_language_tags():
    h = H()
    want = {"واش نتا بخير؟ بغيت نمشي للسوق دابا حيت خاصني الخضرة": "ar-MA-arab",
            "wach nta bikhir? bghit nmchi l souk daba 7it khassni lkhodra": "ar-MA-latn",
            "إن هذا الأمر يتطلب دراسة معمقة لذلك يجب على الجميع أن يشاركوا في هذا العمل الذي بدأناه": "ar-MSA",
            "Je voudrais savoir comment aller à la gare, s'il vous plaît, parce que je suis en retard": "fr",
            "I would like to know how the weather is going to be tomorrow because we are travelling": "en"}
    for text, tag in want.items():
        r = h.classify_language(text)
        assert r["tag"] == tag, (text, r)
        assert 0.0 <= r["confidence"] <= 1.0
    assert h.msa_ratio(list(want)[2]) > h.msa_ratio(list(want)[0])
    # without word evidence the script decides, as in the reference classifier (dataset/langid.cpp:196-237 there):
    # Arabic script -> Standard Arabic at low confidence, Latin script -> other, no letters -> other at zero
    assert h.classify_language("دددددددددددد")["tag"] == "ar-MSA" and h.classify_language("دددددددددددد")["confidence"] == 0.3
    assert h.classify_language(" w w w w w w w w")["tag"] == "other"
    assert h.classify_language("12345 !!!") == dict(h.classify_language(""), tag="other")
    # the verb shapes of Darija count as evidence: a ka- word makes this otherwise formal sentence Darija there too
    assert h.classify_language("إن هذا الأمر يتطلب دراسة معمقة حيث أن النتائج التي تم الحصول عليها ليست كافية")["tag"] == "ar-MA-arab"


def test_dedup_exact_near_and_blocklist():
    h = H()
    d = h.Deduplicator()
    base = "had nhar mchit l souk m3a sahbi w chrina bzaf dyal l7wayj zwinin b taman mzyan bzaf"
    assert d.add(base)
    assert not d.add(base)                                   # exact
    assert not d.add(base + " .")                            # near (one extra shingle)
    assert d.add("chi 7aja khra kamla ma3ndha 7ta 3ala9a m3a dakchi li dazt 9bel f had lista")
    d.add_blocklist_text("what is the capital of morocco and why is it rabat")
    assert not d.add("what is the capital of morocco and why is it rabat")
    assert d.exact_dups == 1 and d.near_dups == 1 and d.blocked == 1 and d.seen == 5
    assert d.is_duplicate(base) and not d.is_duplicate("completely unseen sentence with other words inside of it")


def test_assistant_style_flags():
    h = H()
    f = h.check_assistant_style("As an AI language model, I cannot have opinions.", "chno ban lik?")
    assert f["robotic"] and f["has_boilerplate"] and f["matched_phrases"]
    assert h.has_hard_ai_boilerplate("As an AI language model, I do not have feelings")
    g = h.check_assistant_style("واخا، نمشيو دابا للسوق ونشريو الخضرة", "فين نمشيو؟")
    assert not g["robotic"]
    many = "\n".join("- point %d" % i for i in range(12))
    assert h.check_assistant_style(many, "list")["too_many_bullets"]


# ------------------------------------------------------------------------------------------ shard builder
def test_build_matches_reference_documents(tok, tmp_path):
    from ghassan_b200.data import pipeline as P
    ref, _ = _docs(os.path.join(GOLD, "probe_train_0000.gbin"))
    # the reference's `build` defaults: English style, 0.5 % validation by key hash, masks always written
    rep = P.build_shards(P.iter_inputs(os.path.join(GOLD, "probe.txt")), tok, str(tmp_path), P.BuildConfig(val_ratio=0.005, style_mode="en"))
    mine, s = _docs(str(tmp_path / "train_0000.gbin"))
    assert rep.seen == 60 and rep.kept_docs == 60 and rep.dropped["quality"] == 1 and rep.val_shards == 0 and s.has_mask
    assert mine == ref and len(ref) == 59                    # the same 59 documents in the same order (one fails the quality gate)
    assert open(str(tmp_path / "train_0000.gbin"), "rb").read() == open(os.path.join(GOLD, "probe_train_0000.gbin"), "rb").read()
    assert all(d[0] == 1 and d[-1] == 2 for d in mine)


def test_build_chat_masks_val_split_and_windows(tok, tmp_path):
    from ghassan_b200.data import pipeline as P, synth as S
    rows = list(S.darija_conversations(36, seed=3)) + list(S.english_conversations(20, seed=4))
    rows += rows[:4]                          # the generators never repeat themselves; the builder must catch these
    src = tmp_path / "c.jsonl"
    S.write_jsonl(str(src), rows)
    recs = list(P.iter_inputs(str(src)))
    assert len(recs) == 60 and recs[0].messages and recs[0].messages[0].role == "user"
    rep = P.build_shards(recs, tok, str(tmp_path / "o"), P.BuildConfig(seq_len=48, val_ratio=0.1, style_mode="off"))
    assert rep.dropped["duplicate"] == 4 and rep.kept_docs + rep.dropped["quality"] + rep.dropped["toxicity"] == 60
    assert 0 < rep.val_windows < rep.kept_windows // 3 and rep.train_windows + rep.val_windows == rep.kept_windows   # split by key hash
    docs, s = _docs(str(tmp_path / "o" / "train_0000.gbin"))
    assert s.has_mask and max(len(d) for d in docs) <= 48
    m = np.asarray([s.mask(i) for i in range(s.n_tokens)])
    assert 0 < int(m.sum()) < s.n_tokens                      # only assistant tokens are supervised
    text = P.inspect_shards(str(tmp_path / "o"), tok, 1)
    assert "train_0000.gbin" in text and "loss masks" in text
    with pytest.raises(ValueError):
        P.build_shards([], tok, str(tmp_path / "e"), P.BuildConfig())


REF_DP = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "bin", "data_pipeline")


def _windows_with_masks(folder, prefix):
    h = H()
    out = []
    for name in sorted(n for n in os.listdir(folder) if n.startswith(prefix) and n.endswith(".gbin")):
        s = h.ShardFile()
        ok, why = s.open(os.path.join(folder, name))
        assert ok, why
        t = np.asarray(s.tokens(0, s.n_tokens)).tolist()
        m = [int(s.mask(i)) for i in range(s.n_tokens)] if s.has_mask else [1] * s.n_tokens
        st = 0
        for _ in range(s.n_docs):
            e = s.doc_end_after(st)
            out.append((tuple(t[st:e]), tuple(m[st:e])))
            st = e
    return out


def _is_subsequence(small, big):
    it = iter(big)
    return all(any(x == y for y in it) for x in small)


@pytest.mark.skipif(not os.path.exists(REF_DP), reason="no build of the reference data tool here")
def test_build_reproduces_the_reference_builder_live(tok, tmp_path):
    """The reference's builder and this one on one chat corpus with the same settings (English style, 10 % validation,
    48-token windows): every window the reference wrote appears here with the same tokens and loss mask, in the same
    order and on the same side of the train/validation split.  This builder may keep more (its word lists differ),
    never a different window.  Reference: tools/data_pipeline.cpp (build), src/data/shard_builder.cpp."""
    import subprocess
    from ghassan_b200.data import pipeline as P, synth as S
    rows = list(S.darija_conversations(70, seed=11)) + list(S.english_conversations(50, seed=12))
    rows += rows[:6]
    src = tmp_path / "c.jsonl"
    S.write_jsonl(str(src), rows)
    r = subprocess.run([REF_DP, "build", "--tokenizer", os.path.join(GOLD, "ref_small.gtok"), "--out", str(tmp_path / "r"),
                        "--chat", str(src), "--val-ratio", "0.1", "--seq-len", "48"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rep = P.build_shards(P.iter_inputs(str(src)), tok, str(tmp_path / "o"), P.BuildConfig(seq_len=48, val_ratio=0.1, style_mode="en"))
    def conversations(ws):                     # a conversation's first window opens with <s>
        out = []
        for w in ws:
            if w[0][0] == 1:
                out.append([])
            out[-1].append(w)
        return [tuple(c) for c in out]

    redacted = 0
    for side in ("train_", "val_"):
        ref = conversations(_windows_with_masks(str(tmp_path / "r"), side))
        mine = conversations(_windows_with_masks(str(tmp_path / "o"), side))
        # The reference's IBAN pattern (two letters, two digits, 15+ letters or digits with spaces between) also fires on
        # lower-case Arabizi such as "mo93 riadi bash t3rf" and writes "[iban]" into the training text; this builder's
        # pattern wants upper-case country letters, so those conversations differ and are set aside here.
        clean = [c for c in ref if "[iban]" not in "".join(tok.decode(list(w[0])) for w in c)]
        redacted += len(ref) - len(clean)
        assert clean and _is_subsequence(clean, mine), side
        assert len(mine) <= len(ref) * 1.1, (side, len(ref), len(mine))
    assert redacted <= 6 and rep.dropped["duplicate"] == 6 and rep.dedup["near_dup"] == 0


def test_blocklist_keeps_eval_prompts_out(tok, tmp_path):
    from ghassan_b200.data import pipeline as P
    secret = "what is the tallest mountain in north africa and where exactly is it located"
    recs = [P.Record(text=secret), P.Record(text="lyoum ljow zwin bzaf w bghit nmchi nt3awd m3a s7abi f lb7ar")]
    rep = P.build_shards(recs, tok, str(tmp_path), P.BuildConfig(val_ratio=0.0, style_mode="off", blocklist=[secret]))
    assert rep.kept_docs == 2 and rep.kept_windows == 1 and rep.dedup["blocked"] == 1


def test_readers_accept_common_layouts(tmp_path):
    from ghassan_b200.data import pipeline as P
    (tmp_path / "a.json").write_text(json.dumps([
        {"conversations": [{"from": "human", "value": "salam"}, {"from": "gpt", "value": "wa 3alaykom salam"}]},
        {"instruction": "translate", "input": "hello", "output": "salam"},
        {"prompt": "chno smitek?", "response": "smiti ghassan"},
        {"text": "plain document"}]), encoding="utf-8")
    recs = list(P.iter_inputs(str(tmp_path / "a.json")))
    assert len(recs) == 4
    assert [m.role for m in recs[0].messages] == ["user", "assistant"]
    assert recs[1].messages[-1].content == "salam" and "hello" in recs[1].messages[0].content
    assert recs[2].messages[0].content == "chno smitek?"
    assert recs[3].messages is None and recs[3].text == "plain document"
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    pq.write_table(pa.table({"text": ["wa7ed", "jouj", "tlata"]}), str(tmp_path / "t.parquet"))
    assert [r.text for r in P.read_parquet(str(tmp_path / "t.parquet"), limit=2)] == ["wa7ed", "jouj"]
    assert len(list(P.iter_inputs(str(tmp_path)))) == 7


def test_corpus_stats(tok):
    from ghassan_b200.data import pipeline as P
    st = P.corpus_stats(P.iter_inputs(os.path.join(GOLD, "probe.txt")), tok)
    assert st["documents"] == 60 and st["tokens"] > 0 and st["tokens_per_word"] > 0.5
    assert sum(st["languages"].values()) == 60 and st["scripts"]["latin"] > st["scripts"]["arabic"] > 0


# ------------------------------------------------------------------------------------------ synthesis
def test_synthesis_is_deterministic_and_tagged():
    from ghassan_b200.data import synth as S
    a, b = list(S.darija_conversations(30, seed=9)), list(S.darija_conversations(30, seed=9))
    assert a == b and a != list(S.darija_conversations(30, seed=10))
    h = H()
    for row in a:
        text = " ".join(m["content"] for m in row["messages"])
        arabic = h.script_stats(text)["arabic"]
        assert (arabic == 0) == (row["lang"] == "ar-MA-latn")
        assert len(row["messages"]) % 2 == 0 and "{" not in text
    en = list(S.english_conversations(25, seed=2))
    assert {r["act"] for r in en} >= {"coding", "math"} and all("{" not in r["messages"][1]["content"].replace("```", "") or r["act"] == "coding" for r in en)
    # transliteration: digits for the letters Latin lacks, or letters for lighter typists; deterministic per seed
    assert S.to_arabizi("شنو خبارك؟") == "chnou khbark?" and S.to_arabizi("عندي الحق") == S.to_arabizi("عندي الحق")
    assert "3" in S.to_arabizi("عندي") and "7" in S.to_arabizi("الحق") and "9" in S.to_arabizi("القهوة")
    assert not any("؀" <= ch <= "ۿ" for ch in S.to_arabizi("واش كلشي بخير؟ الحمد لله، ١٢٣"))


def test_native_synthesis_engines_reject_and_count():
    """The native generators: rejection reasons are counted, a conversation never repeats an exchange, worked
    arithmetic is right, and the English style policy pairs a dialog act with the shape of its reply."""
    from ghassan_b200 import _gb200_host as NH
    c = NH.SynthConfig()
    c.seed, c.p_governor, c.p_reasoning, c.max_turns = 11, 0.10, 0.20, 8
    g = NH.DarijaSynth(c)
    convs = g.generate_many(400)
    st = g.stats()
    assert len(convs) == 400 == st["accepted"] and st["attempts"] == 400 + st["rejected_duplicate"] + st["rejected_style"] + \
        st["rejected_entropy"] + st["rejected_template_cap"]
    assert set(st["by_script"]) == {"arab", "latn", "msa"} and len(st["by_domain"]) >= 12
    assert len(NH.DarijaSynth.domains()) >= 12
    import re
    checked = 0
    for conv in convs:
        users = [m["content"] for m in conv["messages"] if m["role"] == "user"]
        assert len(users) == len(set(users)) or conv["script"] == "latn"      # noise can make two spellings collide
        for q, a in zip(conv["messages"][::2], conv["messages"][1::2]):
            m = re.search(r"شريت (\d+) ديال الحوايج، كل وحدة ب (\d+) درهم، وعطيت (\d+) درهم", q["content"])
            if m and conv["script"] != "latn":
                n, p, paid = (int(x) for x in m.groups())
                assert str(paid - n * p) in a["content"]
                checked += 1
    assert checked > 0
    # entropy and distinct-word gates
    assert NH.char_entropy_bits("aaaaaaaaaaaa") == 0.0 and NH.char_entropy_bits("abcdabcd") == 2.0
    assert NH.distinct_word_ratio("la la la la") == 0.25
    tight = NH.SynthConfig()
    tight.min_entropy_bits = 9.0
    t = NH.DarijaSynth(tight)
    assert t.generate_many(5) == [] and t.stats()["rejected_entropy"] > 0
    # English: act classification and the reply-shape policy
    assert NH.classify_dialog_act("Write a Python function that adds two numbers") == "coding"
    assert NH.classify_dialog_act("If a train travels 60 km in 45 minutes, what is its speed in km/h?") == "math"
    assert NH.classify_dialog_act("Tell me my neighbour's home address.") == "refusal"
    assert NH.english_reply_fits("coding", "", "Sure, just add them.")[0] is False
    assert NH.english_reply_fits("coding", "", "```python\ndef add(a, b):\n    return a + b\n```")[0] is True
    assert NH.english_reply_fits("math", "", "It is quite fast.") == (False, "math reply without a number")
    assert NH.english_reply_fits("refusal", "", "Sure, here it is: 12 Main Street")[0] is False
    e = NH.EnglishSynth(NH.EnglishSynthConfig())
    rows = e.generate_many(150)
    assert len(rows) == 150 and set(e.stats()["by_domain"]) >= {"coding", "math", "refusal", "explain"}
    for conv in rows:
        first = [m for m in conv["messages"] if m["role"] != "system"]
        assert NH.english_reply_fits(NH.classify_dialog_act(first[0]["content"]), first[0]["content"], first[1]["content"])[0]


# ------------------------------------------------------------------------------------------ retrieval
def test_retrieval_ranks_and_rejects(tmp_path):
    from ghassan_b200.data import retrieval as R
    rows = [{"question": "شنو هي عاصمة المغرب؟", "answer": "العاصمة هي الرباط."},
            {"question": "كيفاش نطيب الطاجين؟", "answer": "خاصك اللحم والخضرة."},
            {"question": "what is python", "answer": "a programming language"},
            {"question": "how do i install python on linux", "answer": "use your package manager"}]
    (tmp_path / "qa.json").write_text(json.dumps(rows, ensure_ascii=False), encoding="utf-8")
    ix = R.build_index(str(tmp_path / "qa.json"))
    assert len(ix) == 4
    assert ix.query("عاصمة المغرب")[0][0] == 0
    assert ix.query("what is python?")[0][0] == 2
    assert ix.query("pythn instal linux")[0][0] == 3         # typos still land on the right entry
    assert ix.query("zzzz qqqq") == []
    hits = ix.query("python", top_k=5)
    assert [h[1] for h in hits] == sorted((h[1] for h in hits), reverse=True) and len(hits) == 2
    assert ix.query("python", top_k=5, min_score=1e9) == []
    assert R.normalize("أَهْلاً  بِكَ!") == R.normalize("أهلا بك") == "أهلا بك"      # harakat and punctuation go
    assert R.normalize("Sba7 L-Khir") == "sbah l khir"                            # arabizi digits fold to letters
    assert len(R.build_index(str(tmp_path))) == 4            # a directory of .json files
    assert len(R.build_index(str(tmp_path / "missing.json"))) == 0
