"""Command-line front ends of the data side: data_pipeline, train_tokenizer, corpus_stats."""
import json
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden", "text")
TOK = os.path.join(GOLD, "ref_small.gtok")


def test_train_tokenizer_cli_matches_reference_file(tmp_path, capsys):
    """Same corpus, vocabulary size and frequency floor as the reference's trainer run that wrote ref_small.gtok."""
    from ghassan_b200.cli import train_tokenizer as TT
    out = str(tmp_path / "t.gtok")
    assert TT.main(["--input", os.path.join(GOLD, "corpus_small.txt"), "--output", out, "--vocab", "800", "--min-freq", "2"]) == 0
    assert open(out, "rb").read() == open(TOK, "rb").read()
    text = (lambda o: o.out + o.err)(capsys.readouterr())
    assert "fertility" in text and "tokens/word" in text and "fingerprint" in text
    assert TT.main(["--input", str(tmp_path / "missing"), "--output", out]) == 1
    assert TT.main(["--input", out, "--vocab", "0"]) == 2
    out2 = str(tmp_path / "s.gtok")
    assert TT.main(["--synth", "200", "--output", out2, "--vocab", "400", "--keep-case"]) == 0
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.data.tokenizer import Tokenizer
    t = Tokenizer.load(out2)
    assert 272 < t.vocab_size <= 400 and not H.NormalizerConfig.unpack(t.normalizer_bits).lowercase_latin
    capsys.readouterr()


def test_corpus_stats_cli(capsys):
    from ghassan_b200.cli import corpus_stats as CS
    assert CS.main(["--input", os.path.join(GOLD, "probe.txt"), "--tokenizer", TOK, "--dedup", "--pii", "--quality", "--sample", "1"]) == 0
    text = (lambda o: o.out + o.err)(capsys.readouterr())
    assert "documents          : 60" in text and "tokens / word      : 1.114" in text and "ar-MA-latn" in text and "duplicates:" in text
    assert "median tokens    13" in text and "p10/p50/p90/p99  5 / 12 / 19 / 21" in text and "distinct tokens  167 / 800" in text
    assert "personal data:" in text and "quality filter would reject" in text and "---- sample: en ----" in text
    assert CS.main(["--input", os.path.join(GOLD, "probe.txt"), "--limit", "7"]) == 0
    assert "documents          : 7\n" in (lambda o: o.out + o.err)(capsys.readouterr())
    assert CS.main([]) == 2 and CS.main(["--input", "/nonexistent/dir"]) == 1
    assert CS.main(["--input", os.path.join(GOLD, "probe.txt"), "--tokenizer", "/nonexistent.gtok"]) == 1
    capsys.readouterr()


REF_CS = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "bin", "corpus_stats")


@pytest.mark.skipif(not os.path.exists(REF_CS), reason="no build of the reference corpus tool here")
def test_corpus_stats_equals_the_reference_tool(capsys):
    """Both tools on the fixture corpus: every figure outside the language table is the same (totals, fertility,
    script and style shares, lengths, percentiles, vocabulary use); the language table may move one document between
    neighbouring tags, since the word lists are each project's own."""
    import re
    import subprocess
    from ghassan_b200.cli import corpus_stats as CS
    args = ["--input", os.path.join(GOLD, "probe.txt"), "--tokenizer", TOK]
    ref = subprocess.run([REF_CS] + args, capture_output=True, text=True, timeout=120)
    assert ref.returncode == 0, ref.stdout + ref.stderr
    assert CS.main(args) == 0
    mine = capsys.readouterr().out

    def figures(text):
        rows, langs, in_lang = {}, {}, False
        for ln in text.splitlines():
            if ln.startswith("  -- "):
                in_lang = "language distribution" in ln
                continue
            m = re.match(r"^\s+([a-zA-Z][a-zA-Z0-9/ \-]*?)\s*:?\s+([0-9].*)$", ln)
            if not m:
                continue
            (langs if in_lang else rows)[m.group(1).strip()] = m.group(2).strip()
        return rows, langs

    (ra, la), (rb, lb) = figures(ref.stdout), figures(mine)
    ra.pop("analysed in", None)
    assert len(ra) >= 20 and all(rb.get(k) == v for k, v in ra.items()), {k: (v, rb.get(k)) for k, v in ra.items() if rb.get(k) != v}
    assert set(la) == set(lb) and sum(abs(int(la[k].split()[0]) - int(lb[k].split()[0])) for k in la) <= 4


def test_data_pipeline_build_inspect_tokinfo(tmp_path, capsys):
    from ghassan_b200.cli import data_pipeline as DP
    out = str(tmp_path / "shards")
    rc = DP.main(["build", "--tokenizer", TOK, "--out", out, "--text", os.path.join(GOLD, "probe.txt"), "--synth", "30", "--seq-len", "64",
                  "--val-ratio", "0.1", "--style-mode", "off", "--domain", "mix", "--expect-vocab", "800"])
    text = (lambda o: o.out + o.err)(capsys.readouterr())
    assert rc == 0, text
    assert "passed cleaning" in text and sorted(os.listdir(out)) == ["train_mix_0000.gbin", "val_mix_0000.gbin"]
    assert DP.main(["inspect", "--shards", out, "--tokenizer", TOK]) == 0
    assert "train_mix_0000.gbin:" in capsys.readouterr().out
    assert DP.main(["tok-info", "--tokenizer", TOK]) == 0
    info = capsys.readouterr().out
    assert "vocab        : 800" in info and "fingerprint" in info and "lowercase_latin" in info
    with pytest.raises(SystemExit):
        DP.main(["build", "--tokenizer", TOK, "--out", out, "--text", os.path.join(GOLD, "probe.txt"), "--expect-vocab", "801"])
    with pytest.raises(SystemExit):
        DP.main(["build", "--tokenizer", TOK, "--out", out, "--text", os.path.join(GOLD, "probe.txt"), "--keep-case"])
    assert DP.main(["build", "--tokenizer", TOK, "--out", out]) == 1
    capsys.readouterr()


def test_data_pipeline_parquet_modes(tmp_path, capsys):
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    from ghassan_b200 import _gb200_host as H
    from ghassan_b200.cli import data_pipeline as DP
    lake = tmp_path / "lake"
    lake.mkdir()
    qs = ["chno hiya 3asimat lmaghrib nta li 3aref", "kifach n9der nt3ellem lprogrammation b zerba", "fin kayn a7san tajin f mrrakch had l3am"]
    ans = ["l3asima hiya rbat, mdina zwina bzaf 3la lb7ar", "bda b python w dir tamarin kol nhar chwiya bla zerba", "kayn bzaf dyal lblayes zwinin f jam3 lfna w 7daha"]
    pq.write_table(pa.table({"question": qs, "answer": ans}), str(lake / "darija_qa_part0.parquet"))
    pq.write_table(pa.table({"text": ["had nhar zwin bzaf w ljow mzyan l tamchya f lb7ar m3a s7abi", "lbare7 mchit l souk w chrit lkhodra m3a lfawakih b taman mzyan"]}),
                   str(lake / "web_text_part0.parquet"))
    assert DP.main(["parquet", "--probe"]) == 0
    out = str(tmp_path / "o1")
    assert DP.main(["parquet", "--lake", str(lake), "--tokenizer", TOK, "--out", out, "--val-ratio", "0", "--style-mode", "off"]) == 0
    s = H.ShardFile()
    assert s.open(os.path.join(out, "train_0000.gbin"))[0] and s.n_docs == 5 and s.has_mask
    out = str(tmp_path / "o2")
    assert DP.main(["parquet", "--lake", str(lake), "--match", "darija_qa", "--mode", "qa", "--tokenizer", TOK, "--out", out, "--val-ratio", "0",
                    "--style-mode", "off", "--domain", "darija_qa"]) == 0
    s = H.ShardFile()
    assert s.open(os.path.join(out, "train_darija_qa_0000.gbin"))[0] and s.n_docs == 3
    with pytest.raises(SystemExit):
        DP.main(["parquet", "--lake", str(lake), "--match", "web_text", "--mode", "qa", "--tokenizer", TOK, "--out", str(tmp_path / "o3")])
    corpus = str(tmp_path / "c.txt")
    assert DP.main(["parquet-corpus", "--lake", str(lake), "--out", corpus]) == 0
    assert len(open(corpus, encoding="utf-8").read().splitlines()) == 8
    capsys.readouterr()


def test_data_pipeline_csv_json_retrieve_synth(tmp_path, capsys):
    from ghassan_b200.cli import data_pipeline as DP
    root = tmp_path / "csv"
    (root / "sub").mkdir(parents=True)
    (root / "nouns.csv").write_text("n1,n2,eng\nktab,ktoba,book\ndar,dyour,house\nktab,ktoba,book\n", encoding="utf-8")
    (root / "sub" / "qa.csv").write_text("question,answer\nwhat is a book?,ktab\nwhat is a house?,dar\nwhat is a book?,ktab\nsame,same\n,x\n", encoding="utf-8")
    corpus = str(tmp_path / "corpus.txt")
    assert DP.main(["csvs", "--dir", str(root), "--out", corpus]) == 0
    lines = open(corpus, encoding="utf-8").read().splitlines()
    assert {"ktab", "ktoba", "dar", "dyour"} <= set(lines) and "book" not in lines and len(lines) == len(set(lines))
    assert DP.main(["csvs", "--dir", str(root), "--out", corpus, "--with-english"]) == 0
    assert "book" in open(corpus, encoding="utf-8").read().splitlines()
    js = str(tmp_path / "json")
    assert DP.main(["csv2json", "--dir", str(root), "--out", js, "--docs-per-file", "1", "--id-start", "500"]) == 0
    files = sorted(os.listdir(js))
    rows = [r for f in files for r in json.load(open(os.path.join(js, f), encoding="utf-8"))]
    assert {r["id"] for r in rows} == set(range(500, 500 + len(rows))) and all(r["question"] != r["answer"] for r in rows)
    assert len([r for r in rows if r["question"] == "what is a book?"]) == 1 and len(files) == len(rows)
    capsys.readouterr()
    assert DP.main(["retrieve", "--index", js, "--query", "whats a house"]) == 0
    hit = capsys.readouterr().out
    assert "--- hit 1" in hit and "A: dar" in hit.split("--- hit 2")[0]
    assert DP.main(["retrieve", "--index", js, "--query", "zzzzz"]) == 0
    assert DP.main(["retrieve", "--index", str(tmp_path / "nothing"), "--query", "x"]) == 1
    assert DP.main(["jsons", "--dir", js, "--out", corpus]) == 0
    got = open(corpus, encoding="utf-8").read().splitlines()
    assert len(got) == len(set(got)) == len({r["question"] for r in rows} | {r["answer"] for r in rows})   # each distinct side once
    # a table without a known column name has no header: its first row is data, every column a variant
    assert any(r["question"] == "question" and r["answer"] == "answer" for r in rows)
    ref = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "bin", "data_pipeline")
    if os.path.exists(ref):                     # the reference's converters on the same tables write the same bytes
        import subprocess
        (root / "verbs.csv").write_text('eng,darija,darija_ar,n1,id\nto eat,kla,\u0643\u0644\u0627,kayakol,7\n"big, large",kbir,\u0643\u0628\u064a\u0631,,8\n'
                                        'to "go",mcha,,kaymchi,9\n', encoding="utf-8")
        for extra in ([], ["--with-english"]):
            a, b = str(tmp_path / "ca.txt"), str(tmp_path / "cb.txt")
            assert subprocess.run([ref, "csvs", "--dir", str(root), "--out", a] + extra, capture_output=True, timeout=120).returncode == 0
            assert DP.main(["csvs", "--dir", str(root), "--out", b] + extra) == 0
            assert open(a, "rb").read() == open(b, "rb").read()
        ja, jb = str(tmp_path / "ja"), str(tmp_path / "jb")
        assert subprocess.run([ref, "csv2json", "--dir", str(root), "--out", ja, "--docs-per-file", "3"], capture_output=True, timeout=120).returncode == 0
        assert DP.main(["csv2json", "--dir", str(root), "--out", jb, "--docs-per-file", "3"]) == 0
        assert sorted(os.listdir(ja)) == sorted(os.listdir(jb)) and len(os.listdir(ja)) >= 2
        assert all(open(os.path.join(ja, f), "rb").read() == open(os.path.join(jb, f), "rb").read() for f in os.listdir(ja))
        a, b = str(tmp_path / "qa.txt"), str(tmp_path / "qb.txt")
        assert subprocess.run([ref, "jsons", "--dir", ja, "--out", a], capture_output=True, timeout=120).returncode == 0
        assert DP.main(["jsons", "--dir", ja, "--out", b]) == 0
        assert open(a, "rb").read() == open(b, "rb").read()
    assert DP.main(["csvs", "--dir", str(tmp_path / "json")]) == 1
    sy = str(tmp_path / "s.jsonl")
    assert DP.main(["synth", "--out", sy, "--n", "25", "--seed", "5"]) == 0
    assert len(open(sy, encoding="utf-8").read().splitlines()) == 25
    capsys.readouterr()
    assert DP.main(["json", "--input", sy, "--limit", "3"]) == 0
    assert capsys.readouterr().out.count("[chat]") == 3
    assert DP.main(["dump-text", "--input", sy, "--limit", "2"]) == 0
    assert "[chat]" not in capsys.readouterr().out


def test_shipped_synthesis_recipes_drive_the_generator(tmp_path, capsys):
    """The synthesis YAMLs are data_pipeline configs: both sections load, a typo in one is an error, knobs are obeyed."""
    from ghassan_b200.cli import data_pipeline as DP
    from ghassan_b200.data import synth as S
    cfgs = os.path.join(os.path.dirname(__file__), "..", "configs")
    for name, section in (("synthesis_large_200k", "synth"), ("synthesis_billion_scale", "synth"), ("synthesis_billion_scale", "sft_synth")):
        out = str(tmp_path / (name + section + ".jsonl"))
        assert DP.main(["synth", "--config", os.path.join(cfgs, name + ".yaml"), "--section", section, "--n", "6", "--out", out]) == 0
        rows = [json.loads(ln) for ln in open(out, encoding="utf-8")]
        assert len(rows) == 6 and all(r["messages"][-1]["role"] == "assistant" for r in rows)
    typo = tmp_path / "typo.yaml"
    src = open(os.path.join(cfgs, "synthesis_large_200k.yaml"), encoding="utf-8").read()
    typo.write_text(src.replace("  min_turns:", "  p_bogus_typo: 0.5\n  min_turns:", 1), encoding="utf-8")
    assert DP.main(["synth", "--config", str(typo), "--n", "2", "--out", str(tmp_path / "t.jsonl")]) == 1
    assert "p_bogus_typo" in (lambda o: o.out + o.err)(capsys.readouterr())
    assert DP.main(["synth", "--config", os.path.join(cfgs, "synthesis_large_200k.yaml"), "--section", "other", "--out", str(tmp_path / "x")]) == 1
    cfg = S.load_synth_config(os.path.join(cfgs, "synthesis_billion_scale.yaml"), "sft_synth")
    assert cfg.seed == 9999 and cfg.max_turns == 10
    # knobs: script mix, system prompts, turn bounds, template cap, determinism
    c = S.SynthConfig(seed=3, min_turns=4, max_turns=6, p_arabic_script=0.0, p_latin_script=1.0, p_msa=0.0, p_system=1.0,
                      p_french_switch=0.0)
    g = S.DarijaSynthGenerator(c)
    rows = g.generate_many(40)
    assert rows and all(r["lang"] == "ar-MA-latn" and r["messages"][0]["role"] == "system" for r in rows)
    assert all(4 <= len(r["messages"]) - 1 <= 6 for r in rows) and len({json.dumps(r["messages"]) for r in rows}) == len(rows)
    assert [r["messages"] for r in S.DarijaSynthGenerator(c).generate_many(40)] == [r["messages"] for r in rows]
    capped = S.DarijaSynthGenerator(S.SynthConfig(seed=3, max_template_uses=1, max_attempts_multiplier=5))
    few = capped.generate_many(500)
    assert len(few) < 60 and capped.stats.rejected_template_cap > 0 and capped.stats.attempts <= 2500
    assert DP.main(["synth-en", "--n", "7", "--out", str(tmp_path / "en.jsonl")]) == 0
    assert len(open(tmp_path / "en.jsonl", encoding="utf-8").read().splitlines()) == 7
    capsys.readouterr()
