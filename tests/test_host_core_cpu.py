"""Native host runtime: generator, 16-bit codecs, shard files and the stochastic batch sampler."""
import os

import numpy as np
import pytest
import torch


def H():
    from ghassan_b200 import _gb200_host as h
    return h


def _docs(seed, n, lo, hi, vocab):
    r = H().Rng(seed)
    out = []
    for _ in range(n):
        a = np.empty(lo + int(r.below(hi - lo)), dtype=np.int32)
        r.fill_uniform_ids(a, vocab - 16)
        out.append(a + 16)
    return out


# ---------------------------------------------------------------------------------------------- generator
def test_splitmix_and_xoshiro_vectors():
    h = H()
    assert h.splitmix64(0) == 0xE220A8397B1DCDAF          # published splitmix64 first output for state 0
    r = h.Rng(42)
    first = [r.next_u64() for _ in range(3)]
    assert first == [0x15780B2E0C2EC716, 0x6104D9866D113A7E, 0xAE17533239E499A1]
    r2 = h.Rng(42)
    assert [r2.next_u64() for _ in range(3)] == first
    assert h.Rng(43).next_u64() != first[0]


def test_generator_state_round_trip_including_gaussian_spare():
    h = H()
    r = h.Rng(9)
    r.normal()                      # Box-Muller leaves a spare value behind
    st = r.get_state()
    a = [r.normal() for _ in range(5)] + [r.uniform()]
    r2 = h.Rng(1)
    r2.set_state(st)
    b = [r2.normal() for _ in range(5)] + [r2.uniform()]
    assert a == b


def test_distributions():
    r = H().Rng(3)
    u = np.array([r.uniform() for _ in range(20000)])
    assert 0.0 <= u.min() and u.max() < 1.0 and abs(u.mean() - 0.5) < 0.01
    n = np.array([r.normal() for _ in range(20000)])
    assert abs(n.mean()) < 0.03 and abs(n.std() - 1.0) < 0.03
    t = np.array([r.truncated_normal(0.02) for _ in range(5000)])
    assert np.abs(t).max() <= 0.04 + 1e-7 and t.std() > 0.01       # cut at two standard deviations
    b = np.array([r.below(7) for _ in range(7000)])
    assert set(b.tolist()) == set(range(7))


# ---------------------------------------------------------------------------------------------- 16-bit codecs
def test_f16_codec_matches_ieee_on_normal_range():
    h = H()
    rs = np.random.RandomState(0)
    x = (rs.randn(4000) * np.exp(rs.uniform(-8, 8, 4000))).astype(np.float32)
    x = x[(np.abs(x) > 7e-5) & (np.abs(x) < 6e4)]
    bits = h.f32_to_f16_bits(x)
    assert np.array_equal(bits, x.astype(np.float16).view(np.uint16))
    back = h.f16_bits_to_f32(bits)
    assert np.array_equal(back, bits.view(np.float16).astype(np.float32))


def test_f16_special_values():
    h = H()
    enc = lambda v: int(h.f32_to_f16_bits(np.array([v], dtype=np.float32))[0])
    dec = lambda b: float(h.f16_bits_to_f32(np.array([b], dtype=np.uint16))[0])
    assert enc(float("inf")) == 0x7C00
    assert enc(float("-inf")) == 0xFC00
    assert enc(1e6) == 0x7C00                  # overflow saturates to infinity
    nan = enc(float("nan"))
    assert (nan & 0x7C00) == 0x7C00 and (nan & 0x3FF) != 0
    assert enc(0.0) == 0 and enc(-0.0) == 0x8000
    assert dec(0x0001) == pytest.approx(2.0 ** -24)
    assert dec(0x3C00) == 1.0


def test_bf16_codec_matches_torch():
    h = H()
    x = torch.randn(3000) * 37.0
    ref = x.to(torch.bfloat16)
    bits = h.f32_to_bf16_bits(x.numpy())
    assert np.array_equal(bits, ref.view(torch.int16).numpy().view(np.uint16))
    back = h.bf16_bits_to_f32(bits)
    assert np.array_equal(back, ref.float().numpy())


def test_dtype_table():
    h = H()
    for name, size in (("f32", 4), ("f16", 2), ("bf16", 2), ("i32", 4), ("i8", 1), ("u16", 2), ("i64", 8)):
        assert h.dtype_nbytes(h.dtype_id(name), 10) == 10 * size
        assert h.dtype_name(h.dtype_id(name)) == name


# ---------------------------------------------------------------------------------------------- shards
def test_shard_round_trip_and_masks(tmp_path):
    h = H()
    from ghassan_b200.data.loader import write_shard
    docs = _docs(1, 20, 5, 50, 300)
    masks = [(np.arange(len(d)) % 3 == 0).astype(np.uint8) for d in docs]
    p = str(tmp_path / "sft_0000.gbin")
    ntok, ndoc = write_shard(p, docs, 300, masks)
    assert ndoc == 20 and ntok == sum(len(d) for d in docs)
    s = h.ShardFile()
    ok, why = s.open(p)
    assert ok, why
    assert s.n_docs == 20 and s.n_tokens == ntok and s.has_mask
    flat = np.concatenate(docs)
    assert np.array_equal(np.asarray(s.tokens(0, ntok)), flat)
    assert np.array_equal(np.asarray(s.masks(0, ntok)), np.concatenate(masks))
    assert s.doc_start(1) == len(docs[0])
    assert s.doc_end_after(0) == len(docs[0])


def test_shard_refuses_garbage(tmp_path):
    h = H()
    p = str(tmp_path / "bad.gbin")
    open(p, "wb").write(b"not a shard at all" * 10)
    ok, why = h.ShardFile().open(p)
    assert not ok and why
    # a truncated copy of a good shard is refused too
    from ghassan_b200.data.loader import write_shard
    good = str(tmp_path / "good.gbin")
    write_shard(good, _docs(1, 5, 5, 50, 300), 300, None)
    blob = open(good, "rb").read()
    open(p, "wb").write(blob[:len(blob) - 9])
    ok, why = h.ShardFile().open(p)
    assert not ok and why


def test_shard_writer_rejects_out_of_vocab(tmp_path):
    h = H()
    w = h.ShardWriter(str(tmp_path / "x.gbin"), 100, False)
    with pytest.raises(Exception):
        w.add_document(np.array([1, 2, 100], dtype=np.int32))


# ---------------------------------------------------------------------------------------------- sampler
def _loader(tmp, pack, seed=11, B=3, T=32):
    from ghassan_b200.data.loader import DataLoader
    ld = DataLoader(B, T, pack, seed, vocab_size=300, pin=False)
    assert ld.open_glob(tmp, "train")
    return ld


@pytest.fixture()
def shard_dir(tmp_path):
    from ghassan_b200.data.loader import write_shard
    write_shard(str(tmp_path / "train_0000.gbin"), _docs(2, 60, 5, 90, 300), 300, None)
    write_shard(str(tmp_path / "train_0001.gbin"), _docs(3, 40, 5, 90, 300), 300, None)
    return str(tmp_path)


@pytest.mark.parametrize("pack", [False, True])
def test_sampler_is_deterministic_and_resumable(shard_dir, pack):
    a, b = _loader(shard_dir, pack), _loader(shard_dir, pack)
    seq_a = []
    for _ in range(6):
        x, y = a.next(), b.next()
        assert torch.equal(x.ids, y.ids) and torch.equal(x.targets, y.targets) and torch.equal(x.segments, y.segments)
        seq_a.append((x.ids.clone(), x.targets.clone(), x.state))
    # state captured after batch 3 continues with batch 4
    c = _loader(shard_dir, pack, seed=999)
    c.set_state(seq_a[3][2])
    nxt = c.next()
    assert torch.equal(nxt.ids, seq_a[4][0])
    # fast-forward consumes the same stream as drawing
    d = _loader(shard_dir, pack)
    d.fast_forward(4)
    assert torch.equal(d.next().ids, seq_a[4][0])
    # another seed gives another stream
    e = _loader(shard_dir, pack, seed=12)
    assert not torch.equal(e.next().ids, seq_a[0][0])


def test_targets_are_next_tokens_and_unsupervised_marked(shard_dir):
    ld = _loader(shard_dir, True, B=2, T=64)
    for _ in range(4):
        b = ld.next()
        ids, tg, seg = b.ids.view(2, 64), b.targets.view(2, 64), b.segments.view(2, 64)
        sup = tg >= 0
        assert int(sup.sum()) == b.supervised
        for r in range(2):
            for t in range(63):
                if sup[r, t] and seg[r, t] == seg[r, t + 1]:
                    assert tg[r, t] == ids[r, t + 1]
        # packed rows hold several documents: segment ids are non-decreasing runs
        assert bool((seg[:, 1:] >= seg[:, :-1]).all())
        assert int(seg.max()) >= 1
        assert bool((tg[~sup] == -100).all())


def test_unpacked_rows_are_single_documents(shard_dir):
    ld = _loader(shard_dir, False, B=2, T=16)
    b = ld.next()
    assert int(b.segments.max()) == int(b.segments.min())


def test_sft_mask_limits_supervision(tmp_path):
    from ghassan_b200.data.loader import DataLoader, write_shard
    docs = _docs(5, 50, 40, 60, 300)
    masks = [np.concatenate([np.zeros(len(d) // 2, np.uint8), np.ones(len(d) - len(d) // 2, np.uint8)]) for d in docs]
    write_shard(str(tmp_path / "train_0000.gbin"), docs, 300, masks)
    ld = DataLoader(2, 32, True, 4, vocab_size=300, pin=False)
    assert ld.open_glob(str(tmp_path), "train") and ld.all_have_mask
    total = sup = 0
    for _ in range(10):
        b = ld.next()
        total += b.ids.numel()
        sup += b.supervised
    assert 0 < sup < 0.75 * total


def test_mix_follows_weights(tmp_path):
    from ghassan_b200.data.loader import DataLoader, write_shard
    lo = [np.full(40, 20, np.int32) for _ in range(50)]
    hi = [np.full(40, 200, np.int32) for _ in range(50)]
    write_shard(str(tmp_path / "train_a_0000.gbin"), lo, 300, None)
    write_shard(str(tmp_path / "train_b_0000.gbin"), hi, 300, None)
    ld = DataLoader(4, 32, False, 1, vocab_size=300, pin=False)
    assert ld.open_mix(str(tmp_path), {"a": 0.8, "b": 0.2})
    n_a = n = 0
    for _ in range(100):
        b = ld.next()
        first = b.ids.view(4, 32)[:, 0]
        n_a += int((first == 20).sum())
        n += 4
    assert 0.7 < n_a / n < 0.9
    assert ld.mix_report()


def test_rank_streams_differ(shard_dir):
    from ghassan_b200.data.loader import RANK_SEED_STRIDE
    a = _loader(shard_dir, True, seed=5)
    b = _loader(shard_dir, True, seed=5 + RANK_SEED_STRIDE)
    assert not torch.equal(a.next().ids, b.next().ids)
