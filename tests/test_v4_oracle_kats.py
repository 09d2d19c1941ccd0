"""Known-answer tests that pin the V4 cousin-path oracle (``oracle/v4_oracle.c``) to literal
values recorded in the reference's own tests, plus structural properties of each stage.

Reference sources of the literals:
  crates/engine/tests/kernel_v4_indexer.rs:689-726   (f32 accumulate, one bf16 round: 1.125)
  crates/engine/src/v4/select.rs:534-541             (ring order)
  crates/engine/src/v4/select.rs:681-707,714-740     (ties toward the lower index, -1 padding)
  crates/oracles/src/v4oracle/numerics.rs:158-186    (e2m1 tables and the midpoint rule)
  crates/engine/tests/kernel_v4_indexer.rs:287-323   (spread guards), :644-688 (score guard)
"""
import numpy as np
import pytest

from oracle import oracle as orc


def test_e2m1_tables_and_midpoints():
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for code, m in enumerate(mags):
        assert orc.e2m1_decode(code) == m
        assert orc.e2m1_decode(code | 8) == -m
        assert orc.e2m1_encode(m) == code
        if m:
            assert orc.e2m1_encode(-m) == (code | 8)
    # a value on a midpoint goes to the neighbour whose code is even
    for mid, want in [(0.25, 0.0), (0.75, 1.0), (1.25, 1.0), (1.75, 2.0), (2.5, 2.0), (3.5, 4.0), (5.0, 4.0)]:
        assert orc.e2m1_decode(orc.e2m1_encode(mid)) == want
        assert orc.e2m1_decode(orc.e2m1_encode(-mid)) == -want
    assert orc.e2m1_encode(-0.0) == 8


def test_fast_round_scale_rounds_up_to_a_power_of_two():
    inv = np.float32(1.0) / np.float32(6.0)
    assert orc.fast_round_scale(3.0, 1.0 / 3.0) in (1.0, 2.0)  # product may be one ulp off 1.0
    assert orc.fast_round_scale(4.0, 0.25) == 1.0               # exact power stays
    assert orc.fast_round_scale(4.5, 0.25) == 2.0               # anything above rounds up
    assert orc.fast_round_scale(2.0 ** -20, 1.0) == 2.0 ** -20
    s = orc.fast_round_scale(6.0, float(inv))
    assert s in (1.0, 2.0) and s >= np.float32(6.0) * inv


@pytest.mark.parametrize("n", [32, 128, 256])
def test_hadamard_is_the_sylvester_basis_in_natural_order(n):
    scale = np.float32(1.0) / np.sqrt(np.float32(n))
    for i in (0, 1, 2, 5, n // 2, n - 1):
        e = np.zeros(n, np.float32)
        e[i] = 1.0
        got = orc.v4_hadamard(e)
        want = np.array([(-1.0) ** bin(i & j).count("1") for j in range(n)], np.float32) * scale
        assert np.array_equal(got, want)


def test_score_accumulates_in_f32_and_rounds_once():
    heads, hd = 64, 128
    kv = np.zeros(hd, np.float32)
    kv[0] = 1.0
    q = np.zeros((heads, hd), np.float32)
    q[:, 0] = 2.0 ** -9
    q[0, 0] = 1.0
    w = np.ones(heads, np.float32)
    rc, sc = orc.v4_index_score_blocks(q, kv, w, 1, 1, heads, hd)
    assert rc == 0
    assert sc[0, 0] == np.float32(1.125)


def test_score_rounds_to_bf16_before_relu_and_uses_signed_weights():
    heads, hd = 2, 32
    kv = np.zeros(hd, np.float32)
    kv[0] = 1.0
    q = np.zeros((heads, hd), np.float32)
    q[0, 0], q[1, 0] = -3.0, 2.0
    w = np.array([5.0, -0.5], np.float32)
    rc, sc = orc.v4_index_score_blocks(q, kv, w, 1, 1, heads, hd)
    assert rc == 0 and sc[0, 0] == np.float32(-1.0)  # relu kills head 0, head 1 contributes 2 * -0.5


def test_score_and_spread_guards():
    z = np.zeros(1024, np.float32)
    assert orc.v4_index_score_blocks(z, z, z, 0, 1, 1, 1)[0] == 1001
    assert orc.v4_index_score_blocks(z, z, z, 1, 0, 1, 1)[0] == 1005
    assert orc.v4_spread(z, 0)[0] == 1001
    assert orc.v4_spread(np.zeros(512, np.float32), 512)[0] == 1002
    assert orc.v4_spread(np.zeros(96, np.float32), 96)[0] == 1003
    assert orc.v4_spread(np.zeros(16, np.float32), 16)[0] == 1004
    assert orc.v4_spread(np.zeros(128, np.float32), 128)[0] == 0


def test_spread_values_are_fp4_grid_points_times_a_power_of_two():
    rng = np.random.default_rng(5)
    x = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((8, 128)).astype(np.float32)))
    rc, y = orc.v4_spread(x, 128)
    assert rc == 0
    grid = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)
    for row in y:
        for b0 in range(0, 128, 32):
            seg = np.abs(row[b0:b0 + 32])
            if seg.max() == 0:
                continue
            # some power of two s puts every magnitude on the e2m1 grid with the largest in (3, 6]
            s = 2.0 ** np.ceil(np.log2(seg.max() / 6.0))
            assert np.all(np.isin(seg / np.float32(s), grid))


def test_ring_order_literals():
    assert orc.v4_window_row(4, 6).tolist() == [3, 0, 1, 2]
    assert orc.v4_window_row(4, 2).tolist() == [0, 1, 2, -1]
    assert orc.v4_window_row(4, 3).tolist() == [0, 1, 2, 3]
    assert orc.v4_window_row(4, 7).tolist() == [0, 1, 2, 3]


def test_scored_selection_literals():
    scores = np.array([1.0, 1.0, 9.0, 0.5, 1.0], np.float32)
    assert orc.v4_scored_row(scores, 5, 3, 100, 3).tolist() == [100, 101, 102]
    moved = scores.copy()
    moved[4] = 2.0
    assert orc.v4_scored_row(moved, 5, 3, 100, 3).tolist() == [100, 102, 104]
    # the causal limit masks by index; short rows pad with -1
    two = np.array([0.1, 9.0], np.float32)
    assert orc.v4_scored_row(two, 0, 1, 10, 1).tolist() == [-1]
    assert orc.v4_scored_row(two, 1, 1, 10, 1).tolist() == [10]
    assert orc.v4_scored_row(two, 2, 1, 10, 1).tolist() == [11]
    assert orc.v4_scored_row(two, 2, 4, 10, 4).tolist() == [10, 11, -1, -1]
    # total order: -0.0 ranks below +0.0
    z = np.array([-0.0, 0.0, -0.0, 0.0], np.float32)
    assert orc.v4_scored_row(z, 4, 2, 0, 2).tolist() == [1, 3]


def _softmax_attn(q, kv, sink, idx, scale):
    live = idx[idx >= 0]
    k = kv[live].astype(np.float64)
    lg = (q.astype(np.float64) @ k.T) * scale
    mx = lg.max(axis=1, keepdims=True)
    e = np.exp(lg - mx)
    den = e.sum(axis=1, keepdims=True) + np.exp(sink.astype(np.float64)[:, None] - mx)
    return (e / den) @ k


def test_sparse_attn_sink_masks_and_nan():
    rng = np.random.default_rng(11)
    h, d, n, topk = 4, 64, 40, 12
    bf = lambda a: orc.bf16_to_f32(orc.f32_to_bf16(a.astype(np.float32)))
    q, kv = bf(rng.standard_normal((2, h, d))), bf(rng.standard_normal((n, d)))
    sink = rng.standard_normal(h).astype(np.float32)
    idx = np.stack([rng.permutation(n)[:topk], rng.permutation(n)[:topk]]).astype(np.int32)
    idx[0, 3] = -1
    idx[1, :] = -1
    rc, o = orc.v4_sparse_attn(q, kv, sink, idx, 2, h, d, topk, d ** -0.5)
    assert rc == 0
    want = _softmax_attn(q[0], kv, sink, idx[0], d ** -0.5)
    assert np.allclose(o[0], want, rtol=0, atol=np.abs(want).max() / 128)
    assert np.all(np.isnan(o[1]))  # a query that attends to nothing is loud
    # the sink only ever removes mass: with a very negative sink the rows are a plain softmax
    rc, o2 = orc.v4_sparse_attn(q[:1], kv, np.full(h, -1e30, np.float32), idx[:1], 1, h, d, topk, d ** -0.5)
    want2 = _softmax_attn(q[0], kv, np.full(h, -1e30, np.float32), idx[0], d ** -0.5)
    assert np.allclose(o2[0], want2, rtol=0, atol=np.abs(want2).max() / 128)
    assert np.abs(o2[0]).sum() > np.abs(o[0]).sum() * 0.999
    assert orc.v4_sparse_attn(q, kv, sink, idx, 0, h, d, topk, 1.0)[0] == 1001


def test_batched_step_equals_the_row_functions():
    rng = np.random.default_rng(3)
    g = orc.V4Geom(n_heads=4, head_dim=64, window=8, index_heads=4, index_dim=32, index_topk=4, ratio=4,
                   max_comp=16, softmax_scale=64 ** -0.5)
    B = 3
    pos = np.array([5, 30, 63], np.int32)  # n_comp 1 (positional), 7 (scored), 16 (scored, full)
    u16 = lambda *s: orc.f32_to_bf16(rng.standard_normal(s).astype(np.float32))
    q, kvc = u16(B, 4, 64), u16(B, 8 + 16, 64)
    iq = orc.f32_to_bf16(orc.v4_spread(orc.bf16_to_f32(u16(B * 4, 32)), 32)[1]).reshape(B, 4, 32)
    ikv = orc.f32_to_bf16(orc.v4_spread(orc.bf16_to_f32(u16(B * 16, 32)), 32)[1]).reshape(B, 16, 32)
    iw = orc.bf16_to_f32(u16(B, 4))
    sink = rng.standard_normal(4).astype(np.float32)
    sel, out, sc = orc.v4_decode_step_bf16(g, pos, q, kvc, sink, iq, iw, ikv, want_scores=True)
    assert sel[0].tolist() == [0, 1, 2, 3, 4, 5, -1, -1, 8, -1, -1, -1]
    for b in (1, 2):
        n_comp = (pos[b] + 1) // 4
        rc, s = orc.v4_index_score_blocks(orc.bf16_to_f32(iq[b]), orc.bf16_to_f32(ikv[b, :n_comp]), iw[b], 1,
                                          n_comp, 4, 32)
        assert np.array_equal(s[0], sc[b, :n_comp])
        assert sel[b, :8].tolist() == orc.v4_window_row(8, int(pos[b])).tolist()
        assert sel[b, 8:].tolist() == orc.v4_scored_row(s[0], n_comp, 4, 8, 4).tolist()
        rc, o = orc.v4_sparse_attn(orc.bf16_to_f32(q[b]), orc.bf16_to_f32(kvc[b]), sink, sel[b], 1, 4, 64, 12,
                                   64 ** -0.5)
        assert np.array_equal(orc.f32_to_bf16(o[0]), out[b])


def test_e4m3_round_to_nearest_even_round_trip():
    """The V4 act-quant codec: every finite e4m3 value survives; midpoints go to the even mantissa; 448 saturates."""
    tab = orc.e4m3_table()
    vals = tab[np.isfinite(tab)]
    rc, out = orc.act_quant_f8_prefix(np.concatenate([vals, np.zeros(256 - vals.size, np.float32)]), 1, 256, 256, 256)
    # scale: amax 448 -> 448/448 = 1 -> power of two 1: the round trip is the codec itself
    assert rc == 0 and np.array_equal(out[:vals.size], vals)
    row = np.zeros(64, np.float32)
    row[0] = 448.0
    row[1:6] = [17.0, 19.0, 0.0009765625, 0.0029296875, -447.0]   # ties: 17 -> 16, 19 -> 20 (even mantissas)
    rc, out = orc.act_quant_f8_prefix(row, 1, 64, 64, 64)
    assert out[:6].tolist() == [448.0, 16.0, 20.0, 0.0, 0.00390625, -448.0]
    assert orc.act_quant_f8_prefix(row, 1, 64, 48, 32)[0] == 1004
    assert orc.act_quant_f8_prefix(row, 0, 64, 64, 64)[0] == 1001


def test_act_quant_scale_is_a_power_of_two_with_a_floor():
    row = np.full(64, 3e-5, np.float32)     # below the 1e-4 floor: the scale comes from the floor
    rc, out = orc.act_quant_f8_prefix(row, 1, 64, 64, 64)
    s = 2.0 ** np.ceil(np.log2(1e-4 / 448))
    assert np.all(out / np.float32(s) == np.round(out / np.float32(s)))


def _comp_fixture(rng, p, n_pos):
    norm = orc.bf16_to_f32(orc.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(p.d).astype(np.float32)))
    ang = rng.uniform(0, 2 * np.pi, (n_pos, p.rd // 2))
    freqs = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32).reshape(n_pos, p.rd)
    ape = (0.5 * rng.standard_normal((p.ratio, p.cd))).astype(np.float32)
    return norm, freqs, ape


def test_compressor_decode_pools_by_entry_softmax_and_shifts_the_overlap():
    rng = np.random.default_rng(21)
    p = orc.CompGeom.make(ratio=4, d=64, rd=16)
    norm, freqs, ape = _comp_fixture(rng, p, 16)
    kv_state = np.zeros((p.ents, p.cd), np.float32)
    score_state = np.full((p.ents, p.cd), -np.inf, np.float32)
    toks = []
    for pos in range(1, 8):
        kv, sc = rng.standard_normal(p.cd).astype(np.float32), rng.standard_normal(p.cd).astype(np.float32)
        toks.append((pos, kv, sc))
        assert orc.v4_compress_deposit_token(kv, sc, ape, kv_state, score_state, p, pos) == 0
        slot = p.ratio + pos % p.ratio
        assert np.array_equal(kv_state[slot], kv) and np.array_equal(score_state[slot], sc + ape[pos % p.ratio])
        if (pos + 1) % p.ratio:
            assert orc.v4_compress_decode(kv_state, score_state, norm, freqs, p, pos)[0] == 1009
            continue
        before_kv, before_sc = kv_state.copy(), score_state.copy()
        rc, row = orc.v4_compress_decode(kv_state, score_state, norm, freqs, p, pos)
        assert rc == 0
        # the overlap half moved down
        assert np.array_equal(kv_state[:p.ratio], before_kv[p.ratio:]) and np.array_equal(score_state[:p.ratio], before_sc[p.ratio:])
        # reference in float64: entries below ratio give their first d dims, the others their last d
        k = np.concatenate([before_kv[:p.ratio, :p.d], before_kv[p.ratio:, p.d:]]).astype(np.float64)
        s = np.concatenate([before_sc[:p.ratio, :p.d], before_sc[p.ratio:, p.d:]]).astype(np.float64)
        live = np.isfinite(s).any(axis=0)
        w = np.exp(s - s.max(axis=0, where=np.isfinite(s), initial=-1e300))
        pooled = np.where(live, (k * w).sum(axis=0) / np.maximum(w.sum(axis=0), 1e-300), 0.0)
        pooled = orc.bf16_to_f32(orc.f32_to_bf16(pooled.astype(np.float32))).astype(np.float64)
        x = norm * (pooled / np.sqrt((pooled ** 2).mean() + p.eps))
        x = orc.bf16_to_f32(orc.f32_to_bf16(x.astype(np.float32))).astype(np.float64)
        blk = (pos // p.ratio) * p.ratio
        c, sn = freqs[blk, 0::2], freqs[blk, 1::2]
        a, b = x[p.d - p.rd::2].copy(), x[p.d - p.rd + 1::2].copy()
        x[p.d - p.rd::2], x[p.d - p.rd + 1::2] = a * c - b * sn, a * sn + b * c
        assert np.allclose(row, x, rtol=0, atol=np.abs(x).max() / 64)
        assert np.array_equal(row, orc.bf16_to_f32(orc.f32_to_bf16(row)))
    assert orc.v4_compress_decode(kv_state, score_state, norm, freqs, p, 0)[0] == 1007
    bad = orc.CompGeom(4, 2, 64, 128, 7, 16, 1e-6)
    assert orc.v4_compress_decode(kv_state, score_state, norm, freqs, bad, 3)[0] == 1003


def test_compressor_prefill_and_decode_arms_agree():
    """A prompt pooled by the prefill arm and the same tokens fed one at a time after a one-block prompt give the
    same blocks and leave the same state: same entries, same fold order."""
    rng = np.random.default_rng(23)
    p = orc.CompGeom.make(ratio=4, d=64, rd=16)
    norm, freqs, ape = _comp_fixture(rng, p, 16)
    s = 11
    kv = rng.standard_normal((s + 1, p.cd)).astype(np.float32)
    sc = rng.standard_normal((s + 1, p.cd)).astype(np.float32)

    def fresh():
        return np.zeros((p.ents, p.cd), np.float32), np.full((p.ents, p.cd), -np.inf, np.float32)

    # A: the whole prompt through the prefill arm, then one decode token closes block 2
    ka, sa = fresh()
    assert orc.v4_compress_deposit_prefill(kv[:s], sc[:s], ape, ka, sa, p, s) == 0
    rc, blocks_a = orc.v4_compress_prefill(kv[:s], sc[:s], ape, norm, freqs, p, s // p.ratio)
    assert rc == 0 and blocks_a.shape == (2, p.d)
    orc.v4_compress_deposit_token(kv[s], sc[s], ape, ka, sa, p, s)
    rc, b2_a = orc.v4_compress_decode(ka, sa, norm, freqs, p, s)
    assert rc == 0
    # B: one block of prompt, the rest token by token
    kb, sb = fresh()
    orc.v4_compress_deposit_prefill(kv[:4], sc[:4], ape, kb, sb, p, 4)
    rc, blocks_b0 = orc.v4_compress_prefill(kv[:4], sc[:4], ape, norm, freqs, p, 1)
    got = {}
    for pos in range(4, s + 1):
        orc.v4_compress_deposit_token(kv[pos], sc[pos], ape, kb, sb, p, pos)
        if (pos + 1) % p.ratio == 0:
            rc, got[pos // p.ratio] = orc.v4_compress_decode(kb, sb, norm, freqs, p, pos)
    assert np.array_equal(blocks_a[0], blocks_b0[0])
    assert np.array_equal(blocks_a[1], got[1])
    assert np.array_equal(b2_a, got[2])
    assert np.array_equal(ka, kb) and np.array_equal(sa, sb)
    assert orc.v4_compress_prefill(kv, sc, ape, norm, freqs, p, 0)[0] == 1006
    assert orc.v4_compress_deposit_prefill(kv, sc, ape, ka, sa, p, 0) == 1005
