"""The CPU oracle against every literal value the reference's own tests record for this path.

Each case names the reference test it comes from (paths relative to the reference root).
"""
import math

import numpy as np
import pytest

from oracle import oracle as orc


# crates/core/src/routing.rs:207-212 -- the tie rule: value descending, index ascending.
def test_topk_tie_rule_literals():
    s = [0.1, 0.9, 0.5, 0.9]
    assert orc.topk_value_order(s, 3).tolist() == [1, 3, 2]
    assert orc.topk_value_order(s, 10).tolist() == [1, 3, 2, 0]
    # the attend row set is the same selection emitted ascending (kernel_vector.rs:126-131)
    assert orc.index_topk(s, 3).tolist() == [1, 2, 3]


# crates/core/src/routing.rs:259-284 -- bf16 narrowing literals.
def test_bf16_literals():
    L = orc.lib()
    cases = [(0.0, 0x0000), (1.0, 0x3F80), (-2.0, 0xC000), (1.0 + 2.0 ** -8, 0x3F80),
             (1.0 + 2.0 ** -8 + 2.0 ** -16, 0x3F81), (float("inf"), 0x7F80)]
    for x, want in cases:
        assert L.orc_f32_to_bf16(x) == want, (x, hex(L.orc_f32_to_bf16(x)))
    nan_bits = L.orc_f32_to_bf16(float("nan"))
    assert math.isnan(L.orc_bf16_to_f32(nan_bits))
    # vectorised numpy twin used by the tests agrees with the C function
    xs = np.array([c[0] for c in cases], dtype=np.float32)
    assert orc.f32_to_bf16(xs).tolist() == [c[1] for c in cases]


# crates/core/src/routing.rs:338-362 -- e4m3 round trips, saturation, NaN, in-range bound.
def test_e4m3_literals():
    L = orc.lib()
    for v in (0.0, 1.0, -2.0, 448.0, 1.5, 0.0625):
        assert L.orc_e4m3_to_f32(L.orc_f32_to_e4m3(v)) == v
    assert L.orc_e4m3_to_f32(L.orc_f32_to_e4m3(1000.0)) == 448.0
    assert L.orc_e4m3_to_f32(L.orc_f32_to_e4m3(-1000.0)) == -448.0
    assert L.orc_f32_to_e4m3(float("nan")) == 0x7F
    assert math.isnan(L.orc_e4m3_to_f32(0x7F))
    rng = np.random.RandomState(0)
    for x in rng.uniform(-448, 448, 2000).astype(np.float32):
        y = L.orc_e4m3_to_f32(L.orc_f32_to_e4m3(float(x)))
        assert abs(y - float(x)) <= 0.07 * abs(float(x)) + 1e-3


# crates/core/src/num.rs:137-150 -- subnormal rounding is half-AWAY, and m == 8 promotes.
def test_e4m3_subnormal_rule():
    L = orc.lib()
    step = 2.0 ** -9
    assert L.orc_f32_to_e4m3(0.5 * step) == 0x01          # exact tie 0.5 -> 1 (away), RNE would give 0
    assert L.orc_f32_to_e4m3(2.5 * step) == 0x03          # tie 2.5 -> 3 (away), RNE would give 2
    assert L.orc_f32_to_e4m3(7.5 * step) == 0x08          # rounds up into the smallest normal
    assert L.orc_f32_to_e4m3(-2.5 * step) == 0x83
    assert L.orc_f32_to_e4m3(0.49 * step) == 0x00
    assert L.orc_f32_to_e4m3(2.0 ** -11) == 0x00          # below 2^-10 -> signed zero
    assert L.orc_f32_to_e4m3(-(2.0 ** -11)) == 0x80
    # every code decodes and re-encodes to itself (NaN codes aside)
    for c in range(256):
        if (c & 0x7F) == 0x7F:
            continue
        assert L.orc_f32_to_e4m3(L.orc_e4m3_to_f32(c)) == c


# crates/engine/tests/fwd_kernel.rs:140-160 -- the fixture comment records the two block
# amaxes of the Lcg(0xA99E) draw; reproducing them pins the Lcg port and the block fold.
def test_append_kv_fixture_amaxes_and_layout():
    rows, kvl, ropn, pos = 5, 256, 64, 3
    r = orc.Lcg(0xA99E)
    latent = np.array([r.f() * (1.0 if i < 128 else 20.0) for i in range(kvl)], dtype=np.float32)
    rope = r.draws(ropn)
    assert abs(np.abs(latent[:128]).max() - 0.9949) < 5e-5
    assert abs(np.abs(latent[128:]).max() - 19.9455) < 5e-5
    lc8 = np.zeros(rows * kvl, np.uint8)
    ls = np.zeros(rows * 2, np.float32)
    rc = np.zeros(rows * ropn, np.uint16)
    assert orc.append_kv(latent, rope, lc8, ls, rc, pos, kvl, ropn, 2) == 0
    # only row `pos` is written, with three different strides
    mask = np.ones(rows, bool); mask[pos] = False
    assert not lc8.reshape(rows, kvl)[mask].any()
    assert not ls.reshape(rows, 2)[mask].any()
    assert not rc.reshape(rows, ropn)[mask].any()
    assert (lc8.reshape(rows, kvl)[pos] != 0).sum() > kvl // 2
    # each block's extreme lands on the saturation code 0x7e (=448)
    codes = lc8.reshape(rows, kvl)[pos]
    assert (codes[:128] & 0x7F).max() == 0x7E and (codes[128:] & 0x7F).max() == 0x7E
    np.testing.assert_array_equal(ls.reshape(rows, 2)[pos],
                                  np.array([np.abs(latent[:128]).max(), np.abs(latent[128:]).max()],
                                           np.float32) / np.float32(448.0))
    np.testing.assert_array_equal(rc.reshape(rows, ropn)[pos], orc.f32_to_bf16(rope))


# crates/engine/tests/common/reference.rs:141-162 -- the stream is uniform in [-1, 1] and signed.
def test_lcg_range():
    d = orc.Lcg(0x5C04).draws(100000)
    assert d.min() >= -1.0 and d.max() <= 1.0
    assert 0.45 < (d > 0).mean() < 0.55


# crates/core/src/routing.rs:221-256 -- online softmax recurrence == two-pass at n = 200000.
def test_online_softmax_matches_two_pass():
    n = 200000
    r = orc.Lcg(0x1234)
    s = r.draws(n) * 8.0
    v = r.draws(n)
    p = orc.softmax(s)
    want = float((p.astype(np.float64) * v).sum())
    m, l, acc = -np.inf, 0.0, 0.0
    for i in range(0, n, 1000):
        blk = s[i:i + 1000].astype(np.float64)
        m_new = max(m, blk.max())
        corr = math.exp(m - m_new) if m > -np.inf else 0.0
        pe = np.exp(blk - m_new)
        acc = acc * corr + float((pe * v[i:i + 1000]).sum())
        l = l * corr + float(pe.sum())
        m = m_new
    assert abs(acc / l - want) < 1e-4


# crates/engine/tests/kernel_vector.rs:124-212 -- the ten selection shapes; properties the
# reference asserts (strictly ascending, exact count) plus the threshold property.
def _topk_cases():
    rng = orc.Lcg(0x7071C0DE)
    nt = 5185
    relu = np.zeros(nt, np.float32); relu[:300] = (300 - np.arange(300)) * 0.25
    scat = np.zeros(nt, np.float32)
    for j in range(300):
        scat[(j * 7919) % nt] = (300 - j) * 0.25
    dense = rng.draws(nt) * 8.0
    heavy = np.floor(rng.draws(nt) * 4.0)
    ramp = lambda n, m: (np.arange(n) % m).astype(np.float32)
    sz = np.where(np.arange(4096) % 3 == 0, -0.0, 0.0).astype(np.float32)
    neg = -(np.arange(4096) % 11).astype(np.float32)
    return [("signed zeros", sz, 2048), ("negatives", neg, 2048), ("k==nt", ramp(2048, 7), 2048),
            ("k==nt-1", ramp(2049, 7), 2048), ("k>nt", ramp(500, 7), 2048),
            ("single block", ramp(200, 5), 64), ("relu sparse", relu, 2048),
            ("scattered", scat, 2048), ("dense", dense, 2048), ("heavy ties", heavy, 2048)]


@pytest.mark.parametrize("name,scores,k", _topk_cases(), ids=[c[0] for c in _topk_cases()])
def test_topk_selection_properties(name, scores, k):
    rows = orc.index_topk(scores, k)
    n = min(k, scores.size)
    assert rows.size == n
    assert (np.diff(rows.astype(np.int64)) > 0).all()
    sel = np.zeros(scores.size, bool); sel[rows] = True
    if n < scores.size:
        lo = scores[sel].min(); hi = scores[~sel].max()
        assert lo >= hi
        # ties at the boundary go to the lower index
        tied_in = np.nonzero(sel & (scores == lo))[0]
        tied_out = np.nonzero(~sel & (scores == lo))[0]
        if tied_out.size and tied_in.size:
            assert tied_in.max() < tied_out.min()
    if name == "signed zeros":
        assert rows.tolist() == list(range(2048))       # -0.0 ties +0.0, index decides
    if name == "relu sparse":
        assert rows.tolist() == list(range(2048))


# crates/backend/kernels/attn.hip:75-93 -- plan regimes the reference's tests name
# (kernel_attend.rs:270-295): nt=300 -> 4 splits, 704 -> by_grid binds, 4608 -> 16 splits.
def test_split_plan_regimes():
    assert orc.mla_plan_splits(64, 300)[0] == 4
    assert orc.mla_plan_splits(64, 704)[0] == 11
    assert orc.mla_plan_splits(64, 4608)[0] == 16
    assert orc.mla_plan_splits(64, 4608, have_scratch=False)[0] == 1
    assert orc.mla_plan_splits(4, 1)[0] == 1


# crates/engine/tests/kernel_attend.rs:228-304 fixture draw; combine (attn.hip:241-273) of the
# planned splits must reproduce the dense two-pass result.
@pytest.mark.parametrize("seed,H,nt,kvl,rope", [(0x00C0FFEE, 4, 1, 128, 8), (0xB10CC0DE, 20, 130, 512, 64),
                                                 (0x0A5E1102, 64, 300, 512, 64)])
def test_attend_dense_equals_split_combine(seed, H, nt, kvl, rope):
    nb = kvl // 128
    r = orc.Lcg(seed)
    qabs = r.draws(H * kvl); qrope = r.draws(H * rope)
    lc8 = orc.f32_to_e4m3(r.draws(nt * kvl))
    lscale = np.abs(r.draws(nt * nb) * np.float32(0.1)) + np.float32(0.01)
    rc = orc.f32_to_bf16(r.draws(nt * rope))
    scale = np.float32(1.0) / np.sqrt(np.float32(kvl + rope))
    want = orc.mla_attend(qabs, qrope, lc8, lscale, rc, None, H, nt, kvl, rope, nb, scale)
    n_splits, tps = orc.mla_plan_splits(H, nt)
    acc = np.zeros((n_splits, H, kvl), np.float32); ml = np.zeros((n_splits, H, 2), np.float32)
    for s in range(n_splits):
        a, m = orc.mla_attend_partial(qabs, qrope, lc8, lscale, rc, H, s * tps * 16,
                                      min(nt, (s + 1) * tps * 16), kvl, rope, nb, scale)
        acc[s] = a.reshape(H, kvl); ml[s] = m.reshape(H, 2)
    got = orc.attend_combine(acc, ml, H, kvl, n_splits)
    tol = 1e-3 * np.abs(want).max() + 1e-3        # crates/engine/tests/common/scoring.rs:191-194
    assert np.abs(got - want).max() <= tol
    # rows = identity list gives the dense answer bit for bit
    got_rows = orc.mla_attend(qabs, qrope, lc8, lscale, rc, np.arange(nt, dtype=np.uint32), H, nt,
                              kvl, rope, nb, scale)
    np.testing.assert_array_equal(got_rows, want)


# crates/engine/tests/indexer_kernel.rs:214-367 -- DSA (all heads) vs MISA (listed heads)
# must separate on the reference's own fixture, and a float64 recomputation must agree.
def test_index_score_fixture():
    nt, nh, hd = 64, 64, 128
    r = orc.Lcg(0x5C04)
    q = r.draws(nh * hd); w = r.draws(nh)
    kc = orc.f32_to_bf16(r.draws(nt * hd))
    s_all = orc.index_score(q, w, kc, None, nt, nh, nh, hd, 0.75, 0.125)
    s_sub = orc.index_score(q, w, kc, [5, 0, 6, 2], nt, nh, 4, hd, 0.75, 0.125)
    sep = np.abs(s_sub - s_all).max() / np.abs(s_all).max()
    assert sep > 1e-2
    kf = orc.bf16_to_f32(kc).reshape(nt, hd).astype(np.float64)
    dots = kf @ q.reshape(nh, hd).astype(np.float64).T
    ref = (np.maximum(dots * 0.125, 0) * (w.astype(np.float64) * 0.75)).sum(1)
    assert np.abs(ref - s_all).max() <= 1e-5 * np.abs(ref).max()


# crates/engine/tests/fwd_kernel.rs:94-125
def test_gather_rope_fixture():
    h, qh, nope, ropn = 8, 192, 96, 64
    q = orc.Lcg(0x60A7).draws(h * qh)
    got = orc.gather_rope(q, h, qh, nope, ropn)
    want = q.reshape(h, qh)[:, nope:nope + ropn].ravel()
    np.testing.assert_array_equal(got, want)


# crates/engine/tests/indexer_kernel.rs:120-140
def test_index_append_fixture():
    rows, hd, pos = 7, 128, 5
    k = orc.Lcg(0xC0DE).draws(hd) * np.float32(8.0)
    cache = np.zeros(rows * hd, np.uint16)
    orc.index_append(k, cache, pos, hd)
    want = np.zeros((rows, hd), np.uint16); want[pos] = orc.f32_to_bf16(k)
    np.testing.assert_array_equal(cache.reshape(rows, hd), want)


# --- kv_b projections (absorb / value): the reference's six seeded shapes -----------------------------
MLA_SHAPES = [  # (seed, [h, qh, nope, vh, kvl, block]) - crates/engine/tests/kernel_attend.rs:322-331
    (0x77, [4, 128, 128, 64, 256, 128]), (0x78, [3, 64, 48, 32, 37, 128]), (0x79, [2, 32, 16, 8, 64, 2]),
    (0x7a, [2, 32, 16, 8, 64, 4]), (0x7b, [2, 32, 16, 8, 68, 64]), (0x7c, [2, 16, 8, 4, 2, 128]),
]


def _mla_numpy_reference(packed, scale, q, clat, dims):
    """The host references of the reference's test restated independently in numpy
    (kernel_attend.rs:345-390): dequantised kv_b, then a left fold of plain products."""
    h, qh, nope, vh, kvl, block = dims
    rows = h * (nope + vh)
    sc_rows, sc_cols = -(-rows // block), -(-kvl // block)
    r_idx = np.minimum(np.arange(rows) // block, sc_rows - 1)[:, None]
    c_idx = (np.arange(kvl) // block)[None, :]
    kvb = orc.e4m3_table()[packed.reshape(rows, kvl)] * scale.reshape(sc_rows, sc_cols)[r_idx, c_idx]
    kvb = kvb.astype(np.float32)
    absorb = np.zeros((h, kvl), np.float32)
    value = np.zeros((h, vh), np.float32)
    for head in range(h):
        acc = np.zeros(kvl, np.float32)
        for d in range(nope):
            acc = (acc + q[head * qh + d] * kvb[head * (nope + vh) + d]).astype(np.float32)
        absorb[head] = acc
        acc = np.zeros(vh, np.float32)
        for i in range(kvl):
            acc = (acc + clat[head * kvl + i] * kvb[head * (nope + vh) + nope: head * (nope + vh) + nope + vh, i]).astype(np.float32)
        value[head] = acc
    return absorb.ravel(), value.ravel()


@pytest.mark.parametrize("seed,dims", MLA_SHAPES)
def test_mla_absorb_value_match_the_host_reference(seed, dims):
    h, qh, nope, vh, kvl, block = dims
    r = orc.Lcg(seed)
    packed, scale = orc.kvb_fixture(r, h * (nope + vh), kvl, block)      # draw order of check_mla_fp8
    q = r.draws(h * qh)
    clat = r.draws(h * kvl)
    want_abs, want_val = _mla_numpy_reference(packed, scale, q, clat, dims)
    got_abs = orc.mla_absorb_fp8(q, packed, scale, h, qh, nope, vh, kvl, block)[0]
    got_val = orc.mla_value_fp8(clat, packed, scale, h, nope, vh, kvl, block)[0]
    np.testing.assert_array_equal(got_abs.view(np.uint32), want_abs.view(np.uint32))   # same fold, same bits
    np.testing.assert_array_equal(got_val.view(np.uint32), want_val.view(np.uint32))


def test_mla_batched_rows_equal_single_rows():
    """Two q rows through one call == each row alone (kernel_attend.rs:431-493, seed 0xba7c)."""
    h, qh, nope, vh, kvl, block = 3, 20, 12, 8, 16, 4
    r = orc.Lcg(0xBA7C)
    packed, scale = orc.kvb_fixture(r, h * (nope + vh), kvl, block)
    qs = [r.draws(h * qh) for _ in range(2)]
    cs = [r.draws(h * kvl) for _ in range(2)]
    both_a = orc.mla_absorb_fp8(np.concatenate(qs), packed, scale, h, qh, nope, vh, kvl, block, nrow=2)
    both_v = orc.mla_value_fp8(np.concatenate(cs), packed, scale, h, nope, vh, kvl, block, nrow=2)
    for i in range(2):
        np.testing.assert_array_equal(both_a[i], orc.mla_absorb_fp8(qs[i], packed, scale, h, qh, nope, vh, kvl, block)[0])
        np.testing.assert_array_equal(both_v[i], orc.mla_value_fp8(cs[i], packed, scale, h, nope, vh, kvl, block)[0])


# --- indexer front end: fp8 GEMV, layernorm, interleaved RoPE ------------------------------------------
def test_gemv_fp8_literal_kat():
    """crates/artifact/src/quant/fp8.rs:275-284: 2x2 codes [[1,2],[-1,0]], per-element scales."""
    y = orc.gemv_fp8(np.array([3.0, 5.0], np.float32), np.array([0x38, 0x40, 0xB8, 0x00], np.uint8),
                     np.array([10.0, 100.0, 1000.0, 1.0], np.float32), 2, 2, 1)
    assert y[0].tolist() == [1030.0, -3000.0]


@pytest.mark.parametrize("seed,o_dim,i_dim,block", [(0x6E37, 130, 256, 128), (0x6E38, 64, 96, 32), (0x6E39, 7, 37, 4)])
def test_gemv_fp8_matches_an_independent_fold(seed, o_dim, i_dim, block):
    """Draw order weights, scales, x (crates/engine/tests/common/reference.rs:234-247); the ragged
    o_dim = 130 at block 128 is the shape that makes o_dim / block wrong there."""
    r = orc.Lcg(seed)
    packed = orc.f32_to_e4m3(r.draws(o_dim * i_dim))
    sc_rows, sc_cols = -(-o_dim // block), -(-i_dim // block)
    scale = (np.abs(r.draws(sc_rows * sc_cols) * np.float32(0.1)) + np.float32(0.01)).astype(np.float32)
    x = r.draws(i_dim)
    w = (orc.e4m3_table()[packed.reshape(o_dim, i_dim)] *
         scale.reshape(sc_rows, sc_cols)[(np.arange(o_dim) // block)[:, None], (np.arange(i_dim) // block)[None, :]]).astype(np.float32)
    want = np.zeros(o_dim, np.float32)
    for i in range(i_dim):
        want = (want + (w[:, i] * x[i]).astype(np.float32)).astype(np.float32)
    got = orc.gemv_fp8(x, packed, scale, o_dim, i_dim, block)[0]
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    two = orc.gemv_fp8(np.concatenate([x, x[::-1]]), packed, scale, o_dim, i_dim, block, nrow=2)
    np.testing.assert_array_equal(two[0], got)


def test_layernorm_centres_scales_and_biases():
    """crates/engine/tests/indexer_kernel.rs:53-111: n 1024, Lcg(0x1AE6), x + 1.5, w + 1, b * 0.25, eps 1e-6."""
    n = 1024
    r = orc.Lcg(0x1AE6)
    x = (r.draws(n) + np.float32(1.5)).astype(np.float32)
    w = (r.draws(n) + np.float32(1.0)).astype(np.float32)
    b = (r.draws(n) * np.float32(0.25)).astype(np.float32)

    def host(centre, bias):
        mean = np.float32(x.astype(np.float64).sum() / n)
        var = np.float32((x.astype(np.float64) ** 2).sum() / n) - mean * mean
        inv = np.float32(1.0) / np.sqrt(np.float32(var + np.float32(1e-6)))
        m = mean if centre else np.float32(0)
        return ((x - m) * inv * w + (b if bias else 0)).astype(np.float32)

    want = host(True, True)
    rel = lambda a, c: float(np.abs(a - c).max() / np.abs(c).max())
    assert rel(host(False, True), want) > 1e-2 and rel(host(True, False), want) > 1e-2     # the fixture can see both defects
    assert rel(orc.layernorm(x, w, b, 1e-6), want) <= 1e-6


def test_rope_interleave_is_a_permutation_at_position_zero():
    """crates/engine/tests/kernel_vector.rs:280-319: count 5, stride 24, seg 16, theta 1e4, Lcg(0x2909)."""
    count, stride, seg, theta = 5, 24, 16, 10000.0
    half = seg // 2
    base = orc.Lcg(0x2909).draws(count * stride)

    def host(pos):
        v = base.copy()
        for s in range(count):
            row = base[s * stride: s * stride + seg]
            for j in range(half):
                a, b = row[2 * j], row[2 * j + 1]
                ang = pos * theta ** (-2.0 * j / seg)
                cs, sn = np.float32(np.cos(ang)), np.float32(np.sin(ang))
                v[s * stride + j] = a * cs - b * sn
                v[s * stride + half + j] = b * cs + a * sn
        return v

    np.testing.assert_array_equal(orc.rope_interleave(base, count, stride, seg, 0, theta).view(np.uint32), host(0).view(np.uint32))
    got, want = orc.rope_interleave(base, count, stride, seg, 137, theta), host(137)
    assert float(np.abs(got - want).max() / np.abs(want).max()) <= 1e-6
    np.testing.assert_array_equal(got.reshape(count, stride)[:, seg:], base.reshape(count, stride)[:, seg:])   # stride > seg untouched
