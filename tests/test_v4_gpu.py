"""GPU parity of the V4 cousin path (spread, block scorer, selection rows, sparse attention with sink)
against the CPU oracle, through the C ABI. Bit-exact for the spread, the scores and the selected indices;
the reference's own bar (error <= 1/128 of the largest expected element) for the attention output."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as orc
from oracle import v4_workload as wl


def _be():
    from rivoli_b200 import backend as be
    return be


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("d", [32, 128, 256])
def test_spread_is_bit_identical(d):
    be = _be()
    rng = np.random.default_rng(d)
    x = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((97, d)).astype(np.float32)))
    # rows scaled across sixty binades so the power-of-two scale is exercised widely
    x *= (2.0 ** (np.arange(97) % 60 - 30)).astype(np.float32)[:, None]
    x = orc.bf16_to_f32(orc.f32_to_bf16(x))
    x[5] = 0.0
    rc, want = orc.v4_spread(x, d)
    assert rc == 0
    t = dev(x)
    be.launch_act_quant_f4_rotated(t, 97, d)
    assert np.array_equal(bits(t.cpu().numpy()), bits(want))


def test_spread_and_score_guards():
    be = _be()
    t = torch.zeros(1024, device="cuda")
    for rows, d, code in [(0, 128, 1001), (1, 512, 1002), (1, 96, 1003), (1, 16, 1004)]:
        with pytest.raises(be.BackendError) as e:
            be.launch_act_quant_f4_rotated(t, rows, d)
        assert e.value.code == code
    with pytest.raises(be.BackendError) as e:
        be.launch_index_score_blocks(t, t, t, t, 0, 1, 1, 1)
    assert e.value.code == 1001
    with pytest.raises(be.BackendError) as e:
        be.launch_index_score_blocks(t, t, t, t, 1, 0, 1, 1)
    assert e.value.code == 1005
    i = torch.zeros(8, dtype=torch.int32, device="cuda")
    for d, topk, code in [(1025, 8, 1002), (1024, 1 << 20, 1006), (0, 8, 1001)]:
        with pytest.raises(be.BackendError) as e:
            be.launch_gather_attn_shared_kv(t, t, t, i, 1, 1, d, topk, 1.0, t)
        assert e.value.code == code


@pytest.mark.parametrize("s,n_comp,heads,hd", [(1, 1, 64, 128), (3, 37, 64, 128), (2, 301, 5, 32), (2, 19, 70, 24),
                                               (1, 1000, 33, 64)])
def test_block_scores_are_bit_identical(s, n_comp, heads, hd):
    be = _be()
    rng = np.random.default_rng(n_comp)
    if hd % 32 == 0:
        q = orc.v4_spread(orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((s * heads, hd)).astype(np.float32))), hd)[1]
        kv = orc.v4_spread(orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((n_comp, hd)).astype(np.float32))), hd)[1]
    else:
        q = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((s * heads, hd)).astype(np.float32)))
        kv = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((n_comp, hd)).astype(np.float32)))
    w = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((s, heads)).astype(np.float32)))
    if (s, n_comp) == (1, 1):  # the f32-accumulate case: 1 + 63 * 2^-9 rounds once to 1.125
        q[:], kv[:], w[:] = 0, 0, 1
        kv[0, 0] = 1.0
        q[:, 0] = 2.0 ** -9
        q[0, 0] = 1.0
    rc, want = orc.v4_index_score_blocks(q, kv, w, s, n_comp, heads, hd)
    assert rc == 0
    out = torch.zeros((s, n_comp), device="cuda")
    be.launch_index_score_blocks(dev(q), dev(kv), dev(w), out, s, n_comp, heads, hd)
    got = out.cpu().numpy()
    assert np.array_equal(bits(got), bits(want))
    if (s, n_comp) == (1, 1):
        assert got[0, 0] == np.float32(1.125)


def test_unspread_inputs_score_bit_identically():
    """Full-precision bf16 inputs round at every step of the fold: the order and the unfused ops matter."""
    be = _be()
    rng = np.random.default_rng(2)
    s, n_comp, heads, hd = 2, 200, 64, 128
    q = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((s * heads, hd)).astype(np.float32)))
    kv = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((n_comp, hd)).astype(np.float32)))
    w = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((s, heads)).astype(np.float32)))
    rc, want = orc.v4_index_score_blocks(q, kv, w, s, n_comp, heads, hd)
    out = torch.zeros((s, n_comp), device="cuda")
    be.launch_index_score_blocks(dev(q), dev(kv), dev(w), out, s, n_comp, heads, hd)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want))


def test_gather_attn_reference_layout():
    be = _be()
    rng = np.random.default_rng(9)
    m, h, d, n, topk = 3, 8, 512, 300, 160
    bf = lambda a: orc.bf16_to_f32(orc.f32_to_bf16(a.astype(np.float32)))
    q, kv = bf(rng.standard_normal((m, h, d))), bf(rng.standard_normal((n, d)))
    sink = rng.standard_normal(h).astype(np.float32)
    idx = np.stack([rng.permutation(n)[:topk] for _ in range(m)]).astype(np.int32)
    idx[0, ::7] = -1
    idx[2, :] = -1
    rc, want = orc.v4_sparse_attn(q, kv, sink, idx, m, h, d, topk, d ** -0.5)
    out = torch.zeros((m, h, d), device="cuda")
    be.launch_gather_attn_shared_kv(dev(q), dev(kv), dev(sink), dev(idx), m, h, d, topk, d ** -0.5, out)
    got = out.cpu().numpy()
    assert np.all(np.isnan(got[2])) and np.all(np.isnan(want[2]))
    ok, worst = wl.attend_close(orc.f32_to_bf16(got[:2]), orc.f32_to_bf16(want[:2]))
    assert ok, worst
    assert np.array_equal(bits(got[:2]), bits(orc.bf16_to_f32(orc.f32_to_bf16(got[:2]))))  # stored on the bf16 grid


def _run_step(g, inp, force_simt=False, want_scores=True, force_fold=False, want_flags=False, pack=False):
    be = _be()
    from rivoli_b200.v4 import V4DecodeLayer
    B = inp["pos"].size
    bg = be.V4Geom(*[getattr(g, n) for n, _ in orc.V4Geom._fields_])
    layer = V4DecodeLayer(bg, B)
    layer.kv_cache.copy_(dev(inp["kv_cache"]))
    layer.index_kv.copy_(dev(inp["ikv"]))
    layer.sink.copy_(dev(inp["sink"]))
    if pack:   # the int8 + exponent form of the rows, as a cache writer would leave it
        n_rows = (inp["pos"] + 1) // g.ratio
        layer.pack_index_rows(None, dev(n_rows.astype(np.int32)), int(n_rows.max()))
    layer.select(dev(inp["pos"]), dev(inp["iq"]), dev(inp["iw"]), force_fold)
    layer.attend(dev(inp["q"]), force_simt)
    torch.cuda.synchronize()
    res = (layer.sel.cpu().numpy(), layer.out.cpu().numpy(), (layer.scores.cpu().numpy() if want_scores else None))
    return res + (layer.refolded.cpu().numpy(),) if want_flags else res


def test_batched_step_small_shapes():
    g = wl.make_geom(n_heads=4, head_dim=64, window=8, index_heads=4, index_dim=32, index_topk=4, max_comp=16)
    pos = np.array([0, 5, 30, 63, 7, 18], np.int32)
    inp = wl.make_inputs(g, pos.size, pos, seed=1)
    want_sel, want_out, want_sc = orc.v4_decode_step_bf16(g, pos, inp["q"], inp["kv_cache"], inp["sink"], inp["iq"],
                                                          inp["iw"], inp["ikv"], want_scores=True)
    sel, out, sc = _run_step(g, inp)
    assert np.array_equal(sel, want_sel)
    for b in range(pos.size):
        n_comp = (pos[b] + 1) // g.ratio
        if n_comp > g.index_topk:
            assert np.array_equal(bits(sc[b, :n_comp]), bits(want_sc[b, :n_comp]))
    ok, worst = wl.attend_close(out, want_out)
    assert ok, worst


@pytest.mark.parametrize("force_simt,force_fold,pack", [(False, False, False), (True, True, False), (False, False, True)])
def test_batched_step_model_shapes(force_simt, force_fold, pack):
    g = wl.make_geom(max_comp=640, index_topk=96)
    pos = np.array([3, 126, 127, 500, 2559, 1023, 1500, 390], np.int32)  # ring filling / full; positional and scored
    inp = wl.make_inputs(g, pos.size, pos, seed=4)
    inp["iw"][1] = np.abs(inp["iw"][1])
    want_sel, want_out, want_sc = orc.v4_decode_step_bf16(g, pos, inp["q"], inp["kv_cache"], inp["sink"], inp["iq"],
                                                          inp["iw"], inp["ikv"], want_scores=True)
    sel, out, sc, flags = _run_step(g, inp, force_simt, force_fold=force_fold, want_flags=True, pack=pack)
    if not force_fold:
        assert not flags.any()      # spread rows are what the integer scorer takes whole
    assert np.array_equal(sel, want_sel)
    for b in range(pos.size):
        n_comp = (pos[b] + 1) // g.ratio
        if n_comp > g.index_topk:
            assert np.array_equal(bits(sc[b, :n_comp]), bits(want_sc[b, :n_comp]))
    ok, worst = wl.attend_close(out, want_out)
    assert ok, worst


def test_tie_heavy_scores_select_the_lower_blocks():
    """All-zero head weights make every score +0: the selection must be the first index_topk blocks."""
    g = wl.make_geom(max_comp=640, index_topk=96)
    pos = np.array([2559, 2001], np.int32)
    inp = wl.make_inputs(g, 2, pos, seed=6)
    inp["iw"][:] = 0.0
    sel, _, _ = _run_step(g, inp, want_scores=False)
    for b in range(2):
        assert sel[b, g.window:].tolist() == list(range(g.window, g.window + g.index_topk))


def test_fully_masked_row_is_nan_and_masked_slots_are_ignored():
    be = _be()
    g = wl.make_geom(max_comp=64, index_topk=32)
    bg = be.V4Geom(*[getattr(g, n) for n, _ in orc.V4Geom._fields_])
    B, cols = 3, g.window + g.index_topk
    inp = wl.make_inputs(g, B, np.array([200, 200, 200], np.int32), seed=8)
    rng = np.random.default_rng(0)
    sel = np.stack([rng.permutation(g.window + 50)[:cols] for _ in range(B)]).astype(np.int32)
    sel[0, :] = -1
    sel[1, 1::2] = -1
    sel[2, :cols - 3] = -1
    want = np.zeros((B, g.n_heads, g.head_dim), np.uint16)
    for b in range(B):
        rc, o = orc.v4_sparse_attn(orc.bf16_to_f32(inp["q"][b]), orc.bf16_to_f32(inp["kv_cache"][b]), inp["sink"],
                                   sel[b], 1, g.n_heads, g.head_dim, cols, g.softmax_scale)
        want[b] = orc.f32_to_bf16(o[0])
    for force in (False, True):
        out = torch.zeros((B, g.n_heads, g.head_dim), dtype=torch.uint16, device="cuda")
        be.launch_v4_sparse_attend_bf16(bg, B, dev(inp["q"]), dev(inp["kv_cache"]), dev(inp["sink"]), dev(sel), cols,
                                        out, force)
        got = out.cpu().numpy()
        assert np.all(np.isnan(orc.bf16_to_f32(got[0])))
        ok, worst = wl.attend_close(got[1:], want[1:])
        assert ok, (force, worst)


def test_rows_outside_the_integer_form_are_refolded_exactly():
    """Arbitrary bf16 index rows (not spread): the integer scorer must notice and leave them to the ordered fold
    (single columns when a cached row is the problem, the whole sequence when its queries are); scores and indices
    stay bit-exact. One sequence keeps spread rows and stays on the tensor path; one has a single row with one
    block 14 binades above its neighbours."""
    g = wl.make_geom(max_comp=640, index_topk=96)
    pos = np.array([2559, 2559, 2559, 2559], np.int32)
    inp = wl.make_inputs(g, 4, pos, seed=12)
    rng = np.random.default_rng(1)
    inp["ikv"][1] = orc.f32_to_bf16(rng.standard_normal((g.max_comp, g.index_dim)).astype(np.float32))
    inp["iq"][2] = orc.f32_to_bf16(rng.standard_normal((g.index_heads, g.index_dim)).astype(np.float32))
    row = orc.bf16_to_f32(inp["ikv"][3, 17]).copy()
    row[:32] *= np.float32(2.0 ** 14)      # one block of one row 14 binades above its neighbours
    inp["ikv"][3, 17] = orc.f32_to_bf16(row)
    want_sel, want_out, want_sc = orc.v4_decode_step_bf16(g, pos, inp["q"], inp["kv_cache"], inp["sink"], inp["iq"],
                                                          inp["iw"], inp["ikv"], want_scores=True)
    for pack in (False, True):
        sel, out, sc, flags = _run_step(g, inp, want_flags=True, pack=pack)
        assert flags.tolist() == [0, 2, 1, 2]      # bit 0: whole sequence re-folded (its queries); bit 1: some columns
        assert np.array_equal(bits(sc), bits(want_sc))
        assert np.array_equal(sel, want_sel)


# ---- KV compressor, decode arm ------------------------------------------------------------------------
def test_act_quant_f8_prefix_is_bit_identical():
    be = _be()
    rng = np.random.default_rng(31)
    rows, stride, n, block = 37, 512, 448, 64
    x = rng.standard_normal((rows, stride)).astype(np.float32)
    x *= (2.0 ** rng.integers(-20, 12, (rows, 1))).astype(np.float32)
    x[3, :64] = 0.0
    x[4, :64] = 3e-5
    rc, want = orc.act_quant_f8_prefix(x, rows, stride, n, block)
    assert rc == 0
    t = dev(x)
    be.launch_act_quant_f8_prefix(t, t, rows, stride, n, block)
    got = t.cpu().numpy()
    assert np.array_equal(bits(got), bits(want.reshape(rows, stride)))
    assert np.array_equal(got[:, n:], x[:, n:])          # the tail is untouched
    for args, code in [((0, 64, 64, 64), 1001), ((1, 64, 48, 32), 1004), ((1, 32, 64, 64), 1001)]:
        with pytest.raises(be.BackendError) as e:
            be.launch_act_quant_f8_prefix(t, t, *args)
        assert e.value.code == code
    with pytest.raises(be.BackendError) as e:
        be.launch_act_quant_f8_prefix(t, dev(x), 1, 128, 64, 64)
    assert e.value.code == 1002


def _comp_fixture(rng, p, n_pos):
    norm = orc.bf16_to_f32(orc.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(p.d).astype(np.float32)))
    ang = rng.uniform(0, 2 * np.pi, (n_pos, p.rd // 2))
    freqs = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32).reshape(n_pos, p.rd)
    ape = (0.5 * rng.standard_normal((p.ratio, p.cd))).astype(np.float32)
    return norm, freqs, ape


def _row_close(got, want, tol=1.0 / 64.0):
    return float(np.abs(got.astype(np.float64) - want).max() / max(np.abs(want).max(), 1e-30)) <= tol


@pytest.mark.parametrize("ratio,d,rd", [(4, 512, 64), (4, 128, 64), (128, 512, 64)])
def test_compressor_reference_layout_decode(ratio, d, rd):
    """Token by token through rivoli_kv_compress_deposit / _decode against the oracle: state bit-exact, pooled row
    within rounding (expf and the norm's reduction order), guards by code."""
    be = _be()
    rng = np.random.default_rng(ratio + d)
    op = orc.CompGeom.make(ratio=ratio, d=d, rd=rd)
    bp = be.CompGeom(*[getattr(op, n) for n, _ in orc.CompGeom._fields_])
    n_pos = 2 * ratio + 3
    norm, freqs, ape = _comp_fixture(rng, op, n_pos)
    kv_state = np.zeros((op.ents, op.cd), np.float32)
    score_state = np.full((op.ents, op.cd), -np.inf, np.float32)
    d_kv, d_sc = dev(kv_state), dev(score_state)
    d_norm, d_freqs, d_ape = dev(norm), dev(freqs), dev(ape)
    out = torch.zeros(d, device="cuda")
    closed = 0
    for pos in range(1, n_pos):
        kv, sc = rng.standard_normal(op.cd).astype(np.float32), rng.standard_normal(op.cd).astype(np.float32)
        orc.v4_compress_deposit_token(kv, sc, ape, kv_state, score_state, op, pos)
        be.launch_kv_compress_deposit(dev(kv), dev(sc), d_ape, d_kv, d_sc, bp, 1, pos % ratio)
        assert np.array_equal(bits(d_kv.cpu().numpy()), bits(kv_state))
        assert np.array_equal(bits(d_sc.cpu().numpy()), bits(score_state))
        if (pos + 1) % ratio:
            with pytest.raises(be.BackendError) as e:
                be.launch_kv_compress_decode(d_kv, d_sc, d_norm, d_freqs, out, bp, pos)
            assert e.value.code == 1009
            continue
        rc, want = orc.v4_compress_decode(kv_state, score_state, norm, freqs, op, pos)
        be.launch_kv_compress_decode(d_kv, d_sc, d_norm, d_freqs, out, bp, pos)
        got = out.cpu().numpy()
        assert _row_close(got, want), pos
        assert np.array_equal(bits(got), bits(orc.bf16_to_f32(orc.f32_to_bf16(got))))
        assert np.array_equal(bits(d_kv.cpu().numpy()), bits(kv_state))     # the overlap half moved down
        closed += 1
    assert closed == 2
    with pytest.raises(be.BackendError) as e:
        be.launch_kv_compress_decode(d_kv, d_sc, d_norm, d_freqs, out, bp, 0)
    assert e.value.code == 1007
    bad = be.CompGeom(4, 2, 64, 128, 7, 16, 1e-6)
    with pytest.raises(be.BackendError) as e:
        be.launch_kv_compress_deposit(d_kv, d_sc, d_ape, d_kv, d_sc, bad, 1, 0)
    assert e.value.code == 1003
    with pytest.raises(be.BackendError) as e:
        be.launch_kv_compress_deposit(d_kv, d_sc, d_ape, d_kv, d_sc, bp, 1, ratio)
    assert e.value.code == 1008


@pytest.mark.parametrize("rotate,d", [(False, 512), (True, 128)])
def test_compressor_batched_step(rotate, d):
    """Several sequences at different phases of their block, stepped together for a few tokens. The row before the
    finishing quantisation is within rounding of the oracle's; the stored row is EXACTLY the oracle's finish
    (spread, or fp8 block-64 + bf16) applied to the device's own pre-quantisation row; untouched cache rows stay."""
    be = _be()
    rng = np.random.default_rng(40 + d)
    op = orc.CompGeom.make(ratio=4, d=d, rd=64)
    bp = be.CompGeom(*[getattr(op, n) for n, _ in orc.CompGeom._fields_])
    B, steps, cache_rows, row0 = 6, 6, 40, 8
    pos0 = np.array([1, 2, 3, 4, 9, 14], np.int32)
    norm, freqs, ape = _comp_fixture(rng, op, 64)
    kv_state = np.zeros((B, op.ents, op.cd), np.float32)
    score_state = np.full((B, op.ents, op.cd), -np.inf, np.float32)
    # some history so the overlap halves are live
    kv_state[:, : op.ratio] = rng.standard_normal((B, op.ratio, op.cd)).astype(np.float32)
    score_state[:, : op.ratio] = rng.standard_normal((B, op.ratio, op.cd)).astype(np.float32)
    d_kv, d_sc = dev(kv_state), dev(score_state)
    cache = torch.full((B, cache_rows, d), 0x1234, dtype=torch.uint16, device="cuda")
    preq = torch.zeros((B, d), device="cuda")
    packed = torch.zeros((B, cache_rows, 128), dtype=torch.uint8, device="cuda") if rotate else None
    pexp = torch.zeros((B, cache_rows), dtype=torch.int32, device="cuda") if rotate else None
    written = set()
    for t in range(steps):
        pos = pos0 + t
        kvp = rng.standard_normal((B, op.cd)).astype(np.float32)
        scp = rng.standard_normal((B, op.cd)).astype(np.float32)
        be.launch_v4_compress_step_bf16(bp, B, dev(pos), dev(kvp), dev(scp), dev(ape), d_kv, d_sc, dev(norm), dev(freqs),
                                        rotate, cache, cache_rows, row0, preq, packed, pexp)
        got_pre, got_cache = preq.cpu().numpy(), cache.cpu().numpy()
        for b in range(B):
            orc.v4_compress_deposit_token(kvp[b], scp[b], ape, kv_state[b], score_state[b], op, int(pos[b]))
            if (pos[b] + 1) % op.ratio:
                continue
            rc, want = orc.v4_compress_decode(kv_state[b], score_state[b], norm, freqs, op, int(pos[b]))
            assert rc == 0 and _row_close(got_pre[b], want), (t, b)
            if rotate:
                fin = orc.v4_spread(got_pre[b].copy(), d)[1][0]
            else:
                fin = orc.act_quant_f8_prefix(got_pre[b].copy(), 1, d, d - op.rd, 64)[1]
            blk = int(pos[b]) // op.ratio
            assert np.array_equal(got_cache[b, row0 + blk], orc.f32_to_bf16(fin)), (t, b)
            written.add((b, row0 + blk))
            if rotate:   # the int8 + exponent form of the same row: value = int8 * 2^(e - 130), one unit per row
                pk = packed[b, row0 + blk].cpu().numpy().view(np.int8).astype(np.float64)
                e = int(pexp[b, row0 + blk].item()) & 0xffffffff
                if e == 0:
                    assert not fin.any() and not pk.any()
                else:
                    assert e != 0xff and np.array_equal(pk * 2.0 ** (e - 130), fin.astype(np.float64))
                    assert 8 <= np.abs(pk).max() < 128
        assert np.array_equal(bits(d_kv.cpu().numpy()), bits(kv_state))
        assert np.array_equal(bits(d_sc.cpu().numpy()), bits(score_state))
    got_cache = cache.cpu().numpy()
    for b in range(B):
        for r in range(cache_rows):
            if (b, r) not in written:
                assert np.all(got_cache[b, r] == 0x1234)
    assert len(written) >= B


@pytest.mark.parametrize("ratio,d,rd,s", [(4, 512, 64, 23), (4, 128, 64, 9), (128, 512, 64, 300)])
def test_compressor_reference_layout_prefill(ratio, d, rd, s):
    """A prompt through rivoli_kv_compress_deposit (s rows at once) and rivoli_kv_compress_prefill: the state it leaves
    is bit-exact, every pooled block within rounding; then a decode token continues from that state."""
    be = _be()
    rng = np.random.default_rng(s)
    op = orc.CompGeom.make(ratio=ratio, d=d, rd=rd)
    bp = be.CompGeom(*[getattr(op, n) for n, _ in orc.CompGeom._fields_])
    norm, freqs, ape = _comp_fixture(rng, op, s + ratio + 1)
    kv = rng.standard_normal((s, op.cd)).astype(np.float32)
    sc = rng.standard_normal((s, op.cd)).astype(np.float32)
    kv_state = np.zeros((op.ents, op.cd), np.float32)
    score_state = np.full((op.ents, op.cd), -np.inf, np.float32)
    d_kv, d_sc = dev(kv_state), dev(score_state)
    assert orc.v4_compress_deposit_prefill(kv, sc, ape, kv_state, score_state, op, s) == 0
    be.launch_kv_compress_deposit(dev(kv), dev(sc), dev(ape), d_kv, d_sc, bp, s, 0)
    assert np.array_equal(bits(d_kv.cpu().numpy()), bits(kv_state))
    assert np.array_equal(bits(d_sc.cpu().numpy()), bits(score_state))
    nblk = s // ratio
    rc, want = orc.v4_compress_prefill(kv, sc, ape, norm, freqs, op, nblk)
    out = torch.zeros((nblk, d), device="cuda")
    be.launch_kv_compress_prefill(dev(kv), dev(sc), dev(ape), dev(norm), dev(freqs), out, bp, nblk)
    got = out.cpu().numpy()
    for b in range(nblk):
        assert _row_close(got[b], want[b]), b
    assert np.array_equal(bits(got), bits(orc.bf16_to_f32(orc.f32_to_bf16(got))))
    # decode tokens continue from the prompt's state until the open block closes
    row = torch.zeros(d, device="cuda")
    for pos in range(s, (s // ratio + 1) * ratio):
        k1, s1 = rng.standard_normal(op.cd).astype(np.float32), rng.standard_normal(op.cd).astype(np.float32)
        orc.v4_compress_deposit_token(k1, s1, ape, kv_state, score_state, op, pos)
        be.launch_kv_compress_deposit(dev(k1), dev(s1), dev(ape), d_kv, d_sc, bp, 1, pos % ratio)
    pos = (s // ratio + 1) * ratio - 1
    rc, want_row = orc.v4_compress_decode(kv_state, score_state, norm, freqs, op, pos)
    be.launch_kv_compress_decode(d_kv, d_sc, dev(norm), dev(freqs), row, bp, pos)
    assert rc == 0 and _row_close(row.cpu().numpy(), want_row)
    assert np.array_equal(bits(d_kv.cpu().numpy()), bits(kv_state))
    with pytest.raises(be.BackendError) as e:
        be.launch_kv_compress_prefill(dev(kv), dev(sc), dev(ape), dev(norm), dev(freqs), out, bp, 0)
    assert e.value.code == 1006


def test_bench_shape_properties():
    """Batch 128 x context 8192 (the benchmark's shape), inputs made on the device: properties that need no oracle.
    Selection: ring part is the rotation; the 512 ranked blocks are ascending, distinct, and no unselected block
    outranks a selected one under (score descending, index ascending); packed and unpacked rows give the same rows.
    Attention: a row whose only live slot is j returns kv[j] when the sink is far below; reordering the slots of a
    row changes the output only by rounding; masked slots change nothing."""
    be = _be()
    from rivoli_b200.v4 import V4DecodeLayer
    B, ctx = 128, 8192
    g = be.V4Geom.make(max_comp=ctx // 4)
    layer = V4DecodeLayer(g, B)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(77)
    rnd = lambda *shape: torch.randn(shape, generator=gen, device="cuda")
    layer.kv_cache.copy_(rnd(B, layer.kv_rows, g.head_dim).to(torch.bfloat16).view(torch.uint16))
    rows = rnd(B * g.max_comp, g.index_dim).to(torch.bfloat16).float()
    be.launch_act_quant_f4_rotated(rows, B * g.max_comp, g.index_dim)
    layer.index_kv.copy_(rows.to(torch.bfloat16).view(torch.uint16).view(B, g.max_comp, g.index_dim))
    iq = rnd(B * g.index_heads, g.index_dim).to(torch.bfloat16).float()
    be.launch_act_quant_f4_rotated(iq, B * g.index_heads, g.index_dim)
    iq = iq.to(torch.bfloat16).view(torch.uint16).view(B, g.index_heads, g.index_dim).contiguous()
    iw = (rnd(B, g.index_heads) * 0.125).to(torch.bfloat16).float()
    q = rnd(B, g.n_heads, g.head_dim).to(torch.bfloat16).view(torch.uint16)
    layer.sink.copy_(rnd(g.n_heads))
    pos = torch.randint(ctx - 512, ctx, (B,), generator=gen, device="cuda", dtype=torch.int32)
    layer.select(pos, iq, iw)
    sel_a = layer.sel.clone()
    assert not layer.refolded.any().item()
    scores = layer.scores.clone()
    layer.pack_index_rows(None, (pos + 1) // 4, g.max_comp)
    layer.select(pos, iq, iw)
    assert torch.equal(layer.sel, sel_a) and torch.equal(layer.scores.view(torch.int32), scores.view(torch.int32))
    sel, sc, p = sel_a.cpu().numpy(), scores.cpu().numpy(), pos.cpu().numpy()
    W, K = g.window, g.index_topk
    for b in range(0, B, 7):
        assert sel[b, :W].tolist() == orc.v4_window_row(W, int(p[b])).tolist()
        n_comp = (p[b] + 1) // 4
        chosen = sel[b, W:] - W
        assert np.all(np.diff(chosen) > 0) and chosen.min() >= 0 and chosen.max() < n_comp
        key = sc[b, :n_comp].view(np.uint32).astype(np.int64)
        key = np.where(key >> 31, (~key) & 0xffffffff, key | 0x80000000)      # total order on the bits
        rest = np.setdiff1d(np.arange(n_comp), chosen)
        worst_in, best_out = key[chosen].min(), key[rest].max()
        assert worst_in >= best_out
        if worst_in == best_out:   # ties go to the lower index
            assert chosen[key[chosen] == worst_in].max() < rest[key[rest] == best_out].min()
    # attention
    out0 = layer.attend(q).clone()
    assert not torch.isnan(out0.view(torch.bfloat16).float()).any()
    perm = torch.randperm(layer.cols, generator=gen, device="cuda")
    layer.sel.copy_(sel_a[:, perm])
    out1 = layer.attend(q).clone()
    ok, worst = wl.attend_close(out1.cpu().numpy(), out0.cpu().numpy())
    assert ok, worst
    masked = sel_a.clone()
    masked[:, 1::2] = -1
    wide = torch.cat([masked, torch.full_like(masked, -1)], dim=1).contiguous()     # twice as many columns, all masked
    out_n = torch.zeros_like(layer.out)
    be.launch_v4_sparse_attend_bf16(g, B, q, layer.kv_cache, layer.sink, masked, layer.cols, out_n)
    out_w = torch.zeros_like(layer.out)
    be.launch_v4_sparse_attend_bf16(g, B, q, layer.kv_cache, layer.sink, wide, 2 * layer.cols, out_w)
    assert torch.equal(out_n, out_w)
    one = torch.full_like(sel_a, -1)
    one[:, 5] = sel_a[:, 300]
    layer.sink.fill_(-1e30)
    out_1 = torch.zeros_like(layer.out)
    be.launch_v4_sparse_attend_bf16(g, B, q, layer.kv_cache, layer.sink, one, layer.cols, out_1)
    want = layer.kv_cache.view(torch.int16)[torch.arange(B, device="cuda"), sel_a[:, 300].long()]
    assert torch.equal(out_1.view(torch.int16), want[:, None, :].expand(-1, g.n_heads, -1))


def test_token_steps_wire_compressors_selection_and_attention():
    """Twenty decode tokens through V4TokenStep for sequences at different phases. After every token the oracle
    recomputes selection and attention FROM THE DEVICE'S OWN CACHES: rows must match exactly and outputs within the
    attention bar; the caches must have grown by exactly the blocks that closed, at their positional rows."""
    be = _be()
    from rivoli_b200.v4 import V4Compressor, V4DecodeLayer, V4TokenStep
    rng = np.random.default_rng(50)
    g = wl.make_geom(n_heads=4, head_dim=128, window=8, index_heads=4, index_dim=128, index_topk=3, max_comp=32)
    bg = be.V4Geom(*[getattr(g, n) for n, _ in orc.V4Geom._fields_])
    B, steps = 3, 20
    pos0 = np.array([3, 9, 30], np.int32)
    layer = V4DecodeLayer(bg, B)
    layer.sink.copy_(dev(rng.standard_normal(g.n_heads).astype(np.float32)))
    pa, pi = be.CompGeom.make(ratio=4, d=128, rd=64), be.CompGeom.make(ratio=4, d=128, rd=64)
    opa = orc.CompGeom.make(ratio=4, d=128, rd=64)
    na, fa, aa = _comp_fixture(rng, opa, 128)
    ni, fi, ai = _comp_fixture(rng, opa, 128)
    comp_a = V4Compressor(pa, B, dev(aa), dev(na), dev(fa), rotate=False)
    comp_i = V4Compressor(pi, B, dev(ai), dev(ni), dev(fi), rotate=True)
    step = V4TokenStep(layer, comp_a, comp_i)
    # history: earlier blocks already in the caches (random bf16 rows; indexer rows spread), packed form included
    hist = (pos0 + 1) // 4
    kvc = np.zeros((B, layer.kv_rows, 128), np.uint16)
    ikv = np.zeros((B, g.max_comp, 128), np.uint16)
    for b in range(B):
        kvc[b, :8] = orc.f32_to_bf16(rng.standard_normal((8, 128)).astype(np.float32))
        kvc[b, 8:8 + hist[b]] = orc.f32_to_bf16(rng.standard_normal((hist[b], 128)).astype(np.float32))
        if hist[b]:
            rows = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((hist[b], 128)).astype(np.float32)))
            ikv[b, :hist[b]] = orc.f32_to_bf16(orc.v4_spread(rows, 128)[1])
    layer.kv_cache.copy_(dev(kvc)); layer.index_kv.copy_(dev(ikv))
    layer.pack_index_rows(None, dev(hist.astype(np.int32)), int(hist.max()))
    f32 = lambda *s: rng.standard_normal(s).astype(np.float32)
    for t in range(steps):
        pos = pos0 + 1 + t
        q = orc.f32_to_bf16(f32(B, 4, 128))
        iq = orc.f32_to_bf16(orc.v4_spread(orc.bf16_to_f32(orc.f32_to_bf16(f32(B * 4, 128))), 128)[1]).reshape(B, 4, 128)
        iw = orc.bf16_to_f32(orc.f32_to_bf16(f32(B, 4)))
        entry = orc.f32_to_bf16(f32(B, 128))
        out = step(dev(pos), dev(entry), (dev(f32(B, 256)), dev(f32(B, 256))), (dev(f32(B, 256)), dev(f32(B, 256))),
                   dev(q), dev(iq), dev(iw))
        torch.cuda.synchronize()
        kvc_now, ikv_now = layer.kv_cache.cpu().numpy(), layer.index_kv.cpu().numpy()
        assert not layer.refolded.any().item()
        for b in range(B):
            assert np.array_equal(kvc_now[b, pos[b] % 8], entry[b])                       # the ring took the token
            n_comp = (pos[b] + 1) // 4
            assert ikv_now[b, :n_comp].any(axis=1).all() and not ikv_now[b, n_comp:].any()  # blocks by position
            assert kvc_now[b, 8:8 + n_comp].any(axis=1).all() and not kvc_now[b, 8 + n_comp:].any()
        want_sel, want_out = orc.v4_decode_step_bf16(g, pos, q, kvc_now, layer.sink.cpu().numpy(), iq, iw, ikv_now)
        assert np.array_equal(layer.sel.cpu().numpy(), want_sel), t
        ok, worst = wl.attend_close(out.cpu().numpy(), want_out)
        assert ok, (t, worst)
