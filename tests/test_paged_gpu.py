"""The batched / paged / bf16 operators against the oracle on seeded decode states."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import State, attend_close, attend_close_ref, make_geom

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from rivoli_b200 import backend
    backend.lib()
    return backend


def dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(a).cuda()


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.cpu().numpy().view(np.uint16)


def check_mma_attention(got_bits, want_f32):
    """Gate of rivoli_mla_attend_paged_bf16 at the model geometry (tensor-core kernel with q and P each carried
    as two e4m3 terms, ~2^-9 relative, i.e. bf16-class; sequences under 128 rows on the f32 kernel): the
    elementwise form |err| <= 2e-2 |want| + 1e-3 at every row count, the reference's own form
    (max|err| <= 2e-2 max|want| + 1e-3, crates/engine/tests/common/scoring.rs:191-194) and an rms bound of
    0.5 % of rms(want)."""
    ok, worst, rms = attend_close_ref(got_bits, want_f32)
    assert ok, worst
    assert rms <= 5e-3, rms
    ok, worst = attend_close(got_bits, want_f32)
    assert ok, worst


CASES = {
    # the smallest benchmark shape: 1 sequence, 256 cached + 1 appended, H=16, indexer 8x64, k=64, 16-token pages
    "cfg1": dict(seed=0, B=1, ctx=[257], n_heads=16, index_heads=8, index_dim=64, page_tokens=16, top_k=64,
                 pool_factor=1.0),
    # ragged batch, model dims, top-k smaller / larger than the contexts
    "ragged": dict(seed=11, B=5, ctx=[1, 63, 64, 65, 700], top_k=256),
    "dense-equivalent": dict(seed=12, B=3, ctx=[300, 257, 512], top_k=2048),
}


def build(be, case):
    c = dict(CASES[case])
    st = State(c.pop("seed"), c.pop("B"), c.pop("ctx"), **c)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    d = dict(latent_pool=dev(st.latent_pool), latent_scale=dev(st.latent_scale), index_pool=dev(st.index_pool),
             index_scale=dev(st.index_scale), block_table=dev(st.block_table), seq_len=dev(st.seq_len),
             row_pos=dev(st.row_pos))
    return st, g, d


@pytest.mark.parametrize("case", list(CASES))
def test_layer_step_matches_oracle(be, case):
    st, g, d = build(be, case)
    want = st.oracle_step()
    B = st.B
    # 1. append: bit-exact codes and scales, and nothing else in the pool moves
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    be.launch_kv_append_paged(g, dev(st.new_latent), dev(st.new_key), None, d["row_pos"], B, d["block_table"],
                              d["latent_pool"], d["latent_scale"], d["index_pool"], d["index_scale"], status)
    be.device_sync()
    assert int(status.item()) == 0
    np.testing.assert_array_equal(d["latent_pool"].cpu().numpy(), want["latent_pool"])
    np.testing.assert_array_equal(d["latent_scale"].cpu().numpy().view(np.uint32), want["latent_scale"].view(np.uint32))
    np.testing.assert_array_equal(d["index_pool"].cpu().numpy(), want["index_pool"])
    np.testing.assert_array_equal(d["index_scale"].cpu().numpy().view(np.uint32), want["index_scale"].view(np.uint32))
    # 2. q quantisation: bit-exact
    qc = torch.zeros(st.index_q.size, dtype=torch.uint8, device="cuda")
    qs = torch.zeros(B * g.index_heads, dtype=torch.float32, device="cuda")
    be.launch_index_q_quant(dev(st.index_q), B * g.index_heads, g.index_dim, qc, qs)
    be.device_sync()
    np.testing.assert_array_equal(qc.cpu().numpy(), want["qcodes"].ravel())
    np.testing.assert_array_equal(qs.cpu().numpy().view(np.uint32), want["qscales"].view(np.uint32))
    # 3. scores: BIT-exact (fixed fold order), only t < seq_len is defined
    stride = int(st.seq_len.max())
    sc = torch.full((B, stride), float("nan"), dtype=torch.float32, device="cuda")
    be.launch_index_score_paged(g, qc, qs, dev(st.index_w), d["index_pool"], d["index_scale"], d["block_table"],
                                d["seq_len"], B, sc, stride)
    be.device_sync()
    got = sc.cpu().numpy()
    for b in range(B):
        n = st.seq_len[b]
        np.testing.assert_array_equal(got[b, :n].view(np.uint32), want["scores"][b, :n].view(np.uint32))
        assert np.isnan(got[b, n:]).all()
    # 4. top-k: bit-exact indices, sentinel tail
    rows = torch.full((B, g.top_k), -1, dtype=torch.int32, device="cuda")
    n_sel = torch.zeros(B, dtype=torch.int32, device="cuda")
    be.launch_index_topk_batched(sc, stride, d["seq_len"], B, g.top_k, rows, n_sel)
    be.device_sync()
    np.testing.assert_array_equal(n_sel.cpu().numpy(), want["n_sel"])
    np.testing.assert_array_equal(rows.cpu().numpy().view(np.uint32), want["rows"])
    # 5. attention (both implementations) within 2e-2 rel / 1e-3 abs of the oracle's f32 result
    for fn, nbytes in ((be.launch_attend_paged_bf16, be.attend_paged_scratch_bytes(g, B)),
                       (be.launch_attend_simt_paged_bf16, be.attend_simt_scratch_bytes(g, B))):
        out = torch.zeros((B, g.n_heads, g.kv_lora), dtype=torch.bfloat16, device="cuda")
        m = torch.zeros((B, g.n_heads), dtype=torch.float32, device="cuda")
        lse = torch.zeros((B, g.n_heads), dtype=torch.float32, device="cuda")
        scratch = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device="cuda")
        fn(g, dev(st.q), d["latent_pool"], d["latent_scale"], d["block_table"], rows, g.top_k, n_sel, B, out, m,
           lse, scratch)
        be.device_sync()
        if fn is be.launch_attend_paged_bf16 and be.attend_paged_uses_mma(g):
            be.attend_paged_status(g, scratch)
            check_mma_attention(u16(out), want["out_f32"])
        else:
            ok, worst = attend_close(u16(out), want["out_f32"])
            assert ok, worst
        assert np.abs(lse.cpu().numpy() - want["lse"]).max() < 2e-2
        # no-scratch (single split) path
        out2 = torch.zeros_like(out)
        fn(g, dev(st.q), d["latent_pool"], d["latent_scale"], d["block_table"], rows, g.top_k, n_sel, B, out2,
           None, None, None)
        be.device_sync()
        ok, worst = attend_close(u16(out2), want["out_f32"])
        assert ok, worst


def test_dense_attend_and_partial_merge(be):
    """Page-range sharding: attend two halves of each context separately, merge (m, lse, out)."""
    st, g, d = build(be, "ragged")
    want = st.oracle_step()
    B, H, kvl = st.B, g.n_heads, g.kv_lora
    dlp, dls = dev(want["latent_pool"]), dev(want["latent_scale"])
    # dense oracle over the whole prefix
    o_dense, o_f32, _, lse_dense = orc.mla_attend_paged(st.og, st.q, want["latent_pool"], want["latent_scale"],
                                                        st.block_table, None, st.seq_len, want_f32=True)
    out = torch.zeros((B, H, kvl), dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros((B, H), dtype=torch.float32, device="cuda")
    be.launch_attend_paged_bf16(g, dev(st.q), dlp, dls, d["block_table"], None, 0, d["seq_len"], B, out, None, lse,
                                None)
    be.device_sync()
    ok, worst = attend_close(u16(out), o_f32)
    assert ok, worst
    # two shards by row range -> partials -> merge
    parts, lses = [], []
    stride = int(st.seq_len.max())
    for lo_f, hi_f in ((0.0, 0.5), (0.5, 1.0)):
        rows = np.zeros((B, stride), np.uint32); n = np.zeros(B, np.int32)
        for b in range(B):
            lo, hi = int(st.seq_len[b] * lo_f), int(st.seq_len[b] * hi_f)
            n[b] = hi - lo; rows[b, :hi - lo] = np.arange(lo, hi)
        po = torch.zeros((B, H, kvl), dtype=torch.bfloat16, device="cuda")
        pl = torch.zeros((B, H), dtype=torch.float32, device="cuda")
        be.launch_attend_paged_bf16(g, dev(st.q), dlp, dls, d["block_table"], dev(rows), stride, dev(n), B, po,
                                    None, pl, None)
        parts.append(po); lses.append(pl)
    part_out = torch.stack(parts).contiguous(); part_lse = torch.stack(lses).contiguous()
    merged = torch.zeros((B * H, kvl), dtype=torch.bfloat16, device="cuda")
    be.launch_attend_merge_partials(part_out, part_lse, 2, B * H, kvl, merged)
    be.device_sync()
    # GPU merge == oracle merge of the same partials, bit for bit up to bf16 rounding of f32 sums
    want_m = orc.attend_merge_partials(u16(part_out).reshape(2, B * H, kvl), part_lse.cpu().numpy(), kvl)
    diff = np.abs(orc.bf16_to_f32(u16(merged)).reshape(-1) - orc.bf16_to_f32(want_m).reshape(-1))
    assert diff.max() <= 1e-2 * np.abs(orc.bf16_to_f32(want_m)).max()
    # and the merged result is the dense answer (an empty shard for the 1-token sequence included)
    ok, worst = attend_close(u16(merged).reshape(B, H, kvl), o_f32, rel=3e-2, abs_=2e-3)
    assert ok, worst


def test_paged_guards(be):
    g = make_geom(be.DsaGeom, max_pages_per_seq=4, n_pool_pages=8)
    b = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    bad = make_geom(be.DsaGeom, kv_lora=640, max_pages_per_seq=4, n_pool_pages=8)
    for fn, code in ((lambda: be.launch_kv_append_paged(bad, b, b, None, b, 1, b, b, b, b, b), 1004),
                     (lambda: be.launch_kv_append_paged(g, b, b, None, b, 0, b, b, b, b, b), 1001),
                     (lambda: be.launch_index_q_quant(b, 4, 100, b, b), 1004),
                     (lambda: be.launch_index_topk_batched(b, 64, b, 0, 4, b, b), 1001),
                     (lambda: be.launch_attend_merge_partials(b, b, 0, 4, 512, b), 1001)):
        with pytest.raises(be.BackendError) as e:
            fn()
        assert e.value.code == code
    be.device_sync()


def test_append_flags_unmapped_page(be):
    """A block-table entry outside the pool is skipped and reported, never written through."""
    st, g, d = build(be, "cfg1")
    bt = d["block_table"].clone(); bt[0, st.row_pos[0] // g.page_tokens] = g.n_pool_pages + 5
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    before = d["latent_pool"].clone()
    be.launch_kv_append_paged(g, dev(st.new_latent), dev(st.new_key), None, d["row_pos"], 1, bt, d["latent_pool"],
                              d["latent_scale"], d["index_pool"], d["index_scale"], status)
    be.device_sync()
    assert int(status.item()) == 1
    assert torch.equal(before, d["latent_pool"])


# ---- fused tensor-core indexer: rows must be IDENTICAL to the exact chain / the oracle -----------
SELECT_CASES = {
    "model-dims": dict(seed=21, B=4, ctx=[5000, 4097, 129, 2049], top_k=2048),
    "short-topk": dict(seed=22, B=3, ctx=[3000, 1000, 700], top_k=64),
    "p16": dict(seed=23, B=2, ctx=[900, 333], top_k=128, page_tokens=16),
    "cfg1-fallback": dict(seed=0, B=1, ctx=[257], n_heads=16, index_heads=8, index_dim=64, page_tokens=16, top_k=64,
                          pool_factor=1.0),
}


def _select(be, st, g, d, w):
    B = st.B
    stride = int(st.seq_len.max())
    rows = torch.full((B, g.top_k), -1, dtype=torch.int32, device="cuda")
    n_sel = torch.zeros(B, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(be.index_select_scratch_bytes(g, B, stride), dtype=torch.uint8, device="cuda")
    be.launch_index_select_paged(g, dev(st.index_q), dev(w), d["index_pool"], d["index_scale"], d["block_table"],
                                 d["seq_len"], B, stride, rows, n_sel, scratch)
    be.index_select_status(g, B, stride, scratch)
    band = be.index_select_band_stats(g, B, stride, scratch) if be.index_select_uses_mma(g, stride) else None
    return rows.cpu().numpy().view(np.uint32), n_sel.cpu().numpy(), band


@pytest.mark.parametrize("case", list(SELECT_CASES))
def test_fused_select_is_bit_identical(be, case):
    c = dict(SELECT_CASES[case])
    st = State(c.pop("seed"), c.pop("B"), c.pop("ctx"), **c)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    want = st.oracle_step()
    d = dict(index_pool=dev(want["index_pool"]), index_scale=dev(want["index_scale"]),
             block_table=dev(st.block_table), seq_len=dev(st.seq_len))
    rows, n_sel, band = _select(be, st, g, d, st.index_w)
    np.testing.assert_array_equal(n_sel, want["n_sel"])
    np.testing.assert_array_equal(rows, want["rows"])
    if band is not None:
        # the exact re-score touches a small fraction of the cache, not all of it
        for b in range(st.B):
            if st.seq_len[b] > g.top_k:
                assert band[b] <= max(64, st.seq_len[b] // 8), (band, st.seq_len)


def test_fused_select_tie_dominated(be):
    """ReLU makes whole score arrays tie: all-zero head weights (every score exactly 0, the
    index rule decides everything) and a single live head (thousands of exact zeros at the cut)."""
    st = State(31, 2, [4000, 2600], top_k=2048)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    base = st.oracle_step()
    d = dict(index_pool=dev(base["index_pool"]), index_scale=dev(base["index_scale"]),
             block_table=dev(st.block_table), seq_len=dev(st.seq_len))
    for mode in ("zeros", "one-head"):
        w = np.zeros_like(st.index_w)
        if mode == "one-head":
            w[:, 3] = 1.0
        qc, qs = orc.index_q_quant(st.index_q, g.index_dim)
        stride = int(st.seq_len.max())
        sc = orc.index_score_paged(st.og, qc, qs, w, base["index_pool"], base["index_scale"], st.block_table,
                                   st.seq_len, stride)
        want_rows, want_n = orc.index_topk_batched(sc, st.seq_len, g.top_k)
        rows, n_sel, band = _select(be, st, g, d, w)
        np.testing.assert_array_equal(n_sel, want_n)
        np.testing.assert_array_equal(rows, want_rows)
        if mode == "zeros":
            assert (rows[0, :2048] == np.arange(2048)).all()


# ---- tensor-core attention (fp8 MMA, two-term q and P) against the oracle ---------------------------
ATTEND_CASES = {
    "sparse-2048-of-5000": dict(seed=41, B=3, ctx=[5000, 4097, 2500], top_k=2048),
    # both arms of the call in one batch: 1 and 127 rows on the f32 kernel, 128 and up on the tensor cores
    "ragged-tiles": dict(seed=42, B=6, ctx=[1, 127, 128, 129, 300, 1000], top_k=512),
    "every-tile-count": dict(seed=45, B=12, ctx=[128, 200, 256, 257, 384, 511, 640, 768, 1024, 1300, 1700, 2047],
                             top_k=2048),
    "big-batch-one-split": dict(seed=43, B=100, ctx=[200] * 100, top_k=128),
    # batches that split every sequence over a thread-block cluster of 7, 6, 5 and 3 CTAs (148 SMs / B), with sequences
    # of fewer tiles than CTAs and some on the f32 kernel inside the same launch
    "cluster-of-7": dict(seed=46, B=20, ctx=[700, 64, 130, 2] + [300 + 37 * i for i in range(16)], top_k=512),
    "cluster-of-6": dict(seed=47, B=24, ctx=[513, 129] + [200 + 29 * i for i in range(22)], top_k=512),
    "cluster-of-5": dict(seed=48, B=29, ctx=[640] + [150 + 17 * i for i in range(28)], top_k=512),
    "cluster-of-3": dict(seed=49, B=40, ctx=[384, 128, 1] + [140 + 11 * i for i in range(37)], top_k=256),
}


@pytest.mark.parametrize("case", list(ATTEND_CASES))
def test_mma_attention_matches_oracle(be, case):
    c = dict(ATTEND_CASES[case])
    st = State(c.pop("seed"), c.pop("B"), c.pop("ctx"), **c)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    assert be.attend_paged_uses_mma(g)
    want = st.oracle_step()
    B = st.B
    lp, ls, bt = dev(want["latent_pool"]), dev(want["latent_scale"]), dev(st.block_table)
    rows, n_sel = dev(want["rows"]), dev(want["n_sel"])
    out = torch.zeros((B, g.n_heads, g.kv_lora), dtype=torch.bfloat16, device="cuda")
    m = torch.zeros((B, g.n_heads), dtype=torch.float32, device="cuda")
    lse = torch.zeros((B, g.n_heads), dtype=torch.float32, device="cuda")
    scratch = torch.zeros(be.attend_paged_scratch_bytes(g, B), dtype=torch.uint8, device="cuda")
    for _ in range(2):          # twice: barriers, TMEM and scratch must be reusable
        be.launch_attend_paged_bf16(g, dev(st.q), lp, ls, bt, rows, g.top_k, n_sel, B, out, m, lse, scratch)
        be.attend_paged_status(g, scratch)
        check_mma_attention(u16(out), want["out_f32"])
        assert np.abs(lse.cpu().numpy() - want["lse"]).max() < 2e-2
        assert (m.cpu().numpy() <= lse.cpu().numpy() + 1e-4).all()
    # the CUDA-core kernel on the same inputs: both within tolerance of the oracle and close to each other
    out2 = torch.zeros_like(out)
    be.launch_attend_simt_paged_bf16(g, dev(st.q), lp, ls, bt, rows, g.top_k, n_sel, B, out2, None, None, None)
    be.device_sync()
    a, b2 = orc.bf16_to_f32(u16(out)).ravel(), orc.bf16_to_f32(u16(out2)).ravel()
    assert np.abs(a - b2).max() <= 2e-2 * np.abs(b2).max() + 1e-3


def test_mma_attention_dense_long_prefix(be):
    """Dense (rows = NULL) attention over a few thousand tokens: many tiles per split, the
    lagging reference max and the rare O rescale are exercised by a query aligned with one late key."""
    st = State(44, 2, [3000, 2049], top_k=64)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    want = st.oracle_step()
    # make head 0 of sequence 0 attend sharply to a late token: its score towers over the rest
    lat = want["latent_pool"].reshape(-1, 576)
    P = g.page_tokens
    t_late = 2900
    r = st.block_table[0, t_late // P] * P + t_late % P
    code = orc.e4m3_table()[lat[r]] * want["latent_scale"][r]
    q = st.q.copy().reshape(2, 64, 576)
    q[0, 0] = orc.f32_to_bf16((code / np.abs(code).max() * 6.0).astype(np.float32))
    o, o_f32, _, lse_w = orc.mla_attend_paged(st.og, q, want["latent_pool"], want["latent_scale"], st.block_table,
                                              None, st.seq_len, want_f32=True)
    B = 2
    out = torch.zeros((B, 64, 512), dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros((B, 64), dtype=torch.float32, device="cuda")
    scratch = torch.zeros(be.attend_paged_scratch_bytes(g, B), dtype=torch.uint8, device="cuda")
    be.launch_attend_paged_bf16(g, dev(q), dev(want["latent_pool"]), dev(want["latent_scale"]), dev(st.block_table),
                                None, 0, dev(st.seq_len), B, out, None, lse, scratch)
    be.attend_paged_status(g, scratch)
    check_mma_attention(u16(out), o_f32)
    assert np.abs(lse.cpu().numpy() - lse_w).max() < 2e-2


@pytest.mark.parametrize("case", ["ragged", "cfg1"])
def test_fused_append_select_equals_separate_calls(be, case):
    """rivoli_dsa_append_select_paged == rivoli_kv_append_paged + rivoli_index_select_paged: pools,
    scales, selected rows and counts bit for bit (tensor-core path on "ragged", CUDA-core on "cfg1")."""
    st, g, d = build(be, case)
    B = st.B
    stride = int(st.seq_len.max())
    nbytes = be.index_select_scratch_bytes(g, B, stride)

    def run(fused):
        pools = {k: d[k].clone() for k in ("latent_pool", "latent_scale", "index_pool", "index_scale")}
        rows = torch.full((B, g.top_k), -1, dtype=torch.int32, device="cuda")
        n_sel = torch.zeros(B, dtype=torch.int32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        if fused:
            be.launch_dsa_append_select_paged(g, dev(st.new_latent), dev(st.new_key), d["row_pos"], d["block_table"],
                                              pools["latent_pool"], pools["latent_scale"], pools["index_pool"],
                                              pools["index_scale"], status, dev(st.index_q), dev(st.index_w),
                                              d["seq_len"], B, stride, rows, n_sel, scratch)
        else:
            be.launch_kv_append_paged(g, dev(st.new_latent), dev(st.new_key), None, d["row_pos"], B, d["block_table"],
                                      pools["latent_pool"], pools["latent_scale"], pools["index_pool"],
                                      pools["index_scale"], status)
            be.launch_index_select_paged(g, dev(st.index_q), dev(st.index_w), pools["index_pool"], pools["index_scale"],
                                         d["block_table"], d["seq_len"], B, stride, rows, n_sel, scratch)
        be.device_sync()
        be.index_select_status(g, B, stride, scratch)
        assert int(status.item()) == 0
        return pools, rows.cpu().numpy(), n_sel.cpu().numpy()

    pa, ra, na = run(False)
    pb, rb, nb = run(True)
    for k in pa:
        assert torch.equal(pa[k].view(torch.uint8), pb[k].view(torch.uint8)), k
    np.testing.assert_array_equal(na, nb)
    for b in range(B):
        np.testing.assert_array_equal(ra[b, :na[b]], rb[b, :nb[b]])
    want = st.oracle_step()
    np.testing.assert_array_equal(nb, want["n_sel"])
    for b in range(B):
        np.testing.assert_array_equal(rb[b, :nb[b]].view(np.uint32), want["rows"][b, :nb[b]])


def test_empty_and_single_token_sequences(be):
    """A batch holding an empty sequence, a one-token sequence and an ordinary one: the empty one selects
    nothing and attends to zeros (lse = -inf), the others are unaffected by their neighbour."""
    st, g, d = build(be, "ragged")
    B = st.B
    seq_len = st.seq_len.copy()
    seq_len[1] = 0                                   # sequence 1 is empty this step; sequence 0 has one token
    from rivoli_b200.layer import DsaDecodeLayer
    layer = DsaDecodeLayer(g, B, max_ctx=int(g.max_pages_per_seq * g.page_tokens))
    layer.latent_pool.copy_(d["latent_pool"]); layer.latent_scale.copy_(d["latent_scale"])
    layer.index_pool.copy_(d["index_pool"]); layer.index_scale.copy_(d["index_scale"])
    layer.upload_block_table(st.block_table)
    # the step's token is appended everywhere but in the empty sequence
    keep = np.array([b for b in range(B) if b != 1], np.int32)
    layer.append(dev(st.new_latent[keep]), dev(st.new_key[keep]), dev(st.row_pos[keep]), dev(keep))
    sl = dev(seq_len)
    layer.select(dev(st.index_q), dev(st.index_w), sl)
    out = layer.attend(dev(st.q))
    be.device_sync(); layer.check_status()
    n_sel = layer.n_sel.cpu().numpy()
    assert n_sel[1] == 0 and n_sel[0] == 1
    assert int(layer.rows[0, 0]) == 0
    o = out.float().cpu().numpy()
    assert np.all(o[1] == 0.0) and np.all(np.isneginf(layer.out_lse.cpu().numpy()[1]))
    want = st.oracle_step()
    for b in (0, 2, 3, 4):
        np.testing.assert_array_equal(layer.rows[b, :n_sel[b]].cpu().numpy().view(np.uint32), want["rows"][b, :want["n_sel"][b]])
    ok, worst, rms = attend_close_ref(u16(out)[[0, 2, 3, 4]], want["out_f32"][[0, 2, 3, 4]])
    assert ok and rms <= 1e-2, (worst, rms)


# ---- the two arms of rivoli_mla_attend_paged_bf16 and the give-up path of its bounded waits ---------------
def _attend_once(be, st, g, want, rows=None, n_sel=None, dense=False):
    B = st.B
    out = torch.zeros((B, g.n_heads, g.kv_lora), dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros((B, g.n_heads), dtype=torch.float32, device="cuda")
    scratch = torch.zeros(be.attend_paged_scratch_bytes(g, B), dtype=torch.uint8, device="cuda")
    args = (None, 0, dev(st.seq_len)) if dense else (dev(want["rows"]), g.top_k, dev(want["n_sel"]))
    be.launch_attend_paged_bf16(g, dev(st.q), dev(want["latent_pool"]), dev(want["latent_scale"]), dev(st.block_table),
                                *args, B, out, None, lse, scratch)
    return out, lse, scratch


def test_short_sequences_take_the_f32_kernel_and_long_ones_the_tensor_cores(be):
    """One call, both kernels: with the threshold hook at 0 every sequence runs on the tensor cores, so a
    sequence under 128 rows differs (slightly) between the two settings and one at 128 rows or more does not."""
    st = State(46, 4, [40, 127, 128, 900], top_k=2048)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    want = st.oracle_step()
    out_d, lse_d, s1 = _attend_once(be, st, g, want)
    be.attend_paged_status(g, s1)
    check_mma_attention(u16(out_d), want["out_f32"])
    assert np.abs(lse_d.cpu().numpy() - want["lse"]).max() < 2e-2
    be.attend_mma_test_hook(min_rows=0)
    try:
        out_t, _, s2 = _attend_once(be, st, g, want)
        be.attend_paged_status(g, s2)
    finally:
        be.attend_mma_test_hook(min_rows=-1)
    a, b2 = u16(out_d), u16(out_t)
    assert np.array_equal(a[2:], b2[2:]), "sequences of 128 rows and more must not depend on the threshold"
    assert not np.array_equal(a[:2], b2[:2]), "sequences under 128 rows were not routed to the f32 kernel"
    # the f32 arm equals the CUDA-core entry point bit for bit (same kernel, same fold order per head)
    out_s = torch.zeros_like(out_d)
    be.launch_attend_simt_paged_bf16(g, dev(st.q), dev(want["latent_pool"]), dev(want["latent_scale"]),
                                     dev(st.block_table), dev(want["rows"]), g.top_k, dev(want["n_sel"]), st.B, out_s,
                                     None, None, None)
    be.device_sync()
    assert np.array_equal(a[:2], u16(out_s)[:2])


def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_unaffected(be):
    """The give-up path of the bounded waits: one barrier arrival is withheld (test hook), every wait on it runs
    out, the kernel returns through its common exit, the status call reports 1008 and the following ordinary
    call gives the same bits as a call made before."""
    st = State(47, 2, [700, 300], top_k=512)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    want = st.oracle_step()
    good, _, s0 = _attend_once(be, st, g, want)
    be.attend_paged_status(g, s0)
    be.attend_mma_test_hook(min_rows=-1, withhold=1, max_polls=20000)
    try:
        _, _, s1 = _attend_once(be, st, g, want)
        with pytest.raises(be.BackendError) as e:
            be.attend_paged_status(g, s1)
        assert e.value.code == 1008
    finally:
        be.attend_mma_test_hook(min_rows=-1, withhold=0, max_polls=0)
    be.attend_paged_status(g, s1)                      # the error word was cleared by the read above
    again, _, s2 = _attend_once(be, st, g, want)
    be.attend_paged_status(g, s2)
    assert np.array_equal(u16(good), u16(again))


def test_scorer_flags_a_page_outside_the_pool(be):
    """The tensor-core scorer skips a block-table entry that points outside the pool and raises its error word
    (1005 through the status call), like the append kernel does for the same table."""
    st = State(48, 2, [1500, 600], top_k=256)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    want = st.oracle_step()
    assert be.index_select_uses_mma(g, int(st.seq_len.max()))
    bt = st.block_table.copy()
    bt[0, 3] = g.n_pool_pages + 7
    B, stride = st.B, int(st.seq_len.max())
    rows = torch.full((B, g.top_k), -1, dtype=torch.int32, device="cuda")
    n_sel = torch.zeros(B, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(be.index_select_scratch_bytes(g, B, stride), dtype=torch.uint8, device="cuda")
    args = (dev(st.index_q), dev(st.index_w), dev(want["index_pool"]), dev(want["index_scale"]))
    be.launch_index_select_paged(g, *args, dev(bt), dev(st.seq_len), B, stride, rows, n_sel, scratch)
    with pytest.raises(be.BackendError) as e:
        be.index_select_status(g, B, stride, scratch)
    assert e.value.code == 1005
    # the same call on the intact table is clean again and exact
    be.launch_index_select_paged(g, *args, dev(st.block_table), dev(st.seq_len), B, stride, rows, n_sel, scratch)
    be.index_select_status(g, B, stride, scratch)
    np.testing.assert_array_equal(rows.cpu().numpy().view(np.uint32), want["rows"])


def test_fused_step_call_equals_the_separate_operators(be):
    """rivoli_dsa_decode_step_paged == rivoli_dsa_append_select_paged + rivoli_mla_attend_paged_bf16, bit for bit."""
    from rivoli_b200.layer import DsaDecodeLayer
    st = State(49, 3, [3000, 200, 90], top_k=512)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    outs = []
    for fused in (True, False):
        L = DsaDecodeLayer(g, st.B, max_ctx=int(st.seq_len.max()))
        L.latent_pool.copy_(dev(st.latent_pool)); L.latent_scale.copy_(dev(st.latent_scale))
        L.index_pool.copy_(dev(st.index_pool)); L.index_scale.copy_(dev(st.index_scale))
        L.block_table.copy_(dev(st.block_table))
        x = (dev(st.new_latent), dev(st.new_key), dev(st.index_q), dev(st.index_w), dev(st.q), dev(st.row_pos),
             dev(st.seq_len))
        if fused:
            out = L.step(*x)
        else:
            L.append(x[0], x[1], x[5]); L.select(x[2], x[3], x[6]); out = L.attend(x[4])
        be.device_sync()
        L.check_status()
        outs.append((u16(out).copy(), L.rows.cpu().numpy().copy(), L.latent_pool.cpu().numpy().copy()))
    for a, b2 in zip(*outs):
        assert np.array_equal(a, b2)
    want = st.oracle_step()
    check_mma_attention(outs[0][0], want["out_f32"])


def test_host_buffer_pipeline_equals_the_device_resident_step(be):
    """rivoli_dsa_step_host: one packed pinned buffer up, fused step, bf16 output down, slots reused across steps.
    Every step's output equals the device-resident call on the same state, bit for bit, and the cache advances
    identically."""
    from rivoli_b200.layer import DsaDecodeLayer, HostStepPipeline
    st = State(50, 3, [900, 300, 2100], top_k=256)
    P = st.og.page_tokens
    steps = 5
    max_pages = int((st.seq_len.max() + steps + P - 1) // P)
    g = make_geom(be.DsaGeom, **{**st.geom_kw, "max_pages_per_seq": max_pages, "n_pool_pages": 3 * max_pages})
    layers = []
    for _ in range(2):
        L = DsaDecodeLayer(g, st.B, max_ctx=max_pages * P, shuffle_seed=3)
        for b in range(st.B):
            L.reserve(b, int(st.seq_len[b]) + steps)
        L.upload_block_table()
        L.append(dev(st.hist_latent), dev(st.hist_key), dev(st.hist_pos), dev(st.hist_seq))
        layers.append(L)
    be.device_sync()
    ref_layer, pipe_layer = layers
    pipe = HostStepPipeline(pipe_layer, depth=2)
    rng = np.random.RandomState(1)
    W = 576
    bufs = [pipe.new_input_buffer() for _ in range(steps)]
    outs = [pipe.new_output_buffer() for _ in range(steps)]
    pos_dev = [dev((st.seq_len - 1 + i).astype(np.int32)) for i in range(steps)]
    len_dev = [dev((st.seq_len + i).astype(np.int32)) for i in range(steps)]
    torch.cuda.synchronize()
    want, tickets = [], []
    for i in range(steps):
        x = dict(latent=bf16_n(rng, (st.B, W)), index_key=bf16_n(rng, (st.B, 128)), index_q=bf16_n(rng, (st.B, 32, 128)),
                 index_w=torch.from_numpy(orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal((st.B, 32)).astype(np.float32)))),
                 q=bf16_n(rng, (st.B, 64, W)))
        pipe.pack(x, bufs[i])
        tickets.append(pipe.submit(bufs[i], outs[i], pos_dev[i], len_dev[i]))        # never blocks
        xd = {k: v.cuda() for k, v in x.items()}
        want.append(u16(ref_layer.step(xd["latent"], xd["index_key"], xd["index_q"], xd["index_w"], xd["q"], pos_dev[i],
                                       len_dev[i])).copy())
    pipe.wait(tickets[1])
    assert np.array_equal(u16(outs[1]), want[1])
    pipe.drain()
    ref_layer.check_status(); pipe_layer.check_status()
    for i in range(steps):
        assert np.array_equal(u16(outs[i]), want[i]), i
    assert torch.equal(ref_layer.latent_pool, pipe_layer.latent_pool) and torch.equal(ref_layer.index_pool, pipe_layer.index_pool)
    legs = pipe.leg_ms()
    assert all(v >= 0.0 for v in legs.values())


def bf16_n(rng, shape):
    return torch.from_numpy(orc.f32_to_bf16(rng.standard_normal(shape).astype(np.float32)).view(np.int16)).view(torch.bfloat16)
