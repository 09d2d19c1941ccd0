"""Benchmark-sized shapes on the GPU, checked through size-independent properties and through
the oracle on sampled sequences (the oracle runs one 16384-token sequence in well under a
second): append round trip, fused tensor-core selection == exact chain bit for bit,
determinism, attention against the oracle."""
import numpy as np
import pytest
import torch

import bench
from oracle import oracle as orc
from oracle.workload import attend_close, attend_close_ref, make_geom

pytestmark = pytest.mark.gpu


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


@pytest.fixture(scope="module")
def cfg3_like():
    """cfg3 geometry (ctx 16384, k 2048, 64-token pages, 1.25x scattered pool) at batch 16."""
    w = dict(bench.WORKLOADS["cfg3"]); w["B"] = 16
    dev = torch.device("cuda", 0)
    g, layer, gen = bench.build_layer(w, dev, 123)
    x = bench.step_inputs(w, dev, gen)
    return w, g, layer, x


def test_append_round_trip_and_scale_rule(cfg3_like):
    w, g, layer, x = cfg3_like
    B, ctx, P = w["B"], w["ctx"], g.page_tokens
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
    layer.append(x["latent"], x["index_key"], pos)
    torch.cuda.synchronize()
    layer.check_status()
    bt = layer.block_table.cpu().numpy()
    rows = bt[np.arange(B), (ctx - 1) // P].astype(np.int64) * P + (ctx - 1) % P
    tab = torch.from_numpy(orc.e4m3_table()).cuda()
    for pool, scale, src, width in ((layer.latent_pool, layer.latent_scale, x["latent"], 576),
                                    (layer.index_pool, layer.index_scale, x["index_key"], 128)):
        codes = pool.view(-1, width)[torch.from_numpy(rows).cuda()]
        s = scale[torch.from_numpy(rows).cuda()]
        xs = src.float()
        amax = xs.abs().amax(dim=1)
        # scale rule with a true IEEE division (done in numpy: torch divides by a scalar via a reciprocal)
        np.testing.assert_array_equal(s.cpu().numpy(), amax.cpu().numpy() / np.float32(448.0))
        assert int(((codes & 0x7F) == 0x7E).sum()) >= B                   # every row's extreme saturates to 448
        deq = tab[codes.long()] * s[:, None]
        err = (deq - xs).abs()
        assert bool((err <= xs.abs() * 2 ** -4 + s[:, None] * 2 ** -10 + 1e-12).all())   # half an e4m3 ulp


def test_fused_selection_equals_exact_chain_at_full_context(cfg3_like):
    w, g, layer, x = cfg3_like
    B, ctx = w["B"], w["ctx"]
    seq_len = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    layer.select(x["index_q"], x["index_w"], seq_len)
    torch.cuda.synchronize(); layer.check_status()
    rows_f, n_f = layer.rows.clone(), layer.n_sel.clone()
    layer.select(x["index_q"], x["index_w"], seq_len)                      # determinism: same bits again
    torch.cuda.synchronize()
    assert torch.equal(rows_f, layer.rows) and torch.equal(n_f, layer.n_sel)
    layer.select_unfused(x["index_q"], x["index_w"], seq_len)              # exact CUDA-core chain
    torch.cuda.synchronize()
    assert torch.equal(n_f, layer.n_sel)
    assert torch.equal(rows_f, layer.rows), "tensor-core selection differs from the exact chain"
    r = rows_f.cpu().numpy().view(np.uint32).astype(np.int64)
    assert (n_f.cpu().numpy() == 2048).all()
    assert (np.diff(r, axis=1) > 0).all() and r.max() < ctx                # strictly ascending, in range
    # threshold property on the exact scores: min selected >= max unselected
    sc = layer.scores.cpu().numpy()
    for b in (0, B - 1):
        sel = np.zeros(ctx, bool); sel[r[b]] = True
        assert sc[b][sel].min() >= sc[b][~sel].max()
    # oracle on two sampled sequences: scores bit-exact, rows identical
    og = make_geom(orc.Geom, n_heads=g.n_heads, index_heads=g.index_heads, index_dim=g.index_dim,
                   page_tokens=g.page_tokens, top_k=g.top_k, max_pages_per_seq=g.max_pages_per_seq,
                   n_pool_pages=g.n_pool_pages)
    ip, isc = layer.index_pool.cpu().numpy(), layer.index_scale.cpu().numpy()
    bt = layer.block_table.cpu().numpy()
    for b in (1, B - 2):
        qc, qs = orc.index_q_quant(u16(x["index_q"][b:b + 1]), g.index_dim)
        want = orc.index_score_paged(og, qc, qs, x["index_w"][b:b + 1].cpu().numpy(), ip, isc, bt[b:b + 1],
                                     np.array([ctx], np.int32), ctx)
        np.testing.assert_array_equal(want[0].view(np.uint32), sc[b].view(np.uint32))
        np.testing.assert_array_equal(orc.index_topk(want[0], g.top_k), r[b].astype(np.uint32))


def test_attention_at_full_selection_width(cfg3_like):
    w, g, layer, x = cfg3_like
    B, ctx = w["B"], w["ctx"]
    seq_len = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    layer.select(x["index_q"], x["index_w"], seq_len)
    out1 = layer.attend(x["q"]).clone()
    out2 = layer.attend(x["q"]).clone()
    torch.cuda.synchronize(); layer.check_status()
    assert torch.equal(out1, out2)                                          # deterministic
    og = make_geom(orc.Geom, n_heads=g.n_heads, index_heads=g.index_heads, index_dim=g.index_dim,
                   page_tokens=g.page_tokens, top_k=g.top_k, max_pages_per_seq=g.max_pages_per_seq,
                   n_pool_pages=g.n_pool_pages)
    lp, ls = layer.latent_pool.cpu().numpy(), layer.latent_scale.cpu().numpy()
    bt = layer.block_table.cpu().numpy()
    rows = layer.rows.cpu().numpy().view(np.uint32)
    for b in (0, B - 1):
        _, o_f32, _, lse = orc.mla_attend_paged(og, u16(x["q"][b:b + 1]), lp, ls, bt[b:b + 1], rows[b:b + 1],
                                                np.array([2048], np.int32), want_f32=True)
        got = u16(out1[b:b + 1])
        ok, worst = attend_close(got, o_f32)                                # elementwise 2e-2 / 1e-3
        assert ok, worst
        ok, worst, rms = attend_close_ref(got, o_f32)
        assert ok and rms < 5e-3, (worst, rms)
        assert np.abs(layer.out_lse[b].cpu().numpy() - lse[0]).max() < 2e-2
    # softmax weights sum to one: attending a cache of identical rows returns that row (checked on
    # the real cache through the bound |out| <= max |L| over the attended rows)
    tab = orc.e4m3_table()
    b = 0
    r = bt[b, rows[b] // g.page_tokens].astype(np.int64) * g.page_tokens + rows[b] % g.page_tokens
    L = tab[lp.reshape(-1, 576)[r][:, :512]] * ls[r][:, None]
    o = orc.bf16_to_f32(u16(out1[b])).reshape(64, 512)
    assert (np.abs(o) <= np.abs(L).max(0)[None, :] * 1.01 + 1e-3).all()


def test_cfg2_dense_equivalent_shape():
    """The dense-equivalent benchmark shape whole: batch 32, ctx 2048, k = 2048 (selection is the identity)."""
    w = dict(bench.WORKLOADS["cfg2"])
    dev = torch.device("cuda", 0)
    g, layer, gen = bench.build_layer(w, dev, 7)
    x = bench.step_inputs(w, dev, gen)
    B, ctx = w["B"], w["ctx"]
    seq_len = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
    out = layer.step(x["latent"], x["index_key"], x["index_q"], x["index_w"], x["q"], pos, seq_len).clone()
    torch.cuda.synchronize(); layer.check_status()
    assert (layer.n_sel.cpu().numpy() == 2048).all()
    assert (layer.rows.cpu().numpy() == np.arange(2048)[None, :]).all()
    dense = layer.attend(x["q"], dense_len=seq_len).clone()                # rows = NULL path: same result
    torch.cuda.synchronize()
    assert torch.equal(out, dense)
    og = make_geom(orc.Geom, top_k=2048, max_pages_per_seq=g.max_pages_per_seq, n_pool_pages=g.n_pool_pages)
    lp, ls, bt = layer.latent_pool.cpu().numpy(), layer.latent_scale.cpu().numpy(), layer.block_table.cpu().numpy()
    for b in (0, 31):
        _, o_f32, _, _ = orc.mla_attend_paged(og, u16(x["q"][b:b + 1]), lp, ls, bt[b:b + 1], None,
                                              np.array([ctx], np.int32), want_f32=True)
        ok, worst = attend_close(u16(out[b:b + 1]), o_f32)
        assert ok, worst


def test_selection_beyond_16384_tokens_uses_the_wide_kernel_and_stays_exact():
    """Contexts in (16384, 32768] take the 32-keys-per-thread instantiation of the selection kernel: fused
    tensor-core selection == exact CUDA-core chain, bit for bit, on a ragged pair of long contexts."""
    import torch
    from rivoli_b200 import backend as be
    w = dict(bench.WORKLOADS["cfg3"]); w["B"] = 2; w["ctx"] = 30000
    g, layer, gen = bench.build_layer(w, torch.device("cuda", 0), 9)
    x = bench.step_inputs(w, torch.device("cuda", 0), gen)
    seq_len = torch.tensor([30000, 17001], dtype=torch.int32, device="cuda")
    assert be.index_select_uses_mma(g, layer.score_stride)
    layer.select(x["index_q"], x["index_w"], seq_len)
    be.device_sync(); layer.check_status()
    rows_f, n_f = layer.rows.clone(), layer.n_sel.clone()
    layer.select_unfused(x["index_q"], x["index_w"], seq_len)
    be.device_sync()
    assert torch.equal(n_f, layer.n_sel)
    for b in range(2):
        n = int(n_f[b])
        assert n == 2048 and torch.equal(rows_f[b, :n], layer.rows[b, :n])
