"""Continuous batching with eviction churn on the GPU (the 78-layer churn workload at reduced scale): several
layers share one page allocator, every step appends one token per sequence per layer, some
sequences finish and their slots are refilled (pages go back to the free list and are drawn again,
the replacement's context is prefilled through the same append operator). After every step the
selected rows must equal the oracle's bit for bit and the attention output must be within the
tolerance, for every layer - so no stale page, scale or row ever leaks from an evicted sequence."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import attend_close, attend_close_ref, bf16_normal, make_geom

pytestmark = pytest.mark.gpu


def dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(a).cuda()


def test_churn_three_layers_match_oracle():
    from rivoli_b200 import backend as be
    from rivoli_b200.layer import DsaDecodeLayer
    from rivoli_b200.scheduler import ContinuousBatcher, churn_plan
    be.lib()
    n_slots, n_layers, P, top_k, steps = 8, 3, 64, 256, 6
    lo, hi = 60, 900
    max_ctx = hi + steps + 2
    max_pages = (max_ctx + P - 1) // P
    n_pool = int(1.25 * n_slots * max_pages)
    kw = dict(n_heads=64, kv_lora=512, rope_dim=64, index_heads=32, index_dim=128, page_tokens=P, top_k=top_k,
              max_pages_per_seq=max_pages, n_pool_pages=n_pool)
    g, og = make_geom(be.DsaGeom, **kw), make_geom(orc.Geom, **kw)
    W, hd, rows_n = 576, 128, n_pool * P
    sched = ContinuousBatcher(n_slots, n_pool, max_ctx, P, shuffle_seed=9)
    layers = [DsaDecodeLayer(g, n_slots, max_ctx=max_pages * P, pool=sched.pool) for _ in range(n_layers)]
    mirror = [dict(lp=np.zeros(rows_n * W, np.uint8), ls=np.zeros(rows_n, np.float32),
                   ip=np.zeros(rows_n * hd, np.uint8), isc=np.zeros(rows_n, np.float32)) for _ in range(n_layers)]
    rng = np.random.RandomState(5)

    def prefill(slots, lens):
        """Cache contents of freshly admitted sequences, every layer (GPU append + oracle append)."""
        bt = sched.block_table()
        seq = np.concatenate([np.full(n, s, np.int32) for s, n in zip(slots, lens)])
        pos = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])
        for L, M in zip(layers, mirror):
            lat, key = bf16_normal(rng, (seq.size, W)), bf16_normal(rng, (seq.size, hd))
            L.upload_block_table(bt)
            L.append(dev(lat), dev(key), dev(pos), dev(seq))
            assert orc.kv_append_paged(og, lat, key, seq, pos, bt, M["lp"], M["ls"], M["ip"], M["isc"]) == 0

    first = rng.randint(lo, hi + 1, n_slots)
    for s, n in enumerate(first):
        sched.admit(s, int(n))
    prefill(range(n_slots), first)
    for step in range(steps):
        row_pos, seq_len = sched.begin_step()
        bt = sched.block_table()
        for li, (L, M) in enumerate(zip(layers, mirror)):
            lat, key = bf16_normal(rng, (n_slots, W)), bf16_normal(rng, (n_slots, hd))
            iq = bf16_normal(rng, (n_slots, 32, hd))
            iw = orc.bf16_to_f32(bf16_normal(rng, (n_slots, 32)))
            q = bf16_normal(rng, (n_slots, 64, W))
            L.upload_block_table(bt)
            out = L.step(dev(lat), dev(key), dev(iq), dev(iw), dev(q), dev(row_pos), dev(seq_len))
            be.device_sync()
            L.check_status()
            assert orc.kv_append_paged(og, lat, key, None, row_pos, bt, M["lp"], M["ls"], M["ip"], M["isc"]) == 0
            qc, qs = orc.index_q_quant(iq, hd)
            sc = orc.index_score_paged(og, qc, qs, iw, M["ip"], M["isc"], bt, seq_len, int(seq_len.max()))
            rows, n_sel = orc.index_topk_batched(sc, seq_len, top_k)
            _, want, _, _ = orc.mla_attend_paged(og, q, M["lp"], M["ls"], bt, rows, n_sel, want_f32=True)
            got_rows, got_n = L.rows.cpu().numpy().view(np.uint32), L.n_sel.cpu().numpy()
            np.testing.assert_array_equal(got_n, n_sel)
            for b in range(n_slots):
                np.testing.assert_array_equal(got_rows[b, :n_sel[b]], rows[b, :n_sel[b]], err_msg=f"step {step} layer {li} slot {b}")
            ok, worst, rms = attend_close_ref(out.cpu().view(torch.int16).numpy().view(np.uint16), want)
            assert ok and rms <= 5e-3, (step, li, worst, rms)
            ok, worst = attend_close(out.cpu().view(torch.int16).numpy().view(np.uint16), want)   # elementwise 2e-2 / 1e-3
            assert ok, (step, li, worst)
            # the pools themselves: bit-identical everywhere a live sequence has a token
            np.testing.assert_array_equal(L.latent_scale.cpu().numpy().view(np.uint32), M["ls"].view(np.uint32))
            np.testing.assert_array_equal(L.index_pool.cpu().numpy(), M["ip"])
        slots, lens = churn_plan(rng, n_slots, 0.25, lo, hi)      # 2 of 8 slots finish and are refilled
        sched.finish(slots, lens)
        prefill(slots, lens)
    assert sched._next_id == n_slots + steps * 2


def test_shared_layers_attend_over_the_full_layers_selection():
    """A full layer followed by two shared layers: the shared layers run no scorer / top-k, cache only their
    latent rows, and their attention equals the oracle's attention over the FULL layer's rows on their own
    latent cache."""
    from rivoli_b200 import backend as be
    from rivoli_b200.engine import DsaDecodeStack, indexer_layout
    from tests.helpers import State
    be.lib()
    full = indexer_layout(["full", "shared", "shared"], 3, 32, 128, 256)
    states = [State(50 + i, 3, [700, 300, 2100], top_k=256) for i in range(3)]     # same geometry, different contents
    st0 = states[0]
    g = make_geom(be.DsaGeom, **st0.geom_kw)
    stack = DsaDecodeStack(g, st0.B, full, max_ctx=int(g.max_pages_per_seq * g.page_tokens))
    caches = []
    for L, st in zip(stack.layers, states):          # every layer: its own cache contents, ONE page table (layer 0's)
        lp, ls = np.zeros_like(st0.latent_pool), np.zeros_like(st0.latent_scale)
        ip, isc = np.zeros_like(st0.index_pool), np.zeros_like(st0.index_scale)
        assert orc.kv_append_paged(st0.og, st.hist_latent, st.hist_key, st.hist_seq, st.hist_pos, st0.block_table,
                                   lp, ls, ip, isc) == 0
        caches.append((lp, ls, ip, isc))
        L.latent_pool.copy_(dev(lp)); L.latent_scale.copy_(dev(ls))
        L.index_pool.copy_(dev(ip)); L.index_scale.copy_(dev(isc))
        L.upload_block_table(st0.block_table)
    outs = []
    for i, st in enumerate(states):
        outs.append(stack.step_layer(i, dev(st.new_latent), dev(st.new_key) if full[i] else None,
                                     dev(st.index_q) if full[i] else None, dev(st.index_w) if full[i] else None,
                                     dev(st.q), dev(st0.row_pos), dev(st0.seq_len)).clone())
    be.device_sync()
    for L in stack.layers:
        L.check_status()
    want0 = st0.oracle_step()
    rows, n_sel = want0["rows"], want0["n_sel"]
    np.testing.assert_array_equal(stack.layers[0].n_sel.cpu().numpy(), n_sel)
    for i, st in enumerate(states):
        lp, ls, ip, isc = (a.copy() for a in caches[i])
        assert orc.kv_append_paged(st0.og, st.new_latent, st.new_key, None, st0.row_pos, st0.block_table, lp, ls, ip, isc) == 0
        _, want, _, _ = orc.mla_attend_paged(st0.og, st.q, lp, ls, st0.block_table, rows, n_sel, want_f32=True)
        ok, worst, rms = attend_close_ref(outs[i].cpu().view(torch.int16).numpy().view(np.uint16), want)
        assert ok and rms <= 5e-3, (i, worst, rms)
        ok, worst = attend_close(outs[i].cpu().view(torch.int16).numpy().view(np.uint16), want)       # elementwise 2e-2 / 1e-3
        assert ok, (i, worst)


def test_stale_selection_serves_the_previous_tokens_rows():
    """The one-step-stale selection (crates/engine/src/indexer.rs:14-63), batched and on the device: a full layer
    followed by a shared layer, three token-steps. Token t attends over the rows token t-1 selected (verbatim, the
    new token's own row absent); a sequence at or below top_k (nothing stored) attends densely; a request that has
    just taken its slot with a long context serves its fresh selection once. Checked against the oracle step by
    step, for the full layer and for the shared layer that inherits the served rows."""
    from rivoli_b200 import backend as be
    from rivoli_b200.engine import DsaDecodeStack
    from tests.helpers import State
    be.lib()
    k = 256
    states = [State(70 + i, 3, [200, 257, 700], top_k=k) for i in range(2)]          # one cache content per layer
    st0 = states[0]
    og = st0.og
    P = og.page_tokens
    steps = 3
    # room to grow: a pool and table sized for `steps` more tokens
    max_pages = int((st0.seq_len.max() + steps + P - 1) // P)
    g = make_geom(be.DsaGeom, **{**st0.geom_kw, "max_pages_per_seq": max_pages, "n_pool_pages": 3 * max_pages})
    ogs = make_geom(orc.Geom, **{**st0.geom_kw, "max_pages_per_seq": max_pages, "n_pool_pages": 3 * max_pages})
    stack = DsaDecodeStack(g, 3, [True, False], max_ctx=max_pages * P, stale=True)
    W, hd = 576, 128
    rows_n = 3 * max_pages * P
    mirror = []
    seq_len = st0.seq_len.astype(np.int32) - 1                                        # cached tokens before step 0
    for b in range(3):
        stack.pool.reserve(b, int(seq_len[b]))
    bt = stack.pool.block_table()
    for L, st in zip(stack.layers, states):
        lp, ls = np.zeros(rows_n * W, np.uint8), np.zeros(rows_n, np.float32)
        ip, isc = np.zeros(rows_n * hd, np.uint8), np.zeros(rows_n, np.float32)
        assert orc.kv_append_paged(ogs, st.hist_latent, st.hist_key, st.hist_seq, st.hist_pos, bt, lp, ls, ip, isc) == 0
        L.latent_pool.copy_(dev(lp)); L.latent_scale.copy_(dev(ls)); L.index_pool.copy_(dev(ip)); L.index_scale.copy_(dev(isc))
        mirror.append(dict(lp=lp, ls=ls, ip=ip, isc=isc))
    rng = np.random.RandomState(7)
    prev_rows = [None] * 3
    u16 = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16)
    for step in range(steps):
        for b in range(3):
            stack.pool.reserve(b, int(seq_len[b]) + 1)
        row_pos = seq_len.copy()
        seq_len = seq_len + 1
        bt = stack.pool.block_table()
        stack.upload_block_table()
        stack.begin_token(seq_len)
        lat = [bf16_normal(rng, (3, W)) for _ in range(2)]
        key, iq = bf16_normal(rng, (3, hd)), bf16_normal(rng, (3, 32, hd))
        iw = orc.bf16_to_f32(bf16_normal(rng, (3, 32)))
        q = [bf16_normal(rng, (3, 64, W)) for _ in range(2)]
        outs = [stack.step_layer(0, dev(lat[0]), dev(key), dev(iq), dev(iw), dev(q[0]), dev(row_pos), dev(seq_len)).clone(),
                stack.step_layer(1, dev(lat[1]), None, None, None, dev(q[1]), dev(row_pos), dev(seq_len)).clone()]
        be.device_sync()
        for L in stack.layers:
            L.check_status()
        # oracle: append, fresh selection of the full layer, the rows each sequence is SERVED
        M0, M1 = mirror
        assert orc.kv_append_paged(ogs, lat[0], key, None, row_pos, bt, M0["lp"], M0["ls"], M0["ip"], M0["isc"]) == 0
        assert orc.kv_append_paged(ogs, lat[1], np.zeros_like(key), None, row_pos, bt, M1["lp"], M1["ls"], M1["ip"], M1["isc"]) == 0
        qc, qs = orc.index_q_quant(iq, hd)
        sc = orc.index_score_paged(ogs, qc, qs, iw, M0["ip"], M0["isc"], bt, seq_len, int(seq_len.max()))
        fresh, n_fresh = orc.index_topk_batched(sc, seq_len, k)
        stride = int(seq_len.max())
        served = np.zeros((3, stride), np.uint32); n_served = np.zeros(3, np.int32)
        for b in range(3):
            if prev_rows[b] is not None:                      # stored at the previous token
                r = prev_rows[b]
            elif seq_len[b] <= k + 1:                         # nothing stored: dense over the whole prefix
                r = np.arange(seq_len[b], dtype=np.uint32)
            else:                                             # a fresh slot with a long context: its own selection, once
                r = fresh[b, :n_fresh[b]]
            served[b, :r.size] = r; n_served[b] = r.size
            prev_rows[b] = fresh[b, :n_fresh[b]].copy() if seq_len[b] > k else None
        for li, M in enumerate(mirror):
            _, want, _, _ = orc.mla_attend_paged(ogs, q[li], M["lp"], M["ls"], bt, served, n_served, want_f32=True)
            ok, worst = attend_close(u16(outs[li]), want)
            assert ok, (step, li, worst)
    # what was served really was the stale set: sequence 2 attended 256 rows that do NOT contain its newest token
    assert n_served[2] == k and served[2, :k].max() < seq_len[2] - 1
