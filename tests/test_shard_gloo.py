"""Multi-rank host logic on CPU ranks (gloo, world_size 2): page-range sharding with the
candidate exchange and the partial merge must reproduce the single-rank result - indices bit
for bit, output within the merge tolerance. The per-rank arithmetic is the oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as orc
from oracle.workload import State, attend_close, make_geom
from rivoli_b200 import shard


def test_partitions_cover_and_are_disjoint():
    for n, w in ((128, 8), (5, 2), (7, 4), (3, 8)):
        got = [i for r in range(w) for i in shard.shard_sequences(n, w, r)]
        assert got == list(range(n))
        got = [i for r in range(w) for i in shard.page_range(n, w, r)]
        assert got == list(range(n))
    spans = [shard.local_token_span(700, 64, 2, r) for r in range(2)]
    assert spans == [(0, 384), (384, 316)]
    assert shard.local_token_span(10, 64, 4, 3) == (64, 0)          # a rank may hold nothing


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _rank_main(rank, world, port, seed, ctx, k, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        st = State(seed, len(ctx), ctx, top_k=k)
        g = st.og
        P, W, hd = g.page_tokens, st.W, g.index_dim
        B = st.B
        # this rank's slice of every sequence, re-paged into a local pool (local positions from 0)
        spans = [shard.local_token_span(int(n), P, world, rank) for n in st.seq_len]
        max_pages = max(1, max((n + P - 1) // P for _, n in spans))
        lg = make_geom(orc.Geom, **{**st.geom_kw, "max_pages_per_seq": max_pages, "n_pool_pages": max_pages * B})
        pool = orc.Pool(max_pages * B, B, max_pages, P)
        rows_n = max_pages * B * P
        lp, ls = np.zeros(rows_n * W, np.uint8), np.zeros(rows_n, np.float32)
        ip, isc = np.zeros(rows_n * hd, np.uint8), np.zeros(rows_n, np.float32)
        off = np.concatenate([[0], np.cumsum(st.seq_len - 1)])          # history offsets
        lat, key, seqs, poss = [], [], [], []
        for b, (lo, n) in enumerate(spans):
            assert pool.reserve(b, n) == 0
            for t in range(lo, lo + n):
                last = t == st.seq_len[b] - 1
                lat.append(st.new_latent[b] if last else st.hist_latent[off[b] + t])
                key.append(st.new_key[b] if last else st.hist_key[off[b] + t])
                seqs.append(b); poss.append(t - lo)
        bt = pool.block_table()
        if lat:
            assert orc.kv_append_paged(lg, np.stack(lat), np.stack(key), np.array(seqs, np.int32),
                                       np.array(poss, np.int32), bt, lp, ls, ip, isc) == 0
        qc, qs = orc.index_q_quant(st.index_q, hd)

        def score(iq, iw, lens):
            stride = max(1, int(max(n for _, n in spans)))
            return torch.from_numpy(orc.index_score_paged(lg, qc, qs, st.index_w, ip, isc, bt, lens.numpy(), stride))

        def topk(scores, lens, kk):
            r, n = orc.index_topk_batched(scores.numpy(), lens.numpy(), kk)
            r = np.where(np.arange(kk)[None, :] < n[:, None], r, 0)
            return torch.from_numpy(r.astype(np.int64)).to(torch.int32), torch.from_numpy(n)

        def attend(q, rows, n_rows):
            out, m, lse = orc.mla_attend_paged(lg, st.q, lp, ls, bt, rows.numpy().astype(np.uint32), n_rows.numpy())
            return torch.from_numpy(out.view(np.int16)).view(torch.bfloat16), torch.from_numpy(lse)

        def merge(part_out, part_lse):
            o = orc.attend_merge_partials(part_out.view(torch.int16).numpy().view(np.uint16), part_lse.numpy(), g.kv_lora)
            return torch.from_numpy(o.view(np.int16)).view(torch.bfloat16)

        ops = shard.ShardOps(score, topk, attend, merge)
        local_len = torch.tensor([n for _, n in spans], dtype=torch.int32)
        offset = torch.tensor([lo for lo, _ in spans], dtype=torch.int32)
        out, rows_g, n_g = shard.page_range_step(ops, None, None, None, local_len, offset, k)
        ret[rank] = (out.view(torch.int16).numpy().view(np.uint16).copy(), [rows_g[b, :n_g[b]].tolist() for b in range(B)])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ctx,k", [([700, 513, 130], 256), ([300, 64], 2048)])
def test_page_range_shards_reproduce_the_single_rank_step(ctx, k):
    world, seed = 2, 77
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, _free_port(), seed, ctx, k, ret), nprocs=world, join=True)
    st = State(seed, len(ctx), ctx, top_k=k)
    want = st.oracle_step()
    for b in range(len(ctx)):
        union = sorted(ret[0][1][b] + ret[1][1][b])
        assert union == want["rows"][b, :want["n_sel"][b]].tolist()          # exact global top-k, bit for bit
    np.testing.assert_array_equal(ret[0][0], ret[1][0])                      # every rank holds the same merge
    ok, worst = attend_close(ret[0][0].reshape(len(ctx), 64, 512), want["out_f32"], rel=3e-2, abs_=2e-3)
    assert ok, worst
