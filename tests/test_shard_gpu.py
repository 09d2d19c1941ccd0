"""Page-range sharding through the library's ``rivoli_shard_*`` entry points: every shard holds a page range of
every sequence, and the shards together must select exactly the single-rank top-k and merge to the single-rank
output.

* on ONE GPU the ranks are emulated in one process: each shard's phases run one after the other and the two
  all-gathers are a concatenation of the shards' buffers (no kernel of one shard ever waits on another);
* with two or more GPUs the same step runs as one process per GPU with the library's own ``ncclAllGather`` calls
  (``rivoli_shard_step_paged``)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.helpers import State, attend_close, attend_close_ref, make_geom

pytestmark = pytest.mark.gpu

CASES = [([4700, 2513, 130], 2048), ([900, 64, 1], 256)]


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _build_shard(st, rank, world, device, k):
    """This rank's slice of every sequence of ``st`` in a layer of its own (local positions from 0)."""
    from rivoli_b200 import backend as be, shard
    from rivoli_b200.layer import DsaDecodeLayer
    P, B = st.og.page_tokens, st.B
    spans = [shard.local_token_span(int(n), P, world, rank) for n in st.seq_len]
    max_pages = max(1, max((n + P - 1) // P for _, n in spans))
    g = make_geom(be.DsaGeom, **{**st.geom_kw, "max_pages_per_seq": max_pages, "n_pool_pages": max_pages * B})
    layer = DsaDecodeLayer(g, B, device=device, shuffle_seed=5 + rank)
    off = np.concatenate([[0], np.cumsum(st.seq_len - 1)])
    lat, key, seqs, poss = [], [], [], []
    for b, (lo, n) in enumerate(spans):
        layer.reserve(b, n)
        for t in range(lo, lo + n):
            last = t == st.seq_len[b] - 1
            lat.append(st.new_latent[b] if last else st.hist_latent[off[b] + t])
            key.append(st.new_key[b] if last else st.hist_key[off[b] + t])
            seqs.append(b); poss.append(t - lo)
    layer.upload_block_table()

    def dev(a):
        a = np.ascontiguousarray(a)
        return torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).to(device)

    if lat:
        layer.append(dev(np.stack(lat)), dev(np.stack(key)), dev(np.array(poss, np.int32)), dev(np.array(seqs, np.int32)))
    local_len = dev(np.array([n for _, n in spans], np.int32))
    offset = np.array([lo for lo, _ in spans], np.int64)
    return layer, dev, local_len, offset


def _check(st, k, outs, rows_by_rank):
    want = st.oracle_step()
    for b in range(st.B):
        union = sorted(r for rows in rows_by_rank for r in rows[b])
        assert union == want["rows"][b, :want["n_sel"][b]].tolist()          # exact global top-k
    for o in outs[1:]:
        np.testing.assert_array_equal(outs[0], o)                            # every rank holds the same merge
    # bf16 partials per shard, merged: the reference's tolerance form, and elementwise 2e-2 / 1e-3 with a margin
    # for the second bf16 rounding
    ok, worst, rms = attend_close_ref(outs[0].reshape(st.B, 64, 512), want["out_f32"])
    assert ok and rms <= 1e-2, (worst, rms)
    ok, worst = attend_close(outs[0].reshape(st.B, 64, 512), want["out_f32"], rel=3e-2, abs_=2e-3)
    assert ok, worst


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("ctx,k", CASES)
def test_emulated_ranks_on_one_gpu_reproduce_the_single_rank_step(ctx, k, world):
    from rivoli_b200 import backend as be, shard
    be.lib()
    st = State(91, len(ctx), ctx, top_k=k)
    device = torch.device("cuda", 0)
    shards = []
    for rank in range(world):
        layer, dev, local_len, offset = _build_shard(st, rank, world, device, k)
        shards.append((shard.ShardedDecodeStep(layer, rank, world), dev, local_len, offset))
    iq, iw, q = shards[0][1](st.index_q), shards[0][1](st.index_w), shards[0][1](st.q)
    all_cand = torch.cat([s.candidates(iq, iw, ll).clone() for s, _, ll, _ in shards])       # "all-gather" 1
    all_part = torch.cat([s.cut_attend(all_cand, q).clone() for s, _, _, _ in shards])       # "all-gather" 2
    outs, rows = [], []
    for s, _, _, offset in shards:
        o = s.merge(all_part)
        be.device_sync()
        s.layer.check_status()
        outs.append(o.cpu().view(torch.int16).numpy().view(np.uint16).copy())
        n = s.n_mine.cpu().numpy()
        ra = s.rows_att.cpu().numpy().view(np.uint32).astype(np.int64)
        rows.append([(ra[b, :n[b]] + offset[b]).tolist() for b in range(st.B)])
        for b in range(st.B):
            assert np.all(np.diff(ra[b, :n[b]]) > 0)                         # ascending local rows
    _check(st, k, outs, rows)


def test_one_rank_step_equals_the_single_gpu_operators():
    """world = 1 needs no communicator: rivoli_shard_step_paged == select + attend on the same layer."""
    from rivoli_b200 import backend as be, shard
    be.lib()
    ctx, k = [3000, 700, 200], 512
    st = State(92, len(ctx), ctx, top_k=k)
    layer, dev, local_len, offset = _build_shard(st, 0, 1, torch.device("cuda", 0), k)
    step = shard.ShardedDecodeStep(layer, 0, 1)
    out = step.step(dev(st.index_q), dev(st.index_w), dev(st.q), local_len)
    be.device_sync()
    layer.check_status()
    n = step.n_mine.cpu().numpy()
    ra = step.rows_att.cpu().numpy().view(np.uint32).astype(np.int64)
    _check(st, k, [out.cpu().view(torch.int16).numpy().view(np.uint16).copy()], [[ra[b, :n[b]].tolist() for b in range(st.B)]])


def _rank_main(rank, world, port, seed, ctx, k, ret):
    from rivoli_b200 import backend as be, shard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("gloo", rank=rank, world_size=world)          # carries the NCCL id only
    try:
        st = State(seed, len(ctx), ctx, top_k=k)
        layer, dev, local_len, offset = _build_shard(st, rank, world, device, k)
        comm = shard.ShardedDecodeStep.nccl_comm(rank, world)
        step = shard.ShardedDecodeStep(layer, rank, world, comm)
        for _ in range(2):
            out = step.step(dev(st.index_q), dev(st.index_w), dev(st.q), local_len)
        be.device_sync()
        layer.check_status()
        n = step.n_mine.cpu().numpy()
        ra = step.rows_att.cpu().numpy().view(np.uint32).astype(np.int64)
        ret[rank] = (out.cpu().view(torch.int16).numpy().view(np.uint16).copy(),
                     [(ra[b, :n[b]] + offset[b]).tolist() for b in range(st.B)])
        dist.barrier()
        be.shard_nccl_comm_destroy(comm)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ctx,k", CASES)
def test_ranks_on_separate_gpus_exchange_through_nccl(ctx, k):
    world = min(4, torch.cuda.device_count())
    if world < 2:
        pytest.skip("needs two GPUs: one process per GPU, the library's own ncclAllGather between them")
    from rivoli_b200 import backend as be
    be.lib()
    seed = 91
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_rank_main, args=(world, _free_port(), seed, ctx, k, ret), nprocs=world, join=True)
    st = State(seed, len(ctx), ctx, top_k=k)
    _check(st, k, [ret[r][0] for r in range(world)], [ret[r][1] for r in range(world)])
