"""Continuous batching with eviction churn (the 78-layer churn workload at reduced scale): page tables
and free lists stay bit-identical to the oracle's allocator, no page is ever mapped twice,
and a pool sized 1.25x the worst live set never runs dry."""
import numpy as np
import pytest

from oracle import oracle as orc
from rivoli_b200 import backend as be, build
from rivoli_b200.scheduler import ContinuousBatcher, churn_plan


class _OraclePool:
    """The oracle's allocator behind the PagePool interface."""
    def __init__(self, n_pages, n_slots, max_pages, P):
        self.p = orc.Pool(n_pages, n_slots, max_pages, P)
    def shuffle(self, s): self.p.shuffle(s)
    def reserve(self, slot, n): return self.p.reserve(slot, n)
    def release(self, slot): return self.p.release(slot)
    def block_table(self): return self.p.block_table()
    def free_list(self): return self.p.free_list()
    @property
    def n_free(self): return self.p.n_free


def test_churn_matches_oracle_allocator():
    build.build()
    n_slots, P, lo, hi, steps = 32, 64, 512, 4096, 60
    max_ctx = hi + steps + 1
    n_pages = int(1.25 * n_slots * ((max_ctx + P - 1) // P))
    a = ContinuousBatcher(n_slots, n_pages, max_ctx, P, shuffle_seed=4)
    o = ContinuousBatcher(n_slots, n_pages, max_ctx, P, shuffle_seed=4,
                          pool=_OraclePool(n_pages, n_slots, (max_ctx + P - 1) // P, P))
    rng = np.random.RandomState(4)
    for slot, n in enumerate(rng.randint(lo, hi + 1, n_slots)):
        assert a.admit(slot, int(n)) == o.admit(slot, int(n))
    for step in range(steps):
        pa, la = a.begin_step(); po, lo_ = o.begin_step()
        np.testing.assert_array_equal(pa, po); np.testing.assert_array_equal(la, lo_)
        assert (la == pa + 1).all()
        slots, lens = churn_plan(rng, n_slots, 0.10, lo, hi)               # 10 % finish and are replaced
        assert a.finish(slots, lens) == o.finish(slots, lens)
        bt = a.block_table()
        np.testing.assert_array_equal(bt, o.block_table())
        np.testing.assert_array_equal(a.pool.free_list(), o.pool.free_list())
        live = bt[bt >= 0]
        assert len(set(live.tolist())) == live.size and live.size + a.n_free == n_pages
        need = (a.seq_len + P - 1) // P
        assert ((bt >= 0).sum(1) >= need).all()                            # every cached token has a page
    assert a._next_id == n_slots + steps * 3


def test_pool_exhaustion_is_reported_not_hidden():
    build.build()
    a = ContinuousBatcher(2, 4, 64 * 4, 64)
    a.admit(0, 192)
    with pytest.raises(be.BackendError) as e:
        a.admit(1, 128)                                                    # needs 2 pages, 1 left
    assert e.value.code == 1007


def test_replacements_fit_at_pool_capacity_and_a_failed_admit_leaves_the_slot_empty():
    """Three slots of two pages fill a six-page pool. Two finish and are replaced by a one-page and a three-page
    request: that fits only because both finishing slots return their pages before either replacement reserves.
    A request that cannot fit raises 1007 and leaves its slot empty rather than describing pages it gave back."""
    build.build()
    a = ContinuousBatcher(3, 6, 64 * 4, 64)
    for s_ in range(3):
        a.admit(s_, 128)
    assert a.n_free == 0
    a.finish([0, 2], [64 * 3, 64])                 # slot 0 needs 3 pages: its own 2 and one of slot 2's
    assert a.n_free == 0 and a.seq_len.tolist() == [192, 128, 64]
    bt = a.block_table()
    live = bt[bt >= 0]
    assert live.size == 6 and len(set(live.tolist())) == 6
    with pytest.raises(be.BackendError) as e:
        a.admit(1, 64 * 4)                         # 4 pages wanted, 2 come back
    assert e.value.code == 1007
    assert a.seq_id[1] == -1 and a.seq_len[1] == 0
    row_pos, seq_len = a.begin_step()              # the empty slot does not grow
    assert seq_len.tolist() == [193, 0, 65] and row_pos.tolist() == [192, 0, 64]
