"""Host selection arithmetic of the V4 path (rivoli_b200/v4_select.py) against the literal expectations recorded in
the reference's own unit tests (crates/engine/src/v4/select.rs:514-810) and against the oracle's row functions."""
import importlib.util
import os

import numpy as np
import pytest

from oracle import oracle as orc

# the module is pure host arithmetic: load it without importing the package (which binds the CUDA library)
_spec = importlib.util.spec_from_file_location(
    "v4_select", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "rivoli_b200", "v4_select.py"))
vs = importlib.util.module_from_spec(_spec)
import sys
sys.modules["v4_select"] = vs
_spec.loader.exec_module(vs)

at = vs.Extent


def test_multi_row_decode_is_refused():
    with pytest.raises(vs.SelectionError, match="one query row"):
        vs.Sel(8, 0, 512, at(3, 5)).shape()
    assert vs.Sel(8, 0, 512, at(3, 0)).shape() == (3, 3)
    assert vs.Sel(8, 0, 512, at(1, 5)).shape() == (1, 8)


def test_ring_is_read_oldest_first():
    assert vs.window_rows(4, at(1, 6)) == [[3, 0, 1, 2]]
    assert vs.window_rows(4, at(1, 2)) == [[0, 1, 2, -1]]
    for win in (4, 8, 128):
        for sp in (1, win - 2, win - 1, win, 3 * win + 5):
            assert vs.window_rows(win, at(1, sp))[0] == orc.v4_window_row(win, sp).tolist()


def test_prefill_window_is_causal_absolute_positions():
    rows = vs.window_rows(4, at(6, 0))
    assert rows[0] == [0, -1, -1, -1] and rows[2] == [0, 1, 2, -1] and rows[5] == [2, 3, 4, 5]
    assert vs.window_rows(8, at(3, 0)) == [[0, -1, -1], [0, 1, -1], [0, 1, 2]]


def test_prefill_query_reads_only_closed_blocks():
    rows = vs.compressed_rows(2, at(6, 0), 100)
    assert rows[0] == [-1, -1, -1] and rows[1] == [100, -1, -1] and rows[3] == [100, 101, -1] and rows[5] == [100, 101, 102]
    assert vs.compressed_rows(0, at(6, 0), 100) == []
    assert vs.compressed_rows(4, at(1, 19), 8) == [[8, 9, 10, 11, 12]]


def test_cache_row_and_selection_column():
    win, prompt = 128, 16
    pre = at(prompt, 0)
    assert vs.compress_dst(4, win, pre) == (win, 4)
    assert vs.compress_dst(4, vs.compress_offset(win, pre), pre) == (prompt, 4)
    dec = at(1, 47)
    assert vs.compress_dst(4, win, dec) == (win + 11, 1)
    assert vs.compress_dst(4, vs.compress_offset(win, dec), dec) == (win + 11, 1)
    assert [vs.compress_dst(4, 0, at(1, p))[0] for p in (15, 31)] == [3, 7]      # positional, not a running count
    assert vs.compress_dst(4, 0, at(1, 16)) is None and vs.compress_dst(0, 0, at(1, 15)) is None


def test_indexed_layer_refuses_past_its_cap():
    topk = 2
    limit = vs.positional_context_limit(topk)
    assert limit == 12
    assert vs.Sel(8, 4, topk, at(1, limit - 2)).shape() == (1, 8 + 2)
    with pytest.raises(vs.SelectionError, match="index_topk"):
        vs.Sel(8, 4, topk, at(1, limit)).shape()
    assert vs.Sel(8, 2, topk, at(1, limit * 4)).shape()[0] == 1      # no indexer, no cap


def test_below_the_cap_scored_equals_positional():
    for e in (at(1, 19), at(12, 0)):
        s = vs.Sel(8, 4, 512, e)
        rows, cols = s.shape()
        n_comp = cols - len(vs.window_rows(8, e)[0])
        scores = np.arange(rows * n_comp, dtype=np.float32)           # adversarial: newest block scores highest
        comp = vs.scored_rows(scores, n_comp, ratio=4, index_topk=512, at=e, offset=vs.compress_offset(8, e))
        assert np.array_equal(s.gather(), s.gather_scored(comp))


def test_above_the_cap_scores_decide_with_ties_toward_the_lower_index():
    kw = dict(ratio=4, index_topk=3, at=at(1, 19), offset=100)
    assert vs.scored_rows([1.0, 1.0, 9.0, 0.5, 1.0], 5, **kw) == [[100, 101, 102]]
    assert vs.scored_rows([1.0, 1.0, 9.0, 0.5, 2.0], 5, **kw) == [[100, 102, 104]]
    assert vs.scored_rows([-0.0, 0.0, -0.0, 0.0], 4, ratio=4, index_topk=2, at=at(1, 15), offset=0) == [[1, 3]]


def test_prefill_row_cannot_select_a_block_that_closed_after_it():
    scores = [0.1, 9.0] * 8
    kw = dict(ratio=4, index_topk=1, at=at(8, 0), offset=10)
    assert vs.scored_rows(scores, 2, **kw) == [[-1], [-1], [-1], [10], [10], [10], [10], [11]]
    with pytest.raises(vs.SelectionError, match="15 scores"):
        vs.scored_rows(scores[:15], 2, **kw)


def test_ragged_or_short_ranked_rows_are_refused():
    s = vs.Sel(8, 4, 3, at(2, 0))
    with pytest.raises(vs.SelectionError, match="ranked rows"):
        s.gather_scored([[0]])
    with pytest.raises(vs.SelectionError, match="wide"):
        vs.Sel(8, 4, 3, at(8, 0)).gather_scored([[8]] * 7 + [[8, 9]])
    with pytest.raises(vs.SelectionError, match="sliding_window is zero"):
        vs.Sel(0, 4, 3, at(1, 5)).gather_scored([[0]])


def test_scored_rows_match_the_oracle_row_function():
    rng = np.random.default_rng(0)
    for n_comp, k in ((37, 8), (200, 64), (5, 9)):
        sc = orc.bf16_to_f32(orc.f32_to_bf16(rng.standard_normal(n_comp).astype(np.float32)))   # many ties on the bf16 grid
        sc[::5] = sc[0]
        e = at(1, n_comp * 4 - 1)
        got = vs.scored_rows(sc, n_comp, ratio=4, index_topk=k, at=e, offset=128)[0]
        assert got == orc.v4_scored_row(sc, n_comp, k, 128, min(k, n_comp)).tolist()
        # prefill rows use the causal limit
        rows = 12
        m = rng.standard_normal((rows, 3)).astype(np.float32)
        got = vs.scored_rows(m, 3, ratio=4, index_topk=2, at=at(rows, 0), offset=rows)
        for t in range(rows):
            assert got[t] == orc.v4_scored_row(m[t], min((t + 1) // 4, 3), 2, rows, 2).tolist()


def test_decode_rectangle_equals_the_device_layout():
    """gather() at decode is the row the batched kernel writes (before its -1 padding to a fixed width)."""
    s = vs.Sel(8, 4, 4, at(1, 13))            # 3 closed blocks, below the cap
    assert s.gather().tolist() == [[6, 7, 0, 1, 2, 3, 4, 5, 8, 9, 10]]
