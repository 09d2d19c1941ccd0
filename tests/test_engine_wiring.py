"""Host logic of the DSA wiring across layers: indexer layout validation and the lag-by-one
selection state machine (the reference's own host tests, crates/engine/src/indexer.rs:62-88)."""
import pytest

from rivoli_b200.engine import StaleShare, indexer_layout


def test_indexer_layout_accepts_and_rejects_like_the_reference():
    assert indexer_layout(["full", "shared", "shared", "full"], 4, 32, 128, 2048) == [True, False, False, True]
    with pytest.raises(ValueError, match="no DSA indexer dims"):
        indexer_layout(["full"], 1, 0, 128, 2048)
    with pytest.raises(ValueError, match="expected n_layers=3"):
        indexer_layout(["full", "shared"], 3, 32, 128, 2048)
    with pytest.raises(ValueError, match="unknown indexer type"):
        indexer_layout(["full", "sparse"], 2, 32, 128, 2048)
    with pytest.raises(ValueError, match="layer 0 is 'shared'"):
        indexer_layout(["shared", "full"], 2, 32, 128, 2048)


def test_stale_share_serves_the_previous_tokens_selection():
    s = StaleShare(2)
    for nt in range(5, 9):
        served = s.stored(0)
        if nt == 5:
            assert served is None            # the crossing token finds nothing stored
        else:
            assert served == nt - 1          # token nt sees what nt-1 stored
        s.store(0, nt)
        assert s.stored(1) is None           # slab 1 was never stored to
