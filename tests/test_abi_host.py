"""CPU-side checks: the C-ABI library loads and exports every declared symbol, the guard
codes fire before anything touches a device, and the host page allocator matches the
oracle's bit for bit under churn."""
import ctypes
import os
import re

import numpy as np
import pytest

from oracle import oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def be():
    from rivoli_b200 import build
    build.build()
    from rivoli_b200 import backend
    return backend


def test_every_declared_symbol_is_exported(be):
    hdr = open(os.path.join(ROOT, "include", "rivoli_kernels.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = sorted(set(re.findall(r"\b(rivoli_[a-z0-9_]+)\s*\(", hdr)))
    assert len(names) >= 20
    L = be.lib()
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/rivoli_kernels.h but not exported"
    assert be.kernels_arch() == "sm_100a"


def test_geom_layout(be):
    assert ctypes.sizeof(be.DsaGeom) == 48 == ctypes.sizeof(orc.Geom)
    g = be.DsaGeom.make(max_pages_per_seq=4, n_pool_pages=8)
    assert g.n_heads == 64 and abs(g.softmax_scale - 1 / 24.0) < 1e-7
    assert abs(g.index_wscale - 32 ** -0.5) < 1e-7 and abs(g.index_dscale - 128 ** -0.5) < 1e-7


def test_guards_fire_on_the_host(be):
    """Argument guards are decided before any launch, so they work without a GPU
    (pointers are never dereferenced; crates/engine/tests/common/asserts.rs:87-99)."""
    def code(fn):
        with pytest.raises(be.BackendError) as e:
            fn()
        return e.value.code
    assert code(lambda: be.launch_append_kv(0, 0, 0, 0, 0, -1, 256, 64, 2)) == 1001
    assert code(lambda: be.launch_append_kv(0, 0, 0, 0, 0, 0, 160, 64, 2)) == 1002
    assert code(lambda: be.launch_attend(0, 0, 0, 0, 0, None, 8, 16, 640, 64, 5, 1.0, 0, 0)) == 1004
    assert code(lambda: be.launch_attend(0, 0, 0, 0, 0, None, 8, 16, 160, 64, 1, 1.0, 0, 0)) == 1004
    assert code(lambda: be.launch_index_topk(0, 0, 5, 0)) == 1001
    assert code(lambda: be.launch_index_score(0, 0, 0, None, 4, 4, 8, 128, 1.0, 1.0, 0)) == 1001
    assert code(lambda: be.launch_index_append(0, 0, -1, 128)) == 1001
    assert code(lambda: be.launch_gather_rope(0, 0, 0, 1, 0, 1)) == 1001
    e = None
    try:
        be.launch_append_kv(0, 0, 0, 0, 0, 0, 160, 64, 2)
    except be.BackendError as ex:
        e = ex
    assert str(e) == "append_kv: argument guard rejected (1002)"
    assert be.attend_scratch_floats(64, 512) == 16 * 64 * 514


def test_page_pool_matches_oracle_under_churn(be):
    """Continuous-batching churn: 10 % of sequences finish and are replaced each step;
    page tables and free lists stay bit-identical to the oracle's allocator."""
    rng = np.random.RandomState(4)
    B, P, max_pages = 32, 64, 40
    n_pages = 900
    a = be.PagePool(n_pages, B, max_pages, P)
    o = orc.Pool(n_pages, B, max_pages, P)
    a.shuffle(99); o.shuffle(99)
    lens = rng.randint(64, 2000, B)
    for b in range(B):
        a.reserve(b, int(lens[b])); assert o.reserve(b, int(lens[b])) == 0
    for step in range(40):
        for b in rng.choice(B, 3, replace=False):
            a.release(int(b)); o.release(int(b))
            lens[b] = rng.randint(64, 2000)
            a.reserve(int(b), int(lens[b])); assert o.reserve(int(b), int(lens[b])) == 0
        lens += 1
        for b in range(B):
            a.reserve(b, int(lens[b])); assert o.reserve(b, int(lens[b])) == 0
        np.testing.assert_array_equal(a.block_table(), o.block_table())
        np.testing.assert_array_equal(a.free_list(), o.free_list())
    live = a.block_table()[a.block_table() >= 0]
    assert len(set(live.tolist())) == live.size                      # no page mapped twice
    assert live.size + a.n_free == n_pages


def test_page_pool_error_codes(be):
    a = be.PagePool(4, 2, 3, 16)
    a.reserve(0, 48)
    with pytest.raises(be.BackendError) as e:
        a.reserve(0, 49)                                             # row full
    assert e.value.code == 1002
    with pytest.raises(be.BackendError) as e:
        a.reserve(1, 32)                                             # only 1 page left
    assert e.value.code == 1007
    assert a.n_free == 1 and a.seq_pages(1) == 0                     # nothing was mapped
    with pytest.raises(be.BackendError) as e:
        a.reserve(5, 1)
    assert e.value.code == 1001
    a.release(0)
    assert a.n_free == 4 and (a.block_table() == -1).all()
    assert a.free_list().tolist() == [3, 0, 1, 2]                    # LIFO: logical page 0 pushed first
