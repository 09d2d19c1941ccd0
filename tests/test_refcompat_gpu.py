"""The reference-signature operators against the oracle, on the reference's own fixtures
(crates/engine/tests/{fwd_kernel,indexer_kernel,kernel_vector,kernel_attend}.rs)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from rivoli_b200 import backend
    backend.lib()
    return backend


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def zeros(n, dtype):
    return torch.zeros(n, dtype=dtype, device="cuda")


def guard(be, fn, code):
    with pytest.raises(be.BackendError) as e:
        fn()
    assert str(code) in str(e.value) and e.value.code == code


# fwd_kernel.rs:140-214
def test_append_kv_quantizes_one_row_and_leaves_the_slab_alone(be):
    rows, kvl, ropn, pos = 5, 256, 64, 3
    r = orc.Lcg(0xA99E)
    latent = np.array([r.f() * (1.0 if i < 128 else 20.0) for i in range(kvl)], dtype=np.float32)
    rope = r.draws(ropn)
    want_lc8 = np.zeros(rows * kvl, np.uint8); want_ls = np.zeros(rows * 2, np.float32)
    want_rc = np.zeros(rows * ropn, np.uint16)
    orc.append_kv(latent, rope, want_lc8, want_ls, want_rc, pos, kvl, ropn, 2)
    c8, ls, rc = zeros(rows * kvl, torch.uint8), zeros(rows * 2, torch.float32), zeros(rows * ropn, torch.int16)
    be.launch_append_kv(dev(latent), dev(rope), c8, ls, rc, pos, kvl, ropn, 2)
    be.device_sync()
    assert (want_lc8[pos * kvl:(pos + 1) * kvl] != 0).sum() > kvl // 2
    np.testing.assert_array_equal(c8.cpu().numpy(), want_lc8)
    np.testing.assert_array_equal(ls.cpu().numpy().view(np.uint32), want_ls.view(np.uint32))
    np.testing.assert_array_equal(rc.cpu().numpy().view(np.uint16), want_rc)


def test_append_kv_guards(be):
    b = zeros(4096, torch.float32)
    guard(be, lambda: be.launch_append_kv(b, b, b, b, b, -1, 256, 64, 2), 1001)
    guard(be, lambda: be.launch_append_kv(b, b, b, b, b, 0, 160, 64, 2), 1002)
    guard(be, lambda: be.launch_append_kv(b, b, b, b, b, 0, 2048, 64, 2), 1002)
    guard(be, lambda: be.launch_append_kv(b, b, b, b, b, 0, 128, 256, 1), 1002)


# Dense sweep of the e4m3 encoder through append_kv with scale exactly 1 (one element = 448):
# every subnormal tie, every normal tie and their f32 neighbours, saturation and zero edges.
def test_e4m3_encoder_bit_exact_on_ties_and_neighbours(be):
    L = orc.lib()
    vals = []
    for c in range(0x00, 0x7F):
        a, b2 = L.orc_e4m3_to_f32(c), L.orc_e4m3_to_f32(c + 1) if c + 1 < 0x7F else 480.0
        mid = np.float32((a + b2) / 2)
        for x in (a, mid, np.nextafter(mid, np.float32(0)), np.nextafter(mid, np.float32(1000)),
                  np.nextafter(np.float32(a), np.float32(1000))):
            vals += [x, -x]
    vals += [2.0 ** -10, np.nextafter(np.float32(2.0 ** -10), np.float32(0)), 2.0 ** -11, 0.0, -0.0, 447.9, 448.0,
             0.4999999 * 2.0 ** -9, 7.5 * 2.0 ** -9, 7.4999995 * 2.0 ** -9]
    rng = np.random.RandomState(5)
    vals += list(np.exp(rng.uniform(np.log(1e-4), np.log(448), 4000)) * rng.choice([-1, 1], 4000))
    vals = np.array(vals, np.float32)
    vals = vals[np.abs(vals) <= 448]
    n = (len(vals) + 126) // 127
    pad = np.zeros(n * 127, np.float32); pad[:len(vals)] = vals
    lat = np.zeros((n, 128), np.float32); lat[:, :127] = pad.reshape(n, 127); lat[:, 127] = 448.0
    c8, ls, rc = zeros(n * 128, torch.uint8), zeros(n, torch.float32), zeros(n * 8, torch.int16)
    latd, roped = dev(lat), zeros(8, torch.float32)
    for i in range(n):
        be.launch_append_kv(latd[i], roped, c8, ls, rc, i, 128, 8, 1)
    be.device_sync()
    got = c8.cpu().numpy().reshape(n, 128)[:, :127].ravel()[:len(vals)]
    want = orc.f32_to_e4m3(vals)
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, [(float(vals[i]), hex(got[i]), hex(want[i])) for i in bad[:8]]
    assert (ls.cpu().numpy() == 1.0).all()


# fwd_kernel.rs:94-125
def test_gather_rope(be):
    h, qh, nope, ropn = 8, 192, 96, 64
    q = orc.Lcg(0x60A7).draws(h * qh)
    out = zeros(h * ropn, torch.float32)
    be.launch_gather_rope(dev(q), out, h, qh, nope, ropn)
    be.device_sync()
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), orc.gather_rope(q, h, qh, nope, ropn).view(np.uint32))


# indexer_kernel.rs:120-140
def test_index_append_stores_one_bf16_key_row(be):
    rows, hd, pos = 7, 128, 5
    k = orc.Lcg(0xC0DE).draws(hd) * np.float32(8.0)
    want = np.zeros(rows * hd, np.uint16); orc.index_append(k, want, pos, hd)
    cb = zeros(rows * hd, torch.int16)
    be.launch_index_append(dev(k), cb, pos, hd)
    be.device_sync()
    np.testing.assert_array_equal(cb.cpu().numpy().view(np.uint16), want)


# indexer_kernel.rs:214-367
def test_index_score_reduces_over_the_active_heads_only(be):
    nt, nh, hd = 64, 64, 128
    r = orc.Lcg(0x5C04)
    q = r.draws(nh * hd); w = r.draws(nh); kc = orc.f32_to_bf16(r.draws(nt * hd))
    want_all = orc.index_score(q, w, kc, None, nt, nh, nh, hd, 0.75, 0.125)
    sub = np.array([5, 0, 6, 2], np.uint32)
    want_sub = orc.index_score(q, w, kc, sub, nt, nh, 4, hd, 0.75, 0.125)
    qd, wd, kd = dev(q), dev(w), dev(kc.view(np.int16))
    sb = zeros(nt, torch.float32)
    be.launch_index_score(qd, wd, kd, None, nt, nh, nh, hd, 0.75, 0.125, sb)
    be.device_sync()
    got = sb.cpu().numpy()
    assert np.abs(got - want_all).max() <= 1e-5 * np.abs(want_all).max()
    be.launch_index_score(qd, wd, kd, dev(sub.view(np.int32)), nt, nh, 4, hd, 0.75, 0.125, sb)
    be.device_sync()
    got = sb.cpu().numpy()
    assert np.abs(got - want_sub).max() <= 1e-5 * np.abs(want_sub).max()
    guard(be, lambda: be.launch_index_score(qd, wd, kd, None, nt, 4, 8, hd, 0.75, 0.125, sb), 1001)
    guard(be, lambda: be.launch_index_score(qd, wd, kd, None, 0, nh, nh, hd, 0.75, 0.125, sb), 1001)


def _topk_cases():
    from tests.test_oracle_kats import _topk_cases as c
    return c()


# kernel_vector.rs:124-212
@pytest.mark.parametrize("name,scores,k", _topk_cases(), ids=[c[0] for c in _topk_cases()])
def test_index_topk_matches_host_selection(be, name, scores, k):
    n = scores.size
    want = orc.index_topk(scores, k)
    written = min(k, n)
    rb = torch.full((max(n, k),), -1, dtype=torch.int32, device="cuda")     # 0xFFFFFFFF sentinel
    be.launch_index_topk(dev(scores), n, k, rb)
    be.device_sync()
    got = rb.cpu().numpy().view(np.uint32)
    assert want.size == written
    np.testing.assert_array_equal(got[:written], want)
    assert (got[written:] == 0xFFFFFFFF).all(), "wrote past min(k, nt)"
    assert (np.diff(got[:written].astype(np.int64)) > 0).all()


def test_index_topk_guards(be):
    b = zeros(16, torch.float32)
    guard(be, lambda: be.launch_index_topk(b, 0, 4, b), 1001)
    guard(be, lambda: be.launch_index_topk(b, 16, 0, b), 1001)


def _attend_case(be, seed, H, nt, kvl, rope, rows=None):
    nb = kvl // 128
    r = orc.Lcg(seed)
    qabs = r.draws(H * kvl); qrope = r.draws(H * rope)
    lc8 = orc.f32_to_e4m3(r.draws(nt * kvl))
    lscale = np.abs(r.draws(nt * nb) * np.float32(0.1)) + np.float32(0.01)
    rc = orc.f32_to_bf16(r.draws(nt * rope))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(kvl + rope)))
    nr = nt if rows is None else len(rows)
    want = orc.mla_attend(qabs, qrope, lc8, lscale, rc, rows, H, nr, kvl, rope, nb, scale)
    clat = zeros(H * kvl, torch.float32)
    part = zeros(be.attend_scratch_floats(H, kvl), torch.float32)
    rd = None if rows is None else dev(np.asarray(rows, np.uint32).view(np.int32))
    be.launch_attend(dev(qabs), dev(qrope), dev(lc8), dev(lscale), dev(rc.view(np.int16)), rd, H, nr, kvl,
                     rope, nb, scale, clat, part)
    be.device_sync()
    got = clat.cpu().numpy()
    tol = 1e-3 * np.abs(want).max() + 1e-3            # common/scoring.rs:191-194
    assert np.abs(got - want).max() <= tol, (np.abs(got - want).max(), tol)
    # single-split path (no scratch) must agree too
    be.launch_attend(dev(qabs), dev(qrope), dev(lc8), dev(lscale), dev(rc.view(np.int16)), rd, H, nr, kvl,
                     rope, nb, scale, clat, None)
    be.device_sync()
    assert np.abs(clat.cpu().numpy() - want).max() <= tol


# kernel_attend.rs:269-304
@pytest.mark.parametrize("seed,H,nt,kvl,rope", [(0x0A5E1102, 64, 300, 512, 64), (0x5F117BAD, 64, 704, 512, 64),
                                                 (0xC1A39ED0, 64, 4608, 512, 64), (0x00C0FFEE, 4, 1, 128, 8),
                                                 (0xB10CC0DE, 20, 130, 512, 64)])
def test_mla_attend_dense(be, seed, H, nt, kvl, rope):
    _attend_case(be, seed, H, nt, kvl, rope)


# The reference has no test of the rows != null arm (its every launch_attend passes null).
def test_mla_attend_sparse_rows(be):
    rng = np.random.RandomState(3)
    rows = np.sort(rng.choice(704, 200, replace=False)).astype(np.uint32)
    _attend_case(be, 0x5F117BAD, 64, 704, 512, 64, rows=rows)


# kernel_attend.rs:165-189
def test_mla_attend_rejects_unsupported_kvl(be):
    b = zeros(8 * 1024, torch.float32)
    sc = zeros(be.attend_scratch_floats(8, 512), torch.float32)
    be.launch_attend(b, b, b, b, b, None, 8, 16, 512, 64, 4, 1.0, b, sc)
    guard(be, lambda: be.launch_attend(b, b, b, b, b, None, 8, 16, 640, 64, 5, 1.0, b, sc), 1004)
    guard(be, lambda: be.launch_attend(b, b, b, b, b, None, 8, 16, 160, 64, 1, 1.0, b, sc), 1004)
    guard(be, lambda: be.launch_attend(b, b, b, b, b, None, 0, 16, 512, 64, 4, 1.0, b, sc), 1001)
    be.device_sync()
    assert be.attend_scratch_floats(64, 512) == 16 * 64 * 514


def test_mla_attend_takes_more_heads_than_one_block_holds(be):
    """Any head count: 160 heads of width 512 + 64 do not fit one block's shared memory and are tiled over the
    grid (the reference tiles heads in blocks of 16, crates/backend/kernels/attn.hip:119-130)."""
    _attend_case(be, 0x0A5E1102, 160, 300, 512, 64)
    _attend_case(be, 0x5F117BAD, 200, 90, 128, 16)
