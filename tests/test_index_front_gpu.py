"""Indexer front end (fp8 GEMV, LayerNorm, interleaved RoPE, and their batched composition) against
the oracle: reference-layout operators on the reference's fixtures, the batched form at the model
geometry within bf16 rounding."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import bf16_normal

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
    return torch.from_numpy(a).cuda()


@pytest.mark.parametrize("seed,o_dim,i_dim,block", [(0x6E37, 130, 256, 128), (0x6E38, 64, 96, 32), (0x6E39, 7, 37, 4), (0x6E3A, 48, 4224, 128)])
def test_gemv_fp8_is_bit_exact_and_rows_are_independent(be, seed, o_dim, i_dim, block):
    r = orc.Lcg(seed)
    packed = orc.f32_to_e4m3(r.draws(o_dim * i_dim))
    scale = (np.abs(r.draws((-(-o_dim // block)) * (-(-i_dim // block))) * np.float32(0.1)) + np.float32(0.01)).astype(np.float32)
    xs = [r.draws(i_dim), r.draws(i_dim)]
    y2 = torch.zeros(2 * o_dim, dtype=torch.float32, device="cuda")
    be.launch_gemv_fp8(dev(np.concatenate(xs)), dev(packed), dev(scale), o_dim, i_dim, block, 2, y2)
    be.device_sync()
    for i in range(2):
        want = orc.gemv_fp8(xs[i], packed, scale, o_dim, i_dim, block)[0]
        np.testing.assert_array_equal(y2[i * o_dim:(i + 1) * o_dim].cpu().numpy().view(np.uint32), want.view(np.uint32))
    x = torch.zeros(8192, dtype=torch.float32, device="cuda")
    for args, code in (((0, 4, 4, 1), 1001), ((4, 4, 96, 1), 1003), ((4, 4, 4, 3), 1004)):
        with pytest.raises(be.BackendError) as e:
            be.launch_gemv_fp8(x, dev(packed), dev(scale), *args, x)
        assert e.value.code == code


def test_layernorm_and_rope_on_the_reference_fixtures(be):
    n = 1024
    r = orc.Lcg(0x1AE6)
    x = (r.draws(n) + np.float32(1.5)).astype(np.float32)
    w = (r.draws(n) + np.float32(1.0)).astype(np.float32)
    b = (r.draws(n) * np.float32(0.25)).astype(np.float32)
    y = torch.zeros(n, dtype=torch.float32, device="cuda")
    be.launch_layernorm(dev(x), dev(w), dev(b), n, 1e-6, y)
    be.device_sync()
    want = orc.layernorm(x, w, b, 1e-6)
    assert float(np.abs(y.cpu().numpy() - want).max() / np.abs(want).max()) <= 1e-4       # the reference's tolerance
    count, stride, seg, theta = 5, 24, 16, 10000.0
    base = orc.Lcg(0x2909).draws(count * stride)
    for pos, exact in ((0, True), (137, False)):
        v = dev(base.copy())
        be.launch_rope_interleave(v, count, stride, seg, pos, theta)
        be.device_sync()
        want = orc.rope_interleave(base, count, stride, seg, pos, theta)
        if exact:                                         # position 0 is a pure de-interleave permutation
            np.testing.assert_array_equal(v.cpu().numpy().view(np.uint32), want.view(np.uint32))
        else:
            assert float(np.abs(v.cpu().numpy() - want).max() / np.abs(want).max()) <= 1e-6
    for args in ((0, 24, 16), (5, 24, 15), (5, 8, 16)):
        with pytest.raises(be.BackendError) as e:
            be.launch_rope_interleave(dev(base.copy()), *args, 3, theta)
        assert e.value.code == 1001


def _front_weights(seed, hidden, q_lora, nh, hd, block):
    rng = np.random.RandomState(seed)
    def mat(n, k):
        packed = orc.f32_to_e4m3((rng.standard_normal(n * k) * 0.7).astype(np.float32))
        scale = (np.abs(rng.standard_normal((-(-n // block)) * (-(-k // block)))) * 0.01 + 0.004).astype(np.float32)
        return packed, scale
    wk, wk_s = mat(hd, hidden)
    wq, wq_s = mat(nh * hd, q_lora)
    wp, wp_s = mat(nh, hidden)
    kn_w = (rng.standard_normal(hd) * 0.1 + 1.0).astype(np.float32)
    kn_b = (rng.standard_normal(hd) * 0.05).astype(np.float32)
    return dict(wk=wk, wk_scale=wk_s, knorm_w=kn_w, knorm_b=kn_b, wq_b=wq, wq_b_scale=wq_s, wproj=wp, wproj_scale=wp_s), rng


@pytest.mark.parametrize("B,hidden,q_lora,nh,hd", [(128, 6144, 2048, 32, 128), (5, 512, 256, 8, 64)])
def test_batched_front_end_matches_oracle(be, B, hidden, q_lora, nh, hd):
    from rivoli_b200.layer import IndexerFrontEnd
    block, rope_off, rope_seg, theta, eps = 128, 0, 64, 10000.0, 1e-6
    W, rng = _front_weights(9 + B, hidden, q_lora, nh, hd, block)
    x = bf16_normal(rng, (B, hidden))
    qr = bf16_normal(rng, (B, q_lora))
    pos = rng.randint(0, 100000, B).astype(np.int32)
    key, q, w, k32, q32 = orc.index_frontend_bf16(x, qr, pos, nh, hd, rope_off, rope_seg, theta, eps, block, W["wk"], W["wk_scale"],
                                                  W["knorm_w"], W["knorm_b"], W["wq_b"], W["wq_b_scale"], W["wproj"], W["wproj_scale"])
    fg = be.IndexFrontGeom(hidden, q_lora, nh, hd, rope_off, rope_seg, block, eps, theta)
    fe = IndexerFrontEnd(fg, B, {k: dev(v) for k, v in W.items()})
    for simt in (False, True):
        gk, gq, gw = fe.run(dev(x), dev(qr), dev(pos), force_simt=simt)
        be.index_frontend_status()
        _check_front(gk, gq, gw, k32, q32, w)
    assert gk.shape == (B, hd) and gq.shape == (B, nh, hd) and gw.shape == (B, nh)


def _check_front(gk, gq, gw, k32, q32, w):
    # split-K sums (and, on the tensor cores, weights rounded to bf16 after scaling) differ from the oracle's
    # single f32 fold in the low bits; one bf16 rounding on top
    for got, want in ((orc.bf16_to_f32(gk.cpu().view(torch.int16).numpy().view(np.uint16)), k32),
                      (orc.bf16_to_f32(gq.cpu().view(torch.int16).numpy().view(np.uint16)), q32),
                      (gw.cpu().numpy(), w)):
        err = np.abs(got.astype(np.float64) - want)
        tol = 2.0 ** -7 * np.abs(want) + 2e-3 * np.abs(want).max()
        assert (err <= tol).all(), float((err / tol).max())
