"""kv_b projections either side of attention (absorb / value) against the oracle.

* reference-layout f32 operators on the reference's six seeded shapes: bit-exact (same fold);
* the two-row launch equals two one-row launches bit for bit (the reference's own claim);
* guards (the reference's codes);
* the batched bf16 form at the model geometry (64 heads, nope 192, vh 256, kvl 512, rope 64,
  128-blocks): tensor-core kernel within bf16 rounding of the oracle's f32 fold, CUDA-core
  kernel bit-exact, rope segment copied bit for bit, ragged batch sizes.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import bf16_normal
from tests.test_oracle_kats import MLA_SHAPES

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


@pytest.mark.parametrize("seed,dims", MLA_SHAPES)
def test_reference_layout_operators_are_bit_exact(be, seed, dims):
    h, qh, nope, vh, kvl, block = dims
    r = orc.Lcg(seed)
    packed, scale = orc.kvb_fixture(r, h * (nope + vh), kvl, block)
    q, clat = r.draws(h * qh), r.draws(h * kvl)
    qabs = torch.zeros(h * kvl, dtype=torch.float32, device="cuda")
    be.launch_mla_absorb(dev(q), dev(packed), dev(scale), h, qh, nope, vh, kvl, block, 1, qabs)
    be.device_sync()
    want = orc.mla_absorb_fp8(q, packed, scale, h, qh, nope, vh, kvl, block)[0]
    np.testing.assert_array_equal(qabs.cpu().numpy().view(np.uint32), want.view(np.uint32))
    if kvl % 4 == 0:
        ctx = torch.zeros(h * vh, dtype=torch.float32, device="cuda")
        be.launch_mla_value(dev(clat), dev(packed), dev(scale), h, nope, vh, kvl, block, 1, ctx)
        be.device_sync()
        want = orc.mla_value_fp8(clat, packed, scale, h, nope, vh, kvl, block)[0]
        np.testing.assert_array_equal(ctx.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_two_rows_equal_single_rows_and_guards(be):
    h, qh, nope, vh, kvl, block = 3, 20, 12, 8, 16, 4
    r = orc.Lcg(0xBA7C)
    packed, scale = orc.kvb_fixture(r, h * (nope + vh), kvl, block)
    qs = [r.draws(h * qh) for _ in range(2)]
    cs = [r.draws(h * kvl) for _ in range(2)]
    kb, sb = dev(packed), dev(scale)
    a2 = torch.zeros(2 * h * kvl, dtype=torch.float32, device="cuda")
    v2 = torch.zeros(2 * h * vh, dtype=torch.float32, device="cuda")
    be.launch_mla_absorb(dev(np.concatenate(qs)), kb, sb, h, qh, nope, vh, kvl, block, 2, a2)
    be.launch_mla_value(dev(np.concatenate(cs)), kb, sb, h, nope, vh, kvl, block, 2, v2)
    for i in range(2):
        a1 = torch.zeros(h * kvl, dtype=torch.float32, device="cuda")
        v1 = torch.zeros(h * vh, dtype=torch.float32, device="cuda")
        be.launch_mla_absorb(dev(qs[i]), kb, sb, h, qh, nope, vh, kvl, block, 1, a1)
        be.launch_mla_value(dev(cs[i]), kb, sb, h, nope, vh, kvl, block, 1, v1)
        be.device_sync()
        assert torch.equal(a2[i * h * kvl:(i + 1) * h * kvl], a1)
        assert torch.equal(v2[i * h * vh:(i + 1) * h * vh], v1)
    # guards: the reference's codes (kernel_attend.rs:134-160, mla.hip:192-231)
    x = torch.zeros(4096, dtype=torch.float32, device="cuda")
    for kvl2, want in ((64, None), (37, 1002), (66, 1002)):
        if want is None:
            be.launch_mla_value(x, kb, sb, 2, 8, 4, kvl2, 128, 1, x)
        else:
            with pytest.raises(be.BackendError) as e:
                be.launch_mla_value(x, kb, sb, 2, 8, 4, kvl2, 128, 1, x)
            assert e.value.code == want
        be.launch_mla_absorb(x, kb, sb, 2, 32, 8, 4, kvl2, 128, 1, x)       # absorb accepts ragged kvl
    for args, code in (((2, 32, 8, 4, 64, 96, 1), 1003), ((2, 32, 8, 4, 64, 128, 3), 1004), ((0, 32, 8, 4, 64, 128, 1), 1001)):
        with pytest.raises(be.BackendError) as e:
            be.launch_mla_absorb(x, kb, sb, *args, x)
        assert e.value.code == code
    be.device_sync()


GLM = dict(H=64, qh=256, nope=192, vh=256, kvl=512, rope=64, block=128)


def _glm_weights(seed):
    g = GLM
    rng = np.random.RandomState(seed)
    rows = g["H"] * (g["nope"] + g["vh"])
    packed = orc.f32_to_e4m3((rng.standard_normal(rows * g["kvl"]) * 0.7).astype(np.float32))
    scale = (np.abs(rng.standard_normal((rows // 128) * (g["kvl"] // 128))) * 0.01 + 0.002).astype(np.float32)
    return packed, scale, rng


@pytest.mark.parametrize("B", [128, 5, 200])
def test_batched_absorb_and_value_at_model_geometry(be, B):
    g = GLM
    packed, scale, rng = _glm_weights(17 + B)
    q = bf16_normal(rng, (B, g["H"], g["qh"]))
    clat = bf16_normal(rng, (B, g["H"], g["kvl"]))
    want_q, want_q32 = orc.mla_absorb_batched_bf16(q, packed, scale, g["H"], g["qh"], g["nope"], g["vh"], g["kvl"], g["rope"], g["block"])
    want_c, want_c32 = orc.mla_value_batched_bf16(clat, packed, scale, g["H"], g["nope"], g["vh"], g["kvl"], g["block"])
    kb, sb = dev(packed), dev(scale)
    for simt in (False, True):
        q_abs = torch.zeros((B, g["H"], g["kvl"] + g["rope"]), dtype=torch.bfloat16, device="cuda")
        ctx = torch.zeros((B, g["H"], g["vh"]), dtype=torch.bfloat16, device="cuda")
        be.launch_mla_absorb_batched_bf16(dev(q), kb, sb, g["H"], g["qh"], g["nope"], g["vh"], g["kvl"], g["rope"],
                                          g["block"], B, q_abs, force_simt=simt)
        be.launch_mla_value_batched_bf16(dev(clat), kb, sb, g["H"], g["nope"], g["vh"], g["kvl"], g["block"], B, ctx,
                                         force_simt=simt)
        be.kvb_proj_status()
        gq = q_abs.cpu().view(torch.int16).numpy().view(np.uint16)
        gc = ctx.cpu().view(torch.int16).numpy().view(np.uint16)
        np.testing.assert_array_equal(gq[:, :, g["kvl"]:], q[:, :, g["nope"]:g["nope"] + g["rope"]])   # rope rides along
        if simt:                                    # same fold as the oracle: bit-exact
            np.testing.assert_array_equal(gq, want_q)
            np.testing.assert_array_equal(gc, want_c)
        else:                                       # exact products, f32 sums in another order, one bf16 rounding
            for got, want in ((gq[:, :, :g["kvl"]], want_q32), (gc, want_c32)):
                err = np.abs(orc.bf16_to_f32(got).astype(np.float64) - want)
                tol = 2.0 ** -8 * np.abs(want) + 1e-3 * np.abs(want).max()
                assert (err <= tol).all(), float((err / tol).max())
