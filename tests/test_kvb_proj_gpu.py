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


def test_absorb_step_value_chain_matches_oracle(be):
    """A whole attention block of a decode layer: per-head q -> absorb -> (append, select, attend)
    -> value, every stage checked against the oracle fed with the oracle's own previous stage."""
    from rivoli_b200.layer import DsaDecodeLayer, KvbProjection
    from tests.helpers import State, attend_close_ref, make_geom
    g0 = GLM
    st = State(31, 4, [700, 2100, 64, 300], top_k=256)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    packed, scale, rng = _glm_weights(5)
    B = st.B
    q_heads = bf16_normal(rng, (B, g0["H"], g0["qh"]))
    layer = DsaDecodeLayer(g, B, max_ctx=int(g.max_pages_per_seq * g.page_tokens))
    layer.latent_pool.copy_(dev(st.latent_pool)); layer.latent_scale.copy_(dev(st.latent_scale))
    layer.index_pool.copy_(dev(st.index_pool)); layer.index_scale.copy_(dev(st.index_scale))
    layer.upload_block_table(st.block_table)
    proj = KvbProjection(g, B, dev(packed), dev(scale), g0["nope"], g0["vh"])
    q_abs = proj.absorb(dev(q_heads))
    out = layer.step(dev(st.new_latent), dev(st.new_key), dev(st.index_q), dev(st.index_w), q_abs, dev(st.row_pos), dev(st.seq_len))
    ctx = proj.value(out)
    be.device_sync(); layer.check_status(); be.kvb_proj_status()
    # oracle chain
    want_q, _ = orc.mla_absorb_batched_bf16(q_heads, packed, scale, g0["H"], g0["qh"], g0["nope"], g0["vh"], g0["kvl"], g0["rope"], g0["block"])
    got_q = q_abs.cpu().view(torch.int16).numpy().view(np.uint16)
    dq = np.abs(orc.bf16_to_f32(got_q).astype(np.float64) - orc.bf16_to_f32(want_q))
    assert (dq <= 2.0 ** -7 * np.abs(orc.bf16_to_f32(want_q)) + 1e-3 * np.abs(orc.bf16_to_f32(want_q)).max()).all()
    st.q = got_q                                   # the oracle attends with the GPU's absorbed q: stage-wise check
    want = st.oracle_step()
    np.testing.assert_array_equal(layer.n_sel.cpu().numpy(), want["n_sel"])
    ok, worst, rms = attend_close_ref(out.cpu().view(torch.int16).numpy().view(np.uint16), want["out_f32"])
    assert ok and rms <= 1e-2, (worst, rms)
    got_out = out.cpu().view(torch.int16).numpy().view(np.uint16)
    _, want_c32 = orc.mla_value_batched_bf16(got_out, packed, scale, g0["H"], g0["nope"], g0["vh"], g0["kvl"], g0["block"])
    got_c = orc.bf16_to_f32(ctx.cpu().view(torch.int16).numpy().view(np.uint16)).astype(np.float64)
    err = np.abs(got_c - want_c32)
    assert (err <= 2.0 ** -8 * np.abs(want_c32) + 1e-3 * np.abs(want_c32).max()).all(), float(err.max())


def test_absorb_then_dense_attend_back_to_back_on_one_stream(be):
    """q produced by the kernel launched immediately before the attention call (no other launch in between):
    the attention kernel is a programmatic dependent of the absorb kernel and must not read q before that kernel
    has completed. Repeated with fresh q so that a stale read would show."""
    from rivoli_b200.layer import DsaDecodeLayer, KvbProjection
    from tests.helpers import State, attend_close, make_geom
    g0 = GLM
    st = State(33, 3, [1500, 400, 129], top_k=256)
    g = make_geom(be.DsaGeom, **st.geom_kw)
    packed, scale, rng = _glm_weights(6)
    B = st.B
    want0 = st.oracle_step()                       # caches after the append
    layer = DsaDecodeLayer(g, B, max_ctx=int(g.max_pages_per_seq * g.page_tokens))
    layer.latent_pool.copy_(dev(want0["latent_pool"])); layer.latent_scale.copy_(dev(want0["latent_scale"]))
    layer.upload_block_table(st.block_table)
    proj = KvbProjection(g, B, dev(packed), dev(scale), g0["nope"], g0["vh"])
    d_len = dev(st.seq_len)
    stream = torch.cuda.Stream()
    for rep in range(3):
        q_heads = bf16_normal(rng, (B, g0["H"], g0["qh"]))
        dq = dev(q_heads)
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            q_abs = proj.absorb(dq, stream=stream)
            out = layer.attend(q_abs, stream=stream, dense_len=d_len)
        stream.synchronize()
        layer.check_status(); be.kvb_proj_status()
        got_q = q_abs.cpu().view(torch.int16).numpy().view(np.uint16)
        _, o_f32, _, _ = orc.mla_attend_paged(st.og, got_q, want0["latent_pool"], want0["latent_scale"], st.block_table,
                                              None, st.seq_len, want_f32=True)
        ok, worst = attend_close(out.cpu().view(torch.int16).numpy().view(np.uint16), o_f32)
        assert ok, (rep, worst)
