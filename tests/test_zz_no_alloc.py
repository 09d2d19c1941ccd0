"""The allocation-free attention entry point against the ordinary one.

Some hosts of this library may not call cudaMalloc (all device memory already belongs to
their own arenas, or their decode thread must never wait on the allocator), so
``rivoli_mla_attend_static`` keeps the split-KV partials in an array compiled into the
library instead of taking scratch from the caller. This file checks, through the C ABI, that
it returns what ``rivoli_mla_attend`` returns with caller scratch - on two calls in a row with
different inputs, because the built-in array keeps the previous call's partials - and that
shapes beyond the built-in array are refused. Named so that pytest collects it last.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(a).cuda()


def _case(seed, H, nt, kvl, rope):
    nb = kvl // 128
    r = orc.Lcg(seed)
    qabs, qrope = r.draws(H * kvl), r.draws(H * rope)
    lc8 = orc.f32_to_e4m3(r.draws(nt * kvl))
    lscale = np.abs(r.draws(nt * nb) * np.float32(0.1)) + np.float32(0.01)
    rc = orc.f32_to_bf16(r.draws(nt * rope))
    scale = float(np.float32(1.0) / np.sqrt(np.float32(kvl + rope)))
    return dict(qabs=dev(qabs), qrope=dev(qrope), lc8=dev(lc8), lscale=dev(lscale), rc=dev(rc), H=H, nt=nt,
                kvl=kvl, rope=rope, nb=nb, scale=scale)


def test_static_scratch_attend_matches_caller_scratch_attend():
    from rivoli_b200 import backend as be
    be.lib()
    # two calls in a row: many splits first, then fewer splits with other data, so stale partials
    # of the first call sit in the built-in array while the second runs
    for seed, H, nt in ((0xC1A39ED0, 64, 4608), (0x5F117BAD, 64, 704), (0xB10CC0DE, 20, 130)):
        c = _case(seed, H, nt, 512, 64)
        want = torch.zeros(H * 512, dtype=torch.float32, device="cuda")
        part = torch.zeros(be.attend_scratch_floats(H, 512), dtype=torch.float32, device="cuda")
        be.launch_attend(c["qabs"], c["qrope"], c["lc8"], c["lscale"], c["rc"], None, H, nt, 512, 64, c["nb"],
                         c["scale"], want, part)
        be.device_sync()
        got = torch.full((H * 512,), float("nan"), dtype=torch.float32, device="cuda")
        be.launch_attend_static(c["qabs"], c["qrope"], c["lc8"], c["lscale"], c["rc"], None, H, nt, 512, 64,
                                c["nb"], c["scale"], got)
        be.device_sync()
        w, g = want.cpu().numpy(), got.cpu().numpy()
        tol = 1e-3 * np.abs(w).max() + 1e-3          # the attention tolerance of the other tests
        assert np.isfinite(g).all()
        assert np.abs(g - w).max() <= tol
        # and both agree with the oracle
        ref = orc.mla_attend(c["qabs"].cpu().numpy(), c["qrope"].cpu().numpy(), c["lc8"].cpu().numpy(),
                             c["lscale"].cpu().numpy(), c["rc"].cpu().numpy().view(np.uint16), None, H, nt, 512, 64,
                             c["nb"], c["scale"])
        assert np.abs(g - ref).max() <= 1e-3 * np.abs(ref).max() + 1e-3


def test_static_scratch_attend_refuses_what_does_not_fit():
    from rivoli_b200 import backend as be
    b = torch.zeros(1 << 16, dtype=torch.float32, device="cuda")
    for args, code in (((128, 16, 512, 64, 4), 1002),      # more heads than the built-in array holds
                       ((8, 16, 640, 64, 5), 1004),        # same width rule as rivoli_mla_attend
                       ((8, 0, 512, 64, 4), 1001)):
        H, nr, kvl, rope, nb = args
        with pytest.raises(be.BackendError) as e:
            be.launch_attend_static(b, b, b, b, b, None, H, nr, kvl, rope, nb, 1.0, b)
        assert e.value.code == code
    be.device_sync()
