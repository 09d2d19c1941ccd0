"""Seeded synthetic inputs for the V4 cousin path (test and benchmark infrastructure, never imported
by the product package). Values follow the dtypes the reference's path carries: everything bf16-valued,
the indexer's q and compressed rows already through the Hadamard + fp4 spread."""
from __future__ import annotations

import numpy as np

from . import oracle as orc


def make_geom(**kw) -> orc.V4Geom:
    d = dict(n_heads=64, head_dim=512, window=128, index_heads=64, index_dim=128, index_topk=512, ratio=4,
             max_comp=2048)
    d.update(kw)
    if "softmax_scale" not in d:
        d["softmax_scale"] = float(np.float32(d["head_dim"]) ** np.float32(-0.5))
    return orc.V4Geom(**d)


def _bf16(rng, shape, scale=1.0) -> np.ndarray:
    return orc.f32_to_bf16((rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)))


def make_inputs(g: orc.V4Geom, n_seqs: int, pos, seed: int = 0) -> dict:
    """pos: int array [n_seqs] (query positions). Returns numpy arrays in storage dtypes."""
    rng = np.random.default_rng(seed)
    pos = np.asarray(pos, np.int32)
    kv_rows = g.window + g.max_comp
    spread = lambda u16, d: orc.f32_to_bf16(orc.v4_spread(orc.bf16_to_f32(u16).reshape(-1, d), d)[1]).reshape(u16.shape)
    return dict(
        pos=pos,
        q=_bf16(rng, (n_seqs, g.n_heads, g.head_dim)),
        kv_cache=_bf16(rng, (n_seqs, kv_rows, g.head_dim)),
        sink=rng.standard_normal(g.n_heads).astype(np.float32),
        iq=spread(_bf16(rng, (n_seqs, g.index_heads, g.index_dim)), g.index_dim),
        iw=orc.bf16_to_f32(_bf16(rng, (n_seqs, g.index_heads), scale=g.index_heads ** -0.5)),
        ikv=spread(_bf16(rng, (n_seqs, g.max_comp, g.index_dim)), g.index_dim),
    )


def attend_close(got_u16, want_u16, tol=1.0 / 128.0):
    """The reference's bar for this attention (crates/engine/tests/kernel_v4_attend.rs:85-93): error
    relative to the largest expected element, two bf16 ulps. Returns (ok, worst)."""
    got, want = orc.bf16_to_f32(got_u16).astype(np.float64), orc.bf16_to_f32(want_u16).astype(np.float64)
    nan_g, nan_w = np.isnan(got), np.isnan(want)
    if not np.array_equal(nan_g, nan_w):
        return False, float("inf")
    if nan_w.all():
        return True, 0.0
    scale = np.abs(want[~nan_w]).max()
    worst = float(np.abs(got - want)[~nan_w].max() / max(scale, 1e-30))
    return worst <= tol, worst
