"""Seeded synthetic decode-layer state built on the CPU with the oracle (test infrastructure):
the parity tests upload it and compare, and the benchmark's CPU arm times ``oracle_step`` on it."""
from __future__ import annotations

import numpy as np

from oracle import oracle as orc


def bf16_normal(rng: np.random.RandomState, shape) -> np.ndarray:
    """bf16 bit patterns of N(0,1) draws (RNE)."""
    return orc.f32_to_bf16(rng.standard_normal(shape).astype(np.float32))


def make_geom(cls, **kw):
    """Build a Geom / DsaGeom of either binding class with the model's default scales."""
    f32 = np.float32
    d = dict(n_heads=64, kv_lora=512, rope_dim=64, index_heads=32, index_dim=128, page_tokens=64,
             top_k=2048, max_pages_per_seq=1, n_pool_pages=1)
    d.update(kw)
    d.setdefault("softmax_scale", float(f32(1.0) / np.sqrt(f32(d["kv_lora"] + d["rope_dim"]))))
    d.setdefault("index_wscale", float(f32(d["index_heads"]) ** f32(-0.5)))
    d.setdefault("index_dscale", float(f32(d["index_dim"]) ** f32(-0.5)))
    order = ["n_heads", "kv_lora", "rope_dim", "index_heads", "index_dim", "page_tokens", "top_k",
             "max_pages_per_seq", "n_pool_pages", "softmax_scale", "index_wscale", "index_dscale"]
    return cls(*[d[k] for k in order])


class State:
    """A decode-layer state: pools filled by the oracle's append, plus this step's inputs."""

    def __init__(self, seed, B, ctx_lens, *, n_heads=64, index_heads=32, index_dim=128, page_tokens=64,
                 top_k=2048, pool_factor=1.25, kv_lora=512, rope_dim=64):
        rng = np.random.RandomState(seed)
        self.B = B
        ctx_lens = np.asarray(ctx_lens, dtype=np.int32)            # tokens AFTER this step's append
        self.seq_len = ctx_lens
        P = page_tokens
        max_pages = int((ctx_lens.max() + P - 1) // P)
        live = int(((ctx_lens + P - 1) // P).sum())
        n_pool = max(int(np.ceil(live * pool_factor)), live)
        kw = dict(n_heads=n_heads, kv_lora=kv_lora, rope_dim=rope_dim, index_heads=index_heads,
                  index_dim=index_dim, page_tokens=P, top_k=top_k, max_pages_per_seq=max_pages,
                  n_pool_pages=n_pool)
        self.geom_kw = kw
        self.og = make_geom(orc.Geom, **kw)
        W = kv_lora + rope_dim
        self.W = W
        self.pool = orc.Pool(n_pool, B, max_pages, P)
        self.pool.shuffle(seed * 7919 + 17)
        for b in range(B):
            assert self.pool.reserve(b, int(ctx_lens[b])) == 0
        self.block_table = self.pool.block_table()
        rows = n_pool * P
        self.latent_pool = np.zeros(rows * W, np.uint8)
        self.latent_scale = np.zeros(rows, np.float32)
        self.index_pool = np.zeros(rows * index_dim, np.uint8)
        self.index_scale = np.zeros(rows, np.float32)
        # history: every token before the one appended this step
        hist_seq = np.concatenate([np.full(n - 1, b, np.int32) for b, n in enumerate(ctx_lens)])
        hist_pos = np.concatenate([np.arange(n - 1, dtype=np.int32) for n in ctx_lens])
        self.hist_seq, self.hist_pos = hist_seq, hist_pos
        nh_tok = hist_seq.size
        self.hist_latent = bf16_normal(rng, (nh_tok, W))
        self.hist_key = bf16_normal(rng, (nh_tok, index_dim))
        if nh_tok:
            assert orc.kv_append_paged(self.og, self.hist_latent, self.hist_key, hist_seq, hist_pos,
                                       self.block_table, self.latent_pool, self.latent_scale,
                                       self.index_pool, self.index_scale) == 0
        # this step's inputs
        self.new_latent = bf16_normal(rng, (B, W))
        self.new_key = bf16_normal(rng, (B, index_dim))
        self.row_pos = (ctx_lens - 1).astype(np.int32)
        self.index_q = bf16_normal(rng, (B, index_heads, index_dim))
        self.index_w = orc.bf16_to_f32(bf16_normal(rng, (B, index_heads)))   # f32 holding bf16 values
        self.q = bf16_normal(rng, (B, n_heads, W))

    def oracle_step(self):
        """The whole layer-step on the CPU; returns every intermediate for comparison."""
        g = self.og
        lp, ls = self.latent_pool.copy(), self.latent_scale.copy()
        ip, isc = self.index_pool.copy(), self.index_scale.copy()
        assert orc.kv_append_paged(g, self.new_latent, self.new_key, None, self.row_pos, self.block_table,
                                   lp, ls, ip, isc) == 0
        qc, qs = orc.index_q_quant(self.index_q, g.index_dim)
        stride = int(self.seq_len.max())
        scores = orc.index_score_paged(g, qc, qs, self.index_w, ip, isc, self.block_table, self.seq_len, stride)
        rows, n_sel = orc.index_topk_batched(scores, self.seq_len, g.top_k)
        out, out_f32, m, lse = orc.mla_attend_paged(g, self.q, lp, ls, self.block_table, rows, n_sel,
                                                    want_f32=True)
        return dict(latent_pool=lp, latent_scale=ls, index_pool=ip, index_scale=isc, qcodes=qc, qscales=qs,
                    scores=scores, rows=rows, n_sel=n_sel, out=out, out_f32=out_f32, m=m, lse=lse)


def attend_close(got_bf16_bits, want_f32, rel=2e-2, abs_=1e-3):
    """|got - want| <= rel*|want| + abs, elementwise; returns (ok, worst excess ratio)."""
    got = orc.bf16_to_f32(np.asarray(got_bf16_bits, dtype=np.uint16)).astype(np.float64)
    want = np.asarray(want_f32, dtype=np.float64)
    err = np.abs(got.reshape(want.shape) - want)
    tol = rel * np.abs(want) + abs_
    return bool((err <= tol).all()), float((err / tol).max())


def attend_close_ref(got_bf16_bits, want_f32, rel=2e-2, abs_=1e-3):
    """The reference's own tolerance form (crates/engine/tests/common/scoring.rs:191-194):
    max|got - want| <= rel * max|want| + abs, per sequence. Returns (ok, worst err/tol,
    worst rms(err)/rms(want))."""
    got = orc.bf16_to_f32(np.asarray(got_bf16_bits, dtype=np.uint16)).astype(np.float64)
    want = np.asarray(want_f32, dtype=np.float64)
    got = got.reshape(want.shape)
    ok, worst, worst_rms = True, 0.0, 0.0
    for b in range(want.shape[0]):
        err = np.abs(got[b] - want[b])
        tol = rel * np.abs(want[b]).max() + abs_
        ok &= bool(err.max() <= tol)
        worst = max(worst, float(err.max() / tol))
        r = float(np.sqrt((want[b] ** 2).mean()))
        if r > 0:
            worst_rms = max(worst_rms, float(np.sqrt((err ** 2).mean())) / r)
    return ok, worst, worst_rms
