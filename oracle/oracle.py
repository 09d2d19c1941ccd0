"""ctypes binding of the CPU oracle (``liboracle.so``, built from ``rivoli_oracle.c`` and ``v4_oracle.c``).

Test infrastructure only: imported by ``tests/``, by the smoke check and by the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark. The product package never
imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` beside its source if it is missing or stale."""
    srcs = [os.path.join(_HERE, n) for n in ("rivoli_oracle.c", "v4_oracle.c")]
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < max(os.path.getmtime(p) for p in srcs):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


class Geom(C.Structure):
    """Mirror of ``orc_geom`` (same field order as the product's ``DsaGeom``)."""
    _fields_ = [(n, C.c_int32) for n in (
        "n_heads", "kv_lora", "rope_dim", "index_heads", "index_dim", "page_tokens", "top_k",
        "max_pages_per_seq", "n_pool_pages")] + [(n, C.c_float) for n in (
        "softmax_scale", "index_wscale", "index_dscale")]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        L = _lib
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_e4m3.restype = C.c_uint8
        L.orc_f32_to_e4m3.argtypes = [C.c_float]
        L.orc_e4m3_to_f32.restype = C.c_float
        L.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_lcg_next.restype = C.c_float
        L.orc_pool_new.restype = C.c_void_p
        L.orc_pool_block_table.restype = C.POINTER(C.c_int32)
        L.orc_pool_free_list.restype = C.POINTER(C.c_int32)
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


# --- codecs -------------------------------------------------------------------------------------
def f32_to_bf16(x) -> np.ndarray:
    """Vectorised RNE f32 -> bf16 bits (same rule as ``orc_f32_to_bf16``)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    r = ((b >> 16) & 1) + 0x7FFF
    out = ((b + r) >> 16).astype(np.uint16)
    out[nan] = ((b[nan] >> 16) | 0x40).astype(np.uint16)
    return out


def bf16_to_f32(b) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_e4m3(x) -> np.ndarray:
    x = _c(x, np.float32)
    L = lib()
    return np.array([L.orc_f32_to_e4m3(float(v)) for v in x.ravel()], dtype=np.uint8).reshape(x.shape)


def e4m3_table() -> np.ndarray:
    L = lib()
    return np.array([L.orc_e4m3_to_f32(c) for c in range(256)], dtype=np.float32)


class Lcg:
    """The reference tests' deterministic input stream."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed)

    def f(self) -> float:
        return float(lib().orc_lcg_next(C.byref(self.state)))

    def draws(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().orc_lcg_fill(C.byref(self.state), _p(out), C.c_size_t(n))
        return out


# --- reference-layout operators -----------------------------------------------------------------
def append_kv(latent, rope, lc8, lscale, rc, pos, kvl, ropn, n_blocks) -> int:
    return lib().orc_append_kv(_p(_c(latent, np.float32)), _p(_c(rope, np.float32)), _p(lc8),
                               _p(lscale), _p(rc), pos, kvl, ropn, n_blocks)


def gather_rope(q, h, qh, nope, ropn) -> np.ndarray:
    out = np.zeros(h * ropn, dtype=np.float32)
    lib().orc_gather_rope(_p(_c(q, np.float32)), _p(out), h, qh, nope, ropn)
    return out


def index_append(k, kcache, pos, hd) -> None:
    lib().orc_index_append(_p(_c(k, np.float32)), _p(kcache), pos, hd)


def index_score(q, w, kcache, heads, nt, nh, nact, hd, wscale, dscale) -> np.ndarray:
    out = np.zeros(nt, dtype=np.float32)
    hp = None if heads is None else _c(heads, np.uint32)
    lib().orc_index_score(_p(_c(q, np.float32)), _p(_c(w, np.float32)), _p(_c(kcache, np.uint16)),
                          _p(hp), nt, nh, nact, hd, C.c_float(wscale), C.c_float(dscale), _p(out))
    return out


def index_score_f32(q, w, keys, nt, nh, hd, wscale, dscale) -> np.ndarray:
    """The scoring core on f32 keys ``[nt, hd]`` (``orc_index_score`` is this after widening its bf16 keys)."""
    scores = np.zeros(nt, dtype=np.float32)
    lib().orc_index_score_f32(_p(_c(q, np.float32)), _p(_c(w, np.float32)), _p(_c(keys, np.float32)), None,
                              C.c_int(nt), C.c_int(nh), C.c_int(nh), C.c_int(hd), C.c_float(wscale), C.c_float(dscale),
                              _p(scores))
    return scores


def index_topk(scores, k) -> np.ndarray:
    s = _c(scores, np.float32)
    rows = np.zeros(max(min(k, s.size), 1), dtype=np.uint32)
    n = lib().orc_index_topk(_p(s), s.size, k, _p(rows))
    return rows[:n]


def topk_value_order(scores, k) -> np.ndarray:
    s = _c(scores, np.float32)
    rows = np.zeros(max(min(k, s.size), 1), dtype=np.uint32)
    n = lib().orc_topk_value_order(_p(s), s.size, k, _p(rows))
    return rows[:n]


def softmax(v) -> np.ndarray:
    v = _c(v, np.float32).copy()
    lib().orc_softmax(_p(v), v.size)
    return v


def mla_attend(qabs, qrope, lc8, lscale, rc, rows, H, nr, kvl, rope, n_blocks, scale) -> np.ndarray:
    out = np.zeros(H * kvl, dtype=np.float32)
    rp = None if rows is None else _c(rows, np.uint32)
    lib().orc_mla_attend(_p(_c(qabs, np.float32)), _p(_c(qrope, np.float32)), _p(_c(lc8, np.uint8)),
                         _p(_c(lscale, np.float32)), _p(_c(rc, np.uint16)), _p(rp), H, nr, kvl, rope,
                         n_blocks, C.c_float(scale), _p(out))
    return out


def mla_attend_f32(qabs, qrope, lat, rk, H, nr, kvl, rope, scale) -> np.ndarray:
    """The attention core on rows already dequantised to f32 (``lat [nr, kvl]``, ``rk [nr, rope]``)."""
    clat = np.zeros((H, kvl), dtype=np.float32)
    lib().orc_mla_attend_f32(_p(_c(qabs, np.float32)), _p(_c(qrope, np.float32)), _p(_c(lat, np.float32)),
                             _p(_c(rk, np.float32)), C.c_int(H), C.c_int(nr), C.c_int(kvl), C.c_int(rope),
                             C.c_float(scale), _p(clat))
    return clat


def mla_absorb_f32(q, wf, H, qh, nope, vh, kvl, nrow=1) -> np.ndarray:
    """``mla_absorb_fp8`` on weights already dequantised to f32 ``[H*(nope+vh), kvl]``."""
    out = np.zeros((nrow, H * kvl), dtype=np.float32)
    lib().orc_mla_absorb_f32(_p(_c(q, np.float32)), _p(_c(wf, np.float32)), C.c_int(H), C.c_int(qh), C.c_int(nope),
                             C.c_int(vh), C.c_int(kvl), C.c_int(nrow), _p(out))
    return out


def mla_value_f32(clat, wf, H, nope, vh, kvl, nrow=1) -> np.ndarray:
    """``mla_value_fp8`` on weights already dequantised to f32."""
    out = np.zeros((nrow, H * vh), dtype=np.float32)
    lib().orc_mla_value_f32(_p(_c(clat, np.float32)), _p(_c(wf, np.float32)), C.c_int(H), C.c_int(nope), C.c_int(vh),
                            C.c_int(kvl), C.c_int(nrow), _p(out))
    return out


def mla_plan_splits(H, nr, have_scratch=True):
    n, tps = C.c_int(), C.c_int()
    lib().orc_mla_plan_splits(H, nr, int(have_scratch), C.byref(n), C.byref(tps))
    return n.value, tps.value


def mla_attend_partial(qabs, qrope, lc8, lscale, rc, H, r0, r1, kvl, rope, n_blocks, scale):
    acc = np.zeros(H * kvl, dtype=np.float32)
    ml = np.zeros(H * 2, dtype=np.float32)
    lib().orc_mla_attend_partial(_p(_c(qabs, np.float32)), _p(_c(qrope, np.float32)),
                                 _p(_c(lc8, np.uint8)), _p(_c(lscale, np.float32)),
                                 _p(_c(rc, np.uint16)), H, r0, r1, kvl, rope, n_blocks,
                                 C.c_float(scale), _p(acc), _p(ml))
    return acc, ml


def attend_combine(acc, ml, H, kvl, n_splits) -> np.ndarray:
    out = np.zeros(H * kvl, dtype=np.float32)
    lib().orc_attend_combine(_p(_c(acc, np.float32)), _p(_c(ml, np.float32)), H, kvl, n_splits, _p(out))
    return out


# --- paged layout ---------------------------------------------------------------------------------
def kv_append_paged(g: Geom, latent, index_key, row_seq, row_pos, block_table, latent_pool,
                    latent_scale, index_pool, index_scale) -> int:
    latent = _c(latent, np.uint16)
    index_key = _c(index_key, np.uint16)
    row_pos = _c(row_pos, np.int32)
    rs = None if row_seq is None else _c(row_seq, np.int32)
    return lib().orc_kv_append_paged(C.byref(g), _p(latent), _p(index_key), _p(rs), _p(row_pos),
                                     row_pos.size, _p(_c(block_table, np.int32)), _p(latent_pool),
                                     _p(latent_scale), _p(index_pool), _p(index_scale))


def index_q_quant(q_bf16, hd):
    q = _c(q_bf16, np.uint16)
    n = q.size // hd
    codes = np.zeros(q.shape, dtype=np.uint8)
    scales = np.zeros(n, dtype=np.float32)
    lib().orc_index_q_quant(_p(q), n, hd, _p(codes), _p(scales))
    return codes, scales


def index_score_paged(g: Geom, qcodes, qscales, w, index_pool, index_scale, block_table, seq_len,
                      score_stride) -> np.ndarray:
    seq_len = _c(seq_len, np.int32)
    B = seq_len.size
    scores = np.zeros((B, score_stride), dtype=np.float32)
    lib().orc_index_score_paged(C.byref(g), _p(_c(qcodes, np.uint8)), _p(_c(qscales, np.float32)),
                                _p(_c(w, np.float32)), _p(index_pool), _p(index_scale),
                                _p(_c(block_table, np.int32)), _p(seq_len), B, _p(scores), score_stride)
    return scores


def index_topk_batched(scores, seq_len, k):
    scores = _c(scores, np.float32)
    seq_len = _c(seq_len, np.int32)
    B = seq_len.size
    rows = np.full((B, k), 0xFFFFFFFF, dtype=np.uint32)
    n_sel = np.zeros(B, dtype=np.int32)
    lib().orc_index_topk_batched(_p(scores), scores.shape[1], _p(seq_len), B, k, _p(rows), _p(n_sel))
    return rows, n_sel


def mla_attend_paged(g: Geom, q, latent_pool, latent_scale, block_table, rows, n_rows,
                     want_f32=False):
    q = _c(q, np.uint16)
    n_rows = _c(n_rows, np.int32)
    B = n_rows.size
    out = np.zeros((B, g.n_heads, g.kv_lora), dtype=np.uint16)
    out_f32 = np.zeros((B, g.n_heads, g.kv_lora), dtype=np.float32)
    m = np.zeros((B, g.n_heads), dtype=np.float32)
    lse = np.zeros((B, g.n_heads), dtype=np.float32)
    rp, stride = (None, 0) if rows is None else (_c(rows, np.uint32), rows.shape[1])
    lib().orc_mla_attend_paged(C.byref(g), _p(q), _p(latent_pool), _p(latent_scale),
                               _p(_c(block_table, np.int32)), _p(rp), stride, _p(n_rows), B, _p(out),
                               _p(out_f32), _p(m), _p(lse))
    return (out, out_f32, m, lse) if want_f32 else (out, m, lse)


def attend_merge_partials(part_out, part_lse, kvl) -> np.ndarray:
    part_out = _c(part_out, np.uint16)
    part_lse = _c(part_lse, np.float32)
    G = part_out.shape[0]
    n = part_lse.size // G
    out = np.zeros((n, kvl), dtype=np.uint16)
    lib().orc_attend_merge_partials(_p(part_out), _p(part_lse), G, n, kvl, _p(out))
    return out


def mla_absorb_fp8(q, kvb, scale, H, qh, nope, vh, kvl, block, nrow=1) -> np.ndarray:
    """f32 q ``[nrow, H*qh]`` through kv_b's absorb rows -> ``[nrow, H*kvl]`` (mla.hip:12-122)."""
    q, kvb, scale = _c(q, np.float32), _c(kvb, np.uint8), _c(scale, np.float32)
    out = np.zeros((nrow, H * kvl), dtype=np.float32)
    lib().orc_mla_absorb_fp8(_p(q), _p(kvb), _p(scale), H, qh, nope, vh, kvl, block, nrow, _p(out))
    return out


def mla_value_fp8(clat, kvb, scale, H, nope, vh, kvl, block, nrow=1) -> np.ndarray:
    """f32 clat ``[nrow, H*kvl]`` through kv_b's value rows -> ``[nrow, H*vh]`` (mla.hip:138-175)."""
    clat, kvb, scale = _c(clat, np.float32), _c(kvb, np.uint8), _c(scale, np.float32)
    out = np.zeros((nrow, H * vh), dtype=np.float32)
    lib().orc_mla_value_fp8(_p(clat), _p(kvb), _p(scale), H, nope, vh, kvl, block, nrow, _p(out))
    return out


def mla_absorb_batched_bf16(q, kvb, scale, H, qh, nope, vh, kvl, rope, block):
    """bf16 q ``[B, H, qh]`` -> (q_abs bf16 ``[B, H, kvl+rope]``, absorbed part in f32 ``[B, H, kvl]``)."""
    q, kvb, scale = _c(q, np.uint16), _c(kvb, np.uint8), _c(scale, np.float32)
    B = q.size // (H * qh)
    out = np.zeros((B, H, kvl + rope), dtype=np.uint16)
    f32 = np.zeros((B, H, kvl), dtype=np.float32)
    lib().orc_mla_absorb_batched_bf16(_p(q), _p(kvb), _p(scale), H, qh, nope, vh, kvl, rope, block, B, _p(out), _p(f32))
    return out, f32


def mla_value_batched_bf16(clat, kvb, scale, H, nope, vh, kvl, block):
    """bf16 clat ``[B, H, kvl]`` -> (ctx bf16 ``[B, H, vh]``, the same in f32)."""
    clat, kvb, scale = _c(clat, np.uint16), _c(kvb, np.uint8), _c(scale, np.float32)
    B = clat.size // (H * kvl)
    out = np.zeros((B, H, vh), dtype=np.uint16)
    f32 = np.zeros((B, H, vh), dtype=np.float32)
    lib().orc_mla_value_batched_bf16(_p(clat), _p(kvb), _p(scale), H, nope, vh, kvl, block, B, _p(out), _p(f32))
    return out, f32


def gemv_fp8(x, packed, scale, o_dim, i_dim, block, nrow=1) -> np.ndarray:
    """f32 x ``[nrow, i_dim]`` through e4m3 block-scaled ``W[o_dim, i_dim]`` (crates/artifact/src/quant/fp8.rs:32-42)."""
    x, packed, scale = _c(x, np.float32), _c(packed, np.uint8), _c(scale, np.float32)
    y = np.zeros((nrow, o_dim), dtype=np.float32)
    lib().orc_gemv_fp8(_p(x), _p(packed), _p(scale), o_dim, i_dim, block, nrow, _p(y))
    return y


def layernorm(x, w, b, eps) -> np.ndarray:
    x, w, b = _c(x, np.float32), _c(w, np.float32), _c(b, np.float32)
    y = np.zeros_like(x)
    lib().orc_layernorm(_p(x), _p(w), _p(b), x.size, C.c_float(eps), _p(y))
    return y


def rope_interleave(base, count, stride, seg, pos, theta) -> np.ndarray:
    v = _c(base, np.float32).copy()
    lib().orc_rope_interleave(_p(v), count, stride, seg, pos, C.c_double(theta))
    return v


def index_frontend_bf16(x, qr, pos, nh, hd, rope_off, rope_seg, theta, eps, block, wk, wk_s, kn_w, kn_b, wq, wq_s, wp, wp_s):
    """Batched indexer front end; returns (index_key bf16, index_q bf16, index_w f32, key f32, q f32)."""
    x, qr, pos = _c(x, np.uint16), _c(qr, np.uint16), _c(pos, np.int32)
    B = pos.size
    hidden, q_lora = x.size // B, qr.size // B
    key = np.zeros((B, hd), np.uint16); q = np.zeros((B, nh, hd), np.uint16); w = np.zeros((B, nh), np.float32)
    k32 = np.zeros((B, hd), np.float32); q32 = np.zeros((B, nh, hd), np.float32)
    a = [_c(t, np.uint8) if t.dtype == np.uint8 else _c(t, np.float32) for t in (wk, wk_s, kn_w, kn_b, wq, wq_s, wp, wp_s)]
    lib().orc_index_frontend_bf16(_p(x), _p(qr), _p(pos), B, hidden, q_lora, nh, hd, rope_off, rope_seg, C.c_double(theta),
                                  C.c_float(eps), block, *[_p(t) for t in a], _p(key), _p(q), _p(w), _p(k32), _p(q32))
    return key, q, w, k32, q32


def kvb_fixture(r: "Lcg", rows, kvl, block):
    """kv_b bytes then the block-scale grid, drawn in that order
    (crates/engine/tests/kernel_attend.rs:127-132, tests/common/reference.rs:218-220)."""
    packed = f32_to_e4m3(r.draws(rows * kvl))
    n = ((rows + block - 1) // block) * ((kvl + block - 1) // block)
    scale = (np.abs(r.draws(n) * np.float32(0.1)) + np.float32(0.01)).astype(np.float32)
    return packed, scale


class Pool:
    """LIFO page allocator of the oracle (see ``orc_pool_*``)."""

    def __init__(self, n_pages, n_seqs, max_pages_per_seq, page_tokens):
        self._h = C.c_void_p(lib().orc_pool_new(n_pages, n_seqs, max_pages_per_seq, page_tokens))
        self.shape = (n_seqs, max_pages_per_seq)
        self.n_pages = n_pages

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                lib().orc_pool_free(self._h)
                self._h = None
        except Exception:   # interpreter shutdown: module globals may already be gone
            pass

    def shuffle(self, seed):
        lib().orc_pool_shuffle(self._h, C.c_uint64(seed))

    def reserve(self, seq, n_tokens) -> int:
        return lib().orc_pool_reserve(self._h, seq, n_tokens)

    def release(self, seq) -> int:
        return lib().orc_pool_release(self._h, seq)

    @property
    def n_free(self) -> int:
        return lib().orc_pool_n_free(self._h)

    def block_table(self) -> np.ndarray:
        p = lib().orc_pool_block_table(self._h)
        return np.ctypeslib.as_array(p, shape=self.shape).copy()

    def free_list(self) -> np.ndarray:
        p = lib().orc_pool_free_list(self._h)
        return np.ctypeslib.as_array(p, shape=(self.n_pages,))[: self.n_free].copy()


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(int(n))


def num_threads() -> int:
    return lib().orc_num_threads()


# --- V4 cousin path (v4_oracle.c) -----------------------------------------------------------------
class V4Geom(C.Structure):
    """Mirror of ``orc_v4_geom`` (same field order as the product's ``V4Geom``)."""
    _fields_ = [(n, C.c_int32) for n in (
        "n_heads", "head_dim", "window", "index_heads", "index_dim", "index_topk", "ratio",
        "max_comp")] + [("softmax_scale", C.c_float)]


def e2m1_decode(nib: int) -> float:
    f = lib().orc_e2m1_decode
    f.restype, f.argtypes = C.c_float, [C.c_uint8]
    return float(f(nib))


def e2m1_encode(x: float) -> int:
    f = lib().orc_e2m1_encode
    f.restype, f.argtypes = C.c_uint8, [C.c_float]
    return int(f(x))


def fast_round_scale(amax: float, max_inv: float) -> float:
    f = lib().orc_fast_round_scale
    f.restype, f.argtypes = C.c_float, [C.c_float, C.c_float]
    return float(f(amax, max_inv))


def v4_hadamard(row) -> np.ndarray:
    r = _c(row, np.float32).copy()
    lib().orc_v4_hadamard(_p(r), C.c_int(r.size))
    return r


def v4_spread(x, d) -> tuple[int, np.ndarray]:
    """Hadamard + bf16 + fp4 block-32 + bf16 on every row of ``x`` ([rows, d] f32)."""
    r = _c(x, np.float32).reshape(-1, d).copy() if d > 0 and np.size(x) else np.zeros((0, max(d, 1)), np.float32)
    rc = lib().orc_v4_spread(_p(r), C.c_int(r.shape[0]), C.c_int(d))
    return int(rc), r


def v4_index_score_blocks(q, kv, w, s, n_comp, heads, hd) -> tuple[int, np.ndarray]:
    q, kv, w = _c(q, np.float32), _c(kv, np.float32), _c(w, np.float32)
    out = np.zeros((max(s, 0), max(n_comp, 0)), np.float32)
    rc = lib().orc_v4_index_score_blocks(_p(q), _p(kv), _p(w), _p(out), C.c_int(s), C.c_int(n_comp),
                                         C.c_int(heads), C.c_int(hd))
    return int(rc), out


def v4_scored_row(scores, limit, k, offset, width) -> np.ndarray:
    sc = _c(scores, np.float32)
    out = np.zeros(width, np.int32)
    lib().orc_v4_scored_row(_p(sc), C.c_int(limit), C.c_int(k), C.c_int(offset), C.c_int(width), _p(out))
    return out


def v4_window_row(win, start_pos) -> np.ndarray:
    out = np.zeros(win, np.int32)
    lib().orc_v4_window_row(C.c_int(win), C.c_int(start_pos), _p(out))
    return out


def v4_sparse_attn(q, kv, sink, idxs, m, h, d, topk, scale) -> tuple[int, np.ndarray]:
    q, kv, sink = _c(q, np.float32), _c(kv, np.float32), _c(sink, np.float32)
    idxs = _c(idxs, np.int32)
    o = np.zeros((max(m, 0), max(h, 0), max(d, 0)), np.float32)
    rc = lib().orc_v4_sparse_attn(_p(q), _p(kv), _p(sink), _p(idxs), C.c_int(m), C.c_int(h), C.c_int(d),
                                  C.c_int(topk), C.c_float(scale), _p(o))
    return int(rc), o


def v4_decode_step_bf16(g: V4Geom, pos, q, kv_cache, sink, iq, iw, ikv, want_scores=False):
    """Batched decode step over bf16 storage. Returns (sel [B, window+topk] i32, out [B,H,D] u16
    [, scores [B, max_comp] f32])."""
    pos = _c(pos, np.int32)
    B = pos.size
    q, kv_cache, iq, ikv = (_c(a, np.uint16) for a in (q, kv_cache, iq, ikv))
    sink, iw = _c(sink, np.float32), _c(iw, np.float32)
    sel = np.zeros((B, g.window + g.index_topk), np.int32)
    out = np.zeros((B, g.n_heads, g.head_dim), np.uint16)
    sc = np.zeros((B, g.max_comp), np.float32) if want_scores else None
    lib().orc_v4_decode_step_bf16(C.byref(g), C.c_int(B), _p(pos), _p(q), _p(kv_cache), _p(sink), _p(iq),
                                  _p(iw), _p(ikv), _p(sel), _p(sc), _p(out))
    return (sel, out, sc) if want_scores else (sel, out)


class CompGeom(C.Structure):
    """Mirror of ``orc_comp_geom`` (the reference's CompGeom)."""
    _fields_ = [(n, C.c_int32) for n in ("ratio", "coff", "d", "cd", "ents", "rd")] + [("eps", C.c_float)]

    @classmethod
    def make(cls, ratio=4, d=512, rd=64, eps=1e-6):
        coff = 2 if ratio == 4 else 1
        return cls(ratio, coff, d, coff * d, coff * ratio, rd, eps)


def act_quant_f8_prefix(src, rows, row_stride, n, block):
    a = _c(src, np.float32).copy()
    rc = lib().orc_act_quant_f8_prefix(_p(a), _p(a), C.c_int(rows), C.c_int(row_stride), C.c_int(n), C.c_int(block))
    return int(rc), a


def v4_compress_deposit_token(kv, score, ape, kv_state, score_state, p: CompGeom, start_pos) -> int:
    """In place on kv_state / score_state (float32 C-contiguous arrays)."""
    return int(lib().orc_v4_compress_deposit_token(_p(_c(kv, np.float32)), _p(_c(score, np.float32)), _p(_c(ape, np.float32)),
                                                   _p(kv_state), _p(score_state), C.byref(p), C.c_int(start_pos)))


def v4_compress_decode(kv_state, score_state, norm, freqs, p: CompGeom, start_pos):
    """Pools in place (the overlap half moves down). Returns (rc, row before the finishing quantisation)."""
    out = np.zeros(p.d, np.float32)
    rc = lib().orc_v4_compress_decode(_p(kv_state), _p(score_state), _p(_c(norm, np.float32)), _p(_c(freqs, np.float32)),
                                      _p(out), C.byref(p), C.c_int(start_pos))
    return int(rc), out


def v4_compress_deposit_prefill(kv, score, ape, kv_state, score_state, p: CompGeom, s) -> int:
    return int(lib().orc_v4_compress_deposit_prefill(_p(_c(kv, np.float32)), _p(_c(score, np.float32)), _p(_c(ape, np.float32)),
                                                     _p(kv_state), _p(score_state), C.byref(p), C.c_int(s)))


def v4_compress_prefill(kv, score, ape, norm, freqs, p: CompGeom, nblk):
    out = np.zeros((max(nblk, 0), p.d), np.float32)
    rc = lib().orc_v4_compress_prefill(_p(_c(kv, np.float32)), _p(_c(score, np.float32)), _p(_c(ape, np.float32)),
                                       _p(_c(norm, np.float32)), _p(_c(freqs, np.float32)), _p(out), C.byref(p), C.c_int(nblk))
    return int(rc), out
