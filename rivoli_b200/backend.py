"""Host-side mirror of the reference's ``crates/backend`` operator surface for the decode
KV-cache path, bound to ``librivolikernels.so`` through its C ABI.

Names, argument order and error behaviour follow the reference's Rust launchers
(``launch_append_kv``, ``launch_index_append``, ``launch_index_score``,
``launch_index_topk``, ``launch_attend``, ``launch_gather_rope``, ``device_sync``,
``attend_scratch_floats``: crates/backend/src/hip_attn.rs:101-147,443-495 and
crates/backend/src/hip.rs:328-336,425-430): every launcher returns ``None`` on success and
raises :class:`BackendError` whose text is ``"<name>: argument guard rejected (<code>)"``
for a positive return and ``"<name>: CUDA error <n>"`` for a negative one, so a test can
assert the guard code exactly as the reference's ``assert_guard`` does.

Pointer arguments accept a ``torch.Tensor`` (its ``data_ptr()`` is passed), an ``int``
device address, or ``None`` for NULL. There is NO fallback: if the CUDA library is not
built, importing a launcher fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "librivolikernels.so")


class BackendError(RuntimeError):
    """A launcher refused its arguments (``code`` > 0) or the launch failed (``code`` < 0)."""

    def __init__(self, name: str, code: int):
        self.name, self.code = name, code
        if code > 0:
            msg = f"{name}: argument guard rejected ({code})"
        else:
            msg = f"{name}: CUDA error {-code}"
        super().__init__(msg)


class DsaGeom(C.Structure):
    """``DsaGeom`` of include/rivoli_kernels.h (48 bytes, align 4)."""
    _fields_ = [(n, C.c_int32) for n in (
        "n_heads", "kv_lora", "rope_dim", "index_heads", "index_dim", "page_tokens", "top_k",
        "max_pages_per_seq", "n_pool_pages")] + [(n, C.c_float) for n in (
        "softmax_scale", "index_wscale", "index_dscale")]

    @classmethod
    def make(cls, *, n_heads=64, kv_lora=512, rope_dim=64, index_heads=32, index_dim=128,
             page_tokens=64, top_k=2048, max_pages_per_seq, n_pool_pages, softmax_scale=None,
             index_wscale=None, index_dscale=None) -> "DsaGeom":
        import numpy as np
        f32 = np.float32
        return cls(n_heads, kv_lora, rope_dim, index_heads, index_dim, page_tokens, top_k,
                   max_pages_per_seq, n_pool_pages,
                   float(f32(1.0) / np.sqrt(f32(kv_lora + rope_dim))) if softmax_scale is None else softmax_scale,
                   float(f32(index_heads) ** f32(-0.5)) if index_wscale is None else index_wscale,
                   float(f32(index_dim) ** f32(-0.5)) if index_dscale is None else index_dscale)


assert C.sizeof(DsaGeom) == 48 and C.alignment(DsaGeom) == 4

_lib = None


def library_path() -> str:
    return _SO


def lib() -> C.CDLL:
    """The loaded CUDA library. Raises if it has not been built: there is no CPU path."""
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            raise RuntimeError(
                f"{_SO} is missing: build it with `python -m rivoli_b200.build` "
                "(nvcc, sm_100a). rivoli_b200 has no CPU fallback.")
        L = C.CDLL(_SO)
        L.rivoli_mla_attend_scratch_floats.restype = C.c_size_t
        L.rivoli_mla_attend_paged_scratch_bytes.restype = C.c_size_t
        L.rivoli_attend_simt_scratch_bytes.restype = C.c_size_t
        L.rivoli_index_select_scratch_bytes.restype = C.c_size_t
        L.rivoli_index_frontend_scratch_bytes.restype = C.c_size_t
        L.rivoli_v4_select_scratch_bytes.restype = C.c_size_t
        L.rivoli_kernels_arch.restype = C.c_char_p
        L.rivoli_pagepool_create.restype = C.c_void_p
        L.rivoli_pagepool_block_table.restype = C.POINTER(C.c_int32)
        L.rivoli_pagepool_free_list.restype = C.POINTER(C.c_int32)
        for n in ("destroy", "shuffle", "reserve", "release", "n_free", "seq_pages", "block_table", "free_list"):
            getattr(L, f"rivoli_pagepool_{n}").argtypes = None
        _lib = L
    return _lib


def _ptr(x):
    if x is None:
        return C.c_void_p(0)
    if isinstance(x, int):
        return C.c_void_p(x)
    return C.c_void_p(x.data_ptr())


def _stream(s):
    if s is None:
        return C.c_void_p(0)
    if isinstance(s, int):
        return C.c_void_p(s)
    return C.c_void_p(s.cuda_stream)


def ensure_status(r: int, name: str) -> None:
    """0 = ok, positive = argument guard, negative = -(cudaError_t) (hip.rs:328-336)."""
    if r != 0:
        raise BackendError(name, int(r))


# --- Part 1: the reference's launchers ------------------------------------------------------------
def launch_append_kv(latent, rope, lc8, lscale, rc, pos: int, kvl: int, ropn: int, n_blocks: int) -> None:
    ensure_status(lib().rivoli_append_kv(_ptr(latent), _ptr(rope), _ptr(lc8), _ptr(lscale), _ptr(rc),
                                         C.c_int(pos), C.c_int(kvl), C.c_int(ropn), C.c_int(n_blocks)),
                  "append_kv")


def launch_gather_rope(q, qrope, h: int, qh: int, nope: int, ropn: int) -> None:
    ensure_status(lib().rivoli_gather_rope(_ptr(q), _ptr(qrope), C.c_int(h), C.c_int(qh), C.c_int(nope),
                                           C.c_int(ropn)), "gather_rope")


def launch_index_append(k, kcache, pos: int, hd: int) -> None:
    ensure_status(lib().rivoli_index_append(_ptr(k), _ptr(kcache), C.c_int(pos), C.c_int(hd)), "index_append")


def launch_index_score(q, w, kcache, heads, nt: int, nh: int, nact: int, hd: int, wscale: float,
                       dscale: float, scores) -> None:
    ensure_status(lib().rivoli_index_score(_ptr(q), _ptr(w), _ptr(kcache), _ptr(heads), C.c_int(nt),
                                           C.c_int(nh), C.c_int(nact), C.c_int(hd), C.c_float(wscale),
                                           C.c_float(dscale), _ptr(scores)), "index_score")


def launch_index_topk(scores, nt: int, k: int, rows) -> None:
    ensure_status(lib().rivoli_index_topk(_ptr(scores), C.c_int(nt), C.c_int(k), _ptr(rows)), "index_topk")


def launch_attend(qabs, qrope, lc8, lscale, rc, rows, h: int, nr: int, kvl: int, rope: int, n_blocks: int,
                  scale: float, clat, partial) -> None:
    ensure_status(lib().rivoli_mla_attend(_ptr(qabs), _ptr(qrope), _ptr(lc8), _ptr(lscale), _ptr(rc),
                                          _ptr(rows), C.c_int(h), C.c_int(nr), C.c_int(kvl), C.c_int(rope),
                                          C.c_int(n_blocks), C.c_float(scale), _ptr(clat), _ptr(partial)),
                  "mla_attend")


def launch_attend_static(qabs, qrope, lc8, lscale, rc, rows, h: int, nr: int, kvl: int, rope: int, n_blocks: int,
                         scale: float, clat) -> None:
    """``launch_attend`` for callers that cannot lend device scratch: the split partials live in
    an array built into the library (h <= 64, kvl <= 512). One call at a time per device."""
    ensure_status(lib().rivoli_mla_attend_static(_ptr(qabs), _ptr(qrope), _ptr(lc8), _ptr(lscale), _ptr(rc),
                                                 _ptr(rows), C.c_int(h), C.c_int(nr), C.c_int(kvl), C.c_int(rope),
                                                 C.c_int(n_blocks), C.c_float(scale), _ptr(clat)),
                  "mla_attend_static")


def attend_scratch_floats(h: int, kvl: int) -> int:
    return int(lib().rivoli_mla_attend_scratch_floats(C.c_int(h), C.c_int(kvl)))


def device_sync() -> None:
    ensure_status(lib().rivoli_device_sync(), "device_sync")


# --- Part 2: batched / paged / bf16 -----------------------------------------------------------------
def launch_kv_append_paged(g: DsaGeom, latent, index_key, row_seq, row_pos, n_rows: int, block_table,
                           latent_pool, latent_scale, index_pool, index_scale, status=None, stream=None) -> None:
    ensure_status(lib().rivoli_kv_append_paged(C.byref(g), _ptr(latent), _ptr(index_key), _ptr(row_seq),
                                               _ptr(row_pos), C.c_int(n_rows), _ptr(block_table),
                                               _ptr(latent_pool), _ptr(latent_scale), _ptr(index_pool),
                                               _ptr(index_scale), _ptr(status), _stream(stream)),
                  "kv_append_paged")


def launch_index_q_quant(q, n_vec: int, hd: int, codes, scales, stream=None) -> None:
    ensure_status(lib().rivoli_index_q_quant(_ptr(q), C.c_int(n_vec), C.c_int(hd), _ptr(codes), _ptr(scales),
                                             _stream(stream)), "index_q_quant")


def launch_index_score_paged(g: DsaGeom, qcodes, qscales, w, index_pool, index_scale, block_table, seq_len,
                             B: int, scores, score_stride: int, stream=None) -> None:
    ensure_status(lib().rivoli_index_score_paged(C.byref(g), _ptr(qcodes), _ptr(qscales), _ptr(w),
                                                 _ptr(index_pool), _ptr(index_scale), _ptr(block_table),
                                                 _ptr(seq_len), C.c_int(B), _ptr(scores),
                                                 C.c_int(score_stride), _stream(stream)), "index_score_paged")


def launch_index_topk_batched(scores, score_stride: int, seq_len, B: int, k: int, rows, n_sel,
                              stream=None) -> None:
    ensure_status(lib().rivoli_index_topk_batched(_ptr(scores), C.c_int(score_stride), _ptr(seq_len),
                                                  C.c_int(B), C.c_int(k), _ptr(rows), _ptr(n_sel),
                                                  _stream(stream)), "index_topk_batched")


def index_select_scratch_bytes(g: DsaGeom, B: int, score_stride: int) -> int:
    return int(lib().rivoli_index_select_scratch_bytes(C.byref(g), C.c_int(B), C.c_int(score_stride)))


def index_select_uses_mma(g: DsaGeom, score_stride: int) -> bool:
    return bool(lib().rivoli_index_select_uses_mma(C.byref(g), C.c_int(score_stride)))


def launch_index_select_paged(g: DsaGeom, index_q, w, index_pool, index_scale, block_table, seq_len, B: int,
                              score_stride: int, rows, n_sel, scratch, stream=None) -> None:
    """Fused indexer (q quant + scores + exact top-k); rows identical to the unfused chain."""
    ensure_status(lib().rivoli_index_select_paged(C.byref(g), _ptr(index_q), _ptr(w), _ptr(index_pool),
                                                  _ptr(index_scale), _ptr(block_table), _ptr(seq_len),
                                                  C.c_int(B), C.c_int(score_stride), _ptr(rows), _ptr(n_sel),
                                                  _ptr(scratch), _stream(stream)), "index_select_paged")


def launch_dsa_append_select_paged(g: DsaGeom, latent, index_key, row_pos, block_table, latent_pool, latent_scale,
                                   index_pool, index_scale, status, index_q, w, seq_len, B: int, score_stride: int,
                                   rows, n_sel, scratch, stream=None) -> None:
    ensure_status(lib().rivoli_dsa_append_select_paged(
        C.byref(g), _ptr(latent), _ptr(index_key), _ptr(row_pos), _ptr(block_table), _ptr(latent_pool),
        _ptr(latent_scale), _ptr(index_pool), _ptr(index_scale), _ptr(status), _ptr(index_q), _ptr(w), _ptr(seq_len),
        C.c_int(B), C.c_int(score_stride), _ptr(rows), _ptr(n_sel), _ptr(scratch), _stream(stream)),
        "dsa_append_select_paged")


def launch_dsa_decode_step_paged(g: DsaGeom, latent, index_key, row_pos, block_table, latent_pool, latent_scale,
                                 index_pool, index_scale, status, index_q, w, seq_len, B: int, score_stride: int,
                                 rows, n_sel, select_scratch, q, out, out_m, out_lse, attend_scratch,
                                 min_rows_hint: int = 0, stream=None) -> None:
    """One decode layer-step in one call: append, select, attend (``rivoli_dsa_decode_step_paged``)."""
    ensure_status(lib().rivoli_dsa_decode_step_paged(
        C.byref(g), _ptr(latent), _ptr(index_key), _ptr(row_pos), _ptr(block_table), _ptr(latent_pool),
        _ptr(latent_scale), _ptr(index_pool), _ptr(index_scale), _ptr(status), _ptr(index_q), _ptr(w), _ptr(seq_len),
        C.c_int(B), C.c_int(score_stride), _ptr(rows), _ptr(n_sel), _ptr(select_scratch), _ptr(q), _ptr(out),
        _ptr(out_m), _ptr(out_lse), _ptr(attend_scratch), C.c_int(min_rows_hint), _stream(stream)),
        "dsa_decode_step_paged")


class DsaStepState(C.Structure):
    """``DsaStepState`` of include/rivoli_kernels.h: the device pointers of one layer."""
    _fields_ = [(n, C.c_void_p) for n in (
        "block_table", "latent_pool", "latent_scale", "index_pool", "index_scale", "status", "rows", "n_sel",
        "select_scratch", "attend_scratch", "out_m", "out_lse")] + [("score_stride", C.c_int32),
                                                                      ("min_rows_hint", C.c_int32)]


class StepPipe:
    """Handle of the library's host-buffer step pipeline (``rivoli_step_pipe_*`` / ``rivoli_dsa_step_host``)."""

    def __init__(self, g: DsaGeom, B: int, depth: int = 2):
        L = lib()
        L.rivoli_step_pipe_create.restype = C.c_void_p
        L.rivoli_step_pipe_stream.restype = C.c_void_p
        L.rivoli_step_pipe_input_bytes.restype = C.c_size_t
        L.rivoli_step_pipe_output_bytes.restype = C.c_size_t
        L.rivoli_dsa_step_host.restype = C.c_longlong
        self._h = C.c_void_p(L.rivoli_step_pipe_create(C.byref(g), C.c_int(B), C.c_int(depth)))
        if not self._h:
            raise BackendError("step_pipe_create", 1008)
        self.g, self.B, self.depth = g, B, depth
        self.input_bytes = int(L.rivoli_step_pipe_input_bytes(C.byref(g), C.c_int(B)))
        self.output_bytes = int(L.rivoli_step_pipe_output_bytes(C.byref(g), C.c_int(B)))
        off = (C.c_size_t * 5)()
        ensure_status(L.rivoli_step_pipe_input_offsets(C.byref(g), C.c_int(B), off), "step_pipe_input_offsets")
        self.offsets = dict(zip(("latent", "index_key", "index_q", "index_w", "q"), (int(o) for o in off)))

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                lib().rivoli_step_pipe_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def submit(self, state: DsaStepState, host_in, host_out, row_pos, seq_len) -> int:
        t = int(lib().rivoli_dsa_step_host(self._h, C.byref(state), _ptr(host_in), _ptr(host_out), _ptr(row_pos),
                                           _ptr(seq_len)))
        if t < 0:
            raise BackendError("dsa_step_host", -t if -t >= 1000 else t)
        return t

    def wait(self, ticket: int) -> None:
        ensure_status(lib().rivoli_step_pipe_wait(self._h, C.c_longlong(ticket)), "step_pipe_wait")

    def drain(self) -> None:
        ensure_status(lib().rivoli_step_pipe_drain(self._h), "step_pipe_drain")

    def leg_ms(self):
        ms = (C.c_float * 3)()
        ensure_status(lib().rivoli_step_pipe_leg_ms(self._h, ms), "step_pipe_leg_ms")
        return {"upload": float(ms[0]), "kernels_after_upload": float(ms[1]), "download_after_kernels": float(ms[2])}

    def stream(self, which: int) -> int:
        return int(lib().rivoli_step_pipe_stream(self._h, C.c_int(which)) or 0)


def index_select_status(g: DsaGeom, B: int, score_stride: int, scratch, stream=None) -> None:
    """Synchronises; raises BackendError(1008) if a bounded device-side wait gave up, (1005) if a block-table
    entry inside a sequence pointed outside the pool."""
    ensure_status(lib().rivoli_index_select_status(C.byref(g), C.c_int(B), C.c_int(score_stride), _ptr(scratch),
                                                   _stream(stream)), "index_select_status")


def index_select_band_stats(g: DsaGeom, B: int, score_stride: int, scratch, stream=None):
    import numpy as np
    out = np.zeros(B, dtype=np.uint32)
    ensure_status(lib().rivoli_index_select_band_stats(C.byref(g), C.c_int(B), C.c_int(score_stride),
                                                       _ptr(scratch), out.ctypes.data_as(C.c_void_p),
                                                       _stream(stream)), "index_select_band_stats")
    return out


def launch_stale_compose_rows(prev_rows, prev_n, cur_rows, cur_n, mode, seq_len, B: int, k: int, out_rows, out_n,
                              stream=None) -> None:
    ensure_status(lib().rivoli_stale_compose_rows(_ptr(prev_rows), _ptr(prev_n), _ptr(cur_rows), _ptr(cur_n), _ptr(mode),
                                                  _ptr(seq_len), C.c_int(B), C.c_int(k), _ptr(out_rows), _ptr(out_n),
                                                  _stream(stream)), "stale_compose_rows")


def attend_paged_scratch_bytes(g: DsaGeom, B: int) -> int:
    return int(lib().rivoli_mla_attend_paged_scratch_bytes(C.byref(g), C.c_int(B)))


def attend_paged_uses_mma(g: DsaGeom) -> bool:
    return bool(lib().rivoli_mla_attend_paged_uses_mma(C.byref(g)))


def attend_paged_status(g: DsaGeom, scratch, stream=None) -> None:
    """Synchronises; raises BackendError(1008) if the tensor-core attention gave up on a wait."""
    ensure_status(lib().rivoli_mla_attend_paged_status(C.byref(g), _ptr(scratch), _stream(stream)),
                  "mla_attend_paged_status")


def step_set_timing_events(events) -> None:
    """``events``: five ``torch.cuda.Event(enable_timing=True)`` objects (already recorded once, so that their
    handles exist) or ``None`` to switch the hook off. See ``rivoli_dsa_step_set_timing_events``."""
    if events is None:
        lib().rivoli_dsa_step_set_timing_events(None)
        return
    arr = (C.c_void_p * 5)(*[C.c_void_p(e.cuda_event) for e in events])
    lib().rivoli_dsa_step_set_timing_events(arr)


def attend_mma_test_hook(min_rows: int = -1, withhold: int = 0, max_polls: int = 0) -> None:
    """Test hook of the tensor-core attention (see include/rivoli_kernels.h); not for production callers."""
    lib().rivoli_attend_mma_test_hook(C.c_int(min_rows), C.c_int(withhold), C.c_int(max_polls))


def index_select_test_cluster(cluster: int = 0) -> None:
    """Test hook: force the selection kernel's cluster size (1, 2, 4, 8; 0 = the library's plan)."""
    lib().rivoli_index_select_test_cluster(C.c_int(cluster))


def attend_simt_scratch_bytes(g: DsaGeom, B: int) -> int:
    return int(lib().rivoli_attend_simt_scratch_bytes(C.byref(g), C.c_int(B)))


def _attend_paged(fn, name, g, q, latent_pool, latent_scale, block_table, rows, row_stride, n_rows, B, out,
                  out_m, out_lse, scratch, stream):
    ensure_status(fn(C.byref(g), _ptr(q), _ptr(latent_pool), _ptr(latent_scale), _ptr(block_table),
                     _ptr(rows), C.c_int(row_stride), _ptr(n_rows), C.c_int(B), _ptr(out), _ptr(out_m),
                     _ptr(out_lse), _ptr(scratch), _stream(stream)), name)


def launch_attend_paged_bf16(g: DsaGeom, q, latent_pool, latent_scale, block_table, rows, row_stride: int,
                             n_rows, B: int, out, out_m=None, out_lse=None, scratch=None, stream=None) -> None:
    _attend_paged(lib().rivoli_mla_attend_paged_bf16, "mla_attend_paged_bf16", g, q, latent_pool,
                  latent_scale, block_table, rows, row_stride, n_rows, B, out, out_m, out_lse, scratch, stream)


def launch_attend_simt_paged_bf16(g: DsaGeom, q, latent_pool, latent_scale, block_table, rows,
                                  row_stride: int, n_rows, B: int, out, out_m=None, out_lse=None,
                                  scratch=None, stream=None) -> None:
    _attend_paged(lib().rivoli_attend_simt_paged_bf16, "attend_simt_paged_bf16", g, q, latent_pool,
                  latent_scale, block_table, rows, row_stride, n_rows, B, out, out_m, out_lse, scratch, stream)


def launch_attend_merge_partials(part_out, part_lse, G: int, n_vec: int, kvl: int, out, stream=None) -> None:
    ensure_status(lib().rivoli_attend_merge_partials(_ptr(part_out), _ptr(part_lse), C.c_int(G),
                                                     C.c_int(n_vec), C.c_int(kvl), _ptr(out),
                                                     _stream(stream)), "attend_merge_partials")


# --- page-range sharded step --------------------------------------------------------------------------------
def shard_candidate_bytes(g: DsaGeom, B: int) -> int:
    f = lib().rivoli_shard_candidate_bytes
    f.restype = C.c_size_t
    return int(f(C.byref(g), C.c_int(B)))


def shard_partial_bytes(g: DsaGeom, B: int) -> int:
    f = lib().rivoli_shard_partial_bytes
    f.restype = C.c_size_t
    return int(f(C.byref(g), C.c_int(B)))


def shard_scratch_bytes(g: DsaGeom, B: int, world: int) -> int:
    f = lib().rivoli_shard_scratch_bytes
    f.restype = C.c_size_t
    return int(f(C.byref(g), C.c_int(B), C.c_int(world)))


def launch_shard_candidates(g: DsaGeom, index_q, w, index_pool, index_scale, block_table, local_len, B: int,
                            score_stride: int, rows_l, select_scratch, cand, stream=None) -> None:
    ensure_status(lib().rivoli_shard_candidates(C.byref(g), _ptr(index_q), _ptr(w), _ptr(index_pool), _ptr(index_scale),
                                                _ptr(block_table), _ptr(local_len), C.c_int(B), C.c_int(score_stride),
                                                _ptr(rows_l), _ptr(select_scratch), _ptr(cand), _stream(stream)),
                  "shard_candidates")


def launch_shard_cut_attend(g: DsaGeom, all_cand, rank: int, world: int, rows_l, q, latent_pool, latent_scale,
                            block_table, B: int, rows_att, n_mine, part, shard_scratch, attend_scratch,
                            stream=None) -> None:
    ensure_status(lib().rivoli_shard_cut_attend(C.byref(g), _ptr(all_cand), C.c_int(rank), C.c_int(world), _ptr(rows_l),
                                                _ptr(q), _ptr(latent_pool), _ptr(latent_scale), _ptr(block_table),
                                                C.c_int(B), _ptr(rows_att), _ptr(n_mine), _ptr(part), _ptr(shard_scratch),
                                                _ptr(attend_scratch), _stream(stream)), "shard_cut_attend")


def launch_shard_merge(g: DsaGeom, all_part, world: int, B: int, out, stream=None) -> None:
    ensure_status(lib().rivoli_shard_merge(C.byref(g), _ptr(all_part), C.c_int(world), C.c_int(B), _ptr(out),
                                           _stream(stream)), "shard_merge")


def launch_shard_step_paged(g: DsaGeom, comm: int, rank: int, world: int, index_q, w, q, latent_pool, latent_scale,
                            index_pool, index_scale, block_table, local_len, B: int, score_stride: int, rows_l,
                            rows_att, n_mine, out, select_scratch, attend_scratch, shard_scratch, stream=None) -> None:
    ensure_status(lib().rivoli_shard_step_paged(
        C.byref(g), C.c_void_p(comm or 0), C.c_int(rank), C.c_int(world), _ptr(index_q), _ptr(w), _ptr(q),
        _ptr(latent_pool), _ptr(latent_scale), _ptr(index_pool), _ptr(index_scale), _ptr(block_table), _ptr(local_len),
        C.c_int(B), C.c_int(score_stride), _ptr(rows_l), _ptr(rows_att), _ptr(n_mine), _ptr(out), _ptr(select_scratch),
        _ptr(attend_scratch), _ptr(shard_scratch), _stream(stream)), "shard_step_paged")


def shard_nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    ensure_status(lib().rivoli_shard_nccl_unique_id(buf), "shard_nccl_unique_id")
    return buf.raw


def shard_nccl_comm_create(unique_id: bytes, rank: int, world: int) -> int:
    comm = C.c_void_p(0)
    ensure_status(lib().rivoli_shard_nccl_comm_create(C.c_char_p(unique_id), C.c_int(rank), C.c_int(world),
                                                      C.byref(comm)), "shard_nccl_comm_create")
    return int(comm.value or 0)


def shard_nccl_comm_destroy(comm: int) -> None:
    ensure_status(lib().rivoli_shard_nccl_comm_destroy(C.c_void_p(comm)), "shard_nccl_comm_destroy")


# --- Part 3: host page allocator ----------------------------------------------------------------------
class PagePool:
    """LIFO page allocator + per-sequence block tables (host memory; C++ ``rivoli::PagePool``)."""

    def __init__(self, n_pages: int, n_seqs: int, max_pages_per_seq: int, page_tokens: int):
        self._h = C.c_void_p(lib().rivoli_pagepool_create(C.c_int(n_pages), C.c_int(n_seqs),
                                                          C.c_int(max_pages_per_seq), C.c_int(page_tokens)))
        if not self._h:
            raise BackendError("pagepool_create", 1001)
        self.n_pages, self.n_seqs = n_pages, n_seqs
        self.max_pages_per_seq, self.page_tokens = max_pages_per_seq, page_tokens

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                lib().rivoli_pagepool_destroy(self._h)
                self._h = None
        except Exception:   # interpreter shutdown: module globals may already be gone
            pass

    def shuffle(self, seed: int) -> None:
        lib().rivoli_pagepool_shuffle(self._h, C.c_uint64(seed))

    def reserve(self, seq: int, n_tokens: int) -> None:
        ensure_status(lib().rivoli_pagepool_reserve(self._h, C.c_int(seq), C.c_int(n_tokens)), "pagepool_reserve")

    def release(self, seq: int) -> None:
        ensure_status(lib().rivoli_pagepool_release(self._h, C.c_int(seq)), "pagepool_release")

    @property
    def n_free(self) -> int:
        return int(lib().rivoli_pagepool_n_free(self._h))

    def seq_pages(self, seq: int) -> int:
        return int(lib().rivoli_pagepool_seq_pages(self._h, C.c_int(seq)))

    def block_table(self):
        import numpy as np
        p = lib().rivoli_pagepool_block_table(self._h)
        return np.ctypeslib.as_array(p, shape=(self.n_seqs, self.max_pages_per_seq)).copy()

    def free_list(self):
        import numpy as np
        n = self.n_free
        if n == 0:
            return np.zeros(0, dtype=np.int32)
        p = lib().rivoli_pagepool_free_list(self._h)
        return np.ctypeslib.as_array(p, shape=(n,)).copy()


def launch_mla_absorb(q, kvb, kvb_scale, H: int, qh: int, nope: int, vh: int, kvl: int, block: int, nrow: int,
                      qabs) -> None:
    ensure_status(lib().rivoli_mla_absorb_fp8(_ptr(q), _ptr(kvb), _ptr(kvb_scale), C.c_int(H), C.c_int(qh),
                                              C.c_int(nope), C.c_int(vh), C.c_int(kvl), C.c_int(block), C.c_int(nrow),
                                              _ptr(qabs)), "mla_absorb_fp8")


def launch_mla_value(clat, kvb, kvb_scale, H: int, nope: int, vh: int, kvl: int, block: int, nrow: int, ctx) -> None:
    ensure_status(lib().rivoli_mla_value_fp8(_ptr(clat), _ptr(kvb), _ptr(kvb_scale), C.c_int(H), C.c_int(nope),
                                             C.c_int(vh), C.c_int(kvl), C.c_int(block), C.c_int(nrow), _ptr(ctx)),
                  "mla_value_fp8")


def launch_mla_absorb_batched_bf16(q, kvb, kvb_scale, H: int, qh: int, nope: int, vh: int, kvl: int, rope: int,
                                   block: int, B: int, q_abs, force_simt: bool = False, stream=None) -> None:
    ensure_status(lib().rivoli_mla_absorb_batched_bf16(_ptr(q), _ptr(kvb), _ptr(kvb_scale), C.c_int(H), C.c_int(qh),
                                                       C.c_int(nope), C.c_int(vh), C.c_int(kvl), C.c_int(rope),
                                                       C.c_int(block), C.c_int(B), _ptr(q_abs), C.c_int(int(force_simt)),
                                                       _stream(stream)), "mla_absorb_batched_bf16")


def launch_mla_value_batched_bf16(clat, kvb, kvb_scale, H: int, nope: int, vh: int, kvl: int, block: int, B: int, ctx,
                                  force_simt: bool = False, stream=None) -> None:
    ensure_status(lib().rivoli_mla_value_batched_bf16(_ptr(clat), _ptr(kvb), _ptr(kvb_scale), C.c_int(H), C.c_int(nope),
                                                      C.c_int(vh), C.c_int(kvl), C.c_int(block), C.c_int(B), _ptr(ctx),
                                                      C.c_int(int(force_simt)), _stream(stream)),
                  "mla_value_batched_bf16")


def kvb_proj_status(stream=None) -> None:
    ensure_status(lib().rivoli_kvb_proj_status(_stream(stream)), "kvb_proj(status)")


class IndexFrontGeom(C.Structure):
    """``repr(C)`` mirror of ``IndexFrontGeom`` (include/rivoli_kernels.h)."""
    _fields_ = [(n, C.c_int32) for n in ("hidden", "q_lora", "index_heads", "index_dim", "rope_off", "rope_seg", "block")] + \
               [("eps", C.c_float), ("theta", C.c_double)]


def launch_gemv_fp8(x, packed, scale, o_dim: int, i_dim: int, block: int, nrow: int, y) -> None:
    ensure_status(lib().rivoli_gemv_fp8(_ptr(x), _ptr(packed), _ptr(scale), C.c_int(o_dim), C.c_int(i_dim), C.c_int(block),
                                        C.c_int(nrow), _ptr(y)), "gemv_fp8")


def launch_layernorm(x, w, b, n: int, eps: float, y) -> None:
    ensure_status(lib().rivoli_layernorm(_ptr(x), _ptr(w), _ptr(b), C.c_int(n), C.c_float(eps), _ptr(y)), "layernorm")


def launch_rope_interleave(base, count: int, stride: int, seg: int, pos: int, theta: float) -> None:
    ensure_status(lib().rivoli_rope_interleave(_ptr(base), C.c_int(count), C.c_int(stride), C.c_int(seg), C.c_int(pos),
                                               C.c_double(theta)), "rope_interleave")


def index_frontend_scratch_bytes(g: IndexFrontGeom, B: int) -> int:
    return int(lib().rivoli_index_frontend_scratch_bytes(C.byref(g), C.c_int(B)))


def launch_index_frontend_bf16(g: IndexFrontGeom, x, q_resid, pos, B: int, wk, wk_scale, knorm_w, knorm_b, wq_b, wq_b_scale,
                               wproj, wproj_scale, index_key, index_q, index_w, scratch, force_simt: bool = False,
                               stream=None) -> None:
    ensure_status(lib().rivoli_index_frontend_bf16(
        C.byref(g), _ptr(x), _ptr(q_resid), _ptr(pos), C.c_int(B), _ptr(wk), _ptr(wk_scale), _ptr(knorm_w), _ptr(knorm_b),
        _ptr(wq_b), _ptr(wq_b_scale), _ptr(wproj), _ptr(wproj_scale), _ptr(index_key), _ptr(index_q), _ptr(index_w),
        _ptr(scratch), C.c_int(int(force_simt)), _stream(stream)), "index_frontend_bf16")


def index_frontend_status(stream=None) -> None:
    ensure_status(lib().rivoli_index_frontend_status(_stream(stream)), "index_frontend(status)")


class V4Geom(C.Structure):
    """``V4Geom`` of include/rivoli_kernels.h: the V4 cousin path's batched decode geometry."""
    _fields_ = [(n, C.c_int32) for n in (
        "n_heads", "head_dim", "window", "index_heads", "index_dim", "index_topk", "ratio", "max_comp")] + [
        ("softmax_scale", C.c_float)]

    @classmethod
    def make(cls, *, n_heads=64, head_dim=512, window=128, index_heads=64, index_dim=128, index_topk=512, ratio=4,
             max_comp, softmax_scale=None) -> "V4Geom":
        import numpy as np
        return cls(n_heads, head_dim, window, index_heads, index_dim, index_topk, ratio, max_comp,
                   float(np.float32(head_dim) ** np.float32(-0.5)) if softmax_scale is None else softmax_scale)


def launch_act_quant_f4_rotated(x, rows: int, d: int, stream=None) -> None:
    """crates/backend/src/hip.rs launcher of ``rivoli_act_quant_f4_rotated`` (in place on f32 rows)."""
    ensure_status(lib().rivoli_act_quant_f4_rotated(_ptr(x), C.c_int(rows), C.c_int(d), _stream(stream)),
                  "act_quant_f4_rotated")


def launch_index_score_blocks(q, kv, w, score, s: int, n_comp: int, heads: int, hd: int, stream=None) -> None:
    ensure_status(lib().rivoli_index_score_blocks(_ptr(q), _ptr(kv), _ptr(w), _ptr(score), C.c_int(s), C.c_int(n_comp),
                                                  C.c_int(heads), C.c_int(hd), _stream(stream)), "index_score_blocks")


def launch_gather_attn_shared_kv(q, kv, sink, idxs, m: int, h: int, d: int, topk: int, scale: float, o,
                                 stream=None) -> None:
    ensure_status(lib().rivoli_gather_attn_shared_kv(_ptr(q), _ptr(kv), _ptr(sink), _ptr(idxs), C.c_int(m), C.c_int(h),
                                                     C.c_int(d), C.c_int(topk), C.c_float(scale), _ptr(o),
                                                     _stream(stream)), "gather_attn_shared_kv")


def v4_select_scratch_bytes(g: V4Geom, n_seqs: int) -> int:
    return int(lib().rivoli_v4_select_scratch_bytes(C.byref(g), C.c_int(n_seqs)))


def launch_v4_select_blocks_bf16(g: V4Geom, n_seqs: int, pos, index_q, index_w, index_kv, sel, scratch,
                                 force_fold: bool = False, packed=None, packed_exp=None, stream=None) -> None:
    ensure_status(lib().rivoli_v4_select_blocks_bf16(C.byref(g), C.c_int(n_seqs), _ptr(pos), _ptr(index_q), _ptr(index_w),
                                                     _ptr(index_kv), _ptr(packed), _ptr(packed_exp), _ptr(sel),
                                                     _ptr(scratch), C.c_int(int(force_fold)), _stream(stream)),
                  "v4_select_blocks_bf16")


def launch_v4_index_pack_bf16(g: V4Geom, n_seqs: int, row_begin, row_end, max_rows: int, index_kv, packed, packed_exp,
                              stream=None) -> None:
    ensure_status(lib().rivoli_v4_index_pack_bf16(C.byref(g), C.c_int(n_seqs), _ptr(row_begin), _ptr(row_end),
                                                  C.c_int(max_rows), _ptr(index_kv), _ptr(packed), _ptr(packed_exp),
                                                  _stream(stream)), "v4_index_pack_bf16")


def launch_v4_sparse_attend_bf16(g: V4Geom, n_seqs: int, q, kv_cache, sink, sel, cols: int, out,
                                 force_simt: bool = False, stream=None) -> None:
    ensure_status(lib().rivoli_v4_sparse_attend_bf16(C.byref(g), C.c_int(n_seqs), _ptr(q), _ptr(kv_cache), _ptr(sink),
                                                     _ptr(sel), C.c_int(cols), _ptr(out), C.c_int(int(force_simt)),
                                                     _stream(stream)), "v4_sparse_attend_bf16")


class CompGeom(C.Structure):
    """``CompGeom`` of include/rivoli_kernels.h (the reference's crates/backend/src/abi.rs:24-45)."""
    _fields_ = [(n, C.c_int32) for n in ("ratio", "coff", "d", "cd", "ents", "rd")] + [("eps", C.c_float)]

    @classmethod
    def make(cls, *, ratio=4, d=512, rd=64, eps=1e-6) -> "CompGeom":
        coff = 2 if ratio == 4 else 1
        return cls(ratio, coff, d, coff * d, coff * ratio, rd, eps)


class CompFinish(C.Structure):
    _fields_ = [("norm", C.c_void_p), ("freqs", C.c_void_p), ("out", C.c_void_p)]


def launch_act_quant_f8_prefix(src, dst, rows: int, row_stride: int, n: int, block: int, stream=None) -> None:
    ensure_status(lib().rivoli_act_quant_f8_prefix(_ptr(src), _ptr(dst), C.c_int(rows), C.c_int(row_stride), C.c_int(n),
                                                   C.c_int(block), _stream(stream)), "act_quant_f8_prefix")


def launch_kv_compress_deposit(kv, score, ape, kv_state, score_state, p: CompGeom, s: int, slot0: int, stream=None) -> None:
    ensure_status(lib().rivoli_kv_compress_deposit(_ptr(kv), _ptr(score), _ptr(ape), _ptr(kv_state), _ptr(score_state),
                                                   C.byref(p) if p is not None else None, C.c_int(s), C.c_int(slot0),
                                                   _stream(stream)), "kv_compress_deposit")


def launch_kv_compress_prefill(kv, score, ape, norm, freqs, out, p: CompGeom, nblk: int, stream=None) -> None:
    f = CompFinish(_ptr(norm), _ptr(freqs), _ptr(out))
    ensure_status(lib().rivoli_kv_compress_prefill(_ptr(kv), _ptr(score), _ptr(ape), C.byref(f), C.byref(p), C.c_int(nblk),
                                                   _stream(stream)), "kv_compress_prefill")


def launch_kv_compress_decode(kv_state, score_state, norm, freqs, out, p: CompGeom, start_pos: int, stream=None) -> None:
    f = CompFinish(_ptr(norm), _ptr(freqs), _ptr(out))
    ensure_status(lib().rivoli_kv_compress_decode(_ptr(kv_state), _ptr(score_state), C.byref(f), C.byref(p),
                                                  C.c_int(start_pos), _stream(stream)), "kv_compress_decode")


def launch_v4_compress_step_bf16(p: CompGeom, n_seqs: int, pos, kv_proj, score_proj, ape, kv_state, score_state, norm,
                                 freqs, rotate: bool, cache, cache_rows: int, cache_row0: int, prequant=None,
                                 packed=None, packed_exp=None, stream=None) -> None:
    ensure_status(lib().rivoli_v4_compress_step_bf16(
        C.byref(p), C.c_int(n_seqs), _ptr(pos), _ptr(kv_proj), _ptr(score_proj), _ptr(ape), _ptr(kv_state),
        _ptr(score_state), _ptr(norm), _ptr(freqs), C.c_int(int(rotate)), _ptr(cache), C.c_int(cache_rows),
        C.c_int(cache_row0), _ptr(prequant), _ptr(packed), _ptr(packed_exp), _stream(stream)), "v4_compress_step_bf16")


def kernels_arch() -> str:
    return lib().rivoli_kernels_arch().decode()
