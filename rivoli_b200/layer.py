"""One MLA + DSA decode layer's KV-cache path on one GPU: the caller side of the operator
surface, i.e. what ``crates/engine/src/glm/attn.rs:119-222`` does for this path (append the
new token, select rows with the lightning indexer, attend), batched over sequences and
paged.

The layer owns the device pools and the per-step scratch; every buffer is allocated once
in ``__init__`` (the reference allocates all KV slabs and scratch once in
``GlmEngine::new``, crates/engine/src/glm/engine.rs:139-260) and a step allocates nothing.
torch is used for device memory and streams only; all arithmetic is in the CUDA library.
"""
from __future__ import annotations

import numpy as np
import torch

from . import backend as be


class DsaDecodeLayer:
    """Device state of one layer for a batch of ``n_seqs`` sequences.

    Call order per layer-step (the operator order the reference documents for a full
    indexer layer, docs/investigations/rewrite.md:135-137): ``append`` -> ``select`` ->
    ``attend``; ``step`` does the three in order on the current stream.
    """

    def __init__(self, geom: be.DsaGeom, n_seqs: int, device="cuda:0", max_ctx: int | None = None,
                 shuffle_seed: int | None = None, pool: "be.PagePool | None" = None):
        """``pool``: a page allocator shared with other layers of the same model (page ``p`` then names
        row block ``p`` of every layer's pools and paging is done once per step, not per layer);
        by default the layer owns one."""
        be.lib()  # fail loudly if the CUDA library is missing
        self.g = geom
        self.B = n_seqs
        self.dev = torch.device(device)
        P = geom.page_tokens
        self.max_ctx = max_ctx if max_ctx is not None else geom.max_pages_per_seq * P
        rows = geom.n_pool_pages * P
        W = geom.kv_lora + geom.rope_dim
        u8, f32, i32 = torch.uint8, torch.float32, torch.int32
        d = self.dev
        self.latent_pool = torch.zeros(rows * W, dtype=u8, device=d)
        self.latent_scale = torch.zeros(rows, dtype=f32, device=d)
        self.index_pool = torch.zeros(rows * geom.index_dim, dtype=u8, device=d)
        self.index_scale = torch.zeros(rows, dtype=f32, device=d)
        self.block_table = torch.full((n_seqs, geom.max_pages_per_seq), -1, dtype=i32, device=d)
        self.pool = pool if pool is not None else be.PagePool(geom.n_pool_pages, n_seqs, geom.max_pages_per_seq, P)
        if shuffle_seed is not None and pool is None:
            self.pool.shuffle(shuffle_seed)
        # per-step scratch
        self.score_stride = self.max_ctx
        self.scores = torch.zeros((n_seqs, self.score_stride), dtype=f32, device=d)
        self.qcodes = torch.zeros(n_seqs * geom.index_heads * geom.index_dim, dtype=u8, device=d)
        self.qscales = torch.zeros(n_seqs * geom.index_heads, dtype=f32, device=d)
        self.rows = torch.zeros((n_seqs, geom.top_k), dtype=torch.int32, device=d)  # u32 payload
        self.n_sel = torch.zeros(n_seqs, dtype=i32, device=d)
        self.status = torch.zeros(1, dtype=i32, device=d)
        self.out = torch.zeros((n_seqs, geom.n_heads, geom.kv_lora), dtype=torch.bfloat16, device=d)
        self.out_m = torch.zeros((n_seqs, geom.n_heads), dtype=f32, device=d)
        self.out_lse = torch.zeros((n_seqs, geom.n_heads), dtype=f32, device=d)
        nbytes = max(be.attend_paged_scratch_bytes(geom, n_seqs), 16)
        self.scratch = torch.zeros(nbytes, dtype=u8, device=d)
        self.select_scratch = torch.zeros(be.index_select_scratch_bytes(geom, n_seqs, self.score_stride),
                                          dtype=u8, device=d)

    # --- paging -------------------------------------------------------------------------------------
    def reserve(self, seq: int, n_tokens: int) -> None:
        self.pool.reserve(seq, n_tokens)

    def release(self, seq: int) -> None:
        self.pool.release(seq)

    def upload_block_table(self, table: "np.ndarray | None" = None, non_blocking: bool = False) -> None:
        bt = torch.from_numpy(self.pool.block_table() if table is None else table)
        self.block_table.copy_(bt, non_blocking=non_blocking)

    # --- operators ----------------------------------------------------------------------------------
    def append(self, latent: torch.Tensor, index_key: torch.Tensor, row_pos: torch.Tensor,
               row_seq: torch.Tensor | None = None, stream=None) -> None:
        """Quantise and store ``n`` new tokens (bf16 ``[n, kv_lora+rope]`` and ``[n, index_dim]``)."""
        n = latent.shape[0]
        be.launch_kv_append_paged(self.g, latent, index_key, row_seq, row_pos, n, self.block_table,
                                  self.latent_pool, self.latent_scale, self.index_pool, self.index_scale,
                                  self.status, stream)

    def select(self, index_q: torch.Tensor, index_w: torch.Tensor, seq_len: torch.Tensor, stream=None) -> None:
        """Indexer: quantise q, score every cached key, exact top-k -> ``rows``/``n_sel``
        (tensor-core scorer with exact refinement at the cut where the geometry allows)."""
        be.launch_index_select_paged(self.g, index_q, index_w, self.index_pool, self.index_scale,
                                     self.block_table, seq_len, self.B, self.score_stride, self.rows,
                                     self.n_sel, self.select_scratch, stream)

    def select_unfused(self, index_q: torch.Tensor, index_w: torch.Tensor, seq_len: torch.Tensor,
                       stream=None) -> None:
        """The same selection through the three separate operators on CUDA cores."""
        g = self.g
        be.launch_index_q_quant(index_q, self.B * g.index_heads, g.index_dim, self.qcodes, self.qscales, stream)
        be.launch_index_score_paged(g, self.qcodes, self.qscales, index_w, self.index_pool, self.index_scale,
                                    self.block_table, seq_len, self.B, self.scores, self.score_stride, stream)
        be.launch_index_topk_batched(self.scores, self.score_stride, seq_len, self.B, g.top_k, self.rows,
                                     self.n_sel, stream)

    def append_latent_only(self, latent: torch.Tensor, row_pos: torch.Tensor, stream=None) -> None:
        """Cache the step's latent rows of a layer that owns no indexer: the index key that travels with the
        operator is a constant zero row written to this layer's (unused) index pool."""
        n = latent.shape[0]
        if getattr(self, "_zero_key", None) is None or self._zero_key.shape[0] != n:
            self._zero_key = torch.zeros((n, self.g.index_dim), dtype=torch.bfloat16, device=self.dev)
        self.append(latent, self._zero_key, row_pos, None, stream)

    def attend(self, q: torch.Tensor, stream=None, dense_len: torch.Tensor | None = None,
               out: torch.Tensor | None = None, rows_from: "DsaDecodeLayer | None" = None) -> torch.Tensor:
        """Attention over the selected rows (or, with ``dense_len``, over the whole prefix).
        Writes ``self.out`` unless another bf16 ``[B, H, kv_lora]`` buffer is given. ``rows_from``:
        attend over another layer's selection (a layer that shares its predecessor's indexer)."""
        out = self.out if out is None else out
        sel = self if rows_from is None else rows_from
        if dense_len is not None:
            be.launch_attend_paged_bf16(self.g, q, self.latent_pool, self.latent_scale, self.block_table,
                                        None, 0, dense_len, self.B, out, self.out_m, self.out_lse,
                                        self.scratch, stream)
        else:
            be.launch_attend_paged_bf16(self.g, q, self.latent_pool, self.latent_scale, self.block_table,
                                        sel.rows, self.g.top_k, sel.n_sel, self.B, out, self.out_m,
                                        self.out_lse, self.scratch, stream)
        return out

    def step(self, latent, index_key, index_q, index_w, q, row_pos, seq_len, stream=None,
             out: torch.Tensor | None = None, min_rows_hint: int = 0) -> torch.Tensor:
        """One layer-step in one library call: append one token per sequence, select, attend (the append
        rides in the launch that prepares the indexer query; the attention kernel converts ``q`` while the
        selection is still running, which the one-call form makes safe). ``min_rows_hint``: a lower bound the
        caller's scheduler knows for ``min(top_k, seq_len)`` over the batch (0 = unknown)."""
        out = self.out if out is None else out
        be.launch_dsa_decode_step_paged(self.g, latent, index_key, row_pos, self.block_table, self.latent_pool,
                                        self.latent_scale, self.index_pool, self.index_scale, self.status,
                                        index_q, index_w, seq_len, self.B, self.score_stride, self.rows,
                                        self.n_sel, self.select_scratch, q, out, self.out_m, self.out_lse,
                                        self.scratch, min_rows_hint, stream)
        return out

    def check_status(self) -> None:
        """Raise if a kernel flagged a bad block-table entry since the last check (syncs)."""
        be.index_select_status(self.g, self.B, self.score_stride, self.select_scratch)
        be.attend_paged_status(self.g, self.scratch)
        s = int(self.status.item())
        if s:
            self.status.zero_()
            raise be.BackendError("kv_append_paged(status)", 1005)


class KvbProjection:
    """The two contractions through kv_b either side of attention, batched
    (``crates/engine/src/glm/attn.rs:161-173,231-242`` run them per token): ``absorb`` turns the
    per-head query (nope values + rope segment) into the 576-wide row the attention operator
    consumes, ``value`` projects the attention output to per-head values. Weights are the
    reference's fp8 block-scaled kv_b ``[H*(nope+vh), kvl]`` with one f32 scale per 128x128 block."""

    def __init__(self, geom: be.DsaGeom, n_seqs: int, kvb: torch.Tensor, kvb_scale: torch.Tensor, nope: int, vh: int,
                 block: int = 128):
        self.g, self.B, self.kvb, self.scale = geom, n_seqs, kvb, kvb_scale
        self.nope, self.vh, self.block = nope, vh, block
        self.qh = nope + geom.rope_dim
        d = kvb.device
        self.q_abs = torch.zeros((n_seqs, geom.n_heads, geom.kv_lora + geom.rope_dim), dtype=torch.bfloat16, device=d)
        self.ctx = torch.zeros((n_seqs, geom.n_heads, vh), dtype=torch.bfloat16, device=d)

    def absorb(self, q: torch.Tensor, stream=None) -> torch.Tensor:
        g = self.g
        be.launch_mla_absorb_batched_bf16(q, self.kvb, self.scale, g.n_heads, self.qh, self.nope, self.vh, g.kv_lora,
                                          g.rope_dim, self.block, self.B, self.q_abs, stream=stream)
        return self.q_abs

    def value(self, clat: torch.Tensor, stream=None) -> torch.Tensor:
        g = self.g
        be.launch_mla_value_batched_bf16(clat, self.kvb, self.scale, g.n_heads, self.nope, self.vh, g.kv_lora,
                                         self.block, self.B, self.ctx, stream=stream)
        return self.ctx


class IndexerFrontEnd:
    """Produces what the indexer of a decode layer consumes - index key, index queries and head
    weights - from the layer's hidden state and the compressed query (``crates/backend/kernels/indexer.hip:1-13``),
    batched over sequences. Weights are fp8 block-scaled; ``positions`` are the tokens' positions."""

    def __init__(self, fg: be.IndexFrontGeom, n_seqs: int, weights: dict, device="cuda:0"):
        self.fg, self.B, self.w = fg, n_seqs, weights
        d = torch.device(device)
        self.index_key = torch.zeros((n_seqs, fg.index_dim), dtype=torch.bfloat16, device=d)
        self.index_q = torch.zeros((n_seqs, fg.index_heads, fg.index_dim), dtype=torch.bfloat16, device=d)
        self.index_w = torch.zeros((n_seqs, fg.index_heads), dtype=torch.float32, device=d)
        self.scratch = torch.zeros(max(be.index_frontend_scratch_bytes(fg, n_seqs), 16), dtype=torch.uint8, device=d)

    def run(self, x: torch.Tensor, q_resid: torch.Tensor, positions: torch.Tensor, stream=None, force_simt: bool = False):
        w = self.w
        be.launch_index_frontend_bf16(self.fg, x, q_resid, positions, self.B, w["wk"], w["wk_scale"], w["knorm_w"],
                                      w["knorm_b"], w["wq_b"], w["wq_b_scale"], w["wproj"], w["wproj_scale"],
                                      self.index_key, self.index_q, self.index_w, self.scratch, force_simt, stream)
        return self.index_key, self.index_q, self.index_w


class HostStepPipeline:
    """Layer-steps for a caller whose activations live in HOST memory (pinned): a thin caller of the library's
    ``rivoli_dsa_step_host``. Every step copies ONE packed input buffer host->device, runs the fused decode step
    and copies the attention output device->host; the three legs run on three streams with ``depth`` device-side
    slots inside the library, so the upload of step ``i+1`` and the download of step ``i-1`` overlap the kernels
    of step ``i`` and results equal the serial order.

    ``pack`` lays the five inputs out in one pinned buffer (the layout ``rivoli_step_pipe_input_offsets``
    gives). The caller owns the pinned buffers and must not reuse an output buffer before ``wait(ticket)`` (or
    ``drain()``) has returned for the step that fills it. The layer's pools and the ``row_pos`` / ``seq_len``
    device arrays must be complete before the first ``submit`` (the pipe's streams do not synchronise with
    other streams)."""
    KEYS = ("latent", "index_key", "index_q", "index_w", "q")

    def __init__(self, layer: DsaDecodeLayer, depth: int = 2, min_rows_hint: int = 0):
        self.layer, self.depth = layer, depth
        self.pipe = be.StepPipe(layer.g, layer.B, depth)
        L = layer
        p = lambda t: t.data_ptr()
        self.state = be.DsaStepState(p(L.block_table), p(L.latent_pool), p(L.latent_scale), p(L.index_pool),
                                     p(L.index_scale), p(L.status), p(L.rows), p(L.n_sel), p(L.select_scratch),
                                     p(L.scratch), p(L.out_m), p(L.out_lse), L.score_stride, min_rows_hint)

    def new_input_buffer(self) -> torch.Tensor:
        return torch.zeros(self.pipe.input_bytes, dtype=torch.uint8).pin_memory()

    def new_output_buffer(self) -> torch.Tensor:
        g = self.layer.g
        return torch.zeros((self.layer.B, g.n_heads, g.kv_lora), dtype=torch.bfloat16).pin_memory()

    def pack(self, host_in: dict, buf: torch.Tensor | None = None) -> torch.Tensor:
        """Copy the five host tensors into one packed pinned buffer (host-side memcpy)."""
        buf = self.new_input_buffer() if buf is None else buf
        for k in self.KEYS:
            src = host_in[k].contiguous().view(torch.uint8).reshape(-1)
            o = self.pipe.offsets[k]
            buf[o:o + src.numel()].copy_(src)
        return buf

    def submit(self, packed_in: torch.Tensor, host_out: torch.Tensor, row_pos: torch.Tensor, seq_len: torch.Tensor) -> int:
        """Enqueue one layer-step; returns a ticket for ``wait``. Never blocks the host."""
        return self.pipe.submit(self.state, packed_in, host_out, row_pos, seq_len)

    def wait(self, ticket: int) -> None:
        self.pipe.wait(ticket)

    def drain(self) -> None:
        self.pipe.drain()

    def leg_ms(self):
        return self.pipe.leg_ms()


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> numpy uint16 bit patterns (host)."""
    return t.detach().cpu().view(torch.int16).numpy().view(np.uint16)
