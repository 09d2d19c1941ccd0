"""Engine-side wiring of DSA across the layers of a model: which layers own an indexer, which
reuse their predecessor's selection, and the optional one-step-stale selection.

Mirrors the reference's host logic for this: the per-layer ``indexer_types`` ("full" owns an
indexer, "shared" reuses the nearest preceding full layer's rows;
``crates/artifact/src/glm_config.rs:176-209``) and the lag-by-one ``StaleShare`` state machine
(``crates/engine/src/indexer.rs:14-63``). The reference has not wired the indexer into its GLM
decode loop yet (``crates/core/src/legality.rs:333-335``); the call order here is the one its
design note gives (``docs/investigations/rewrite.md:135-137``): append, then - on full layers only -
score and top-k, then attention over the layer's (own or inherited) rows.
"""
from __future__ import annotations

import torch

from . import backend as be
from .layer import DsaDecodeLayer


def indexer_layout(indexer_types, n_layers: int, index_n_heads: int, index_head_dim: int, index_topk: int) -> list[bool]:
    """Validate the indexer configuration; returns per-layer flags (True = full). Same rejections as the
    reference: missing dims, wrong length, unknown type, shared first layer."""
    if 0 in (index_n_heads, index_head_dim, index_topk):
        raise ValueError("config has no DSA indexer dims (index_n_heads/index_head_dim/index_topk)")
    if len(indexer_types) != n_layers:
        raise ValueError(f"indexer_types has {len(indexer_types)} entries, expected n_layers={n_layers}")
    full = []
    for t in indexer_types:
        if t not in ("full", "shared"):
            raise ValueError(f"unknown indexer type {t!r}")
        full.append(t == "full")
    if not full[0]:
        raise ValueError("layer 0 is 'shared' but has no preceding full layer")
    return full


class StaleShare:
    """Row count of the selection each indexer slab stored at the PREVIOUS token, per sequence slot (``None`` =
    nothing stored: serve dense). Read with ``stored`` before ``store`` overwrites it - what token ``t`` serves
    is what token ``t-1`` computed (the reference's lag-by-one state machine, ``crates/engine/src/indexer.rs:14-63``,
    kept per sequence of the batch; with ``n_seqs = 1`` it is that type)."""

    def __init__(self, n_slabs: int, n_seqs: int = 1):
        self.n_seqs = n_seqs
        self.nr: list[list[int | None]] = [[None] * n_seqs for _ in range(n_slabs)]

    def stored(self, slab: int, seq: int = 0):
        return self.nr[slab][seq]

    def store(self, slab: int, nr, seq: int = 0) -> None:
        self.nr[slab][seq] = nr

    def reset(self, seq: int) -> None:
        """A new request takes the slot: nothing of its predecessor's may be served."""
        for slab in self.nr:
            slab[seq] = None


class DsaDecodeStack:
    """The KV-cache path of ``len(full)`` decoder layers for one batch of sequences: every layer has its own
    latent pool, full layers also an index pool and a selection; all layers share ONE page allocator and
    block table. A shared layer attends over the rows its nearest preceding full layer selected this step
    and runs no scorer or top-k at all."""

    def __init__(self, geom: be.DsaGeom, n_seqs: int, full: list[bool], device="cuda:0", max_ctx: int | None = None,
                 shuffle_seed: int | None = None, stale: bool = False):
        """``stale``: serve every full layer's selection one token late (``StaleShare``): the attention of token
        ``t`` uses the rows token ``t-1`` selected, so the indexer of a token is off the critical path of its
        own attention; a sequence whose previous token selected nothing (context at or below ``top_k``) attends
        densely, and a request that has just taken its slot serves its fresh selection once."""
        if not full or not full[0]:
            raise ValueError("layer 0 must be a full layer")
        self.full = list(full)
        self.stale = StaleShare(sum(self.full), n_seqs) if stale else None
        self.pool = be.PagePool(geom.n_pool_pages, n_seqs, geom.max_pages_per_seq, geom.page_tokens)
        if shuffle_seed is not None:
            self.pool.shuffle(shuffle_seed)
        self.layers = [DsaDecodeLayer(geom, n_seqs, device=device, max_ctx=max_ctx, pool=self.pool) for _ in full]
        for L in self.layers[1:]:           # ONE device block table for the whole stack: one upload per step
            L.block_table = self.layers[0].block_table
        self.owner = []                     # index of the full layer whose rows layer i attends over
        last = 0
        for i, f in enumerate(full):
            if f:
                last = i
            self.owner.append(last)
        self.slab = {i: n for n, i in enumerate(i for i, f in enumerate(full) if f)}   # full layer -> indexer slab
        if stale:
            g, d = geom, self.layers[0].dev
            for i in self.slab:             # per full layer: last token's rows, the rows being served, the modes
                L = self.layers[i]
                L.prev_rows, L.prev_n = torch.zeros_like(L.rows), torch.zeros_like(L.n_sel)
                L.serve_rows, L.serve_n = torch.zeros_like(L.rows), torch.zeros_like(L.n_sel)
                L.mode = torch.zeros(n_seqs, dtype=torch.int32, device=d)
                L.mode_host = torch.zeros(n_seqs, dtype=torch.int32).pin_memory()

    def upload_block_table(self) -> None:
        self.layers[0].upload_block_table(self.pool.block_table())

    def step_layer(self, i: int, latent, index_key, index_q, index_w, q, row_pos, seq_len, stream=None,
                   min_rows_hint: int = 0):
        """One layer-step of layer ``i``. Shared layers ignore ``index_key``/``index_q``/``index_w`` (they may be
        None) and cache only the latent row. ``min_rows_hint``: see ``DsaDecodeLayer.step``."""
        L = self.layers[i]
        if self.full[i] and self.stale is None:
            return L.step(latent, index_key, index_q, index_w, q, row_pos, seq_len, stream=stream,
                          min_rows_hint=min_rows_hint)
        if self.full[i]:
            return self._step_full_stale(i, latent, index_key, index_q, index_w, q, row_pos, seq_len, stream)
        src = self.layers[self.owner[i]]
        L.append_latent_only(latent, row_pos, stream=stream)
        if self.stale is not None:          # a shared layer serves what its full layer serves at this token
            return L.attend(q, stream=stream, rows_from=_Served(src))
        return L.attend(q, stream=stream, rows_from=src)

    def _step_full_stale(self, i, latent, index_key, index_q, index_w, q, row_pos, seq_len, stream, seq_len_host=None):
        """Full layer under the stale selection: select into the layer's row buffer as usual, but attend over the
        rows composed from LAST token's selection; then this token's selection becomes the stored one."""
        L, slab, k = self.layers[i], self.slab[i], self.layers[i].g.top_k
        nt = self.seq_len_host if seq_len_host is None else seq_len_host    # tokens after this step's append (host)
        if nt is None:
            raise ValueError("stale selection needs the host copy of seq_len: call begin_token(seq_len_host) first")
        for b in range(L.B):
            st = self.stale.stored(slab, b)
            n = int(nt[b])
            # 0: serve the stored rows; 2: dense (nothing stored and the prefix is at most one token past top_k);
            # 1: a request that has just taken the slot with a long context serves its fresh selection once
            L.mode_host[b] = 0 if st is not None else (2 if n <= k + 1 else 1)
        L.mode.copy_(L.mode_host, non_blocking=True)
        be.launch_dsa_append_select_paged(L.g, latent, index_key, row_pos, L.block_table, L.latent_pool, L.latent_scale,
                                          L.index_pool, L.index_scale, L.status, index_q, index_w, seq_len, L.B,
                                          L.score_stride, L.rows, L.n_sel, L.select_scratch, stream)
        be.launch_stale_compose_rows(L.prev_rows, L.prev_n, L.rows, L.n_sel, L.mode, seq_len, L.B, k, L.serve_rows,
                                     L.serve_n, stream)
        out = L.attend(q, stream=stream, rows_from=_Served(L))
        L.prev_rows, L.rows = L.rows, L.prev_rows       # this token's selection is what the next token serves
        L.prev_n, L.n_sel = L.n_sel, L.prev_n
        for b in range(L.B):
            n = int(nt[b])
            self.stale.store(slab, k if n > k else None, b)   # at or below top_k the indexer stores no selection
        return out

    seq_len_host = None

    def begin_token(self, seq_len_host) -> None:
        """Host copy of the sequence lengths AFTER this token's append (the scheduler's own array): the stale
        selection decides on the host what every sequence serves, without reading anything back from the device."""
        self.seq_len_host = seq_len_host

    def reset_slot(self, seq: int) -> None:
        if self.stale is not None:
            self.stale.reset(seq)


class _Served:
    """The (rows, n_sel) pair a layer serves under the stale selection, in the shape ``attend(rows_from=...)`` reads."""

    def __init__(self, layer):
        self.rows, self.n_sel = layer.serve_rows, layer.serve_n
