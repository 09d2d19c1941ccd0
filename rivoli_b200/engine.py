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
    """Row count of the selection each indexer slab stored at the PREVIOUS token (``None`` = nothing
    stored: serve dense). Read with ``stored`` before ``store`` overwrites it - what token ``t`` serves
    is what token ``t-1`` computed."""

    def __init__(self, n_slabs: int):
        self.nr: list[int | None] = [None] * n_slabs

    def stored(self, slab: int):
        return self.nr[slab]

    def store(self, slab: int, nr: int) -> None:
        self.nr[slab] = nr


class DsaDecodeStack:
    """The KV-cache path of ``len(full)`` decoder layers for one batch of sequences: every layer has its own
    latent pool, full layers also an index pool and a selection; all layers share ONE page allocator and
    block table. A shared layer attends over the rows its nearest preceding full layer selected this step
    and runs no scorer or top-k at all."""

    def __init__(self, geom: be.DsaGeom, n_seqs: int, full: list[bool], device="cuda:0", max_ctx: int | None = None,
                 shuffle_seed: int | None = None):
        if not full or not full[0]:
            raise ValueError("layer 0 must be a full layer")
        self.full = list(full)
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

    def upload_block_table(self) -> None:
        self.layers[0].upload_block_table(self.pool.block_table())

    def step_layer(self, i: int, latent, index_key, index_q, index_w, q, row_pos, seq_len, stream=None):
        """One layer-step of layer ``i``. Shared layers ignore ``index_key``/``index_q``/``index_w`` (they may be
        None) and cache only the latent row."""
        L = self.layers[i]
        if self.full[i]:
            return L.step(latent, index_key, index_q, index_w, q, row_pos, seq_len, stream=stream)
        src = self.layers[self.owner[i]]
        L.append_latent_only(latent, row_pos, stream=stream)
        return L.attend(q, stream=stream, rows_from=src)
