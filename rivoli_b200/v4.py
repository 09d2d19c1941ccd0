"""Caller-side sequencing of the V4 cousin path's decode step: selection rows, then sparse attention.

Mirrors what ``crates/engine/src/v4/blocksel.rs:361-417`` (scored selection) and
``crates/engine/src/v4/attn.rs`` (the gather-attention call) do per layer, batched over sequences and
over bf16 storage. Device memory is owned here through torch; every launch goes through the C ABI.
"""
from __future__ import annotations

import torch

from . import backend as be


class V4DecodeLayer:
    """One layer's ring + compressed KV, the indexer's compressed rows, and the two launches of a step."""

    def __init__(self, g: be.V4Geom, n_seqs: int, device="cuda"):
        self.g, self.B = g, n_seqs
        dev = torch.device(device)
        self.kv_rows = g.window + g.max_comp
        self.kv_cache = torch.zeros((n_seqs, self.kv_rows, g.head_dim), dtype=torch.uint16, device=dev)
        self.index_kv = torch.zeros((n_seqs, g.max_comp, g.index_dim), dtype=torch.uint16, device=dev)
        self.sink = torch.zeros(g.n_heads, dtype=torch.float32, device=dev)
        self.cols = g.window + g.index_topk
        self.sel = torch.full((n_seqs, self.cols), -1, dtype=torch.int32, device=dev)
        self.out = torch.zeros((n_seqs, g.n_heads, g.head_dim), dtype=torch.uint16, device=dev)
        self.packed = self.packed_exp = None   # optional int8 form of index_kv (pack_index_rows)
        # score rows f32 [B][max_comp] of the sequences that ranked, then one flag per sequence
        self.scratch = torch.zeros(be.v4_select_scratch_bytes(g, n_seqs) // 4, dtype=torch.float32, device=dev)

    @property
    def scores(self):
        return self.scratch[: self.B * self.g.max_comp].view(self.B, self.g.max_comp)

    @property
    def refolded(self):
        """Per sequence after the last select(): bit 0 = the integer scorer handed the whole sequence to the ordered
        CUDA-core fold (its queries were not of the integer form), bit 1 = some of its columns were re-scored."""
        return self.scratch[self.B * self.g.max_comp:].view(torch.int32)

    def pack_index_rows(self, row_begin, row_end, max_rows: int, stream=None):
        """Write the int8 + exponent form of index_kv rows [row_begin[b], row_end[b]) (call it when rows enter the
        cache); select() uses it from then on. Only for index_dim == 128."""
        if self.packed is None:
            dev = self.index_kv.device
            self.packed = torch.zeros((self.B, self.g.max_comp, 128), dtype=torch.uint8, device=dev)
            self.packed_exp = torch.zeros((self.B, self.g.max_comp), dtype=torch.int32, device=dev)
        be.launch_v4_index_pack_bf16(self.g, self.B, row_begin, row_end, max_rows, self.index_kv, self.packed,
                                     self.packed_exp, stream)

    def select(self, pos, index_q, index_w, force_fold: bool = False, stream=None):
        be.launch_v4_select_blocks_bf16(self.g, self.B, pos, index_q, index_w, self.index_kv, self.sel, self.scratch,
                                        force_fold, self.packed, self.packed_exp, stream)
        return self.sel

    def attend(self, q, force_simt: bool = False, stream=None):
        be.launch_v4_sparse_attend_bf16(self.g, self.B, q, self.kv_cache, self.sink, self.sel, self.cols, self.out,
                                        force_simt, stream)
        return self.out

    def step(self, pos, q, index_q, index_w, stream=None):
        """Selection then attention for one decode step; returns the bf16 output [B, H, D]."""
        self.select(pos, index_q, index_w, False, stream)
        return self.attend(q, False, stream)


class V4Compressor:
    """Pooling state and parameters of one KV compressor for a batch of sequences (decode arm).

    ``rotate`` selects the finish: the Hadamard + fp4 spread (the indexer's compressor) or the fp8 block-64
    quantisation of the un-rotated dims (the attention compressor). Mirrors the per-step part of
    ``crates/engine/src/v4/kvcompress.rs``.
    """

    def __init__(self, p: be.CompGeom, n_seqs: int, ape, norm, freqs, rotate: bool, device="cuda"):
        dev = torch.device(device)
        self.p, self.B, self.rotate = p, n_seqs, bool(rotate)
        self.kv_state = torch.zeros((n_seqs, p.ents, p.cd), dtype=torch.float32, device=dev)
        self.score_state = torch.full((n_seqs, p.ents, p.cd), float("-inf"), dtype=torch.float32, device=dev)
        self.ape, self.norm, self.freqs = ape, norm, freqs

    def step(self, pos, kv_proj, score_proj, cache, cache_rows: int, cache_row0: int, packed=None, packed_exp=None,
             prequant=None, stream=None):
        be.launch_v4_compress_step_bf16(self.p, self.B, pos, kv_proj, score_proj, self.ape, self.kv_state,
                                        self.score_state, self.norm, self.freqs, self.rotate, cache, cache_rows,
                                        cache_row0, prequant, packed, packed_exp, stream)


class V4TokenStep:
    """One decode token through a V4 layer, in the reference's order (crates/oracles/src/v4oracle/attention.rs:197-232):
    the indexer's compressor ingests the token, the selection rows are built, the token's entry goes into the ring,
    the attention compressor ingests the token, then the sparse attention runs."""

    def __init__(self, layer: V4DecodeLayer, attn_comp: V4Compressor, index_comp: V4Compressor, pack_index: bool = True):
        self.layer, self.attn_comp, self.index_comp = layer, attn_comp, index_comp
        g = layer.g
        if pack_index and g.index_dim == 128:
            dev = layer.index_kv.device
            layer.packed = torch.zeros((layer.B, g.max_comp, 128), dtype=torch.uint8, device=dev)
            layer.packed_exp = torch.zeros((layer.B, g.max_comp), dtype=torch.int32, device=dev)
        self._seq = torch.arange(layer.B, device=layer.kv_cache.device)

    def __call__(self, pos, kv_entry, attn_proj, index_proj, q, index_q, index_w, stream=None):
        """pos i32 [B]; kv_entry bf16 bits [B, head_dim] (the token's window entry); attn_proj / index_proj =
        (kv_proj, score_proj) f32 [B, cd] of the two compressors; q, index_q, index_w as for V4DecodeLayer.step."""
        L, g = self.layer, self.layer.g
        self.index_comp.step(pos, index_proj[0], index_proj[1], L.index_kv, g.max_comp, 0, L.packed, L.packed_exp,
                             stream=stream)
        L.select(pos, index_q, index_w, False, stream)
        # ring write: slot pos % window (plain device copy: torch indexes int16 views of the bf16 bits)
        L.kv_cache.view(torch.int16)[self._seq, (pos % g.window).long()] = kv_entry.view(torch.int16)
        self.attn_comp.step(pos, attn_proj[0], attn_proj[1], L.kv_cache, L.kv_rows, g.window, stream=stream)
        return L.attend(q, False, stream)
