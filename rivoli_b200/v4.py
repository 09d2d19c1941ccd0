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
        """Per sequence: 1 if the integer scorer handed it to the ordered CUDA-core fold in the last select()."""
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
