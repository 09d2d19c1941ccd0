"""Host-side selection arithmetic of the V4 cousin path: which cache rows a query row may read.

Mirror of the reference's ``crates/engine/src/v4/select.rs`` (same names, argument meaning and refusals):
the ring order, the positional block columns, the scored block columns, and the rectangle that
``gather_attn_shared_kv`` receives. Pure integer / ordering work on the host; the batched decode form of the
same rules runs on the device (``rivoli_v4_select_blocks_bf16``), this module covers the prefill rows and
the one-sequence call shape of the reference.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

INDEXED_RATIO = 4  # the only compressor ratio that carries an indexer (crates/engine/src/v4/geometry.rs:86-131)


class SelectionError(ValueError):
    """A refusal of select.rs (the text names the same condition)."""


@dataclass(frozen=True)
class Extent:
    """select.rs:26-86. ``seqlen`` rows starting at ``start_pos``; start_pos == 0 is the prefill."""
    seqlen: int
    start_pos: int

    def is_prefill(self) -> bool:
        return self.start_pos == 0

    def query_rows(self) -> int:
        return self.seqlen if self.is_prefill() else 1

    def end_pos(self) -> int:
        return self.start_pos + self.query_rows()

    def check_single_row_decode(self) -> None:
        if not (self.is_prefill() or self.seqlen == 1):
            raise SelectionError(f"v4 selection: decode consumes one query row (the bsz=1 scope cut), got {self.seqlen}")


def compressor_ratio(ratio: int):
    """LayerKind::compressor_ratio: None for a plain layer (ratio 0)."""
    return None if ratio == 0 else ratio


def has_indexer(ratio: int) -> bool:
    return ratio == INDEXED_RATIO


def positional_context_limit(index_topk: int) -> int:
    """select.rs:106-108: past this many positions an indexed layer's block set is decided by scores."""
    return INDEXED_RATIO * (index_topk + 1)


def _rows_from(rows: int, cols: int, cell) -> list[list[int]]:
    out = []
    for t in range(rows):
        r = []
        for j in range(cols):
            v = cell(t, j)
            r.append(-1 if v is None else int(v))
        out.append(r)
    return out


def window_rows(win: int, at: Extent) -> list[list[int]]:
    """select.rs:195-218. Prefill: absolute positions, the last ``win`` of them, causally masked. Decode: ring
    slots, oldest first once the ring is full, live slots then -1 before that."""
    sp = at.start_pos
    if at.is_prefill():
        def cell(t, j):
            v = max(t - (win - 1), 0) + j
            return v if v <= t else None
        return _rows_from(at.seqlen, min(win, at.seqlen), cell)
    if sp >= win - 1:
        cut = sp % win
        return [list(range(cut + 1, win)) + list(range(0, cut + 1))]
    return _rows_from(1, win, lambda _t, j: j if j <= sp else None)


def compressed_rows(ratio: int, at: Extent, offset: int) -> list[list[int]]:
    """select.rs:224-246. Block c covers positions [c*ratio, (c+1)*ratio): a prefill row t may read it only once it
    is complete, c < (t+1)/ratio; a decode step sees every closed block."""
    r = compressor_ratio(ratio)
    if r is None:
        return []
    if not at.is_prefill():
        return _rows_from(1, at.end_pos() // r, lambda _t, c: c + offset)
    return _rows_from(at.seqlen, at.seqlen // r, lambda t, c: c + offset if c < (t + 1) // r else None)


def compress_offset(window: int, at: Extent) -> int:
    """select.rs:268-270: selection-space base of the compressed columns."""
    return at.seqlen if at.is_prefill() else window


def should_compress(ratio: int, at: Extent) -> bool:
    r = compressor_ratio(ratio)
    if r is None:
        return False
    return at.seqlen >= r if at.is_prefill() else (at.start_pos + 1) % r == 0


def compress_dst(ratio: int, region_base: int, at: Extent):
    """select.rs:316-327: (first row, count) of the blocks this step emits, by POSITION, or None."""
    r = compressor_ratio(ratio)
    if r is None or not should_compress(ratio, at):
        return None
    return (region_base, at.seqlen // r) if at.is_prefill() else (region_base + at.start_pos // r, 1)


def _total_key(scores: np.ndarray) -> np.ndarray:
    """f32 total order (sign-magnitude), what ``total_cmp`` ranks by: -0.0 below +0.0."""
    b = np.ascontiguousarray(scores, np.float32).view(np.uint32).astype(np.int64)
    return np.where(b >> 31, (~b) & 0xFFFFFFFF, b | 0x80000000)


def scored_rows(scores, n_comp: int, *, ratio: int, index_topk: int, at: Extent, offset: int) -> list[list[int]]:
    """select.rs:153-190. One ranked row per query row from the score matrix [rows, n_comp]: the best
    min(index_topk, n_comp) causally legal blocks by score (descending, ties toward the lower block), emitted
    ascending, shifted by ``offset``, padded with -1."""
    at.check_single_row_decode()
    r = compressor_ratio(ratio)
    if r is None:
        raise SelectionError("scored selection on a layer with no compressor")
    rows = at.query_rows()
    scores = np.asarray(scores, np.float32).reshape(-1)
    if scores.size != rows * n_comp:
        raise SelectionError(f"v4 scored selection: {scores.size} scores for [{rows}, {n_comp}]")
    k = min(index_topk, n_comp)
    out = []
    for t in range(rows):
        row = scores[t * n_comp:(t + 1) * n_comp]
        limit = min((t + 1) // r, n_comp) if at.is_prefill() else n_comp
        key = _total_key(row[:limit])
        order = np.lexsort((np.arange(limit), -key))[:k]     # key descending, index ascending on ties
        sel = sorted(int(c) + offset for c in order)
        out.append(sel + [-1] * (k - len(sel)))
    return out


@dataclass(frozen=True)
class Sel:
    """select.rs:329-447: the rectangle [query rows, window columns + compressed columns] of one layer step."""
    win: int
    ratio: int
    index_topk: int
    at: Extent

    def _n_comp(self) -> int:
        r = compressor_ratio(self.ratio)
        if r is None:
            return 0
        live = self.at.end_pos() // r
        if has_indexer(self.ratio) and live > self.index_topk:
            raise SelectionError(
                f"v4 selection: {live} compressed blocks at position {self.at.end_pos()} exceeds index_topk "
                f"{self.index_topk} on an indexed layer. Past {positional_context_limit(self.index_topk)} positions the "
                "block set is decided by the indexer's SCORES - the scored path (gather_scored) is how it is answered")
        return live

    def shape(self) -> tuple[int, int]:
        self.at.check_single_row_decode()
        if self.win <= 0:
            raise SelectionError("v4 selection: sliding_window is zero")
        win_cols = min(self.at.seqlen, self.win) if self.at.is_prefill() else self.win
        return self.at.query_rows(), win_cols + self._n_comp()

    def gather(self) -> np.ndarray:
        """Positional rectangle (legal while the closed blocks fit index_topk on an indexed layer)."""
        rows, cols = self.shape()
        win = window_rows(self.win, self.at)
        n_comp = cols - (len(win[0]) if win else 0)
        comp = compressed_rows(self.ratio, self.at, compress_offset(self.win, self.at)) if n_comp else []
        return _assemble(win, comp, rows, cols)

    def gather_scored(self, comp: list[list[int]]) -> np.ndarray:
        """Rectangle whose compressed columns are the ranked rows of :func:`scored_rows`."""
        self.at.check_single_row_decode()
        rows = self.at.query_rows()
        if len(comp) != rows:
            raise SelectionError(f"v4 scored selection: {len(comp)} ranked rows for {rows} query rows")
        if self.win <= 0:
            raise SelectionError("v4 selection: sliding_window is zero")
        win = window_rows(self.win, self.at)
        cols = (len(win[0]) if win else 0) + (len(comp[0]) if comp else 0)
        return _assemble(win, comp, rows, cols)


def _assemble(win, comp, rows: int, cols: int) -> np.ndarray:
    out = np.full((rows, cols), -1, np.int32)
    for t, w in enumerate(win):
        c = comp[t] if t < len(comp) else []
        if len(w) + len(c) != cols:
            raise SelectionError(f"v4 selection: row {t} is {len(w) + len(c)} wide ({len(w)} window + {len(c)} compressed), "
                                 f"the rectangle is {cols}")
        out[t, :len(w)] = w
        out[t, len(w):] = c
    if len(win) != rows:
        raise SelectionError(f"v4 selection: wrote {len(win) * cols} entries, {rows}x{cols} needs {rows * cols}")
    return out
