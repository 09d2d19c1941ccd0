"""Continuous batching over the shared page pool: the host-side bookkeeping of a decode step
with sequences finishing and being replaced (eviction churn).

The reference decodes one sequence and has no scheduler; its nearest idiom is the
allocate-once ownership of KV slabs (crates/engine/src/glm/engine.rs:139-260) and the LIFO
free list of its expert arena (crates/core/src/arena.rs:131-149). Here every sequence slot of
the batch owns the pages its context needs; one decode step grows every live sequence by one
token (a page is drawn from the free list when a sequence crosses a page boundary), and a
slot whose sequence finishes returns its pages (logical page 0 first) before the replacement
sequence reserves its own. All layers of a model share one block table - page ``p`` names
row block ``p`` of every layer's pool - so paging is done once per step, not per layer.

Deterministic by construction: the order of releases and reservations is slot order, so page
tables are a pure function of the call history (and comparable bit for bit with the oracle).
"""
from __future__ import annotations

import numpy as np

from . import backend as be


class ContinuousBatcher:
    def __init__(self, n_slots: int, n_pool_pages: int, max_ctx: int, page_tokens: int = 64,
                 shuffle_seed: int | None = None, pool=None):
        self.P = page_tokens
        self.max_pages = (max_ctx + page_tokens - 1) // page_tokens
        self.pool = pool if pool is not None else be.PagePool(n_pool_pages, n_slots, self.max_pages, page_tokens)
        if shuffle_seed is not None:
            self.pool.shuffle(shuffle_seed)
        self.n_slots = n_slots
        self.seq_len = np.zeros(n_slots, dtype=np.int32)       # tokens cached per slot
        self.seq_id = np.full(n_slots, -1, dtype=np.int64)     # which request occupies the slot
        self._next_id = 0

    def _reserve(self, slot: int, n_tokens: int) -> None:
        r = self.pool.reserve(slot, n_tokens)
        if r not in (None, 0):                                  # the oracle's pool returns codes
            raise be.BackendError("pagepool_reserve", int(r))

    def _evict(self, slot: int) -> None:
        """Return the slot's pages and mark it empty (its bookkeeping never describes pages it no longer owns)."""
        if self.seq_id[slot] >= 0:
            self.pool.release(slot)
        self.seq_id[slot] = -1
        self.seq_len[slot] = 0

    def _place(self, slot: int, context_len: int) -> int:
        self._reserve(slot, context_len)                        # raises with the slot still marked empty
        self.seq_len[slot] = context_len
        self.seq_id[slot] = self._next_id
        self._next_id += 1
        return int(self.seq_id[slot])

    def admit(self, slot: int, context_len: int) -> int:
        """Place a new request with ``context_len`` prefilled tokens in ``slot``; returns its id. If the pool
        cannot hold it the slot is left empty (1007 is raised)."""
        self._evict(slot)
        return self._place(slot, context_len)

    def begin_step(self):
        """Grow every live sequence by the token this step appends. Returns ``(row_pos, seq_len)``:
        the position each slot writes (its old length) and the length after the append. A slot counts as
        grown as soon as its page is reserved, so a failure part-way leaves lengths and pages in step."""
        row_pos = self.seq_len.copy()
        for slot in np.nonzero(self.seq_id >= 0)[0]:
            self._reserve(int(slot), int(self.seq_len[slot]) + 1)
            self.seq_len[slot] += 1
        return row_pos, self.seq_len.copy()

    def finish(self, slots, new_context_lens) -> list[int]:
        """Sequences in ``slots`` end and replacements with the given prefilled context lengths take their
        slots. Every finishing slot returns its pages FIRST (slot order), then the replacements reserve (slot
        order): near a full pool a replacement can use the pages of a slot that finishes later in the list,
        and the order stays a pure function of the call. Returns the new ids."""
        order = np.argsort(np.asarray(slots), kind="stable")
        for i in order:
            self._evict(int(slots[i]))
        return [self._place(int(slots[i]), int(new_context_lens[i])) for i in order]

    def block_table(self) -> np.ndarray:
        return self.pool.block_table()

    @property
    def n_free(self) -> int:
        return self.pool.n_free


def churn_plan(rng: np.random.RandomState, n_slots: int, frac: float, lo: int, hi: int):
    """Which slots finish this step and the context lengths of their replacements (seeded)."""
    n = max(1, int(round(n_slots * frac)))
    slots = np.sort(rng.choice(n_slots, n, replace=False))
    return slots, rng.randint(lo, hi + 1, n)
