"""Multi-GPU partitioning of the decode KV-cache path: one process per GPU.

Two partitions, as the path allows:

* **by sequence** (batched decode): sequences are independent, each rank owns its slice of
  the batch with its own pools and page allocator; there is NO collective on the data path.
* **by KV page range** (one long context): rank ``g`` of ``G`` holds the logical pages
  ``[g*n/G, (g+1)*n/G)`` of every sequence. A layer-step is then

    1. local indexer scores (exact, bit-reproducible) and a local top-k candidate list;
    2. ONE small all-gather of the candidates ``(score, global index)`` - every token of the
       global top-k is in its shard's local top-k, so the exact global cut (ties -> lower
       global index) is decided identically on every rank from the gathered lists;
    3. local attention over the surviving local rows -> normalised partial ``out`` (bf16) and
       ``lse``;
    4. ONE all-gather of the partials and the merge ``w_g = exp(lse_g - max lse)`` in ascending
       shard order (the reference's split combine, crates/backend/kernels/attn.hip:241-273).

The arithmetic is injected (``ops``): on GPUs it is the CUDA library, in the CPU tests it is
the oracle, so the partition logic and the collectives are exercised with ``gloo`` ranks
without any device.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def shard_sequences(n_seqs: int, world: int, rank: int) -> range:
    """Contiguous slice of sequence ids owned by ``rank`` (sizes differ by at most one)."""
    base, rem = divmod(n_seqs, world)
    lo = rank * base + min(rank, rem)
    return range(lo, lo + base + (1 if rank < rem else 0))


def page_range(n_pages: int, world: int, rank: int) -> range:
    """Logical pages of a sequence held by ``rank``."""
    base, rem = divmod(n_pages, world)
    lo = rank * base + min(rank, rem)
    return range(lo, lo + base + (1 if rank < rem else 0))


def local_token_span(seq_len: int, page_tokens: int, world: int, rank: int) -> tuple[int, int]:
    """``(first_token, n_tokens)`` of the tokens of a ``seq_len`` context that live on ``rank``."""
    n_pages = (seq_len + page_tokens - 1) // page_tokens
    pr = page_range(n_pages, world, rank)
    lo = pr.start * page_tokens
    hi = min(seq_len, pr.stop * page_tokens)
    return lo, max(0, hi - lo)


@dataclass
class ShardOps:
    """The per-rank arithmetic of a page-range step.

    score(index_q, index_w, local_len) -> f32 [B, stride]      exact local scores
    topk(scores, lens, k)              -> (rows u32-as-i32 [B, k], n_sel i32 [B])   ascending, exact
    attend(q, rows, n_rows)            -> (out bf16-bits [B, H, kvl], lse f32 [B, H])
    merge(part_out [G, B*H, kvl], part_lse [G, B*H]) -> out [B*H, kvl]
    """
    score: callable
    topk: callable
    attend: callable
    merge: callable


def _all_gather(t: torch.Tensor, group=None) -> torch.Tensor:
    world = dist.get_world_size(group)
    if t.is_cuda and dist.get_backend(group) == "gloo":
        # CPU transport for device tensors (ranks that share one GPU cannot form an NCCL group)
        return _all_gather(t.cpu(), group).to(t.device)
    out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather(list(out.unbind(0)), t.contiguous(), group=group)   # views of `out`: filled in place
    return out


def page_range_step(ops: ShardOps, index_q, index_w, q, local_len: torch.Tensor, token_offset: torch.Tensor,
                    k: int, group=None):
    """One layer-step (select + attend) of a page-range shard. Returns ``(out, rows_global, n_global)``.

    ``local_len[b]`` = tokens of sequence ``b`` on this rank, ``token_offset[b]`` = global index
    of its first local token. The merged output is identical on every rank; ``rows_global`` are
    this rank's surviving rows as GLOBAL token indices (ascending), ``n_global`` their count.
    """
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    B = local_len.numel()
    # 1. local exact scores and local candidates (ascending local indices)
    scores = ops.score(index_q, index_w, local_len)                       # [B, stride]
    rows_l, n_l = ops.topk(scores, local_len, k)                          # [B, k], [B]
    cols = torch.arange(k, device=scores.device).unsqueeze(0)
    live = cols < n_l.unsqueeze(1)
    idx = rows_l.to(torch.int64).clamp_(0, scores.shape[1] - 1)
    cand_score = torch.where(live, scores.gather(1, idx), torch.full_like(scores[:, :1], float("-inf")).expand(B, k))
    # 2. exchange candidates; the concatenation [rank 0 | rank 1 | ...] is ascending in global index,
    #    so "lower position wins a tie" IS "lower global index wins a tie"
    all_score = _all_gather(cand_score, group)                            # [G, B, k]
    all_n = _all_gather(n_l, group)                                       # [G, B]
    cat = all_score.permute(1, 0, 2).reshape(B, world * k).contiguous()
    # compact each row: candidates of rank g occupy [g*k, g*k + n_g); dead slots carry -inf and sit
    # AFTER every live slot of their rank, so their positions never beat a live tie
    sel_pos, n_glob = ops.topk(cat, torch.full_like(all_n[0], world * k), k)  # positions in cat, ascending
    pos = sel_pos.to(torch.int64)
    valid = torch.arange(k, device=pos.device).unsqueeze(0) < n_glob.unsqueeze(1)
    # -inf padding is selected only when fewer than k live candidates exist (and then possibly at
    # positions BEFORE later ranks' live ones); it is dropped by its score, not by its rank
    picked_score = cat.gather(1, pos.clamp(0, world * k - 1))
    valid &= picked_score > float("-inf")
    mine = valid & (pos >= rank * k) & (pos < (rank + 1) * k)
    # surviving local rows, ascending (pos ascending within a rank's segment == local index ascending)
    slot = (pos - rank * k).clamp(0, k - 1)
    local_rows = rows_l.to(torch.int64).gather(1, slot)
    n_mine = mine.sum(1).to(torch.int32)
    order = torch.argsort((~mine).to(torch.int8), dim=1, stable=True)     # mine first, order kept
    rows_att = local_rows.gather(1, order).to(torch.int32)
    # 3. local partial attention
    part_out, part_lse = ops.attend(q, rows_att, n_mine)
    # 4. merge
    H, kvl = part_out.shape[1], part_out.shape[2]
    g_out = _all_gather(part_out.reshape(B * H, kvl), group)
    g_lse = _all_gather(part_lse.reshape(B * H), group)
    out = ops.merge(g_out, g_lse).reshape(B, H, kvl)
    rows_global = rows_att.to(torch.int64) + token_offset.to(torch.int64).unsqueeze(1)
    return out, rows_global, n_mine


class ShardedDecodeStep:
    """A page-range shard's layer-step through the CUDA library (``rivoli_shard_*``): this rank's ``DsaDecodeLayer``
    holds its slice of every sequence at local positions ``0 .. n-1``. ``step`` runs the three phases around two
    NCCL all-gathers inside the library (``rivoli_shard_step_paged``) on the communicator created by
    ``nccl_comm``; ``candidates`` / ``cut_attend`` / ``merge`` are the phases on their own, for a host that
    exchanges the two small buffers itself."""

    def __init__(self, layer, rank: int, world: int, comm: int = 0):
        from . import backend as be
        self.be, self.layer, self.rank, self.world, self.comm = be, layer, rank, world, comm
        g, B, d = layer.g, layer.B, layer.dev
        u8 = torch.uint8
        self.shard_scratch = torch.zeros(be.shard_scratch_bytes(g, B, world), dtype=u8, device=d)
        self.cand = torch.zeros(be.shard_candidate_bytes(g, B), dtype=u8, device=d)
        self.part = torch.zeros(be.shard_partial_bytes(g, B), dtype=u8, device=d)
        self.rows_l = torch.zeros((B, g.top_k), dtype=torch.int32, device=d)
        self.rows_att = torch.zeros((B, g.top_k), dtype=torch.int32, device=d)
        self.n_mine = torch.zeros(B, dtype=torch.int32, device=d)
        self.out = torch.zeros((B, g.n_heads, g.kv_lora), dtype=torch.bfloat16, device=d)

    @staticmethod
    def nccl_comm(rank: int, world: int, group=None) -> int:
        """An NCCL communicator for the library: rank 0 makes the id, ``torch.distributed`` carries it."""
        from . import backend as be
        box = [be.shard_nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=group)
        return be.shard_nccl_comm_create(box[0], rank, world)

    def step(self, index_q, index_w, q, local_len, stream=None) -> torch.Tensor:
        L, g = self.layer, self.layer.g
        self.be.launch_shard_step_paged(g, self.comm, self.rank, self.world, index_q, index_w, q, L.latent_pool,
                                        L.latent_scale, L.index_pool, L.index_scale, L.block_table, local_len, L.B,
                                        L.score_stride, self.rows_l, self.rows_att, self.n_mine, self.out,
                                        L.select_scratch, L.scratch, self.shard_scratch, stream)
        return self.out

    def candidates(self, index_q, index_w, local_len, stream=None) -> torch.Tensor:
        L = self.layer
        self.be.launch_shard_candidates(L.g, index_q, index_w, L.index_pool, L.index_scale, L.block_table, local_len, L.B,
                                        L.score_stride, self.rows_l, L.select_scratch, self.cand, stream)
        return self.cand

    def cut_attend(self, all_cand, q, stream=None) -> torch.Tensor:
        L = self.layer
        self.be.launch_shard_cut_attend(L.g, all_cand, self.rank, self.world, self.rows_l, q, L.latent_pool,
                                        L.latent_scale, L.block_table, L.B, self.rows_att, self.n_mine, self.part,
                                        self.shard_scratch, L.scratch, stream)
        return self.part

    def merge(self, all_part, stream=None) -> torch.Tensor:
        self.be.launch_shard_merge(self.layer.g, all_part, self.world, self.layer.B, self.out, stream)
        return self.out
