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


def gpu_shard_ops(layer) -> ShardOps:
    """The CUDA library as the arithmetic of a page-range shard. ``layer`` is this rank's
    ``DsaDecodeLayer`` holding the rank's slice of every sequence at local positions 0..n-1."""
    from . import backend as be
    g, B, dev = layer.g, layer.B, layer.dev

    def score(index_q, index_w, local_len):
        be.launch_index_q_quant(index_q, B * g.index_heads, g.index_dim, layer.qcodes, layer.qscales)
        be.launch_index_score_paged(g, layer.qcodes, layer.qscales, index_w, layer.index_pool, layer.index_scale,
                                    layer.block_table, local_len, B, layer.scores, layer.score_stride)
        return layer.scores

    def topk(scores, lens, k):
        rows = torch.zeros((B, k), dtype=torch.int32, device=dev)
        n = torch.zeros(B, dtype=torch.int32, device=dev)
        scores = scores.contiguous()
        be.launch_index_topk_batched(scores, scores.shape[1], lens.contiguous(), B, k, rows, n)
        return rows, n

    def attend(q, rows, n_rows):
        rows = rows.contiguous()
        be.launch_attend_paged_bf16(g, q, layer.latent_pool, layer.latent_scale, layer.block_table, rows,
                                    rows.shape[1], n_rows.contiguous(), B, layer.out, layer.out_m, layer.out_lse,
                                    layer.scratch)
        return layer.out, layer.out_lse

    def merge(part_out, part_lse):
        G, n_vec, kvl = part_out.shape
        out = torch.empty((n_vec, kvl), dtype=torch.bfloat16, device=dev)
        be.launch_attend_merge_partials(part_out.contiguous(), part_lse.contiguous(), G, n_vec, kvl, out)
        return out

    return ShardOps(score, topk, attend, merge)
