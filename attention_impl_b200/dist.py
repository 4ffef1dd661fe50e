"""Multi-GPU sharding of the decode path (one process per GPU, torch.distributed / NCCL).

Two schemes, both absent from the reference (it has no multi-GPU code):

* head sharding: rank r owns heads [r*H/G, (r+1)*H/G) of every token; its KV pool is
  ``[slots, (H/G)*D]``.  (sequence, head) units are independent, so there is NO collective.
* KV split: rank r owns a contiguous 1/G slice of every sequence's cached tokens (its own pool
  and slot table); each rank reduces its slice to one fp32 row ``[o[D], m, l]`` per (sequence,
  head), the rows are all-gathered (B*H*(D+2) floats per rank, ~1 MB at B=64, H=32) and every
  rank folds them, plus the current token, with the log-sum-exp combine kernel.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def head_shard(num_heads: int, world: int, rank: int) -> Tuple[int, int]:
    """Half-open head range owned by ``rank``."""
    if num_heads % world:
        raise ValueError(f"num_heads={num_heads} is not divisible by world={world}")
    per = num_heads // world
    return rank * per, (rank + 1) * per


def slice_heads(x: torch.Tensor, num_heads: int, world: int, rank: int) -> torch.Tensor:
    """Columns of a ``[rows, H*D]`` tensor that belong to ``rank``'s heads (contiguous copy)."""
    h0, h1 = head_shard(num_heads, world, rank)
    D = x.size(1) // num_heads
    return x[:, h0 * D:h1 * D].contiguous()


def kv_split_bounds(lengths: torch.Tensor, world: int, rank: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per sequence, the half-open range (relative to the sequence start) of cached tokens that
    ``rank`` owns: ``[n*r//G, n*(r+1)//G)``.  Ranges of all ranks tile ``[0, n)`` without gaps."""
    n = lengths.to(torch.int64)
    return n * rank // world, n * (rank + 1) // world


def plan_kv_split(cache_indices: torch.Tensor, offsets: torch.Tensor, world: int, rank: int):
    """Slot table and inclusive cumulative offsets of ``rank``'s slice of every sequence.

    ``cache_indices`` int32 [T] and ``offsets`` int32 [B] describe the whole batch (reference
    layout).  Returns ``(local_indices int32 [T_r], local_offsets int32 [B])`` on the inputs'
    device.  Pure index arithmetic; no synchronisation besides what torch needs for the result size.
    """
    off = offsets.to(torch.int64)
    beg = torch.cat([off.new_zeros(1), off[:-1]])
    lo, hi = kv_split_bounds(off - beg, world, rank)
    cnt = hi - lo
    local_off = cnt.cumsum(0)
    total = int(local_off[-1].item()) if cnt.numel() else 0
    # token t of the local stream belongs to sequence seq[t] at local position t - local_beg[seq[t]]
    seq = torch.repeat_interleave(torch.arange(cnt.numel(), device=cnt.device), cnt, output_size=total)
    local_beg = local_off - cnt
    pos = torch.arange(total, device=cnt.device) - local_beg[seq]
    src = beg[seq] + lo[seq] + pos
    return cache_indices[src].contiguous(), local_off.to(torch.int32)


def gather_partials(part: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather one ``[B, H, D+2]`` fp32 partial per rank into ``[G, B, H, D+2]`` (rank order)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return part.unsqueeze(0)
    G = dist.get_world_size(group)
    part = part.contiguous()
    out = torch.empty((G * part.size(0),) + tuple(part.shape[1:]), dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(out, part, group=group)     # concatenation along dim 0, rank order
    return out.view((G,) + tuple(part.shape))


def kv_split_decode(Q, K, V, K_cache_local, V_cache_local, local_indices, local_offsets, num_heads: int, *,
                    scale: Optional[float] = None, k_scale=None, v_scale=None, chunk: Optional[int] = None,
                    group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Decode with every sequence's KV split across the ranks of ``group``.

    Q, K, V ``[B, H*D]`` are replicated; ``K_cache_local``/``V_cache_local`` is this rank's pool and
    ``local_indices``/``local_offsets`` its slot table (see :func:`plan_kv_split`).  Returns the
    full ``[B, H*D]`` output on every rank.
    """
    from . import ops
    part = ops.paged_decode_partial(Q, K_cache_local, V_cache_local, local_indices, local_offsets, num_heads,
                                    scale=scale, chunk=chunk, k_scale=k_scale, v_scale=v_scale)
    parts = gather_partials(part, group)
    return ops.lse_combine(parts, Q, K, V, num_heads=num_heads, scale=scale)
