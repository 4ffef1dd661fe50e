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


class KvSplitExchange:
    """KV-split decode whose partial rows travel by plain stores into the peers' memory (NVLink)
    instead of an NCCL all-gather.

    Set-up (collective over ``group``): a symmetric buffer ``[2, G, B, H, D+2]`` fp32 (two halves used
    on alternate steps, so a rank that is one step ahead never overwrites rows a slower peer is
    still combining) and ``G`` arrival counters per rank, mapped into every process with
    ``torch.distributed._symmetric_memory``.

    ``fused=True`` (default), three launches per step: the partial kernel; the local combine, which
    stores each (sequence, head) row straight into every rank's slot ``[parity, my_rank]`` and bumps
    that rank's counter for me; the final combine, whose CTAs wait for the counters themselves
    (bounded; ``FLAG_TIMEOUT`` in ``err_flag``) and whose last CTA takes the arrivals off again.
    ``fused=False``, five launches: partial, local combine, a push kernel, a one-warp wait kernel,
    final combine.  Either way the counters return to where they were, so every step has the same
    arguments: :meth:`capture` records the step for each of the two buffer halves as a CUDA graph and
    :meth:`replay` launches them alternately.  No host synchronisation, no NCCL call.
    """

    def __init__(self, batch: int, num_heads: int, head_dim: int, device, group=None, fused: bool = True):
        import ctypes
        import torch.distributed._symmetric_memory as symm
        from . import _lib
        self._lib, self._ct = _lib, ctypes
        self.group = group if group is not None else dist.group.WORLD
        self.G, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.B, self.H, self.D = batch, num_heads, head_dim
        G = self.G
        self.row_elems = batch * num_heads * (head_dim + 2)
        self.row_bytes = self.row_elems * 4
        if self.row_bytes % 16:
            raise ValueError("B*H*(D+2)*4 must be a multiple of 16 bytes")
        self.parts = symm.empty((2, G, batch, num_heads, head_dim + 2), dtype=torch.float32, device=device)
        self.flags = symm.empty((32,), dtype=torch.int32, device=device)
        self.parts.zero_()
        self.flags.zero_()
        torch.cuda.synchronize(device)
        self._h_parts = symm.rendezvous(self.parts, self.group)
        self._h_flags = symm.rendezvous(self.flags, self.group)
        dist.barrier(self.group)
        part_ptrs, flag_ptrs = list(self._h_parts.buffer_ptrs), list(self._h_flags.buffer_ptrs)
        PtrArr = ctypes.c_void_p * G
        self._dst = []
        for parity in range(2):     # my slot [parity, rank] in every rank's buffer
            self._dst.append(PtrArr(*[part_ptrs[g] + (parity * G + self.rank) * self.row_bytes for g in range(G)]))
        self._flag = PtrArr(*[flag_ptrs[g] + 4 * self.rank for g in range(G)])
        self.ctas_per_push = _lib.lib.attn_b200_peer_push_ctas(self.row_bytes)
        self.step = 0
        self.err_flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.fused = fused
        self._done = self.flags[31:]            # local scratch of the fused wait (never written by peers)
        self._ws = None

    def decode(self, Q, K, V, K_cache_local, V_cache_local, local_indices, local_offsets, *, scale=None,
               k_scale=None, v_scale=None, chunk=None, _parity=None) -> torch.Tensor:
        from . import ops
        lib, check = self._lib.lib, self._lib.check
        parity = self.step & 1 if _parity is None else _parity
        if _parity is None:
            self.step += 1
        stream = torch.cuda.current_stream().cuda_stream
        if self.fused:
            return self._decode_fused(Q, K, V, K_cache_local, V_cache_local, local_indices, local_offsets, parity,
                                      scale, k_scale, v_scale, chunk, stream)
        part = ops.paged_decode_partial(Q, K_cache_local, V_cache_local, local_indices, local_offsets, self.H,
                                        scale=scale, chunk=chunk, k_scale=k_scale, v_scale=v_scale)
        check(lib.attn_b200_peer_push(part.data_ptr(), self.row_bytes, self._dst[parity], self._flag, self.G, stream),
              "peer_push")
        check(lib.attn_b200_wait_flags_consume(self.flags.data_ptr(), self.G, self.ctas_per_push,
                                               self.err_flag.data_ptr(), stream), "wait_flags_consume")
        return ops.lse_combine(self.parts[parity], Q, K, V, num_heads=self.H, scale=scale)

    def _decode_fused(self, Q, K, V, Kc, Vc, ci, off, parity, scale, k_scale, v_scale, chunk, stream):
        import math
        from . import ops
        lib, check = self._lib.lib, self._lib.check
        B, H, D = self.B, self.H, self.D
        Hkv = Kc.size(1) // D
        kvd = ops._kv_code(Kc, Q)
        qd = ops._dtype_code(Q, "Q")
        T = ci.numel()
        if scale is None:
            scale = 1.0 / math.sqrt(D)
        if chunk is None:
            chunk = ops.pick_chunk(B, Hkv, D, T, Q.device, group=H // Hkv, kv_dtype=kvd)
        need = ops.decode_workspace_bytes(B, H, D, T, chunk)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=Q.device)
        check(lib.attn_b200_paged_decode_partial_push(
            Q.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), ci.data_ptr(), off.data_ptr(), self._ws.data_ptr(),
            self._ws.numel(), B, H, Hkv, D, T, Kc.size(0), 1, 0, chunk, float(scale), ops._ptr(k_scale),
            ops._ptr(v_scale), qd, kvd, self._dst[parity], self._flag, self.G, self.err_flag.data_ptr(), stream),
            "paged_decode_partial_push")
        out = torch.empty_like(Q)
        check(lib.attn_b200_lse_combine_wait(
            self.parts[parity].data_ptr(), self.G, Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), B, H,
            K.size(1) // D, D, float(scale), qd, self.flags.data_ptr(), self._done.data_ptr(),
            self.err_flag.data_ptr(), stream), "lse_combine_wait")
        return out

    def capture(self, Q, K, V, K_cache_local, V_cache_local, local_indices, local_offsets, **kw) -> None:
        """Record the step on these (static) tensors as two CUDA graphs, one per buffer half.  The
        caller refreshes the tensors' contents between replays; every rank must capture and replay in
        step with the others (a replay is one exchange)."""
        args = (Q, K, V, K_cache_local, V_cache_local, local_indices, local_offsets)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):          # warm-up outside capture: two real steps, parity stays aligned
            for _ in range(2):
                self.decode(*args, **kw)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self._graphs, self._graph_out = [], []
        for parity in range(2):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = self.decode(*args, _parity=parity, **kw)
            self._graphs.append(g)
            self._graph_out.append(out)

    def replay(self) -> torch.Tensor:
        """One captured step; returns the graph's output tensor for this buffer half."""
        parity = self.step & 1
        self.step += 1
        self._graphs[parity].replay()
        return self._graph_out[parity]
