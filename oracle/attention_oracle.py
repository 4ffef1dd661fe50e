"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, with plain torch on host tensors, the arithmetic that the
reference project (ita9naiwa/attention-impl) uses as ITS OWN ground truth: the
pure-torch functions inside its test files.  Nothing under ``oracle/`` is part
of the product: only ``tests/``, ``__graft_entry__.smoke()`` and the CPU legs of
``bench.py`` may import it, and only as the checker / the timed CPU baseline.

Parity status: pinned.  ``tests/golden/*.npz`` were produced by importing the
reference's own test modules (``tests/golden/make_golden.py``) and calling its
functions on seeded inputs; ``tests/test_oracle_golden.py`` checks every
function here against those vectors.  The two places where the reference's
torch function cannot be used literally are stated on the function:

* ``paged_decode``: the reference function hard-codes two cached tokens per
  sequence and forgets to apply ``scale`` although the reference CUDA kernel
  applies it.  The golden vectors pin the unscaled two-token form
  (``scale=1.0``); ragged lengths and ``scale = D**-0.5`` are generalisations.
* ``packed_prefill``: the reference only tests equal lengths; the ragged form
  applies the same per-sequence math to each slice.

Every function takes an optional ``compute_dtype``.  ``None`` evaluates in the
tensors' own dtype exactly as the reference test does (torch CPU half/bfloat16
matmul rounds each result tensor to that dtype).  ``torch.float32`` /
``torch.float64`` evaluates the same formula on up-cast inputs; that is the
"exact" answer a kernel with fp32 accumulation is compared with.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

E4M3_MAX = 448.0


def _starts(offsets: torch.Tensor) -> Tuple[List[int], List[int]]:
    """Inclusive cumulative lengths -> (begin, end) lists.

    Follows paged_attention_kernel.cu:35-37 and :123-125: sequence ``b`` covers
    ``[offsets[b-1], offsets[b])`` with ``offsets[-1] == 0``.
    """
    ends = [int(x) for x in offsets.tolist()]
    begs = [0] + ends[:-1]
    return begs, ends


# --------------------------------------------------------------------------------------
# a1: KV-paged single-query decode
# --------------------------------------------------------------------------------------
def paged_decode(
    Q: torch.Tensor,
    K: torch.Tensor,
    V: torch.Tensor,
    K_cache: torch.Tensor,
    V_cache: torch.Tensor,
    cache_indices: torch.Tensor,
    offsets: torch.Tensor,
    num_heads: int,
    scale: Optional[float] = None,
    compute_dtype: Optional[torch.dtype] = None,
    block_size: int = 1,
):
    """Single-query attention over slot-addressed KV rows plus the new token.

    Follows tests/test_kv_paged_attention.py:21-43 (gather rows by
    ``cache_indices``, append the new token's k/v LAST, softmax, P @ V),
    generalised from its fixed two tokens per sequence (:28-29) to ragged
    lengths through ``offsets``, with ``scale`` applied to every score as the
    reference kernel does (paged_attention_kernel.cu:134,141,269).  Pass
    ``scale=1.0`` for the literal (unscaled) reference function.

    Returns ``S, P`` as float64 ``[B, H, max_ctx + 1]`` (new token's entry at
    index ``ctx_b``, zero tail; paged_attention_kernel.cu:261-262) and ``O``
    ``[B, H*D]`` in Q's dtype.

    Two generalisations the reference does not have (it is multi-head with one slot per token):
    the pools and K, V may carry ``Hkv < H`` heads (query head h uses KV head ``h // (H // Hkv)``),
    and with ``block_size > 1`` ``cache_indices`` is a block table ``[B, max_blocks]``, token t of
    sequence b living in row ``table[b, t // block_size] * block_size + t % block_size``.
    """
    B, dim = Q.shape
    H = num_heads
    D = dim // H
    Hkv = K_cache.shape[1] // D
    g = H // Hkv
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    cd = compute_dtype or Q.dtype
    begs, ends = _starts(offsets)
    max_ctx = max([e - b for b, e in zip(begs, ends)] + [0])
    S_out = torch.zeros(B, H, max_ctx + 1, dtype=torch.float64)
    P_out = torch.zeros(B, H, max_ctx + 1, dtype=torch.float64)
    O = torch.empty(B, dim, dtype=Q.dtype)
    idx = cache_indices.long()
    for b in range(B):
        n = ends[b] - begs[b]
        if block_size > 1:
            t = torch.arange(n)
            rows = idx[b, t // block_size] * block_size + t % block_size
        else:
            rows = idx[begs[b]:ends[b]]
        q = Q[b].to(cd).reshape(H, D)
        k_all = torch.cat([K_cache[rows].to(cd).reshape(n, Hkv, D), K[b].to(cd).reshape(1, Hkv, D)], 0)
        v_all = torch.cat([V_cache[rows].to(cd).reshape(n, Hkv, D), V[b].to(cd).reshape(1, Hkv, D)], 0)
        k_all = k_all.permute(1, 0, 2).repeat_interleave(g, dim=0)  # [H, n+1, D]
        v_all = v_all.permute(1, 0, 2).repeat_interleave(g, dim=0)
        s = torch.matmul(k_all, q.unsqueeze(-1)).squeeze(-1) * scale  # [H, n+1]
        p = s.softmax(dim=-1)
        o = torch.matmul(p.unsqueeze(1), v_all).squeeze(1)  # [H, D]
        S_out[b, :, : n + 1] = s.double()
        P_out[b, :, : n + 1] = p.double()
        O[b] = o.reshape(dim).to(Q.dtype)
    return S_out, P_out, O


def paged_decode_partial(Q, K_cache, V_cache, cache_indices, offsets, num_heads, scale=None):
    """fp32 partial rows ``[B, H, D+2] = [o[D] un-normalised, m (log2 domain), l]`` of a decode over
    the given tokens only (no new token).  Not in the reference; this is the quantity one rank of a
    KV-split group exchanges, defined so that ``lse_combine`` of the partials of a partition of the
    tokens plus the new token equals ``paged_decode``."""
    B, dim = Q.shape
    H, D = num_heads, dim // num_heads
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    begs, ends = _starts(offsets)
    out = torch.zeros(B, H, D + 2, dtype=torch.float32)
    idx = cache_indices.long()
    log2e = 1.4426950408889634
    for b in range(B):
        rows = idx[begs[b]:ends[b]]
        n = rows.numel()
        if n == 0:
            out[b, :, D] = float("-inf")
            continue
        q = Q[b].float().reshape(H, D)
        k = K_cache[rows].float().reshape(n, H, D).permute(1, 0, 2)
        v = V_cache[rows].float().reshape(n, H, D).permute(1, 0, 2)
        s = torch.matmul(k, q.unsqueeze(-1)).squeeze(-1) * (scale * log2e)  # [H, n]
        m = s.max(dim=-1).values
        p = torch.exp2(s - m.unsqueeze(-1))
        out[b, :, :D] = torch.matmul(p.unsqueeze(1), v).squeeze(1)
        out[b, :, D] = m
        out[b, :, D + 1] = p.sum(-1)
    return out


def lse_combine(parts, Q, K, V, num_heads, scale=None):
    """Fold partial rows ``[G, B, H, D+2]`` and the new token (K, V) into ``[B, H*D]`` (fp32)."""
    G, B, H, RS = parts.shape
    D = RS - 2
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    log2e = 1.4426950408889634
    q = Q.float().reshape(B, H, D)
    s_new = (q * K.float().reshape(B, H, D)).sum(-1) * (scale * log2e)       # [B, H]
    m_all = torch.cat([parts[..., D], s_new.unsqueeze(0)], 0)                   # [G+1, B, H]
    M = m_all.max(0).values
    w = torch.exp2(m_all - M)                                                    # exp2(-inf) = 0
    num = (parts[..., :D] * w[:G].unsqueeze(-1)).sum(0) + w[G].unsqueeze(-1) * V.float().reshape(B, H, D)
    den = (parts[..., D + 1] * w[:G]).sum(0) + w[G]
    return (num / den.unsqueeze(-1)).reshape(B, H * D)


def quantize_e4m3_per_head(x: torch.Tensor, num_heads: int):
    """Per-head absmax e4m3 quantisation of a ``[rows, H*D]`` pool.

    Not in the reference (it has no FP8 path); defined by the workload
    description: ``scale_h = absmax(x[:, h, :]) / 448``, ``x8 = rn_e4m3(x / scale_h)``.
    Returns ``(x8 as torch.float8_e4m3fn [rows, H*D], scale float32 [H])``.
    """
    rows, dim = x.shape
    D = dim // num_heads
    xf = x.float().reshape(rows, num_heads, D)
    amax = xf.abs().amax(dim=(0, 2)).clamp_min(1e-12)
    sc = (amax / E4M3_MAX).float()
    x8 = (xf / sc.view(1, num_heads, 1)).to(torch.float8_e4m3fn).reshape(rows, dim)
    return x8, sc


def dequantize_e4m3_per_head(x8: torch.Tensor, sc: torch.Tensor, num_heads: int, dtype=torch.float32):
    rows, dim = x8.shape
    D = dim // num_heads
    return (x8.float().reshape(rows, num_heads, D) * sc.view(1, num_heads, 1).float()).reshape(rows, dim).to(dtype)


# --------------------------------------------------------------------------------------
# a5: single query over a contiguous cache
# --------------------------------------------------------------------------------------
def single_query(Q, K, V, K_cache, V_cache, num_heads: int, compute_dtype=None):
    """Follows tests/test_single_query_attention.py:9-32 with ``num_heads``
    actually used and NO scale (the function computes ``scale`` at :12 and never
    applies it; the reference kernel does not either, attention_kernel.cu:129,143).
    S, P are ``[B, H, ctx+1]`` in the input dtype, O ``[B, H*D]``.
    """
    B, dim = Q.shape
    _, ctx, _ = K_cache.shape
    H, D = num_heads, dim // num_heads
    cd = compute_dtype or Q.dtype
    q = Q.to(cd).reshape(B, H, D)
    k = K.to(cd).reshape(B, H, D)
    v = V.to(cd).reshape(B, H, D)
    kc = K_cache.to(cd).reshape(B, ctx, H, D).permute(0, 2, 1, 3)
    vc = V_cache.to(cd).reshape(B, ctx, H, D).permute(0, 2, 1, 3)
    new_k = torch.cat([kc, k.unsqueeze(2)], dim=2)
    new_v = torch.cat([vc, v.unsqueeze(2)], dim=2)
    S = torch.matmul(new_k, q.unsqueeze(-1)).squeeze(-1)
    P = S.softmax(dim=-1)
    O = torch.matmul(P.unsqueeze(2), new_v).squeeze(2).reshape(B, dim)
    return S, P, O.to(Q.dtype)


# --------------------------------------------------------------------------------------
# a4 / a2: dense masked attention, packed causal prefill
# --------------------------------------------------------------------------------------
def dense_mha(Q, K, V, mask, num_heads: int, fill: float = 100000.0, compute_dtype=None, out_dtype=None):
    """Follows tests/test_naive_attention.py:13-25 (``fill=100000``) and
    tests/test_packed_attention.py:9-22 (``fill=10000``):
    ``S = scale * Q K^T + (mask - 1) * fill``, ``P = softmax(S)``, ``O = P V``,
    ``scale = (dim/num_heads) ** -0.5``.  Q, K, V ``[B, L, H*D]``; mask ``[B, L, L]`` or None.
    O is returned in ``out_dtype`` (default: Q's dtype).
    """
    B, L, dim = Q.shape
    H, D = num_heads, dim // num_heads
    cd = compute_dtype or Q.dtype
    q = Q.to(cd).reshape(B, L, H, D).permute(0, 2, 1, 3).reshape(B * H, L, D)
    k = K.to(cd).reshape(B, L, H, D).permute(0, 2, 1, 3).reshape(B * H, L, D)
    scale = (dim / num_heads) ** -0.5
    S = torch.bmm(q, k.permute(0, 2, 1)).reshape(B, H, L, L)
    S = S * scale
    if mask is not None:
        S = S + (mask.to(cd).unsqueeze(1) - 1) * fill
    P = S.softmax(dim=-1)
    O = torch.matmul(P, V.to(cd).reshape(B, L, H, D).permute(0, 2, 1, 3))
    O = O.permute(0, 2, 1, 3).reshape(B, L, dim)
    return S, P, O.to(out_dtype or Q.dtype)


def packed_prefill(Q, K, V, offsets, num_heads: int, compute_dtype=None, out_dtype=None):
    """Causal attention per sequence slice of a packed ``[sum L, H*D]`` buffer.

    Per slice this is ``dense_mha`` with a lower-triangular mask and fill 10000
    (tests/test_packed_attention.py:9-22, mask built at :40); key j is visible
    to query i iff j <= i (paged_attention_kernel.cu:47).  Returns O only.
    """
    begs, ends = _starts(offsets)
    O = torch.zeros(Q.shape, dtype=out_dtype or Q.dtype)
    cd = compute_dtype or Q.dtype
    for b, e in zip(begs, ends):
        L = e - b
        if L == 0:
            continue
        mask = torch.tril(torch.ones(L, L, dtype=cd)).unsqueeze(0)
        _, _, o = dense_mha(Q[b:e].unsqueeze(0), K[b:e].unsqueeze(0), V[b:e].unsqueeze(0), mask,
                            num_heads, fill=10000.0, compute_dtype=compute_dtype, out_dtype=O.dtype)
        O[b:e] = o[0]
    return O


def paged_prefill(Q, K_cache, V_cache, cache_indices, kv_offsets, q_offsets, num_heads, scale=None,
                  compute_dtype=None, out_dtype=None):
    """Chunked prefill through the slot table (not in the reference; the packed-prefill math of
    tests/test_packed_attention.py:9-22 applied to gathered rows): per sequence, the query rows are
    its last ``q_len`` tokens and see key j iff ``j <= kv_len - q_len + i``."""
    nq, dim = Q.shape
    H, D = num_heads, dim // num_heads
    Hkv = K_cache.shape[1] // D
    g = H // Hkv
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    cd = compute_dtype or Q.dtype
    qb, qe = _starts(q_offsets)
    kb, ke = _starts(kv_offsets)
    O = torch.zeros(Q.shape, dtype=out_dtype or Q.dtype)
    idx = cache_indices.long()
    for b in range(len(qe)):
        lq, lk = qe[b] - qb[b], ke[b] - kb[b]
        if lq == 0:
            continue
        rows = idx[kb[b]:ke[b]]
        q = Q[qb[b]:qe[b]].to(cd).reshape(lq, H, D).permute(1, 0, 2)
        k = K_cache[rows].to(cd).reshape(lk, Hkv, D).permute(1, 0, 2).repeat_interleave(g, dim=0)
        v = V_cache[rows].to(cd).reshape(lk, Hkv, D).permute(1, 0, 2).repeat_interleave(g, dim=0)
        S = torch.matmul(q, k.transpose(-1, -2)) * scale
        vis = torch.arange(lk).unsqueeze(0) <= (lk - lq + torch.arange(lq)).unsqueeze(1)
        S = S.masked_fill(~vis.unsqueeze(0), float("-inf"))
        P = S.softmax(dim=-1)
        O[qb[b]:qe[b]] = torch.matmul(P, v).permute(1, 0, 2).reshape(lq, dim).to(O.dtype)
    return O


# --------------------------------------------------------------------------------------
# a3: rotary embedding
# --------------------------------------------------------------------------------------
def rope_tables(rot_dim: int, max_pos: int, base: float = 10000.0, dtype=torch.float16):
    """cos/sin tables ``[max_pos, rot_dim/2]`` exactly as the reference's kernel-side
    module builds them (tests/test_rotary_embedding.py:57,65-71): fp32 outer
    product of positions and ``inv_freq``, ``cos``/``sin`` in fp32, then cast.
    """
    inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2).float() / rot_dim))
    t = torch.arange(max_pos, dtype=inv_freq.dtype)
    freqs = torch.outer(t, inv_freq)
    return freqs.cos().to(dtype), freqs.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """tests/test_rotary_embedding.py:43-48."""
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope(q, k, positions, cos, sin, head_dim: int):
    """NeoX-pairing rotary embedding; returns new tensors (the kernel is in place).

    Follows tests/test_rotary_embedding.py:32-48: ``x * cos + rotate_half(x) * sin``
    evaluated in the tensors' dtype (three roundings per element for fp16, as
    the reference kernel's ``scalar_t`` arithmetic, rotary_embedding.cu:33-34),
    on the first ``rot_dim = 2 * cos.shape[1]`` dims of every head, the rest
    passed through (tests/test_rotary_embedding.py:131-135).  ``cos``/``sin`` are
    the ``[max_pos, rot_dim/2]`` tables the kernel itself receives; the full-width
    table is ``cat(table, table)`` (:29).
    """
    N = q.shape[0]
    rh = cos.shape[1]
    rot = 2 * rh
    pos = positions.long()
    c = torch.cat((cos, cos), dim=-1)[pos].unsqueeze(1)  # [N, 1, rot]
    s = torch.cat((sin, sin), dim=-1)[pos].unsqueeze(1)

    def one(x):
        xh = x.reshape(N, -1, head_dim)
        xr, xp = xh[..., :rot], xh[..., rot:]
        xr = xr * c + rotate_half(xr) * s
        return torch.cat((xr, xp), dim=-1).reshape(N, -1)

    return one(q), one(k)
