"""GPU: KV-paged decode and single-query attention through the drop-in API vs the CPU oracle.

Tolerance: <= 2e-3 max-abs on O for fp16/bf16 inputs against the oracle evaluated in fp32 on the
same (rounded) inputs; the same-dtype oracle (the reference's literal torch math) is checked with
the dtype's own rounding added.  FP8 KV: <= 2e-2 relative against the oracle on dequantised KV.
"""
import math

import pytest
import torch

from oracle import attention_oracle as orc
from conftest import load_golden
from helpers import decode_inputs, uniform_lens

pytestmark = pytest.mark.gpu

TOL16 = 2e-3


def _gpu(*ts):
    return [t.cuda() for t in ts]


def _decode(Q, K, V, Kc, Vc, ci, off, H, **kw):
    import lm_ops
    S, P, O = lm_ops.paged_kv_attention_forward(*_gpu(Q, K, V, Kc, Vc, ci, off), H, **kw)
    torch.cuda.synchronize()
    return S.cpu(), P.cpu(), O.cpu()


@pytest.mark.parametrize("tag", ["paged_ref_shape", "paged_f32"])
def test_paged_decode_golden_unscaled(tag):
    """The reference's own torch function (unscaled, two cached tokens per sequence)."""
    g = load_golden(tag)
    S, P, O = _decode(g["Q"], g["K"], g["V"], g["K_cache"], g["V_cache"], g["cache_indices"], g["offsets"],
                      int(g["num_heads"]), scale=1.0)
    assert (S.float() - g["S"]).abs().max() < 1e-5
    assert (P.float() - g["P"]).abs().max() < 1e-5
    assert (O - g["O"]).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_paged_decode_small_batch_workload(dtype):
    """B=8, H=32, D=128, ctx ~ U[128,1024], 16384-slot pool, scale 1/sqrt(128)."""
    B, H, D = 8, 32, 128
    lens = uniform_lens(B, 128, 1024, seed=1)
    inp = decode_inputs(B, H, D, lens, 16384, dtype, seed=1001)
    S, P, O = _decode(*inp, H)
    S32, P32, O32 = orc.paged_decode(*inp, H, compute_dtype=torch.float32)
    tol = TOL16 if dtype == torch.float16 else 8e-3   # bf16 output rounding: half-ulp 3.9e-3 at |O|<1
    assert (O.float() - O32.float()).abs().max() <= tol
    # fp32-evaluated comparison without the output rounding of the oracle
    _, _, O64 = orc.paged_decode(*[t.double() if t.is_floating_point() else t for t in inp], H)
    assert (O.double() - O64).abs().max() <= (TOL16 if dtype == torch.float16 else 8e-3)
    assert (S - S32).abs().max() < 2e-4 * math.sqrt(D)
    assert (P - P32).abs().max() < 1e-4
    # the reference's literal same-dtype torch math
    _, _, Oh = orc.paged_decode(*inp, H)
    assert (O.float() - Oh.float()).abs().max() <= 4 * tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("H,D", [(2, 2), (4, 16), (8, 64), (3, 40), (16, 128), (4, 256), (1, 128)])
@pytest.mark.parametrize("chunk", [None, 32, 64])
def test_paged_decode_ragged_shapes(dtype, H, D, chunk):
    """Ragged lengths incl. empty sequences, length 1, chunk-boundary lengths."""
    lens = [0, 1, 31, 32, 33, 64, 0, 100, 257, 5]
    B = len(lens)
    inp = decode_inputs(B, H, D, lens, 1024, dtype, seed=H * 1000 + D)
    S, P, O = _decode(*inp, H, chunk=chunk)
    S32, P32, O32 = orc.paged_decode(*inp, H, compute_dtype=torch.float32)
    tol = {torch.float16: TOL16, torch.bfloat16: 1.6e-2, torch.float32: 2e-5}[dtype]
    assert (O.float() - O32.float()).abs().max() <= tol
    assert (P - P32).abs().max() < 2e-4
    # tail beyond ctx_b + 1 stays zero like the reference's zero-initialised buffers
    for b, n in enumerate(lens):
        assert S[b, :, n + 1:].abs().sum() == 0 and P[b, :, n + 1:].abs().sum() == 0
    assert torch.allclose(P.sum(-1), torch.ones(B, H, dtype=torch.float64), atol=1e-5)


def test_paged_decode_without_sp_matches_with_sp():
    lens = uniform_lens(6, 10, 700, seed=4)
    inp = decode_inputs(6, 8, 128, lens, 4096, torch.float16, seed=77)
    _, _, O1 = _decode(*inp, 8)
    S, P, O2 = _decode(*inp, 8, return_sp=False)
    assert S.numel() == 0 and P.numel() == 0
    assert torch.equal(O1, O2)


def test_paged_decode_chunk_invariance():
    """Split-KV must not change the answer beyond fp32 reassociation."""
    lens = uniform_lens(4, 900, 3000, seed=9)
    inp = decode_inputs(4, 8, 128, lens, 16384, torch.float16, seed=5)
    outs = [_decode(*inp, 8, return_sp=False, chunk=c)[2].float() for c in (32, 256, 2048)]
    assert (outs[0] - outs[1]).abs().max() < 1e-3 and (outs[0] - outs[2]).abs().max() < 1e-3


def test_paged_decode_fp8_kv():
    """e4m3 KV with per-head absmax scales: <= 2e-2 relative vs the oracle on dequantised KV."""
    import lm_ops
    B, H, D = 6, 8, 128
    lens = uniform_lens(B, 300, 2000, seed=11)
    Q, K, V, Kc, Vc, ci, off = decode_inputs(B, H, D, lens, 16384, torch.float16, seed=12)
    K8, ks = orc.quantize_e4m3_per_head(Kc, H)
    V8, vs = orc.quantize_e4m3_per_head(Vc, H)
    Kd = orc.dequantize_e4m3_per_head(K8, ks, H)
    Vd = orc.dequantize_e4m3_per_head(V8, vs, H)
    _, _, Oref = orc.paged_decode(Q.float(), K.float(), V.float(), Kd, Vd, ci, off, H)
    for kw in ({}, {"chunk": 64}):
        _, _, O = lm_ops.paged_kv_attention_forward(Q.cuda(), K.cuda(), V.cuda(), K8.cuda(), V8.cuda(), ci.cuda(),
                                                    off.cuda(), H, return_sp=False, k_scale=ks.cuda(),
                                                    v_scale=vs.cuda(), **kw)
        rel = (O.cpu().float() - Oref).norm() / Oref.norm()
        assert rel <= 2e-2
        assert (O.cpu().float() - Oref).abs().max() <= 2e-2 * Oref.abs().max()


def test_paged_decode_bad_slot_is_flagged():
    import lm_ops
    Q, K, V, Kc, Vc, ci, off = decode_inputs(2, 8, 128, [40, 50], 256, torch.float16, seed=3)
    ci[7] = 100000
    ci[60] = -5
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    _, _, O = lm_ops.paged_kv_attention_forward(*_gpu(Q, K, V, Kc, Vc, ci, off), 8, return_sp=False, err_flag=flag)
    assert int(flag.item()) & 1
    assert torch.isfinite(O).all()


def test_partial_plus_combine_equals_decode():
    """KV split into 3 slices per sequence -> partials -> combine == one-shot decode."""
    import attention_impl_b200 as A
    B, H, D, G = 5, 8, 128, 3
    lens = uniform_lens(B, 50, 900, seed=21)
    Q, K, V, Kc, Vc, ci, off = decode_inputs(B, H, D, lens, 8192, torch.float16, seed=22)
    _, _, O_full = _decode(Q, K, V, Kc, Vc, ci, off, H, return_sp=False)
    parts = []
    begs = [0] + off.tolist()[:-1]
    for r in range(G):
        idx, ln = [], []
        for b, n in enumerate(lens):
            lo, hi = n * r // G, n * (r + 1) // G
            idx.append(ci[begs[b] + lo: begs[b] + hi])
            ln.append(hi - lo)
        ci_r = torch.cat(idx)
        off_r = torch.tensor(ln).cumsum(0).int()
        parts.append(A.paged_decode_partial(Q.cuda(), Kc.cuda(), Vc.cuda(), ci_r.cuda(), off_r.cuda(), H))
    O = A.lse_combine(torch.stack(parts).contiguous(), Q.cuda(), K.cuda(), V.cuda(), num_heads=H)
    assert (O.cpu().float() - O_full.float()).abs().max() < 1e-3


@pytest.mark.parametrize("tag", ["single_f32", "single_f16"])
def test_single_query_golden(tag):
    import lm_ops
    g = load_golden(tag)
    S, P, O = lm_ops.single_query_attention(*_gpu(g["Q"], g["K"], g["V"], g["K_cache"], g["V_cache"]),
                                            int(g["num_heads"]))
    tol = 1e-5 if g["Q"].dtype == torch.float32 else 2e-3
    assert (O.cpu().float() - g["O"].float()).abs().max() <= tol
    assert (P.cpu().float() - g["P"].float()).abs().max() <= tol
    assert (S.cpu().float() - g["S"].float()).abs().max() <= tol * 4


@pytest.mark.parametrize("batch_size", [1, 4, 8])
@pytest.mark.parametrize("context_size", [256, 512])
@pytest.mark.parametrize("dim", [32, 64, 256])
@pytest.mark.parametrize("num_heads", [1, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_single_query_reference_matrix(batch_size, context_size, dim, num_heads, dtype):
    """The reference's parameter grid (tests/test_single_query_attention.py:35-39), with non-zero
    caches, num_heads actually passed, and the result asserted."""
    import lm_ops
    gen = torch.Generator().manual_seed(batch_size * 7 + dim)
    Q, K, V = ((torch.randn(batch_size, dim, generator=gen) * 0.1).to(dtype) for _ in range(3))
    Kc, Vc = ((torch.randn(batch_size, context_size, dim, generator=gen) * 0.1).to(dtype) for _ in range(2))
    S1, P1, O1 = orc.single_query(Q, K, V, Kc, Vc, num_heads, compute_dtype=torch.float32)
    S2, P2, O2 = lm_ops.single_query_attention(*_gpu(Q, K, V, Kc, Vc), num_heads)
    assert torch.allclose(O1.float(), O2.cpu().float(), atol=1e-2)     # the reference's tolerance
    assert (O1.float() - O2.cpu().float()).abs().max() <= (2e-3 if dtype == torch.float16 else 1e-5)


def test_decode_graph_replays_with_changing_lengths():
    """One captured graph, two steps with different context lengths and slot tables."""
    import attention_impl_b200 as A
    B, H, D, cap = 8, 32, 128, 8192
    g = torch.Generator().manual_seed(41)
    Kc, Vc = (torch.randn(16384, H * D, generator=g).half().cuda() for _ in range(2))
    graph = A.PagedDecodeGraph(Kc, Vc, B, H, cap)
    for seed, (lo, hi) in ((1, (128, 1024)), (2, (1, 300))):
        lens = uniform_lens(B, lo, hi, seed=seed)
        Q, K, V, _, _, ci, off = decode_inputs(B, H, D, lens, 16384, torch.float16, seed=seed)
        graph.q.copy_(Q); graph.k.copy_(K); graph.v.copy_(V)
        graph.cache_indices[: ci.numel()].copy_(ci)
        graph.offsets.copy_(off)
        O = graph.replay().clone()
        _, _, O_ref = A.paged_kv_attention_forward(Q.cuda(), K.cuda(), V.cuda(), Kc, Vc, ci.cuda(), off.cuda(), H,
                                                   return_sp=False)
        assert (O.float() - O_ref.float()).abs().max() < 1e-3
        _, _, O32 = orc.paged_decode(Q, K, V, Kc.cpu(), Vc.cpu(), ci, off, H, compute_dtype=torch.float32)
        assert (O.cpu().float() - O32.float()).abs().max() <= TOL16


def test_paged_decode_pool_beyond_int32_element_offsets():
    """600 000 slots x 4096 elements: element offsets exceed 2^31 (the reference's int index
    overflows past 524 288 slots, paged_attention_kernel.cu:132).  Only the rows that are used are
    non-zero; the oracle runs on the gathered rows."""
    import lm_ops
    B, H, D = 3, 32, 128
    n_slots = 600_000
    lens = [700, 1, 333]
    g = torch.Generator().manual_seed(123)
    T = sum(lens)
    Kc = torch.zeros(n_slots, H * D, dtype=torch.float16, device="cuda")
    Vc = torch.zeros(n_slots, H * D, dtype=torch.float16, device="cuda")
    # all slots in the upper part of the pool, beyond the 32-bit element range
    ci = (torch.randperm(60_000, generator=g)[:T] + 530_000).int()
    rows_k = torch.randn(T, H * D, generator=g).half()
    rows_v = torch.randn(T, H * D, generator=g).half()
    Kc[ci.long().cuda()] = rows_k.cuda()
    Vc[ci.long().cuda()] = rows_v.cuda()
    Q, K, V = (torch.randn(B, H * D, generator=g).half() for _ in range(3))
    off = torch.tensor(lens).cumsum(0).int()
    _, _, O = lm_ops.paged_kv_attention_forward(Q.cuda(), K.cuda(), V.cuda(), Kc, Vc, ci.cuda(), off.cuda(), H,
                                                return_sp=False)
    _, _, O32 = orc.paged_decode(Q, K, V, rows_k, rows_v, torch.arange(T).int(), off, H, compute_dtype=torch.float32)
    assert (O.cpu().float() - O32.float()).abs().max() <= TOL16


def _gqa_inputs(B, Hq, Hkv, D, lens, n_slots, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    Q = torch.randn(B, Hq * D, generator=g).to(dtype)
    K, V = (torch.randn(B, Hkv * D, generator=g).to(dtype) for _ in range(2))
    Kc, Vc = (torch.randn(n_slots, Hkv * D, generator=g).to(dtype) for _ in range(2))
    ci = torch.randperm(n_slots, generator=g)[: sum(lens)].int()
    off = torch.tensor(lens).cumsum(0).int()
    return Q, K, V, Kc, Vc, ci, off


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 4, 128), (32, 8, 128), (16, 2, 128), (8, 2, 64), (6, 2, 128), (12, 4, 48)])
def test_paged_decode_grouped_query(dtype, Hq, Hkv, D):
    """Fewer KV heads than query heads (not in the reference): group sizes 2, 4, 8 take the fast kernel,
    3 and head_dim 48 the generic one."""
    lens = [0, 1, 40, 129, 700]
    inp = _gqa_inputs(len(lens), Hq, Hkv, D, lens, 2048, dtype, seed=Hq * 10 + Hkv)
    S, P, O = _decode(*inp, Hq)
    S32, P32, O32 = orc.paged_decode(*inp, Hq, compute_dtype=torch.float32)
    tol = TOL16 if dtype == torch.float16 else 1.6e-2
    assert (O.float() - O32.float()).abs().max() <= tol
    assert (P - P32).abs().max() < 2e-4


def test_paged_decode_grouped_query_fp8():
    B, Hq, Hkv, D = 4, 32, 8, 128
    lens = uniform_lens(B, 100, 1500, seed=6)
    Q, K, V, Kc, Vc, ci, off = _gqa_inputs(B, Hq, Hkv, D, lens, 8192, torch.float16, seed=7)
    K8, ks = orc.quantize_e4m3_per_head(Kc, Hkv)
    V8, vs = orc.quantize_e4m3_per_head(Vc, Hkv)
    Kd, Vd = orc.dequantize_e4m3_per_head(K8, ks, Hkv), orc.dequantize_e4m3_per_head(V8, vs, Hkv)
    _, _, Oref = orc.paged_decode(Q.float(), K.float(), V.float(), Kd, Vd, ci, off, Hq)
    import lm_ops
    _, _, O = lm_ops.paged_kv_attention_forward(Q.cuda(), K.cuda(), V.cuda(), K8.cuda(), V8.cuda(), ci.cuda(),
                                                off.cuda(), Hq, return_sp=False, k_scale=ks.cuda(), v_scale=vs.cuda())
    assert (O.cpu().float() - Oref).norm() / Oref.norm() <= 2e-2


@pytest.mark.parametrize("block_size", [4, 16, 64])
@pytest.mark.parametrize("Hq,Hkv", [(8, 8), (16, 4)])
def test_paged_decode_block_table(block_size, Hq, Hkv):
    """KV blocks of several tokens addressed through a [B, max_blocks] block table."""
    import lm_ops
    B, D = 5, 128
    lens = [1, block_size, block_size + 1, 333, 0]
    n_blocks = 128
    g = torch.Generator().manual_seed(block_size)
    max_blocks = max((n + block_size - 1) // block_size for n in lens)
    perm = torch.randperm(n_blocks, generator=g)
    table = torch.full((B, max_blocks), -1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(lens):
        nb = (n + block_size - 1) // block_size
        table[b, :nb] = perm[nxt:nxt + nb].int()
        nxt += nb
    Q = torch.randn(B, Hq * D, generator=g).half()
    K, V = (torch.randn(B, Hkv * D, generator=g).half() for _ in range(2))
    Kc, Vc = (torch.randn(n_blocks * block_size, Hkv * D, generator=g).half() for _ in range(2))
    off = torch.tensor(lens).cumsum(0).int()
    S, P, O = lm_ops.paged_kv_attention_forward(Q.cuda(), K.cuda(), V.cuda(), Kc.cuda(), Vc.cuda(), table.cuda(),
                                                off.cuda(), Hq, block_size=block_size)
    tbl = table.clamp(min=0)
    S32, P32, O32 = orc.paged_decode(Q, K, V, Kc, Vc, tbl, off, Hq, compute_dtype=torch.float32,
                                     block_size=block_size)
    assert (O.cpu().float() - O32.float()).abs().max() <= TOL16
    assert (P.cpu() - P32).abs().max() < 2e-4


def test_host_staged_decoder_matches_direct_call():
    """Inputs in pinned host memory, uploads overlapped with compute in sequence groups."""
    import attention_impl_b200 as A
    B, H, D = 12, 8, 128
    lens = uniform_lens(B, 1, 900, seed=77)
    Q, K, V, Kc, Vc, ci, off = decode_inputs(B, H, D, lens, 16384, torch.float16, seed=78)
    Kd, Vd = Kc.cuda(), Vc.cuda()
    dec = A.HostStagedDecoder(Kd, Vd, H, B, ci.numel(), n_groups=3)
    out = torch.empty(B, H * D, dtype=torch.float16).pin_memory()
    pins = [t.pin_memory() for t in (Q, K, V, ci, off)]
    for _ in range(2):          # staging buffers are reused across steps
        out.zero_()
        dec(*pins, out)
        _, _, O_ref = A.paged_kv_attention_forward(Q.cuda(), K.cuda(), V.cuda(), Kd, Vd, ci.cuda(), off.cuda(), H,
                                                   return_sp=False)
        assert (out.float() - O_ref.cpu().float()).abs().max() < 1e-3
