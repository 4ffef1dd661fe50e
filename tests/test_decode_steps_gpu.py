"""GPU: captured decode steps (grouped-query pools; RoPE -> cache append -> attention -> combine in
one graph), the host-staged decoder with a prefetched slot table, and the e4m3 path at long context.

Every case goes through the drop-in modules / the C ABI and is compared with the CPU oracle
(fp16: <= 2e-3 max-abs against the fp32-evaluated oracle; bf16: its output rounding added; e4m3
KV: <= 2e-2 relative against the oracle on dequantised KV).
"""
import pytest
import torch

from oracle import attention_oracle as orc
from helpers import decode_inputs, uniform_lens

pytestmark = pytest.mark.gpu

TOL16 = 2e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("H,D", [(32, 128), (3, 128), (8, 64), (4, 256)])
def test_single_launch_decode_ragged(dtype, H, D):
    """One CTA per (sequence, head), combine in shared memory: ragged lengths incl. empty sequences,
    sequences shorter than one warp tile, longer than one round of the CTA's eight warps."""
    import attention_impl_b200 as A
    lens = [0, 1, 15, 16, 17, 127, 128, 129, 0, 700, 1030, 5]
    inp = decode_inputs(len(lens), H, D, lens, 4096, dtype, seed=H * 10 + D)
    args = [t.cuda() for t in inp]
    _, _, O = A.paged_kv_attention_forward(*args, H, return_sp=False, single_launch=True)
    _, _, O32 = orc.paged_decode(*inp, H, compute_dtype=torch.float32)
    tol = TOL16 if dtype == torch.float16 else 1.6e-2
    assert torch.isfinite(O).all()
    assert (O.cpu().float() - O32.float()).abs().max() <= tol
    _, _, O2 = A.paged_kv_attention_forward(*args, H, return_sp=False, single_launch=False)
    assert (O.float() - O2.float()).abs().max() <= (1e-3 if dtype == torch.float16 else 1.6e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_tables_ready_steps_chained_in_one_graph(dtype):
    """Four decode steps back to back in one CUDA graph, each over its own pool, with `tables_ready`:
    every partial kernel is a programmatic dependent of the previous step's combine and reads the slot
    table and the offsets before that kernel has finished.  Each step's output equals the plain call's
    bit for bit and the oracle within tolerance; a bad slot is still flagged."""
    import attention_impl_b200 as A
    B, H, D = 8, 32, 128
    lens = [0, 1, 31, 32, 33, 700, 1024, 129]
    steps = []
    for s_ in range(4):
        inp = decode_inputs(B, H, D, lens, 4096, dtype, seed=50 + s_)
        steps.append((inp, [t.cuda() for t in inp], torch.empty(B, H * D, dtype=dtype, device="cuda")))
    T = sum(lens)
    chunk = 32
    ws = torch.empty(A.ops.decode_workspace_bytes(B, H, D, T, chunk), dtype=torch.uint8, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")

    def many():
        for _, a, out in steps:
            A.paged_kv_attention_forward(*a, H, return_sp=False, chunk=chunk, workspace=ws, out=out,
                                         tables_ready=True, err_flag=flag)
    g = A.ops.capture_graph(torch.device("cuda"), many)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    tol = TOL16 if dtype == torch.float16 else 1.6e-2
    for inp, a, out in steps:
        _, _, O32 = orc.paged_decode(*inp, H, compute_dtype=torch.float32)
        assert (out.cpu().float() - O32.float()).abs().max() <= tol
        _, _, plain = A.paged_kv_attention_forward(*a, H, return_sp=False, chunk=chunk, single_launch=False)
        assert torch.equal(out, plain)
    # eager, right behind a kernel that writes q (the case the flag allows): same bits again
    inp, a, out = steps[0]
    q2 = a[0].clone()
    q2.mul_(1.0)
    _, _, O = A.paged_kv_attention_forward(q2, *a[1:], H, return_sp=False, chunk=chunk, single_launch=False,
                                           tables_ready=True)
    assert torch.equal(O, out)
    ci = a[5].clone()
    ci[40] = -7
    torch.cuda.synchronize()      # the flag's contract: the tables are not written by the kernel just before the call
    A.paged_kv_attention_forward(*a[:5], ci, a[6], H, return_sp=False, chunk=chunk, single_launch=False,
                                 tables_ready=True, err_flag=flag)
    assert int(flag.item()) & 1


def test_single_launch_decode_small_batch_workload_and_its_choice():
    """B=8, H=32, D=128, ctx ~ U[128,1024]: the heuristic picks the single-launch form by itself; bad
    slots are flagged and skipped; cases it does not cover are refused when forced."""
    import attention_impl_b200 as A
    from attention_impl_b200 import _lib
    B, H, D = 8, 32, 128
    lens = uniform_lens(B, 128, 1024, seed=1)
    inp = decode_inputs(B, H, D, lens, 16384, torch.float16, seed=1001)
    T = sum(lens)
    assert _lib.lib.attn_b200_paged_decode_single_launch_ok(B, H, H, D, T, 1, _lib.F16, _lib.F16, 148) == 1
    assert _lib.lib.attn_b200_paged_decode_single_launch_ok(256, H, H, D, 4_600_000, 1, _lib.F16, _lib.F16, 148) == 0
    assert _lib.lib.attn_b200_paged_decode_single_launch_ok(B, H, 8, D, T, 1, _lib.F16, _lib.F16, 148) == 0
    args = [t.cuda() for t in inp]
    _, _, O = A.paged_kv_attention_forward(*args, H, return_sp=False)                 # auto: single launch
    _, _, O32 = orc.paged_decode(*inp, H, compute_dtype=torch.float32)
    assert (O.cpu().float() - O32.float()).abs().max() <= TOL16
    ci = inp[5].clone()
    ci[3] = 10 ** 6
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    _, _, Ob = A.paged_kv_attention_forward(*args[:5], ci.cuda(), args[6], H, return_sp=False, single_launch=True,
                                            err_flag=flag)
    assert int(flag.item()) & 1 and torch.isfinite(Ob).all()
    with pytest.raises(RuntimeError):
        A.paged_kv_attention_forward(*[a.float() if a.is_floating_point() else a for a in args], H, return_sp=False,
                                     single_launch=True)
    with pytest.raises(RuntimeError, match="single_launch=True"):
        A.paged_kv_attention_forward(*args, H, single_launch=True)


def test_decode_graph_grouped_query_pools():
    """A captured step over pools with fewer KV heads than query heads (head_dim given explicitly)."""
    import attention_impl_b200 as A
    B, H, Hkv, D, cap = 4, 16, 4, 128, 4096
    g = torch.Generator().manual_seed(5)
    Kc, Vc = (torch.randn(8192, Hkv * D, generator=g).half().cuda() for _ in range(2))
    graph = A.PagedDecodeGraph(Kc, Vc, B, H, cap, head_dim=D)
    assert graph.q.shape == (B, H * D) and graph.k.shape == (B, Hkv * D)
    for seed in (1, 2):
        lens = uniform_lens(B, 1, 900, seed=seed)
        gg = torch.Generator().manual_seed(seed)
        Q = torch.randn(B, H * D, generator=gg).half()
        K, V = (torch.randn(B, Hkv * D, generator=gg).half() for _ in range(2))
        ci = torch.randperm(8192, generator=gg)[: sum(lens)].int()
        off = torch.tensor(lens).cumsum(0).int()
        graph.host_q.copy_(Q); graph.host_k.copy_(K); graph.host_v.copy_(V)
        graph.host_cache_indices[: ci.numel()].copy_(ci); graph.host_offsets.copy_(off)
        graph.upload(ci.numel())
        O = graph.replay().clone()
        _, _, O32 = orc.paged_decode(Q, K, V, Kc.cpu(), Vc.cpu(), ci, off, H, compute_dtype=torch.float32)
        assert (O.cpu().float() - O32.float()).abs().max() <= TOL16
    with pytest.raises(RuntimeError, match="head count"):
        A.PagedDecodeGraph(Kc, Vc, B, 6, cap, head_dim=D)


@pytest.mark.parametrize("fp8", [False, True])
def test_decode_step_graph_three_growing_steps(fp8):
    """RoPE -> cache append -> attention -> combine replayed from one graph for three consecutive
    steps of growing sequences; every step's output and the pool rows it wrote are compared with
    the oracle (rope + scatter + paged_decode)."""
    import attention_impl_b200 as A
    B, H, D, n_slots, max_pos = 5, 8, 128, 4096, 2048
    g = torch.Generator().manual_seed(77)
    lens = [0, 1, 70, 300, 33]
    Kc, Vc = (torch.randn(n_slots, H * D, generator=g).half() for _ in range(2))
    cos, sin = orc.rope_tables(D, max_pos)
    perm = torch.randperm(n_slots - 1, generator=g) + 1           # slot 0 stays out of use
    seq_slots, nxt = [], 0
    for n in lens:
        seq_slots.append(perm[nxt:nxt + n].tolist())
        nxt += n
    if fp8:
        K8, ks = orc.quantize_e4m3_per_head(Kc, H)
        V8, vs = orc.quantize_e4m3_per_head(Vc, H)
        Kd, Vd = K8.cuda(), V8.cuda()
        Kref, Vref = orc.dequantize_e4m3_per_head(K8, ks, H), orc.dequantize_e4m3_per_head(V8, vs, H)
        kw = dict(k_scale=ks.cuda(), v_scale=vs.cuda(), dtype=torch.float16)
    else:
        Kd, Vd = Kc.cuda(), Vc.cuda()
        Kref, Vref = Kc.clone().float(), Vc.clone().float()
        kw = {}
    row0 = (Kd[0].clone(), Vd[0].clone())
    step = A.DecodeStepGraph(Kd, Vd, cos.cuda(), sin.cuda(), B, H, D, max_tokens=1024, **kw)
    assert torch.equal(Kd[0].view(torch.uint8), row0[0].view(torch.uint8))      # the capture's warm-up left no trace
    assert torch.equal(Vd[0].view(torch.uint8), row0[1].view(torch.uint8))
    for s in range(3):
        q, k, v = (torch.randn(B, H * D, generator=g).half() for _ in range(3))
        pos = torch.tensor([len(x) for x in seq_slots], dtype=torch.int32)
        new = perm[nxt:nxt + B].int()
        nxt += B
        ci = torch.tensor([x for sl in seq_slots for x in sl], dtype=torch.int32)
        off = torch.tensor([len(x) for x in seq_slots]).cumsum(0).int()
        h = step.host
        h["q"].copy_(q); h["k"].copy_(k); h["v"].copy_(v); h["positions"].copy_(pos); h["new_slots"].copy_(new)
        h["cache_indices"][: ci.numel()].copy_(ci); h["offsets"].copy_(off)
        step.upload(ci.numel())
        O = step.replay().clone()
        torch.cuda.synchronize()
        assert int(step.err_flag.item()) == 0
        # oracle: rotate, attend over the cache as it was BEFORE the append, then append
        q_r, k_r = orc.rope(q, k, pos, cos, sin, D)
        _, _, O_ref = orc.paged_decode(q_r.float(), k_r.float(), v.float(), Kref, Vref, ci, off, H)
        if fp8:
            assert (O.cpu().float() - O_ref).norm() / O_ref.norm() <= 2e-2
            Kq = (k_r.float().reshape(B, H, D) / ks.view(1, H, 1)).to(torch.float8_e4m3fn).reshape(B, H * D)
            Vq = (v.float().reshape(B, H, D) / vs.view(1, H, 1)).to(torch.float8_e4m3fn).reshape(B, H * D)
            Kgot, Vgot = Kd[new.long().cuda()].cpu(), Vd[new.long().cuda()].cpu()
            # same codes, except where x / scale and x * (1 / scale) fall on either side of a rounding boundary
            for got, exp in ((Kgot, Kq), (Vgot, Vq)):
                dcode = (got.view(torch.uint8).int() - exp.view(torch.uint8).int()).abs()
                assert dcode.max() <= 1 and (dcode > 0).float().mean() < 0.01
            Kref[new.long()] = orc.dequantize_e4m3_per_head(Kgot, ks, H)
            Vref[new.long()] = orc.dequantize_e4m3_per_head(Vgot, vs, H)
        else:
            assert (O.cpu().float() - O_ref).abs().max() <= TOL16
            assert torch.equal(step.q.cpu(), q_r) and torch.equal(step.k.cpu(), k_r)
            assert torch.equal(Kd[new.long().cuda()].cpu(), k_r) and torch.equal(Vd[new.long().cuda()].cpu(), v)
            Kref[new.long()] = k_r.float()
            Vref[new.long()] = v.float()
        for b in range(B):
            seq_slots[b].append(int(new[b]))


def test_host_staged_decoder_with_prefetched_table():
    """The next step's slot table travels during the current step; three steps of growing sequences."""
    import attention_impl_b200 as A
    B, H, D = 7, 8, 128
    g = torch.Generator().manual_seed(9)
    Kc, Vc = (torch.randn(8192, H * D, generator=g).half() for _ in range(2))
    Kd, Vd = Kc.cuda(), Vc.cuda()
    lens0 = uniform_lens(B, 1, 500, seed=3)
    perm = torch.randperm(8192, generator=g)
    tables = []
    for s in range(3):
        lens = [n + s for n in lens0]
        ci = perm[1000 * s: 1000 * s + sum(lens)].int().pin_memory()      # a different table every step
        off = torch.tensor(lens).cumsum(0).int().pin_memory()
        tables.append((ci, off))
    dec = A.HostStagedDecoder(Kd, Vd, H, B, max(t[0].numel() for t in tables), n_groups=2)
    out = torch.empty(B, H * D, dtype=torch.float16).pin_memory()
    for s, (ci, off) in enumerate(tables):
        Q, K, V = (torch.randn(B, H * D, generator=g).half().pin_memory() for _ in range(3))
        dec(Q, K, V, ci, off, out, next_table=tables[s + 1] if s + 1 < len(tables) else None)
        _, _, O32 = orc.paged_decode(Q, K, V, Kc, Vc, ci, off, H, compute_dtype=torch.float32)
        assert (out.float() - O32.float()).abs().max() <= TOL16, f"step {s}"


@pytest.mark.parametrize("Hq,Hkv", [(8, 8), (16, 4)])
def test_fp8_decode_long_context_absmax_scales(Hq, Hkv):
    """One 40 000-token sequence, K/V ~ N(0,1) quantised to e4m3 with per-head absmax scales (codes
    up to +-448), multi-head kernel and the grouped-query tensor-core kernel: <= 2e-2 relative and
    <= 2e-2 of max |O| against the oracle on dequantised KV."""
    import lm_ops
    D, n = 128, 40_000
    g = torch.Generator().manual_seed(Hq)
    Q = torch.randn(1, Hq * D, generator=g).half()
    K, V = (torch.randn(1, Hkv * D, generator=g).half() for _ in range(2))
    Kc, Vc = (torch.randn(n + 100, Hkv * D, generator=g) for _ in range(2))
    K8, ks = orc.quantize_e4m3_per_head(Kc, Hkv)
    V8, vs = orc.quantize_e4m3_per_head(Vc, Hkv)
    assert int(K8.view(torch.uint8).max()) >= 0x7E - 0 and float(K8.float().abs().max()) == 448.0
    ci = torch.randperm(n + 100, generator=g)[:n].int()
    off = torch.tensor([n]).int()
    Kd, Vd = orc.dequantize_e4m3_per_head(K8, ks, Hkv), orc.dequantize_e4m3_per_head(V8, vs, Hkv)
    _, _, Oref = orc.paged_decode(Q.float(), K.float(), V.float(), Kd, Vd, ci, off, Hq)
    _, _, O = lm_ops.paged_kv_attention_forward(Q.cuda(), K.cuda(), V.cuda(), K8.cuda(), V8.cuda(), ci.cuda(),
                                                off.cuda(), Hq, return_sp=False, k_scale=ks.cuda(), v_scale=vs.cuda())
    err = O.cpu().float() - Oref
    assert err.norm() / Oref.norm() <= 2e-2
    assert err.abs().max() <= 2e-2 * Oref.abs().max()
