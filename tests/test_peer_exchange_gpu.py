"""GPU (one device): the peer-store exchange kernels of the KV-split path.

The multi-GPU form needs one process per GPU; here every "peer" buffer is a local allocation, which
exercises the same kernels: stores into n destinations, one counter bump per CTA and destination,
and the bounded wait (including the case where it runs out: a counter nothing ever sets).
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_push_lands_in_every_destination_and_counts_ctas():
    from attention_impl_b200 import _lib
    lib = _lib.lib
    n_peers, n = 3, 64 * 32 * 130              # a [B=64, H=32, D+2] partial
    src = torch.randn(n, device="cuda")
    dst = [torch.zeros(2, n, device="cuda") for _ in range(n_peers)]      # slot 1 of each peer
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(n_peers)]
    Ptr = ctypes.c_void_p * n_peers
    d = Ptr(*[t[1].data_ptr() for t in dst])
    f = Ptr(*[t[5:].data_ptr() for t in flags])                              # "my rank" = 5
    stream = torch.cuda.current_stream().cuda_stream
    ctas = lib.attn_b200_peer_push_ctas(n * 4)
    assert ctas == (n * 4 // 16 + 1023) // 1024
    for step in (1, 2):
        _lib.check(lib.attn_b200_peer_push(src.data_ptr(), n * 4, d, f, n_peers, stream), "peer_push")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        _lib.check(lib.attn_b200_wait_flags(flags[0][5:].data_ptr(), 1, step * ctas, err.data_ptr(), stream),
                   "wait_flags")
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        for t, fl in zip(dst, flags):
            assert torch.equal(t[1], src) and t[0].abs().sum() == 0
            assert fl.tolist() == [0, 0, 0, 0, 0, step * ctas, 0, 0]


def test_wait_gives_up_with_a_status_instead_of_hanging():
    from attention_impl_b200 import _lib
    lib = _lib.lib
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    flags[0] = 7
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(lib.attn_b200_wait_flags(flags.data_ptr(), 2, 7, err.data_ptr(), None), "wait_flags")
    torch.cuda.synchronize()                       # flags[1] never reaches 7: bounded wait, about a second
    assert int(err.item()) & _lib.FLAG_TIMEOUT
    # the context is still usable
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0


def test_consuming_wait_takes_its_count_off_and_keeps_early_arrivals():
    """The graph-replayable wait: the same `count` every step; arrivals of a peer that is one push ahead
    stay on the counter for the next step."""
    from attention_impl_b200 import _lib
    lib = _lib.lib
    n = 64 * 32 * 130
    src = torch.randn(n, device="cuda")
    dst = torch.zeros(n, device="cuda")
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    Ptr = ctypes.c_void_p * 1
    d, f = Ptr(dst.data_ptr()), Ptr(flags[2:].data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    ctas = lib.attn_b200_peer_push_ctas(n * 4)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    # the "peer" pushes twice before the local rank waits once: one step ahead
    for _ in range(2):
        _lib.check(lib.attn_b200_peer_push(src.data_ptr(), n * 4, d, f, 1, stream), "peer_push")
    _lib.check(lib.attn_b200_wait_flags_consume(flags[2:].data_ptr(), 1, ctas, err.data_ptr(), stream), "wait")
    torch.cuda.synchronize()
    assert flags.tolist() == [0, 0, ctas, 0] and int(err.item()) == 0
    _lib.check(lib.attn_b200_wait_flags_consume(flags[2:].data_ptr(), 1, ctas, err.data_ptr(), stream), "wait")
    torch.cuda.synchronize()
    assert flags.tolist() == [0, 0, 0, 0] and int(err.item()) == 0
    # captured once, replayed three times with constant arguments
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            st = s.cuda_stream
            _lib.check(lib.attn_b200_peer_push(src.data_ptr(), n * 4, d, f, 1, st), "peer_push")
            _lib.check(lib.attn_b200_wait_flags_consume(flags[2:].data_ptr(), 1, ctas, err.data_ptr(), st), "wait")
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert flags.tolist() == [0, 0, 0, 0] and int(err.item()) == 0 and torch.equal(dst, src)


def _split_tables(ci, off, G):
    from attention_impl_b200 import dist as adist
    return [adist.plan_kv_split(ci, off, G, r) for r in range(G)]


def test_fused_exchange_three_ranks_emulated_on_one_device():
    """The three-launch exchange (partial -> combine that pushes -> combine that waits) with three
    "ranks" played one after the other on one device: each rank's rows go into every rank's gather
    buffer, each rank's final combine finds its counters already complete, the result equals the
    oracle's one-shot decode, and the counters are back at zero afterwards (twice in a row)."""
    import attention_impl_b200 as A
    from attention_impl_b200 import _lib
    from oracle import attention_oracle as orc
    from helpers import decode_inputs, uniform_lens
    lib = _lib.lib
    G, B, H, D = 3, 5, 8, 128
    RS = D + 2
    stream = torch.cuda.current_stream().cuda_stream
    parts = [torch.zeros(G, B, H, RS, device="cuda") for _ in range(G)]         # rank g's gather buffer
    flags = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(G)]
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    Ptr = ctypes.c_void_p * G
    for seed in (1, 2):
        lens = uniform_lens(B, 0, 700, seed=seed)
        Q, K, V, Kc, Vc, ci, off = decode_inputs(B, H, D, lens, 4096, torch.float16, seed=seed)
        Qd, Kd, Vd, Kcd, Vcd = (t.cuda() for t in (Q, K, V, Kc, Vc))
        for r, (ci_r, off_r) in enumerate(_split_tables(ci, off, G)):
            ci_r, off_r = ci_r.cuda(), off_r.cuda()
            T = max(1, ci_r.numel())
            chunk = 64
            ws = torch.empty(A.ops.decode_workspace_bytes(B, H, D, T, chunk), dtype=torch.uint8, device="cuda")
            dst = Ptr(*[parts[g][r].data_ptr() for g in range(G)])
            flg = Ptr(*[flags[g][r:].data_ptr() for g in range(G)])
            _lib.check(lib.attn_b200_paged_decode_partial_push(
                Qd.data_ptr(), Kcd.data_ptr(), Vcd.data_ptr(), ci_r.data_ptr(), off_r.data_ptr(), ws.data_ptr(),
                ws.numel(), B, H, H, D, ci_r.numel(), Kcd.size(0), 1, 0, chunk, D ** -0.5, None, None, _lib.F16,
                _lib.F16, dst, flg, G, err.data_ptr(), stream), "partial_push")
        torch.cuda.synchronize()
        for g in range(G):
            assert flags[g][:G].tolist() == [B * H] * G
        _, _, O32 = orc.paged_decode(Q, K, V, Kc, Vc, ci, off, H, compute_dtype=torch.float32)
        for g in range(G):
            out = torch.empty_like(Qd)
            _lib.check(lib.attn_b200_lse_combine_wait(
                parts[g].data_ptr(), G, Qd.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), out.data_ptr(), B, H, H, D,
                D ** -0.5, _lib.F16, flags[g].data_ptr(), flags[g][31:].data_ptr(), err.data_ptr(), stream), "combine_wait")
            torch.cuda.synchronize()
            assert int(err.item()) == 0
            assert flags[g].abs().sum().item() == 0                      # arrivals consumed, ticket counter reset
            assert (out.cpu().float() - O32.float()).abs().max() <= 2e-3


def test_fused_exchange_wait_gives_up_with_a_status():
    """A counter that nothing ever completes: every CTA's wait runs out (about a second), the kernel
    raises the timeout flag, still ends, and the context stays usable."""
    from attention_impl_b200 import _lib
    lib = _lib.lib
    B, H, D, G = 2, 4, 128, 2
    parts = torch.zeros(G, B, H, D + 2, device="cuda")
    parts[..., D] = float("-inf")
    flags = torch.zeros(32, dtype=torch.int32, device="cuda")
    flags[0] = B * H                                                    # rank 0 arrived, rank 1 never does
    q = torch.randn(B, H * D, device="cuda").half()
    out = torch.empty_like(q)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(lib.attn_b200_lse_combine_wait(parts.data_ptr(), G, q.data_ptr(), q.data_ptr(), q.data_ptr(),
                                              out.data_ptr(), B, H, H, D, 1.0, _lib.F16, flags.data_ptr(),
                                              flags[31:].data_ptr(), err.data_ptr(), None), "combine_wait")
    torch.cuda.synchronize()
    assert int(err.item()) & _lib.FLAG_TIMEOUT
    assert torch.equal(out, q)                                          # only the current token: out = v_new
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0
