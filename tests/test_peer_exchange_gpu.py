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
