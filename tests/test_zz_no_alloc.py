"""GPU: the decode entry point that brings its own scratch (for hosts that may not allocate).

Collected last on purpose (file name), so a run that stops at the first failure has already run
everything else.  The call goes straight through the C ABI with ctypes: the caller supplies the
inputs and the output buffer, the library supplies the split-KV scratch from a fixed array in its
device image.  Both entry points run the same kernels on the same chunking, so their outputs must
be bit-identical, on two calls in a row, the second with other inputs so that stale scratch
contents from the first call would show; each is also held to the decode tolerance against the
CPU oracle, so that a mix-up that hit both entry points alike would show too.
"""
import pytest
import torch

from oracle import attention_oracle as orc
from helpers import decode_inputs, uniform_lens

pytestmark = pytest.mark.gpu

TOL = 2e-3   # the fp16 decode tolerance used across the decode tests (max-abs against the fp32-evaluated oracle)


def _call_pair(seed, B, H, D, lo, hi, chunk):
    from attention_impl_b200 import _lib
    lib = _lib.lib
    lens = uniform_lens(B, lo, hi, seed=seed)
    host = decode_inputs(B, H, D, lens, 16384, torch.float16, seed=seed)
    Q, K, V, Kc, Vc, ci, off = [t.cuda() for t in host]
    T = ci.numel()
    scale = D ** -0.5
    stream = torch.cuda.current_stream().cuda_stream
    need = lib.attn_b200_paged_decode_workspace_bytes(B, H, D, T, chunk)
    assert need <= _lib.STATIC_SCRATCH_BYTES
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    out_ref = torch.empty_like(Q)
    out_new = torch.full_like(Q, float("nan"))
    _lib.check(lib.attn_b200_paged_decode(
        Q.data_ptr(), K.data_ptr(), V.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), ci.data_ptr(), off.data_ptr(),
        out_ref.data_ptr(), ws.data_ptr(), need, None, None, 0, B, H, H, D, T, Kc.size(0), 0, 1, 0, chunk, scale, None,
        None, _lib.F16, _lib.F16, 3, None, stream), "paged_decode")
    _lib.check(lib.attn_b200_paged_decode_static_scratch(
        Q.data_ptr(), K.data_ptr(), V.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), ci.data_ptr(), off.data_ptr(),
        out_new.data_ptr(), B, H, D, T, Kc.size(0), chunk, scale, None, None, _lib.F16, _lib.F16, None, stream),
        "paged_decode_static_scratch")
    torch.cuda.synchronize()
    _, _, O32 = orc.paged_decode(*host, H, compute_dtype=torch.float32)
    return out_ref.cpu(), out_new.cpu(), O32.float()


def test_static_scratch_decode_matches_regular_entry_point_twice():
    ref1, new1, orc1 = _call_pair(seed=31, B=8, H=32, D=128, lo=128, hi=1024, chunk=32)
    assert torch.equal(ref1, new1)
    assert (new1.float() - orc1).abs().max() <= TOL
    # second call, different shapes and chunking: leftovers of the first call must not matter
    ref2, new2, orc2 = _call_pair(seed=32, B=5, H=8, D=128, lo=1, hi=700, chunk=64)
    assert torch.equal(ref2, new2)
    assert (new2.float() - orc2).abs().max() <= TOL


def test_static_scratch_rejects_sizes_beyond_its_limit():
    from attention_impl_b200 import _lib
    lib = _lib.lib
    # 256 sequences x 32 heads with 4.6 M tokens needs ~80 MB of partial rows: over the 16 MiB limit
    assert lib.attn_b200_paged_decode_workspace_bytes(256, 32, 128, 4_600_000, 1024) > _lib.STATIC_SCRATCH_BYTES
    x = torch.zeros(16, device="cuda")
    rc = lib.attn_b200_paged_decode_static_scratch(
        x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
        x.data_ptr(), 256, 32, 128, 4_600_000, 4_600_000, 1024, 1.0, None, None, _lib.F16, _lib.F16, None, None)
    assert rc == -5
    with pytest.raises(RuntimeError, match="beyond a documented limit"):
        _lib.check(rc, "paged_decode_static_scratch")
