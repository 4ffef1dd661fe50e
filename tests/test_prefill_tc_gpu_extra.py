"""GPU: more shapes for the persistent tensor-core prefill (work-item grouping and ring wrap-around)."""
import pytest
import torch

from oracle import attention_oracle as orc
from helpers import prefill_inputs

pytestmark = pytest.mark.gpu


def _run(Q, K, V, off, H, **kw):
    import lm_ops
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    O = lm_ops.packed_attention(Q.cuda(), K.cuda(), V.cuda(), off.cuda(), H, return_sp=False, err_flag=flag, **kw)[2]
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    return O.cpu()


def test_many_tiny_sequences_odd_head_count():
    """300 sequences of 1..40 tokens, 3 heads: 900 (sequence, head) combinations do not fill the last
    group of 16 work items; every item is a single half-empty query tile."""
    g = torch.Generator().manual_seed(9)
    lens = torch.randint(1, 41, (300,), generator=g).tolist()
    H = 3
    Q, K, V, off = prefill_inputs(lens, H, 128, torch.float16, seed=13)
    O = _run(Q, K, V, off, H, out_dtype=torch.float32)
    O32 = orc.packed_prefill(Q, K, V, off, H, compute_dtype=torch.float32, out_dtype=torch.float32)
    assert (O - O32).abs().max() <= 2e-3


def test_fewer_items_than_sms_and_exact_tile_multiples():
    """One head, lengths that are exact multiples of 128 and 256 (no partial tiles; the upper query tile
    of a pair is present or absent exactly at the boundary)."""
    lens = [128, 256, 384, 512]
    H = 1
    Q, K, V, off = prefill_inputs(lens, H, 128, torch.bfloat16, seed=17)
    O = _run(Q, K, V, off, H, out_dtype=torch.float32)
    O32 = orc.packed_prefill(Q, K, V, off, H, compute_dtype=torch.float32, out_dtype=torch.float32)
    assert (O - O32).abs().max() <= 1e-2


def test_pair_kernel_matches_persistent_kernel_bitwise():
    """The two kernels run the same arithmetic in the same order per row: identical bits.  The kernel is
    chosen once per process (environment variable), so the pair kernel runs in a child process."""
    import os, subprocess, sys, tempfile
    lens = [700, 33, 1500, 256, 90]
    H = 4
    Q, K, V, off = prefill_inputs(lens, H, 128, torch.bfloat16, seed=23)
    O = _run(Q, K, V, off, H)
    with tempfile.TemporaryDirectory() as d:
        torch.save((Q, K, V, off), os.path.join(d, "in.pt"))
        code = (
            "import sys, torch; sys.path[:0] = %r\n"
            "import lm_ops\n"
            "Q, K, V, off = torch.load(%r)\n"
            "O = lm_ops.packed_attention(Q.cuda(), K.cuda(), V.cuda(), off.cuda(), %d, return_sp=False)[2]\n"
            "torch.save(O.cpu(), %r)\n" % (sys.path, os.path.join(d, "in.pt"), H, os.path.join(d, "out.pt")))
        env = dict(os.environ, ATTN_B200_PREFILL_VERSION="2")
        subprocess.run([sys.executable, "-c", code], check=True, env=env, timeout=300)
        O2 = torch.load(os.path.join(d, "out.pt"))
    assert torch.equal(O, O2)
