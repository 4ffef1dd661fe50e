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
    assert (O - O32).abs().max() <= 2e-3
