"""GPU: dense masked attention and packed causal prefill (generic path) vs the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc
from conftest import load_golden
from helpers import prefill_inputs

pytestmark = pytest.mark.gpu


def _gpu(*ts):
    return [t.cuda() for t in ts]


@pytest.mark.parametrize("tag", ["naive_f32", "naive_f16", "naive_f32_std1"])
def test_naive_golden(tag):
    import lm_ops
    g = load_golden(tag)
    S, P, O = lm_ops.naive_attention_forward(*_gpu(g["Q"], g["K"], g["V"], g["mask"]), int(g["num_heads"]))
    tol = 1e-5 if g["Q"].dtype == torch.float32 else 2e-3
    assert (O.cpu().float() - g["O"].float()).abs().max() <= tol
    assert (P.cpu().float() - g["P"].float()).abs().max() <= tol
    fin = torch.isfinite(g["S"])
    assert torch.equal(torch.isfinite(S.cpu()), fin)
    assert (S.cpu().float()[fin] - g["S"].float()[fin]).abs().max() <= max(tol, 1e-2 if fin.all() else tol) * 8


@pytest.mark.parametrize("batch_size", [1, 4, 8])
@pytest.mark.parametrize("context_size", [256, 512])
@pytest.mark.parametrize("dim", [32, 64])
@pytest.mark.parametrize("num_heads", [1, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_naive_reference_matrix(batch_size, context_size, dim, num_heads, dtype):
    """The reference's grid and tolerance (tests/test_naive_attention.py:27-36): std 0.1, tril mask."""
    import lm_ops
    gen = torch.Generator().manual_seed(context_size + dim + num_heads)
    Q, K, V = ((torch.randn(batch_size, context_size, dim, generator=gen) * 0.1).to(dtype) for _ in range(3))
    mask = torch.from_numpy(np.tril(np.ones(context_size))).reshape(1, context_size, context_size) \
        .repeat(batch_size, 1, 1).to(dtype)
    S1, P1, O1 = orc.dense_mha(Q, K, V, mask, num_heads, fill=100000.0, compute_dtype=torch.float32)
    S2, P2, O2 = lm_ops.naive_attention_forward(*_gpu(Q, K, V, mask), num_heads)
    assert torch.allclose(O1.float(), O2.cpu().float(), atol=1e-2)
    assert (O1.float() - O2.cpu().float()).abs().max() <= (2e-3 if dtype == torch.float16 else 1e-5)


def test_naive_arbitrary_mask():
    import lm_ops
    gen = torch.Generator().manual_seed(8)
    B, L, dim, H = 2, 70, 48, 3
    Q, K, V = (torch.randn(B, L, dim, generator=gen) for _ in range(3))
    mask = (torch.rand(B, L, L, generator=gen) > 0.3).float()
    mask[:, :, 0] = 1   # every row keeps at least one key
    _, P1, O1 = orc.dense_mha(Q, K, V, mask, H)
    _, P2, O2 = lm_ops.naive_attention_forward(*_gpu(Q, K, V, mask), H)
    assert (O1 - O2.cpu()).abs().max() < 1e-5 and (P1 - P2.cpu()).abs().max() < 1e-5


@pytest.mark.parametrize("tag", ["packed_f16", "packed_f32"])
def test_packed_golden(tag):
    import lm_ops
    g = load_golden(tag)
    _, _, O = lm_ops.packed_attention(*_gpu(g["Q"], g["K"], g["V"], g["offsets"]), int(g["num_heads"]))
    tol = 1e-5 if g["Q"].dtype == torch.float32 else 2e-3
    assert (O.cpu().float() - g["O"].float()).abs().max() <= tol


@pytest.mark.parametrize("batch_size", [16, 32])
@pytest.mark.parametrize("context_size", [32, 64])
@pytest.mark.parametrize("dim", [32, 64, 128])
@pytest.mark.parametrize("num_heads", [4, 8])
def test_packed_reference_matrix_equal_lengths(batch_size, context_size, dim, num_heads):
    """The reference's grid and tolerance (tests/test_packed_attention.py:26-43), fp16, std 0.1."""
    import lm_ops
    lens = [context_size] * batch_size
    Q, K, V, off = prefill_inputs(lens, num_heads, dim // num_heads, torch.float16, seed=dim + batch_size, std=0.1)
    S, P, O2 = lm_ops.packed_attention(*_gpu(Q, K, V, off), num_heads)
    O1 = orc.packed_prefill(Q, K, V, off, num_heads, compute_dtype=torch.float32)
    assert S.shape == (batch_size, num_heads, context_size, context_size)
    assert torch.allclose(O1.float(), O2.cpu().float(), atol=2e-2)
    assert (O1.float() - O2.cpu().float()).abs().max() <= 2e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("H,D", [(4, 8), (2, 64), (2, 128)])
def test_packed_ragged_generic(dtype, H, D):
    """Varlen (untested by the reference): ragged lengths incl. 0 and 1, N(0,1) inputs."""
    import lm_ops
    lens = [5, 0, 1, 130, 64, 257]
    Q, K, V, off = prefill_inputs(lens, H, D, dtype, seed=H * D)
    S, P, O = lm_ops.packed_attention(*_gpu(Q, K, V, off), H, force_generic=True)
    O32 = orc.packed_prefill(Q, K, V, off, H, compute_dtype=torch.float32, out_dtype=torch.float32)
    tol = {torch.float16: 2e-3, torch.bfloat16: 1.6e-2, torch.float32: 2e-5}[dtype]
    assert (O.cpu().float() - O32).abs().max() <= tol
    # P rows are causal distributions
    Pc = P.cpu().float()
    beg = 0
    for b, n in enumerate(lens):
        if n:
            rows = Pc[b, :, :n, :n]
            assert torch.allclose(rows.sum(-1), torch.ones(H, n), atol=2e-2 if dtype != torch.float32 else 1e-5)
            assert rows.triu(1).abs().max() == 0
        beg += n
