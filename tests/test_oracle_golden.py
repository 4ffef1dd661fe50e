"""CPU: the oracle restatement reproduces the reference's own torch functions.

The golden vectors were produced by tests/golden/make_golden.py, which imports the
reference's test modules and calls their functions unchanged.  Same torch build =>
the comparison is bit-exact; across torch builds matmul blocking may differ in the
last ulp, so a tolerance of a few ulp of the dtype is allowed and stated per case.
"""
import pytest
import torch

from oracle import attention_oracle as orc
from conftest import load_golden


def _close(a, b, tol):
    a, b = a.double(), b.double()
    fin = torch.isfinite(b)
    assert torch.equal(torch.isfinite(a), fin)
    assert torch.equal(a[~fin], b[~fin])
    assert (a[fin] - b[fin]).abs().max().item() <= tol


@pytest.mark.parametrize("tag,tol", [("naive_f32", 1e-6), ("naive_f16", 1e-3), ("naive_f32_std1", 2e-6)])
def test_naive_matches_reference(tag, tol):
    g = load_golden(tag)
    S, P, O = orc.dense_mha(g["Q"], g["K"], g["V"], g["mask"], int(g["num_heads"]), fill=100000.0)
    _close(S, g["S"], tol * 10)
    _close(P, g["P"], tol)
    _close(O, g["O"], tol)


@pytest.mark.parametrize("tag,tol", [("packed_f16", 1e-3), ("packed_f32", 2e-6)])
def test_packed_matches_reference(tag, tol):
    g = load_golden(tag)
    O = orc.packed_prefill(g["Q"], g["K"], g["V"], g["offsets"], int(g["num_heads"]))
    _close(O, g["O"], tol)


@pytest.mark.parametrize("tag,tol", [("single_f32", 2e-6), ("single_f16", 1e-3)])
def test_single_query_matches_reference(tag, tol):
    g = load_golden(tag)
    S, P, O = orc.single_query(g["Q"], g["K"], g["V"], g["K_cache"], g["V_cache"], int(g["num_heads"]))
    _close(S, g["S"], tol * 4)
    _close(P, g["P"], tol)
    _close(O, g["O"], tol)


@pytest.mark.parametrize("tag", ["paged_ref_shape", "paged_f32"])
def test_paged_decode_matches_reference_unscaled(tag):
    """The reference torch function never applies its scale: scale=1.0 is the literal form."""
    g = load_golden(tag)
    S, P, O = orc.paged_decode(g["Q"], g["K"], g["V"], g["K_cache"], g["V_cache"], g["cache_indices"],
                               g["offsets"], int(g["num_heads"]), scale=1.0)
    _close(S.float(), g["S"], 2e-6)
    _close(P.float(), g["P"], 2e-6)
    _close(O, g["O"], 2e-6)


@pytest.mark.parametrize("tag", ["rope_full", "rope_partial", "rope_big_pos"])
def test_rope_matches_reference_bit_exact(tag):
    g = load_golden(tag)
    q, k = orc.rope(g["q"], g["k"], g["positions"], g["cos"], g["sin"], int(g["head_dim"]))
    assert torch.equal(q.view(torch.int16), g["q_out"].view(torch.int16))
    assert torch.equal(k.view(torch.int16), g["k_out"].view(torch.int16))
    # the table builder reproduces the rows the reference module built
    rot = 2 * g["cos"].shape[1]
    cos, sin = orc.rope_tables(rot, int(g["max_pos"]))
    rows = g["orig_positions"].long() if g["cos"].shape[0] != int(g["max_pos"]) else slice(None)
    assert torch.equal(cos[rows], g["cos"]) and torch.equal(sin[rows], g["sin"])


def test_paged_decode_ragged_equals_dense_per_sequence():
    """Ragged generalisation: each sequence equals single_query on its gathered rows."""
    gen = torch.Generator().manual_seed(3)
    B, H, D, slots = 4, 2, 8, 64
    lens = [0, 5, 1, 9]
    Q, K, V = (torch.randn(B, H * D, generator=gen) for _ in range(3))
    Kc, Vc = (torch.randn(slots, H * D, generator=gen) for _ in range(2))
    ci = torch.randperm(slots, generator=gen)[: sum(lens)].int()
    off = torch.tensor(lens).cumsum(0).int()
    S, P, O = orc.paged_decode(Q, K, V, Kc, Vc, ci, off, H, scale=1.0)
    beg = 0
    for b, n in enumerate(lens):
        rows = ci[beg:beg + n].long()
        s1, p1, o1 = orc.single_query(Q[b:b + 1], K[b:b + 1], V[b:b + 1], Kc[rows].unsqueeze(0),
                                      Vc[rows].unsqueeze(0), H)
        assert torch.allclose(O[b], o1[0], atol=1e-6)
        assert torch.allclose(P[b, :, : n + 1].float(), p1[0], atol=1e-6)
        assert P[b, :, n + 1:].abs().sum() == 0
        beg += n


def test_e4m3_roundtrip_within_format_error():
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(200, 4 * 16, generator=gen)
    x8, sc = orc.quantize_e4m3_per_head(x, 4)
    y = orc.dequantize_e4m3_per_head(x8, sc, 4)
    # e4m3 has 3 mantissa bits: relative error <= 2^-4 for normals
    assert ((y - x).abs() <= x.abs() * 0.0625 + sc.max() * 2 ** -9 * 1.01).all()
