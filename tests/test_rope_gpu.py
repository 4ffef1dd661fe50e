"""GPU: rotary embedding through the drop-in API vs the CPU oracle (bit-exact)."""
import pytest
import torch

from oracle import attention_oracle as orc
from conftest import load_golden

pytestmark = pytest.mark.gpu


def _run(q, k, pos, cos, sin, head_dim):
    import lm_ops
    qd, kd = q.cuda().clone(), k.cuda().clone()
    lm_ops.rotary_embedding_inplace(qd, kd, pos.cuda(), cos.cuda(), sin.cuda(), head_dim)
    torch.cuda.synchronize()
    return qd.cpu(), kd.cpu()


def _bits(x):
    return x.view(torch.int16) if x.element_size() == 2 else x.view(torch.int32)


@pytest.mark.parametrize("tag", ["rope_full", "rope_partial", "rope_big_pos"])
def test_rope_golden_bit_exact(tag):
    g = load_golden(tag)
    q, k = _run(g["q"], g["k"], g["positions"], g["cos"], g["sin"], int(g["head_dim"]))
    assert torch.equal(_bits(q), _bits(g["q_out"]))
    assert torch.equal(_bits(k), _bits(g["k_out"]))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("N,Hq,Hk,hd,rot", [
    (4, 1, 1, 16, 16), (4, 1, 1, 32, 32), (4, 1, 1, 64, 64),          # reference: rot_dim == head_dim
    (4, 1, 1, 16, 8), (4, 4, 4, 32, 4), (4, 8, 8, 64, 32),            # reference: partial rotary
    (257, 32, 32, 128, 128), (33, 8, 2, 128, 64), (19, 3, 5, 80, 48), (7, 2, 2, 24, 12),
])
def test_rope_matches_oracle_bit_exact(dtype, N, Hq, Hk, hd, rot):
    gen = torch.Generator().manual_seed(N * 131 + hd)
    max_pos = 8192
    q = torch.randn(N, Hq * hd, generator=gen).to(dtype)
    k = torch.randn(N, Hk * hd, generator=gen).to(dtype)
    pos = torch.randint(0, max_pos, (N,), generator=gen).int()
    cos, sin = orc.rope_tables(rot, max_pos, dtype=dtype)
    q_ref, k_ref = orc.rope(q, k, pos, cos, sin, hd)
    q_out, k_out = _run(q, k, pos, cos, sin, hd)
    assert torch.equal(_bits(q_out), _bits(q_ref))
    assert torch.equal(_bits(k_out), _bits(k_ref))


def test_rope_workload_shape_sampled_bit_exact():
    """Full workload shape [16384, 32*128] fp16, positions in [0, 8191]; the oracle checks a
    seeded sample of 512 tokens, the untouched-property is checked on all."""
    import lm_ops
    N, H, hd = 16384, 32, 128
    gen = torch.Generator().manual_seed(2)
    q = torch.randn(N, H * hd, generator=gen).half()
    k = torch.randn(N, H * hd, generator=gen).half()
    pos = torch.randint(0, 8192, (N,), generator=gen).int()
    cos, sin = orc.rope_tables(hd, 8192)
    qd, kd = q.cuda(), k.cuda()
    lm_ops.rotary_embedding_inplace(qd, kd, pos.cuda(), cos.cuda(), sin.cuda(), hd)
    sel = torch.randperm(N, generator=gen)[:512]
    q_ref, k_ref = orc.rope(q[sel], k[sel], pos[sel], cos, sin, hd)
    assert torch.equal(_bits(qd.cpu()[sel]), _bits(q_ref))
    assert torch.equal(_bits(kd.cpu()[sel]), _bits(k_ref))
    # rotation preserves the norm of each (d, d+64) pair up to fp16 rounding
    n0 = (q.float().reshape(N, H, 2, 64) ** 2).sum(2)
    n1 = (qd.cpu().float().reshape(N, H, 2, 64) ** 2).sum(2)
    assert ((n0 - n1).abs() <= 1e-2 * (1 + n0)).all()


def test_rope_bad_position_is_flagged_not_dereferenced():
    import attention_impl_b200 as A
    q = torch.randn(4, 64).half().cuda()
    k = q.clone()
    q0 = q.clone()
    cos, sin = orc.rope_tables(64, 16)
    pos = torch.tensor([0, 99, 3, -1], dtype=torch.int32).cuda()
    with pytest.raises(RuntimeError, match="outside"):
        A.rotary_embedding_inplace(q, k, pos, cos.cuda(), sin.cuda(), 64, check_positions=True)
    assert torch.equal(q[1], q0[1]) and torch.equal(q[3], q0[3])   # skipped rows untouched


def test_rope_empty_input():
    import lm_ops
    cos, sin = orc.rope_tables(64, 16)
    q = torch.empty(0, 64, dtype=torch.float16, device="cuda")
    lm_ops.rotary_embedding_inplace(q, q.clone(), torch.empty(0, dtype=torch.int32, device="cuda"),
                                    cos.cuda(), sin.cuda(), 64)


@pytest.mark.parametrize("num_heads,head_dim,rot_dim", [(1, 16, 16), (1, 32, 32), (1, 64, 64), (1, 16, 8), (4, 32, 4), (8, 64, 32)])
def test_rope_reference_suite_shapes(num_heads, head_dim, rot_dim):
    """The reference's own cases (tests/test_rotary_embedding.py:79-142): 4 tokens, positions
    arange(4), a 32-position table, std 0.1, atol 1e-3 against the torch module that rounds the angles
    to fp16 before cos/sin (its own table, :27-30) -- and, unlike the reference, k is checked as well."""
    import lm_ops
    gen = torch.Generator().manual_seed(head_dim + rot_dim)
    n, max_pos = 4, 32
    q = (torch.randn(n, num_heads * head_dim, generator=gen) * 0.1).half()
    k = (torch.randn(n, num_heads * head_dim, generator=gen) * 0.1).half()
    pos = torch.arange(n).int()
    cos, sin = orc.rope_tables(rot_dim, max_pos)                       # the kernel-side table (:65-71)
    inv_freq = 1.0 / (10000 ** (torch.arange(0, rot_dim, 2).float() / rot_dim))
    emb = torch.cat((torch.outer(torch.arange(max_pos).float(), inv_freq),) * 2, dim=-1).half()
    ref_cos, ref_sin = emb.cos().half(), emb.sin().half()                # the torch module's table (:27-30)

    def ref(x):
        xh = x.reshape(n, num_heads, head_dim)
        xr = xh[..., :rot_dim]
        c, s_ = ref_cos[pos.long()].unsqueeze(1), ref_sin[pos.long()].unsqueeze(1)
        xr = xr * c + orc.rotate_half(xr) * s_
        return torch.cat((xr, xh[..., rot_dim:]), dim=-1).reshape(n, -1)
    qd, kd = q.cuda(), k.cuda()
    lm_ops.rotary_embedding_inplace(qd, kd, pos.cuda(), cos.cuda(), sin.cuda(), head_dim)
    assert torch.allclose(ref(q).float(), qd.cpu().float(), atol=1e-3)
    assert torch.allclose(ref(k).float(), kd.cpu().float(), atol=1e-3)
