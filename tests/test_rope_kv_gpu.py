"""GPU: rotary embedding fused with the KV-cache append vs the oracle (rope, then scatter)."""
import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def _inputs(N, Hq, Hk, hd, rot, dtype, slots, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(N, Hq * hd, generator=g).to(dtype)
    k = torch.randn(N, Hk * hd, generator=g).to(dtype)
    v = torch.randn(N, Hk * hd, generator=g).to(dtype)
    pos = torch.randint(0, 4096, (N,), generator=g).int()
    sl = torch.randperm(slots, generator=g)[:N].int()
    cos, sin = orc.rope_tables(rot, 4096, dtype=dtype)
    return q, k, v, pos, sl, cos, sin


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N,Hq,Hk,hd,rot", [(37, 32, 32, 128, 128), (64, 8, 2, 128, 64), (5, 4, 4, 64, 32), (300, 2, 2, 256, 256)])
def test_rope_write_kv_bit_exact(dtype, N, Hq, Hk, hd, rot):
    import attention_impl_b200 as A
    slots = 1024
    q, k, v, pos, sl, cos, sin = _inputs(N, Hq, Hk, hd, rot, dtype, slots, seed=N + hd)
    q_ref, k_ref = orc.rope(q, k, pos, cos, sin, hd)
    Kc = torch.zeros(slots, Hk * hd, dtype=dtype, device="cuda")
    Vc = torch.zeros_like(Kc)
    qd, kd = q.cuda(), k.cuda()
    A.rope_and_cache_write(qd, kd, v.cuda(), pos.cuda(), cos.cuda(), sin.cuda(), sl.cuda(), Kc, Vc, hd)
    assert torch.equal(qd.cpu().view(torch.int16), q_ref.view(torch.int16))
    assert torch.equal(kd.cpu().view(torch.int16), k_ref.view(torch.int16))
    Kc_ref = torch.zeros(slots, Hk * hd, dtype=dtype)
    Vc_ref = torch.zeros_like(Kc_ref)
    Kc_ref[sl.long()] = k_ref
    Vc_ref[sl.long()] = v
    assert torch.equal(Kc.cpu().view(torch.int16), Kc_ref.view(torch.int16))
    assert torch.equal(Vc.cpu().view(torch.int16), Vc_ref.view(torch.int16))


def test_rope_write_kv_e4m3_pool_and_decode_roundtrip():
    """Append quantised rows, then decode from the pool: the written format is the one decode reads."""
    import attention_impl_b200 as A
    N, H, hd = 200, 8, 128
    slots = 512
    q, k, v, pos, sl, cos, sin = _inputs(N, H, H, hd, hd, torch.float16, slots, seed=9)
    _, k_ref = orc.rope(q, k, pos, cos, sin, hd)
    ks = (k_ref.float().reshape(N, H, hd).abs().amax(dim=(0, 2)) / 448.0)
    vs = (v.float().reshape(N, H, hd).abs().amax(dim=(0, 2)) / 448.0)
    K8 = torch.zeros(slots, H * hd, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    V8 = torch.zeros(slots, H * hd, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    A.rope_and_cache_write(q.cuda(), k.cuda(), v.cuda(), pos.cuda(), cos.cuda(), sin.cuda(), sl.cuda(), K8, V8, hd,
                           k_scale=ks.cuda(), v_scale=vs.cuda())
    exp_k = (k_ref.float().reshape(N, H, hd) / ks.view(1, H, 1)).to(torch.float8_e4m3fn).reshape(N, H * hd)
    exp_v = (v.float().reshape(N, H, hd) / vs.view(1, H, 1)).to(torch.float8_e4m3fn).reshape(N, H * hd)
    got_k = K8.cpu()[sl.long()]
    got_v = V8.cpu()[sl.long()]
    # identical codes except where fp32 division vs multiplication by the reciprocal lands on the
    # other side of a rounding boundary (1 code apart, rare)
    dk = (got_k.view(torch.uint8).int() - exp_k.view(torch.uint8).int()).abs()
    dv = (got_v.view(torch.uint8).int() - exp_v.view(torch.uint8).int()).abs()
    assert dk.max() <= 1 and dv.max() <= 1
    assert (dk > 0).float().mean() < 0.01 and (dv > 0).float().mean() < 0.01
    # decode one sequence made of all N appended tokens from the quantised pool
    g = torch.Generator().manual_seed(1)
    Q1, K1, V1 = (torch.randn(1, H * hd, generator=g).half() for _ in range(3))
    off = torch.tensor([N], dtype=torch.int32)
    _, _, O = A.paged_kv_attention_forward(Q1.cuda(), K1.cuda(), V1.cuda(), K8, V8, sl.cuda(), off.cuda(), H,
                                           return_sp=False, k_scale=ks.cuda(), v_scale=vs.cuda())
    Kd = orc.dequantize_e4m3_per_head(K8.cpu(), ks, H)
    Vd = orc.dequantize_e4m3_per_head(V8.cpu(), vs, H)
    _, _, O_ref = orc.paged_decode(Q1.float(), K1.float(), V1.float(), Kd, Vd, sl, off, H)
    assert (O.cpu().float() - O_ref).norm() / O_ref.norm() <= 2e-2


def test_rope_write_kv_bad_slot_flagged():
    import attention_impl_b200 as A
    q, k, v, pos, sl, cos, sin = _inputs(4, 2, 2, 64, 64, torch.float16, 16, seed=3)
    sl[2] = 999
    Kc = torch.zeros(16, 128, dtype=torch.float16, device="cuda")
    Vc = torch.zeros_like(Kc)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    A.rope_and_cache_write(q.cuda(), k.cuda(), v.cuda(), pos.cuda(), cos.cuda(), sin.cuda(), sl.cuda(), Kc, Vc, 64,
                           err_flag=flag)
    assert int(flag.item()) & 1


def test_rope_write_kv_bad_position_leaves_token_and_slot_untouched():
    """A position outside the table: the token's q and k stay un-rotated and NOTHING of it reaches
    the pools (no new v beside a stale k); the other tokens are processed as usual."""
    import attention_impl_b200 as A
    N, H, hd, slots = 6, 2, 64, 32
    q, k, v, pos, sl, cos, sin = _inputs(N, H, H, hd, hd, torch.float16, slots, seed=5)
    pos[3] = 4096                      # one past the table
    pos[5] = -1
    Kc = torch.full((slots, H * hd), 7.0, dtype=torch.float16, device="cuda")
    Vc = torch.full_like(Kc, -7.0)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    qd, kd = q.cuda(), k.cuda()
    A.rope_and_cache_write(qd, kd, v.cuda(), pos.cuda(), cos.cuda(), sin.cuda(), sl.cuda(), Kc, Vc, hd, err_flag=flag)
    assert int(flag.item()) == 2
    good = [0, 1, 2, 4]
    q_ref, k_ref = orc.rope(q[good], k[good], pos[good], cos, sin, hd)
    assert torch.equal(qd.cpu()[good], q_ref) and torch.equal(kd.cpu()[good], k_ref)
    for t in (3, 5):
        assert torch.equal(qd.cpu()[t], q[t]) and torch.equal(kd.cpu()[t], k[t])
        assert (Kc[sl[t]] == 7.0).all() and (Vc[sl[t]] == -7.0).all()
    assert torch.equal(Kc.cpu()[sl[good].long()], k_ref) and torch.equal(Vc.cpu()[sl[good].long()], v[good])
