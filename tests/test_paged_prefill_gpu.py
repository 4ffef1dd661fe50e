"""GPU: chunked / prefix-cached prefill through the slot table vs the oracle, and its two limits
(whole-sequence chunk == packed prefill, one-row chunk == paged decode)."""
import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def _inputs(q_lens, kv_lens, H, Hkv, D, dtype, n_slots, seed):
    g = torch.Generator().manual_seed(seed)
    Q = torch.randn(sum(q_lens), H * D, generator=g).to(dtype)
    Kc, Vc = (torch.randn(n_slots, Hkv * D, generator=g).to(dtype) for _ in range(2))
    ci = torch.randperm(n_slots, generator=g)[: sum(kv_lens)].int()
    return Q, Kc, Vc, ci, torch.tensor(kv_lens).cumsum(0).int(), torch.tensor(q_lens).cumsum(0).int()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("H,Hkv,D", [(4, 4, 128), (8, 2, 128), (4, 4, 64), (6, 3, 40)])
def test_paged_prefill_matches_oracle(dtype, H, Hkv, D):
    import attention_impl_b200 as A
    q_lens = [1, 17, 128, 0, 200, 64]
    kv_lens = [50, 17, 300, 0, 200, 1000]
    Q, Kc, Vc, ci, kvo, qo = _inputs(q_lens, kv_lens, H, Hkv, D, dtype, 4096, seed=H * D)
    O = A.paged_prefill_attention(Q.cuda(), Kc.cuda(), Vc.cuda(), ci.cuda(), kvo.cuda(), qo.cuda(), H)
    O32 = orc.paged_prefill(Q, Kc, Vc, ci, kvo, qo, H, compute_dtype=torch.float32, out_dtype=torch.float32)
    tol = {torch.float16: 2e-3, torch.bfloat16: 1.6e-2, torch.float32: 2e-5}[dtype]
    assert (O.cpu().float() - O32).abs().max() <= tol


def test_paged_prefill_limits_equal_packed_prefill_and_decode():
    import attention_impl_b200 as A
    H, D = 4, 128
    lens = [130, 64, 257]
    Q, Kc, Vc, ci, kvo, qo = _inputs(lens, lens, H, H, D, torch.float16, 1024, seed=5)
    # whole sequence as the chunk == packed causal prefill on the gathered rows
    O = A.paged_prefill_attention(Q.cuda(), Kc.cuda(), Vc.cuda(), ci.cuda(), kvo.cuda(), qo.cuda(), H)
    Kg, Vg = Kc[ci.long()], Vc[ci.long()]
    _, _, Op = A.paged_attention_forward(Q.cuda(), Kg.cuda(), Vg.cuda(), qo.cuda(), H, return_sp=False)
    assert (O.float() - Op.float()).abs().max() <= 2e-3
    # one query row per sequence == paged decode whose current token is the last cached one
    q1 = torch.tensor([1, 1, 1]).cumsum(0).int()
    Q1 = Q[(qo - 1).long()]
    O1 = A.paged_prefill_attention(Q1.cuda(), Kc.cuda(), Vc.cuda(), ci.cuda(), kvo.cuda(), q1.cuda(), H)
    begs = [0] + kvo.tolist()[:-1]
    ci_ctx = torch.cat([ci[b:e - 1] for b, e in zip(begs, kvo.tolist())])
    last = ci[(kvo - 1).long()].long()
    off_ctx = torch.tensor([n - 1 for n in lens]).cumsum(0).int()
    _, _, Od = A.paged_kv_attention_forward(Q1.cuda(), Kc[last].cuda(), Vc[last].cuda(), Kc.cuda(), Vc.cuda(),
                                            ci_ctx.cuda(), off_ctx.cuda(), H, return_sp=False)
    assert (O1.float() - Od.float()).abs().max() <= 2e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv", [(4, 4), (8, 2)])
def test_paged_prefill_tensor_core_path(dtype, H, Hkv):
    """head_dim 128, 16-bit: tcgen05 kernel with gathered K/V; also against the generic kernel."""
    import attention_impl_b200 as A
    q_lens = [256, 1, 300, 128, 513, 77]
    kv_lens = [256, 700, 300, 1500, 513, 2048]
    Q, Kc, Vc, ci, kvo, qo = _inputs(q_lens, kv_lens, H, Hkv, 128, dtype, 8192, seed=H + Hkv)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = (Q.cuda(), Kc.cuda(), Vc.cuda(), ci.cuda(), kvo.cuda(), qo.cuda(), H)
    O = A.paged_prefill_attention(*args, err_flag=flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    O32 = orc.paged_prefill(Q, Kc, Vc, ci, kvo, qo, H, compute_dtype=torch.float32, out_dtype=torch.float32)
    tol = 2e-3 if dtype == torch.float16 else 1.6e-2
    assert (O.cpu().float() - O32).abs().max() <= tol
    Og = A.paged_prefill_attention(*args, force_generic=True)
    assert (O.float() - Og.float()).abs().max() <= tol
