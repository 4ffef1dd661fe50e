"""GPU: grouped-query decode on the tensor cores (G = 2, 4 or 8 query heads per KV head, head_dim 128,
fp16 / bf16 / e4m3 pools; taken when S and P are not requested) against the CPU oracle."""
import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def _inputs(Hq, Hkv, D, lens, n_slots, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    Q = torch.randn(B, Hq * D, generator=g).to(dtype)
    K, V = (torch.randn(B, Hkv * D, generator=g).to(dtype) for _ in range(2))
    Kc, Vc = (torch.randn(n_slots, Hkv * D, generator=g).to(dtype) for _ in range(2))
    ci = torch.randperm(n_slots, generator=g)[: sum(lens)].int()
    off = torch.tensor(lens).cumsum(0).int()
    return Q, K, V, Kc, Vc, ci, off


def _run(inp, Hq, **kw):
    import lm_ops
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    O = lm_ops.paged_kv_attention_forward(*[t.cuda() for t in inp], Hq, return_sp=False, err_flag=flag, **kw)[2]
    torch.cuda.synchronize()
    return O.cpu(), int(flag.item())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (16, 2), (32, 8), (40, 5), (24, 3), (8, 4), (6, 3)])
@pytest.mark.parametrize("chunk", [None, 32, 64, 1024])
def test_gqa_mma_matches_oracle(dtype, Hq, Hkv, chunk):
    """Ragged lengths around the 16-token tile (0, 1, 15, 16, 17 ...), KV head counts that do and do not
    fill a CTA of four warps, every chunk length class."""
    lens = [0, 1, 15, 16, 17, 31, 33, 700, 2049]
    inp = _inputs(Hq, Hkv, 128, lens, 4096, dtype, seed=Hq * 7 + Hkv)
    O, flag = _run(inp, Hq, chunk=chunk)
    assert flag == 0
    O32 = orc.paged_decode(*inp, Hq, compute_dtype=torch.float32)[2]
    tol = 2e-3 if dtype == torch.float16 else 1.6e-2
    assert (O.float() - O32.float()).abs().max() <= tol


def test_gqa_mma_equals_cuda_core_kernel_closely():
    """Same inputs through the CUDA-core kernel (taken when S and P are requested)."""
    import lm_ops
    lens = [5, 300, 1500, 64]
    inp = _inputs(32, 4, 128, lens, 4096, torch.float16, seed=3)
    O, _ = _run(inp, 32)
    O_cc = lm_ops.paged_kv_attention_forward(*[t.cuda() for t in inp], 32)[2].cpu()
    assert (O.float() - O_cc.float()).abs().max() <= 1e-3


@pytest.mark.parametrize("qdtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("G", [2, 4, 8])
def test_gqa_mma_e4m3(G, qdtype):
    Hkv, D = 6, 128
    Hq = Hkv * G
    lens = [0, 1, 17, 100, 1500, 3000]
    Q, K, V, Kc, Vc, ci, off = _inputs(Hq, Hkv, D, lens, 8192, qdtype, seed=11 + G)
    Kc, Vc = Kc.float(), Vc.float()
    K8, ks = orc.quantize_e4m3_per_head(Kc, Hkv)
    V8, vs = orc.quantize_e4m3_per_head(Vc, Hkv)
    Kd, Vd = orc.dequantize_e4m3_per_head(K8, ks, Hkv), orc.dequantize_e4m3_per_head(V8, vs, Hkv)
    Oref = orc.paged_decode(Q.float(), K.float(), V.float(), Kd, Vd, ci, off, Hq)[2]
    O, flag = _run((Q, K, V, K8, V8, ci, off), Hq, k_scale=ks.cuda(), v_scale=vs.cuda())
    assert flag == 0
    assert (O.float() - Oref).norm() / Oref.norm() <= 2e-2
    assert (O.float() - Oref).abs().max() <= 2e-2


@pytest.mark.parametrize("block_size", [16, 64])
def test_gqa_mma_block_table(block_size):
    import lm_ops
    B, D, Hq, Hkv = 4, 128, 32, 4
    lens = [1, block_size + 1, 333, 0]
    n_blocks = 64
    g = torch.Generator().manual_seed(block_size)
    max_blocks = max((n + block_size - 1) // block_size for n in lens)
    perm = torch.randperm(n_blocks, generator=g)
    table = torch.full((B, max_blocks), -1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(lens):
        nb = (n + block_size - 1) // block_size
        table[b, :nb] = perm[nxt:nxt + nb].int()
        nxt += nb
    Q = torch.randn(B, Hq * D, generator=g).half()
    K, V = (torch.randn(B, Hkv * D, generator=g).half() for _ in range(2))
    Kc, Vc = (torch.randn(n_blocks * block_size, Hkv * D, generator=g).half() for _ in range(2))
    off = torch.tensor(lens).cumsum(0).int()
    O = lm_ops.paged_kv_attention_forward(Q.cuda(), K.cuda(), V.cuda(), Kc.cuda(), Vc.cuda(), table.cuda(),
                                          off.cuda(), Hq, block_size=block_size, return_sp=False)[2]
    O32 = orc.paged_decode(Q, K, V, Kc, Vc, table.clamp(min=0), off, Hq, compute_dtype=torch.float32,
                           block_size=block_size)[2]
    assert (O.cpu().float() - O32.float()).abs().max() <= 2e-3


def test_gqa_mma_bad_slots_are_skipped_and_flagged():
    from attention_impl_b200 import _lib
    lens = [40, 200]
    Q, K, V, Kc, Vc, ci, off = _inputs(16, 2, 128, lens, 512, torch.float16, seed=5)
    ci = ci.clone()
    ci[7] = -3
    ci[100] = 512
    O, flag = _run((Q, K, V, Kc, Vc, ci, off), 16)
    assert flag & _lib.FLAG_BAD_SLOT
    # the oracle on the sequences with those two tokens removed
    keep = torch.ones(sum(lens), dtype=torch.bool)
    keep[7] = keep[100] = False
    ci2 = ci[keep]
    off2 = torch.tensor([39, 39 + 199]).int()
    O32 = orc.paged_decode(Q, K, V, Kc, Vc, ci2, off2, 16, compute_dtype=torch.float32)[2]
    assert (O.float() - O32.float()).abs().max() <= 2e-3
