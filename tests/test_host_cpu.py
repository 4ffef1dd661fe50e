"""CPU: host-side logic around the C ABI that needs no GPU — the operators' argument checks (the
reference's messages, `util.cuh:4-6`), the benchmark's e4m3 quantiser against the oracle's, the
single-launch heuristic's stated range, and the JSON contract of `bench.py --impl reference`."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_operators_reject_host_tensors_like_the_reference():
    import attention_impl_b200 as A
    q = torch.zeros(2, 256, dtype=torch.float16)
    kc = torch.zeros(16, 256, dtype=torch.float16)
    ci = torch.zeros(4, dtype=torch.int32)
    off = torch.tensor([2, 4], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="Q must be a CUDA tensor"):
        A.paged_kv_attention_forward(q, q, q, kc, kc, ci, off, 2)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        A.paged_attention_forward(q, q, q, off, 2)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        A.rotary_embedding_inplace(q, q, torch.zeros(2, dtype=torch.int32), torch.zeros(8, 64, dtype=torch.float16),
                                   torch.zeros(8, 64, dtype=torch.float16), 128)


def test_dropin_modules_export_the_reference_names():
    sys.path.insert(0, os.path.join(ROOT, "attention_impl_b200", "dropin"))
    try:
        import lm_ops
        import attention
        import paged_attention
        import rotary_embedding
    finally:
        sys.path.pop(0)
    for name in ("naive_attention_forward", "single_query_attention", "packed_attention",
                 "paged_kv_attention_forward", "rotary_embedding_inplace"):
        assert callable(getattr(lm_ops, name))
    assert callable(attention.naive_attention_forward) and callable(attention.kv_attention_forward)
    assert callable(paged_attention.paged_attention_forward) and callable(paged_attention.paged_kv_attention_forward)
    assert callable(rotary_embedding.rotary_embedding_inplace)


def test_bench_quantiser_matches_the_oracle():
    """bench.py quantises the long-context pools itself (it may not call the oracle outside its CPU legs):
    same codes and scales as the oracle's per-head absmax quantiser, on a case with several chunks."""
    sys.path.insert(0, ROOT)
    import bench
    from oracle import attention_oracle as orc
    g = torch.Generator().manual_seed(5)
    x = torch.randn(1000, 4 * 32, generator=g).half()
    codes, scales = bench.quantize_e4m3_per_head(x, 4, rows_per_chunk=256)
    ref_codes, ref_scales = orc.quantize_e4m3_per_head(x, 4)
    assert torch.allclose(scales.float().cpu(), ref_scales.float(), rtol=1e-6, atol=0)
    assert torch.equal(codes.view(torch.uint8).cpu(), ref_codes.view(torch.uint8))
    back = orc.dequantize_e4m3_per_head(ref_codes, ref_scales, 4)
    assert (back - x.float()).abs().max() <= x.float().abs().max() / 16       # e4m3: 3 mantissa bits


def test_single_launch_heuristic_range():
    from attention_impl_b200 import _lib
    ok = _lib.lib.attn_b200_paged_decode_single_launch_ok
    F16, E4M3 = _lib.F16, _lib.E4M3
    assert ok(8, 32, 32, 128, 8 * 1024, 1, F16, F16, 148) == 1          # 256 CTAs, 1024 tokens of capacity each
    assert ok(8, 32, 32, 128, 8 * 1025 + 8, 1, F16, F16, 148) == 0      # longer sequences: a CTA would hold the step
    assert ok(4, 32, 32, 128, 2048, 1, F16, F16, 148) == 0              # 128 CTAs do not fill 148 SMs
    assert ok(10, 32, 32, 128, 4096, 1, F16, F16, 148) == 0             # 320 CTAs: more than one wave
    assert ok(8, 32, 32, 128, 4096, 16, F16, F16, 148) == 0             # block tables
    assert ok(8, 32, 32, 128, 4096, 1, F16, E4M3, 148) == 0             # e4m3 pools


def test_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: the oracle on a bounded sample, one JSON line."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0"], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    d = json.loads(line)
    assert d["impl"] == "reference" and d["metric"] == "paged_decode_kv_read_bandwidth" and d["unit"] == "TB/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["value"] > 0 and d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["config"]["workload"] == "large_batch_paged_decode"
