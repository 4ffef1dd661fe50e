"""CPU: the C-ABI library loads, exports every symbol the header declares, and validates arguments
before touching the GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "attn_b200.h")


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(attn_b200_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for s in ("attn_b200_rope_inplace", "attn_b200_paged_decode", "attn_b200_lse_combine",
              "attn_b200_varlen_prefill", "attn_b200_dense_attention", "attn_b200_strerror"):
        assert s in syms


def test_library_exports_every_declared_symbol():
    from attention_impl_b200 import _lib
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for s in declared_symbols():
        assert hasattr(raw, s), f"{s} declared in include/attn_b200.h but not exported"
    # and the Python prototype table covers the header one to one
    assert sorted(_lib.PROTOTYPES) == declared_symbols()


def test_argument_errors_are_reported_without_a_gpu():
    from attention_impl_b200 import _lib
    lib = _lib.lib
    assert lib.attn_b200_abi_version() == _lib.ABI_VERSION
    assert lib.attn_b200_strerror(0) == b"ok"
    # null pointers -> EINVAL before any CUDA call
    assert lib.attn_b200_rope_inplace(None, None, None, None, None, 4, 1, 1, 16, 8, 32, 0, None, None) == -1
    assert lib.attn_b200_rope_inplace(None, None, None, None, None, 0, 1, 1, 16, 8, 32, 0, None, None) == 0
    assert lib.attn_b200_paged_decode(None, None, None, None, None, None, None, None, None, 0, None, None, 0,
                                      1, 1, 1, 128, 0, 1, 0, 1, 0, 32, 1.0, None, None, 0, 0, 3, None, None) == -1
    assert lib.attn_b200_lse_combine(None, 1, None, None, None, None, 1, 1, 1, 128, 1.0, 0, None) == -1
    assert lib.attn_b200_varlen_prefill(None, None, None, None, None, None, None, 1, 1, 1, 1, 128, 1.0, 0, 0, 0,
                                        None, None) == -1
    assert lib.attn_b200_dense_attention(None, None, None, None, None, None, None, 1, 1, 1, 1, 1.0, 1.0, 0,
                                         None) == -1
    with pytest.raises(RuntimeError, match="invalid argument"):
        _lib.check(-1, "x")


def test_chunk_heuristic_and_workspace_size():
    from attention_impl_b200 import _lib
    lib = _lib.lib
    # small batch: smallest chunk so that the machine is filled
    assert lib.attn_b200_paged_decode_pick_chunk(8, 32, 128, 4608, 148) == 32
    # large batch: largest chunk
    assert lib.attn_b200_paged_decode_pick_chunk(256, 32, 128, 4_330_000, 148) == 1024
    n_units = 4608 // 32 + 8 + 1
    assert lib.attn_b200_paged_decode_workspace_bytes(8, 32, 128, 4608, 32) == n_units * 32 * 130 * 4


def test_ops_reject_cpu_tensors_like_the_reference():
    import torch
    import attention_impl_b200 as A
    q = torch.zeros(2, 8)
    with pytest.raises(RuntimeError, match="Q must be a CUDA tensor"):
        A.naive_attention_forward(q.reshape(1, 2, 8), q.reshape(1, 2, 8), q.reshape(1, 2, 8), torch.zeros(1, 2, 2), 1)
    with pytest.raises(RuntimeError, match="Q must be a CUDA tensor"):
        A.rotary_embedding_inplace(q, q, torch.zeros(2, dtype=torch.int32), q, q, 8)


def test_dropin_module_names_resolve():
    import attention
    import lm_ops
    import paged_attention
    import rotary_embedding
    assert lm_ops.single_query_attention is attention.kv_attention_forward
    assert lm_ops.packed_attention is paged_attention.paged_attention_forward
    assert lm_ops.rotary_embedding_inplace is rotary_embedding.rotary_embedding_inplace
    assert lm_ops.paged_kv_attention_forward is paged_attention.paged_kv_attention_forward
    assert lm_ops.naive_attention_forward is attention.naive_attention_forward
