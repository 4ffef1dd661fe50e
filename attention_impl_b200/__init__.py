"""attention_impl_b200: sm_100a kernels behind the operator API of ita9naiwa/attention-impl.

Importing the package loads ``lib/libattn_b200.so``; it raises if the library is not built.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from .ops import (DecodeStepGraph, HostStagedDecoder, PagedDecodeGraph, kv_attention_forward, lse_combine, naive_attention_forward, paged_attention_forward,  # noqa: F401
                  paged_decode_partial, paged_kv_attention_forward, paged_prefill_attention, rope_and_cache_write,
                  rotary_embedding_inplace)

__all__ = ["naive_attention_forward", "kv_attention_forward", "paged_attention_forward",
           "paged_kv_attention_forward", "rotary_embedding_inplace", "paged_decode_partial", "lse_combine", "PagedDecodeGraph", "DecodeStepGraph", "rope_and_cache_write", "HostStagedDecoder", "paged_prefill_attention"]
