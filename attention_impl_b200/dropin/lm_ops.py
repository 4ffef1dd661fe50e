"""The aggregator module the reference's tests import but the reference does not ship.

Name mapping (import sites: tests/test_naive_attention.py:7, tests/test_single_query_attention.py:4,
tests/test_packed_attention.py:5, tests/test_kv_paged_attention.py:4, tests/test_rotary_embedding.py:4):
``single_query_attention`` is ``attention.kv_attention_forward`` and ``packed_attention`` is
``paged_attention.paged_attention_forward`` (their call sites match those argument lists).
"""
from attention_impl_b200.ops import kv_attention_forward as single_query_attention  # noqa: F401
from attention_impl_b200.ops import naive_attention_forward  # noqa: F401
from attention_impl_b200.ops import paged_attention_forward as packed_attention  # noqa: F401
from attention_impl_b200.ops import paged_kv_attention_forward, rotary_embedding_inplace  # noqa: F401
