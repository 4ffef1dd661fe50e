"""Drop-in for the reference extension module ``paged_attention`` (setup.py:10-12, paged_attention_kernel.cu:296-299)."""
from attention_impl_b200.ops import paged_attention_forward, paged_kv_attention_forward  # noqa: F401
