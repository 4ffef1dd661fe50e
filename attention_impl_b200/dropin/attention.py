"""Drop-in for the reference extension module ``attention`` (setup.py:7-9, attention_kernel.cu:282-285)."""
from attention_impl_b200.ops import kv_attention_forward, naive_attention_forward  # noqa: F401
