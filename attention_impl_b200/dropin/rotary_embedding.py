"""Drop-in for the reference extension module ``rotary_embedding`` (setup.py:13-15, rotary_embedding.cu:80-84)."""
from attention_impl_b200.ops import rotary_embedding_inplace  # noqa: F401
