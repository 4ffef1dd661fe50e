"""ctypes binding of libattn_b200.so (the C ABI declared in include/attn_b200.h).

There is no fallback: if the library is missing or fails to load, importing this
module raises, and every op of the package is unusable.  Build it with
``python attention_impl_b200/build.py``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libattn_b200.so")

F16, BF16, F32, E4M3 = 0, 1, 2, 3
FLAG_BAD_SLOT, FLAG_BAD_POSITION, FLAG_BAD_OFFSETS, FLAG_TIMEOUT = 1, 2, 4, 8
DECODE_TABLES_READY = 0x100      # or-ed into `stages` of attn_b200_paged_decode
ABI_VERSION = 4
STATIC_SCRATCH_BYTES = 16 << 20

_vp, _i32, _i64, _f32, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/attn_b200.h one to one
PROTOTYPES = {
    "attn_b200_strerror": (C.c_char_p, [_i32]),
    "attn_b200_abi_version": (_i32, []),
    "attn_b200_rope_inplace": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i64, _i32, _vp, _vp]),
    "attn_b200_rope_write_kv": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i64,
                                       _i64, _i32, _i32, _vp, _vp, _vp, _vp]),
    "attn_b200_paged_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp, _i64,
                                      _i32, _i32, _i32, _i32, _i64, _i64, _i32, _i32, _i32, _i32, _f32, _vp, _vp,
                                      _i32, _i32, _i32, _vp, _vp]),
    "attn_b200_paged_decode_workspace_bytes": (_sz, [_i32, _i32, _i32, _i64, _i32]),
    "attn_b200_paged_decode_single_launch_ok": (_i32, [_i32, _i32, _i32, _i32, _i64, _i32, _i32, _i32, _i32]),
    "attn_b200_paged_decode_pick_chunk": (_i32, [_i32, _i32, _i32, _i64, _i32]),
    "attn_b200_paged_decode_pick_chunk_gqa": (_i32, [_i32, _i32, _i32, _i32, _i32, _i64, _i32]),
    "attn_b200_paged_decode_partial": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i32, _i32, _i32, _i32, _i64,
                                              _i64, _i32, _i32, _i32, _f32, _vp, _vp, _i32, _i32, _vp, _vp]),
    "attn_b200_paged_decode_static_scratch": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i64,
                                                     _i64, _i32, _f32, _vp, _vp, _i32, _i32, _vp, _vp]),
    "attn_b200_peer_push_ctas": (_i32, [_sz]),
    "attn_b200_peer_push": (_i32, [_vp, _sz, _vp, _vp, _i32, _vp]),
    "attn_b200_wait_flags": (_i32, [_vp, _i32, _i32, _vp, _vp]),
    "attn_b200_wait_flags_consume": (_i32, [_vp, _i32, _i32, _vp, _vp]),
    "attn_b200_paged_decode_partial_push": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _i32, _i32, _i32, _i32, _i64, _i64,
                                                   _i32, _i32, _i32, _f32, _vp, _vp, _i32, _i32, _vp, _vp, _i32, _vp,
                                                   _vp]),
    "attn_b200_lse_combine_wait": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _i32, _vp, _vp,
                                          _vp, _vp]),
    "attn_b200_lse_combine": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _i32, _vp]),
    "attn_b200_varlen_prefill": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _i32, _f32,
                                        _i32, _i32, _i32, _vp, _vp]),
    "attn_b200_paged_prefill": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i32, _i32, _i32, _i32, _i32,
                                       _i64, _f32, _i32, _i32, _vp, _vp]),
    "attn_b200_dense_attention": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _f32,
                                         _i32, _vp]),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: the CUDA library is not built. Run `python attention_impl_b200/build.py` "
            "(needs nvcc); attention_impl_b200 has no CPU or eager fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype, fn.argtypes = res, args
    got = lib.attn_b200_abi_version()
    if got != ABI_VERSION:
        raise ImportError(f"libattn_b200.so has ABI version {got}, this package expects {ABI_VERSION}: rebuild")
    return lib


lib = _load()


def check(status: int, what: str) -> None:
    """Raise RuntimeError (what the reference's AT_ASSERTM surfaces as in Python) on failure."""
    if status != 0:
        raise RuntimeError(f"{what}: {lib.attn_b200_strerror(status).decode()} (status {status})")
