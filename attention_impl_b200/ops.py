"""Host-side mirror of the reference's five operators, calling libattn_b200 through its C ABI.

Names, positional argument order and return arity follow the reference's pybind blocks
(attention_kernel.cu:282-285, paged_attention_kernel.cu:296-299, rotary_embedding.cu:80-84).
Extra behaviour is keyword-only and defaults to the reference's.  torch is used for device
memory and the current stream only; all arithmetic happens in the CUDA library.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from . import _lib
from ._lib import lib, check

_DT = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}
_FP8 = tuple(t for t in (getattr(torch, "float8_e4m3fn", None),) if t is not None)


def _check_input(x: torch.Tensor, name: str) -> None:
    # same wording as the reference's CHECK_INPUT (util.cuh:4-6)
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not x.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _dtype_code(x: torch.Tensor, name: str) -> int:
    if x.dtype not in _DT:
        raise RuntimeError(f"{name}: dtype {x.dtype} is not supported (float16, bfloat16, float32; "
                           "float64 inputs are rejected on purpose)")
    return _DT[x.dtype]


def _int32(x: torch.Tensor, name: str) -> None:
    _check_input(x, name)
    if x.dtype != torch.int32:
        raise RuntimeError(f"{name} must be int32 (expected scalar type Int but found {x.dtype})")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    # the raw handle of the current stream of the current device (the short way when torch has it:
    # torch.cuda.current_stream() costs several microseconds of Python per call)
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(x: Optional[torch.Tensor]) -> Optional[int]:
    return None if x is None else x.data_ptr()


_SM_COUNT: dict = {}


def sm_count(device) -> int:
    key = device.index if isinstance(device, torch.device) and device.index is not None else device
    n = _SM_COUNT.get(key)
    if n is None:
        n = _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


class _on_device:
    """`with torch.cuda.device(dev)` that does nothing when dev is already current (the usual case;
    the context manager costs a few microseconds each way)."""
    __slots__ = ("ctx",)

    def __init__(self, dev: torch.device):
        self.ctx = None if dev.index is None or dev.index == torch.cuda.current_device() else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            return self.ctx.__exit__(*exc)
        return False


_EMPTY_F64: dict = {}


def _empty_f64(dev: torch.device) -> torch.Tensor:
    """The placeholder returned for S and P when they are not requested (one per device)."""
    t = _EMPTY_F64.get(dev)
    if t is None:
        t = _EMPTY_F64[dev] = torch.empty(0, dtype=torch.float64, device=dev)
    return t


# ----------------------------------------------------------------------------------------------
# rotary embedding
# ----------------------------------------------------------------------------------------------
def rotary_embedding_inplace(Q, K, positions, cos, sin, head_dim: int, *, check_positions: bool = False) -> None:
    """In-place NeoX rotary embedding on Q and K (rotary_embedding.cu:40-77).

    Q ``[N, Hq*head_dim]``, K ``[N, Hk*head_dim]`` (the reference assumes Hk == Hq; any Hk works
    here), positions int32 ``[N]``, cos/sin ``[max_pos, rot_half]`` in Q's dtype.
    ``check_positions=True`` synchronises and raises if a position was outside the table
    (such rows are skipped by the kernel either way).
    """
    for t, n in ((Q, "Q"), (K, "K"), (positions, "positions"), (cos, "cos"), (sin, "sin")):
        _check_input(t, n)
    _int32(positions, "positions")
    dt = _dtype_code(Q, "Q")
    if K.dtype != Q.dtype or cos.dtype != Q.dtype or sin.dtype != Q.dtype:
        raise RuntimeError("K, cos and sin must have Q's dtype")
    n_tokens = Q.size(0)
    rot_half = cos.size(1)
    if Q.size(1) % head_dim or K.size(1) % head_dim:
        raise RuntimeError("Q.size(1) and K.size(1) must be multiples of head_dim")
    flag = torch.zeros(1, dtype=torch.int32, device=Q.device) if check_positions else None
    with _on_device(Q.device):
        check(lib.attn_b200_rope_inplace(Q.data_ptr(), K.data_ptr(), positions.data_ptr(), cos.data_ptr(),
                                         sin.data_ptr(), n_tokens, Q.size(1) // head_dim, K.size(1) // head_dim,
                                         head_dim, rot_half, cos.size(0), dt, _ptr(flag), _stream()),
              "rotary_embedding_inplace")
    if flag is not None and int(flag.item()) & _lib.FLAG_BAD_POSITION:
        raise RuntimeError("rotary_embedding_inplace: a position is outside [0, cos.size(0))")


def rope_and_cache_write(Q, K, V, positions, cos, sin, slots, K_cache, V_cache, head_dim: int, *,
                         k_scale=None, v_scale=None, err_flag: Optional[torch.Tensor] = None) -> None:
    """Rotate Q and K in place (as :func:`rotary_embedding_inplace`) and append the rotated K and V
    of every token to the KV pools at ``slots`` (int32 ``[N]``).  With ``k_scale``/``v_scale`` (float32
    ``[Hk]``) the pools are ``float8_e4m3fn`` and receive ``x / scale`` rounded to nearest.  This is the
    step the reference leaves to its caller before ``paged_kv_attention_forward``."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (cos, "cos"), (sin, "sin"), (K_cache, "K_cache"), (V_cache, "V_cache")):
        _check_input(t, n)
    _int32(positions, "positions")
    _int32(slots, "slots")
    dt = _dtype_code(Q, "Q")
    if any(t.dtype != Q.dtype for t in (K, V, cos, sin)):
        raise RuntimeError("K, V, cos and sin must have Q's dtype")
    kvd = _kv_code(K_cache, Q)
    n = Q.size(0)
    hk = K.size(1) // head_dim
    if V.shape != K.shape or K_cache.size(1) != K.size(1) or V_cache.shape != K_cache.shape:
        raise RuntimeError("V must match K, and the pools must be [slots, Hk*head_dim]")
    with _on_device(Q.device):
        check(lib.attn_b200_rope_write_kv(Q.data_ptr(), K.data_ptr(), V.data_ptr(), positions.data_ptr(),
                                          cos.data_ptr(), sin.data_ptr(), slots.data_ptr(), K_cache.data_ptr(),
                                          V_cache.data_ptr(), n, Q.size(1) // head_dim, hk, head_dim, cos.size(1),
                                          cos.size(0), K_cache.size(0), dt, kvd, _ptr(k_scale), _ptr(v_scale),
                                          _ptr(err_flag), _stream()), "rope_and_cache_write")


# ----------------------------------------------------------------------------------------------
# paged decode
# ----------------------------------------------------------------------------------------------
def _kv_code(kc: torch.Tensor, q: torch.Tensor) -> int:
    if kc.dtype in _FP8 or kc.dtype == torch.uint8:
        if q.dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError("FP8 KV needs float16 or bfloat16 queries")
        return _lib.E4M3
    if kc.dtype != q.dtype:
        raise RuntimeError("K_cache/V_cache must have Q's dtype (or be float8_e4m3fn)")
    return _DT[q.dtype]


def pick_chunk(B: int, H: int, D: int, n_tokens: int, device, group: int = 1, kv_dtype: int = 0) -> int:
    """Chunk length for ``H`` KV heads serving ``group`` query heads each (``kv_dtype``: ABI dtype code)."""
    if group > 1:
        return lib.attn_b200_paged_decode_pick_chunk_gqa(B, H, group, D, kv_dtype, n_tokens, sm_count(device))
    return lib.attn_b200_paged_decode_pick_chunk(B, H, D, n_tokens, sm_count(device))


def decode_workspace_bytes(B: int, H: int, D: int, n_tokens: int, chunk: int) -> int:
    return lib.attn_b200_paged_decode_workspace_bytes(B, H, D, n_tokens, chunk)


def paged_kv_attention_forward(Q, K, V, K_cache, V_cache, cache_indices, offsets, num_heads: int, *,
                               scale: Optional[float] = None, return_sp: bool = True,
                               chunk: Optional[int] = None, k_scale=None, v_scale=None,
                               max_context_len: Optional[int] = None, workspace: Optional[torch.Tensor] = None,
                               out: Optional[torch.Tensor] = None,
                               err_flag: Optional[torch.Tensor] = None, stages: int = 3,
                               block_size: int = 1, single_launch: Optional[bool] = None,
                               tables_ready: bool = False) -> List[torch.Tensor]:
    """KV-paged single-query attention, block_size = 1 (paged_attention_kernel.cu:237-294).

    Q, K, V ``[B, H*D]`` (the current token); K_cache, V_cache ``[slots, H*D]``; cache_indices
    int32 ``[T]``; offsets int32 ``[B]`` inclusive cumulative context lengths.  Returns
    ``[S, P, O]`` with S, P float64 ``[B, H, max_ctx+1]`` like the reference.  ``scale`` defaults
    to ``1/sqrt(D)`` as in the reference launcher (:269).

    Keyword-only extensions: ``return_sp=False`` skips S/P (empty placeholders are returned) and
    with it the one device->host sync needed to size them (``max_context_len`` also avoids it);
    ``k_scale``/``v_scale`` float32 ``[H]`` select the FP8-e4m3 KV path; ``chunk`` overrides the
    split-KV chunk length; ``workspace``/``out`` let a caller reuse buffers; ``stages`` (1 = partial
    kernel only, 2 = combine only, 3 = both) exists so a benchmark can time the two kernels apart.
    Grouped-query attention: K, V and the pools may have fewer heads than Q (``Hkv = K_cache.size(1) //
    D`` must divide ``num_heads``); query head h reads KV head ``h // (num_heads // Hkv)``.
    ``block_size > 1``: ``cache_indices`` is a block table int32 ``[B, max_blocks]`` and token t of
    sequence b lives in pool row ``cache_indices[b, t // block_size] * block_size + t % block_size``.
    ``single_launch``: run the step as ONE kernel, a CTA per (sequence, head) that combines in shared
    memory (multi-head attention over 16-bit pools, per-token table, head_dim 64/128/256, no S/P).
    ``None`` (default) takes it for an EAGER call when S and P are not requested and the library's
    heuristic covers the case: the (sequence, head) pairs alone fill the machine in one wave and
    sequences are short (a batch of 8 with 32 heads).  There the host bounds the call (23 us against
    27 us per call for the two launches and their scratch allocation).  While the stream is being
    captured into a CUDA graph the default is the two-kernel form, whose step is shorter on the GPU
    (18 against 21 us at that shape).  ``True`` forces the single launch (RuntimeError if the case is
    not covered), ``False`` the two kernels.
    ``tables_ready=True`` is the caller's statement that ``cache_indices`` and ``offsets`` were complete
    before the kernel that precedes this call on the stream started (they were uploaded, not written
    by that kernel): the multi-head partial kernel then reads them while that kernel still runs.
    """
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (K_cache, "K_cache"), (V_cache, "V_cache")):
        _check_input(t, n)
    _int32(cache_indices, "cache_indices")
    _int32(offsets, "offsets")
    qd = _dtype_code(Q, "Q")
    kvd = _kv_code(K_cache, Q)
    if V_cache.dtype != K_cache.dtype or K.dtype != Q.dtype or V.dtype != Q.dtype:
        raise RuntimeError("dtype mismatch between Q/K/V or K_cache/V_cache")
    B, dim = Q.shape
    if dim % num_heads:
        raise RuntimeError("Q.size(1) must be a multiple of num_heads")
    H, D = num_heads, dim // num_heads
    if offsets.numel() != B:
        raise RuntimeError("offsets must have one entry per sequence")
    if K_cache.size(1) % D or V_cache.shape != K_cache.shape:
        raise RuntimeError("K_cache/V_cache must be [slots, Hkv*D]")
    Hkv = K_cache.size(1) // D
    if H % Hkv or K.size(1) != Hkv * D or V.size(1) != Hkv * D:
        raise RuntimeError("K, V and the pools must have Hkv*D columns with Hkv dividing num_heads")
    if block_size > 1:
        if cache_indices.dim() != 2 or cache_indices.size(0) != B:
            raise RuntimeError("block_size > 1 needs a block table [B, max_blocks]")
        max_blocks = cache_indices.size(1)
        T = B * max_blocks * block_size          # token capacity; the lengths come from offsets
    else:
        max_blocks = 0
        T = cache_indices.numel()
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if kvd == _lib.E4M3:
        if k_scale is None or v_scale is None:
            raise RuntimeError("FP8 KV needs k_scale and v_scale (float32 [H])")
        for t, n in ((k_scale, "k_scale"), (v_scale, "v_scale")):
            _check_input(t, n)
            if t.dtype != torch.float32 or t.numel() != Hkv:
                raise RuntimeError(f"{n} must be float32 [Hkv]")
    dev = Q.device
    with _on_device(dev):
        if single_launch is None:
            single_launch = (not return_sp and stages == 3 and not torch.cuda.is_current_stream_capturing()
                             and bool(lib.attn_b200_paged_decode_single_launch_ok(
                                 B, H, Hkv, D, T, block_size, qd, kvd, sm_count(dev))))
        elif single_launch and return_sp:
            raise RuntimeError("single_launch=True does not produce S and P: pass return_sp=False")
        if single_launch:
            stages = 4
            if chunk is None:
                chunk = 32                       # unused by the single launch, only range-checked
        if chunk is None:
            chunk = pick_chunk(B, Hkv, D, T, dev, group=H // Hkv, kv_dtype=kvd)
        need = 0 if single_launch else decode_workspace_bytes(B, H, D, T, chunk)
        if single_launch:
            workspace = None
        elif workspace is None:
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        elif workspace.numel() * workspace.element_size() < need:
            raise RuntimeError(f"workspace too small: {need} bytes needed")
        O = torch.empty_like(Q) if out is None else out
        if return_sp:
            if max_context_len is None:
                lens = torch.diff(offsets, prepend=offsets.new_zeros(1))
                max_context_len = int(lens.max().item()) if B > 0 else 0
            S = torch.zeros(B, H, max_context_len + 1, dtype=torch.float64, device=dev)
            P = torch.zeros_like(S)
            stride = max_context_len + 1
        else:
            S = P = _empty_f64(dev)
            stride = 0
        check(lib.attn_b200_paged_decode(
            Q.data_ptr(), K.data_ptr(), V.data_ptr(), K_cache.data_ptr(), V_cache.data_ptr(),
            cache_indices.data_ptr(), offsets.data_ptr(), O.data_ptr(), _ptr(workspace),
            0 if workspace is None else workspace.numel() * workspace.element_size(),
            S.data_ptr() if return_sp else None, P.data_ptr() if return_sp else None, stride,
            B, H, Hkv, D, T, K_cache.size(0), 0, block_size, max_blocks, chunk, float(scale), _ptr(k_scale),
            _ptr(v_scale), qd, kvd, stages | (_lib.DECODE_TABLES_READY if tables_ready else 0), _ptr(err_flag),
            _stream()), "paged_kv_attention_forward")
    return [S, P, O]


class _StepArena:
    """One device buffer and one pinned host mirror holding all per-step inputs of a captured decode
    step, so that a step needs a single host->device copy.  ``fields``: name -> (shape, dtype)."""

    def __init__(self, fields, device):
        self.names, starts, sizes = [], [0], []
        for name, (shape, dtype) in fields.items():
            n = math.prod(shape) * torch.empty(0, dtype=dtype).element_size()
            self.names.append(name)
            sizes.append(n)
            starts.append((starts[-1] + n + 255) // 256 * 256)
        self.starts, self.sizes = starts, sizes
        self.dev = torch.zeros(starts[-1], dtype=torch.uint8, device=device)
        self.host = torch.zeros(starts[-1], dtype=torch.uint8).pin_memory()
        self.d, self.h = {}, {}
        for i, (name, (shape, dtype)) in enumerate(fields.items()):
            for buf, out in ((self.dev, self.d), (self.host, self.h)):
                out[name] = buf[starts[i]:starts[i] + sizes[i]].view(dtype).view(*shape)

    def start_of(self, name: str) -> int:
        return self.starts[self.names.index(name)]

    def upload(self, end: Optional[int] = None) -> None:
        if end is None:
            self.dev.copy_(self.host, non_blocking=True)
        else:
            self.dev[:end].copy_(self.host[:end], non_blocking=True)


def capture_graph(device, call):
    """Run ``call`` once on a side stream (module load, attribute set-up), then record it."""
    with torch.cuda.device(device):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            call()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            call()
    return graph


class PagedDecodeGraph:
    """A paged decode step captured in a CUDA graph: one graph launch per step instead of kernel
    launches plus the Python wrapper, which is what bounds small batches (a B=8 step is ~20 us of
    GPU work).  Not in the reference; it is how a serving loop would call this path.

    The kernels take sequence lengths from the device-side ``offsets`` and derive their grid from
    the slot-table CAPACITY, so one captured graph serves every step whose total context fits
    ``max_tokens``: write the step's q/k/v, slot table (first ``offsets[-1]`` entries) and offsets
    into the static tensors (``q``, ``k``, ``v``, ``cache_indices``, ``offsets``) — or into their
    pinned host mirrors (``host_q`` ...) followed by :meth:`upload`, one copy for all five — call
    :meth:`replay`, read ``out``.  The KV pools are captured by address.

    ``head_dim`` must be given for grouped-query pools (``K_cache.size(1) == Hkv * head_dim`` with
    ``Hkv < num_heads``); it defaults to ``K_cache.size(1) // num_heads`` (multi-head attention).
    """

    def __init__(self, K_cache, V_cache, batch: int, num_heads: int, max_tokens: int, *, dtype=None,
                 head_dim: Optional[int] = None, scale: Optional[float] = None, chunk: Optional[int] = None,
                 k_scale=None, v_scale=None):
        dev = K_cache.device
        dtype = dtype or (K_cache.dtype if K_cache.dtype in _DT else torch.float16)
        H = num_heads
        D = head_dim or K_cache.size(1) // H
        if D <= 0 or K_cache.size(1) % D:
            raise RuntimeError("K_cache.size(1) must be a multiple of head_dim")
        Hkv = K_cache.size(1) // D
        if H % Hkv:
            raise RuntimeError("the pools' head count must divide num_heads (pass head_dim for grouped-query pools)")
        self.H, self.Hkv, self.D, self.max_tokens = H, Hkv, D, max_tokens
        self._arena = _StepArena({"q": ((batch, H * D), dtype), "k": ((batch, Hkv * D), dtype),
                                  "v": ((batch, Hkv * D), dtype), "cache_indices": ((max_tokens,), torch.int32),
                                  "offsets": ((batch,), torch.int32)}, dev)
        d, h = self._arena.d, self._arena.h
        self.q, self.k, self.v, self.cache_indices, self.offsets = (d[n] for n in self._arena.names)
        self.host_q, self.host_k, self.host_v, self.host_cache_indices, self.host_offsets = (
            h[n] for n in self._arena.names)
        self.arena, self.host_arena = self._arena.dev, self._arena.host
        self._ci_start = self._arena.start_of("cache_indices")
        self.out = torch.zeros(batch, H * D, dtype=dtype, device=dev)
        kvd = _kv_code(K_cache, self.q)
        self.chunk = chunk or pick_chunk(batch, Hkv, D, max_tokens, dev, group=H // Hkv, kv_dtype=kvd)
        self.workspace = torch.empty(decode_workspace_bytes(batch, H, D, max_tokens, self.chunk), dtype=torch.uint8,
                                     device=dev)
        # tables_ready: the slot table and the offsets are written into the arena before the graph is launched
        kw = dict(scale=scale, return_sp=False, chunk=self.chunk, k_scale=k_scale, v_scale=v_scale,
                  workspace=self.workspace, out=self.out, tables_ready=True, single_launch=False)
        self._pools = (K_cache, V_cache)
        self.graph = capture_graph(dev, lambda: paged_kv_attention_forward(
            self.q, self.k, self.v, K_cache, V_cache, self.cache_indices, self.offsets, H, **kw))

    def upload(self, n_tokens: Optional[int] = None) -> None:
        """Copy the pinned host mirror (``host_q`` ... ``host_offsets``) to the device arena in one
        transfer; with ``n_tokens`` the unused tail of the slot table is skipped (offsets, which sit
        after it, then go in a second small copy)."""
        if n_tokens is None or n_tokens >= self.max_tokens:
            self._arena.upload()
        else:
            self._arena.upload(self._ci_start + 4 * n_tokens)
            self.offsets.copy_(self.host_offsets, non_blocking=True)

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.out


class DecodeStepGraph:
    """The whole decode step of a serving loop in one CUDA graph: rotary embedding of the current
    token's q and k, append of the rotated k and of v to the KV pools, paged attention over the
    cached tokens plus the current one, combine.  It is the caller-side sequence around the
    reference's operator, which receives the current token's k, v as arguments
    (paged_attention_kernel.cu:137-146, 179-185) and leaves both the rotation and the append to its
    caller.

    Per step the caller fills the pinned host mirrors ``host["q"|"k"|"v"]`` (``[batch, H*D]`` /
    ``[batch, Hkv*D]``, un-rotated), ``host["positions"]`` (int32 ``[batch]``), ``host["new_slots"]``
    (int32 ``[batch]``: the pool row that receives each sequence's current token),
    ``host["cache_indices"]`` (int32, the slots of the tokens cached BEFORE this step, concatenated)
    and ``host["offsets"]`` (int32 ``[batch]``, inclusive cumulative counts of those), then calls
    :meth:`upload` and :meth:`replay`.  ``out`` holds the attention output; ``q``/``k`` on the device
    hold the rotated values.  For the next step the caller appends ``new_slots[b]`` to sequence b's
    slots.  One captured graph serves every step whose cached tokens fit ``max_tokens``.
    With float8 pools pass ``k_scale``/``v_scale`` (float32 ``[Hkv]``).
    """

    def __init__(self, K_cache, V_cache, cos, sin, batch: int, num_heads: int, head_dim: int, max_tokens: int, *,
                 dtype=None, scale: Optional[float] = None, chunk: Optional[int] = None, k_scale=None, v_scale=None):
        dev = K_cache.device
        dtype = dtype or (K_cache.dtype if K_cache.dtype in _DT else torch.float16)
        H, D = num_heads, head_dim
        if K_cache.size(1) % D:
            raise RuntimeError("K_cache.size(1) must be a multiple of head_dim")
        Hkv = K_cache.size(1) // D
        if H % Hkv:
            raise RuntimeError("the pools' head count must divide num_heads")
        self.H, self.Hkv, self.D, self.max_tokens = H, Hkv, D, max_tokens
        self._arena = _StepArena({"q": ((batch, H * D), dtype), "k": ((batch, Hkv * D), dtype),
                                  "v": ((batch, Hkv * D), dtype), "positions": ((batch,), torch.int32),
                                  "new_slots": ((batch,), torch.int32), "offsets": ((batch,), torch.int32),
                                  "cache_indices": ((max_tokens,), torch.int32)}, dev)
        self.dev_in, self.host = self._arena.d, self._arena.h
        self.q, self.k = self.dev_in["q"], self.dev_in["k"]
        self.out = torch.zeros(batch, H * D, dtype=dtype, device=dev)
        self.err_flag = torch.zeros(1, dtype=torch.int32, device=dev)
        kvd = _kv_code(K_cache, self.q)
        self.chunk = chunk or pick_chunk(batch, Hkv, D, max_tokens, dev, group=H // Hkv, kv_dtype=kvd)
        self.workspace = torch.empty(decode_workspace_bytes(batch, H, D, max_tokens, self.chunk), dtype=torch.uint8,
                                     device=dev)
        self._keep = (K_cache, V_cache, cos, sin, k_scale, v_scale)
        d = self.dev_in

        def step():
            rope_and_cache_write(d["q"], d["k"], d["v"], d["positions"], cos, sin, d["new_slots"], K_cache, V_cache,
                                 D, k_scale=k_scale, v_scale=v_scale, err_flag=self.err_flag)
            paged_kv_attention_forward(d["q"], d["k"], d["v"], K_cache, V_cache, d["cache_indices"], d["offsets"], H,
                                       scale=scale, return_sp=False, chunk=self.chunk, k_scale=k_scale,
                                       v_scale=v_scale, workspace=self.workspace, out=self.out,
                                       err_flag=self.err_flag, single_launch=False,
                                       tables_ready=True)   # tables: uploaded, not made by the RoPE kernel

        # the warm-up run inside capture_graph executes a real step on whatever the arena holds (zeros:
        # position 0, slot 0, no cached tokens): the caller's first upload overwrites all of it, but
        # pool row 0 receives one bogus append, so put it back afterwards
        row0 = (K_cache[0].clone(), V_cache[0].clone())
        self.graph = capture_graph(dev, step)
        K_cache[0].copy_(row0[0])
        V_cache[0].copy_(row0[1])
        self.err_flag.zero_()

    def upload(self, n_tokens: Optional[int] = None) -> None:
        """One host->device copy of all per-step inputs; ``n_tokens`` (cached tokens this step) skips the
        unused tail of the slot table, which is the last field of the arena."""
        if n_tokens is None or n_tokens >= self.max_tokens:
            self._arena.upload()
        else:
            self._arena.upload(self._arena.start_of("cache_indices") + 4 * n_tokens)

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.out


class HostStagedDecoder:
    """Paged decode whose per-step inputs live in pinned HOST memory, with the uploads overlapped
    with compute.  (The slot table is the bulk of the traffic: 4 bytes per context token per step.)

    Two forms of overlap.  Within a step, the batch is cut into ``n_groups`` runs of sequences with
    about equal token counts; while group g is decoded, group g+1's q/k/v rows, slot-table slice and
    offsets travel on a copy stream, and each group's output rows go back as soon as they exist.
    Across steps, a decode loop knows the NEXT step's slot table while the current step runs (it is
    this step's table plus one slot per sequence): pass it as ``next_table=(cache_indices, offsets)``
    and it is uploaded into the second of two device buffers during this step's kernels; the next
    call, given those same host tensors, finds its table already resident, uploads only q/k/v and
    runs the batch as one group.

    ``Q, K, V`` pinned ``[B, H*D]``, ``cache_indices`` pinned int32 ``[T]``, ``offsets`` pinned int32 ``[B]``
    (inclusive cumulative lengths), ``out`` pinned ``[B, H*D]``.  The KV pools stay on the device.
    """

    def __init__(self, K_cache, V_cache, num_heads: int, max_batch: int, max_tokens: int, *, dtype=None,
                 n_groups: int = 4, scale: Optional[float] = None, k_scale=None, v_scale=None):
        dev = K_cache.device
        self.dev, self.H, self.n_groups = dev, num_heads, n_groups
        self.Kc, self.Vc, self.kw = K_cache, V_cache, dict(scale=scale, k_scale=k_scale, v_scale=v_scale)
        dtype = dtype or (K_cache.dtype if K_cache.dtype in _DT else torch.float16)
        dim_kv = K_cache.size(1)
        self.dim_q = None
        self.dtype = dtype
        # two table buffers: one in use by the running step, one receiving the next step's table
        self.d_ci = [torch.empty(max_tokens, dtype=torch.int32, device=dev) for _ in range(2)]
        self.d_off = [torch.empty(max_batch, dtype=torch.int32, device=dev) for _ in range(2)]
        self.h_off = torch.empty(max_batch, dtype=torch.int32).pin_memory()     # offsets rebased per group
        self.d_q = self.d_k = self.d_v = self.d_o = None
        self.max_batch, self.dim_kv = max_batch, dim_kv
        self.cur = 0                 # table buffer of the running step
        self._staged = None          # (cache_indices.data_ptr(), offsets.data_ptr(), T) resident in buffer 1 - cur
        with _on_device(dev):
            self.copy_stream = torch.cuda.Stream()
            self.events = [torch.cuda.Event() for _ in range(n_groups)]
            self.table_event = torch.cuda.Event()
            self.done_event = torch.cuda.Event()

    def _ensure(self, dim_q):
        if self.dim_q != dim_q:
            dev, B = self.dev, self.max_batch
            self.dim_q = dim_q
            self.d_q = torch.empty(B, dim_q, dtype=self.dtype, device=dev)
            self.d_k = torch.empty(B, self.dim_kv, dtype=self.dtype, device=dev)
            self.d_v = torch.empty(B, self.dim_kv, dtype=self.dtype, device=dev)
            self.d_o = torch.empty(B, dim_q, dtype=self.dtype, device=dev)

    def __call__(self, Q, K, V, cache_indices, offsets, out, next_table=None) -> None:
        """Enqueues everything; returns after the last output row has been copied (it synchronises
        the compute stream once, at the end)."""
        B = Q.size(0)
        self._ensure(Q.size(1))
        cur = torch.cuda.current_stream(self.dev)
        key = (cache_indices.data_ptr(), offsets.data_ptr(), cache_indices.numel())
        resident = self._staged == key
        if resident:
            self.cur ^= 1
        self._staged = None
        d_ci, d_off = self.d_ci[self.cur], self.d_off[self.cur]
        self.copy_stream.wait_stream(cur)           # staging buffers free again
        if resident:
            T = cache_indices.numel()
            with torch.cuda.stream(self.copy_stream):
                self.d_q[:B].copy_(Q, non_blocking=True)
                self.d_k[:B].copy_(K, non_blocking=True)
                self.d_v[:B].copy_(V, non_blocking=True)
                self.events[0].record(self.copy_stream)
            spans = [(0, B, 0, T)]
            cur.wait_event(self.table_event)        # the table upload of the previous call
        else:
            ends = offsets[:B].tolist()
            T = ends[-1] if B else 0
            # group boundaries (sequence indices) at about equal token counts
            bounds, g = [0], 1
            for b, e in enumerate(ends):
                if g < self.n_groups and e >= T * g / self.n_groups and b + 1 < B:
                    bounds.append(b + 1)
                    g += 1
            bounds.append(B)
            spans = []
            with torch.cuda.stream(self.copy_stream):
                for i in range(len(bounds) - 1):
                    b0, b1 = bounds[i], bounds[i + 1]
                    t0 = ends[b0 - 1] if b0 else 0
                    t1 = ends[b1 - 1]
                    self.h_off[b0:b1] = offsets[b0:b1] - t0
                    self.d_q[b0:b1].copy_(Q[b0:b1], non_blocking=True)
                    self.d_k[b0:b1].copy_(K[b0:b1], non_blocking=True)
                    self.d_v[b0:b1].copy_(V[b0:b1], non_blocking=True)
                    d_ci[t0:t1].copy_(cache_indices[t0:t1], non_blocking=True)
                    d_off[b0:b1].copy_(self.h_off[b0:b1], non_blocking=True)
                    self.events[i].record(self.copy_stream)
                    spans.append((b0, b1, t0, t1))
        if next_table is not None:                  # travels while this step's kernels run
            nci, noff = next_table
            with torch.cuda.stream(self.copy_stream):
                self.d_ci[self.cur ^ 1][:nci.numel()].copy_(nci, non_blocking=True)
                self.d_off[self.cur ^ 1][:noff.numel()].copy_(noff, non_blocking=True)
                self.table_event.record(self.copy_stream)
            self._staged = (nci.data_ptr(), noff.data_ptr(), nci.numel())
        for i, (b0, b1, t0, t1) in enumerate(spans):
            cur.wait_event(self.events[i])
            paged_kv_attention_forward(self.d_q[b0:b1], self.d_k[b0:b1], self.d_v[b0:b1], self.Kc, self.Vc,
                                       d_ci[t0:t1], d_off[b0:b1], self.H, return_sp=False,
                                       out=self.d_o[b0:b1], **self.kw)
            out[b0:b1].copy_(self.d_o[b0:b1], non_blocking=True)
        self.done_event.record(cur)
        self.done_event.synchronize()


def paged_decode_partial(Q, K_cache, V_cache, cache_indices, offsets, num_heads: int, *,
                         scale: Optional[float] = None, chunk: Optional[int] = None, k_scale=None, v_scale=None,
                         workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One KV-split rank's share of a decode: float32 ``[B, H, D+2]`` rows ``[o[D], m, l]``
    (un-normalised numerator, log2-domain maximum, denominator) over the rank's own tokens,
    without the new token.  Feed the gathered rows of all ranks to :func:`lse_combine`."""
    for t, n in ((Q, "Q"), (K_cache, "K_cache"), (V_cache, "V_cache")):
        _check_input(t, n)
    _int32(cache_indices, "cache_indices")
    _int32(offsets, "offsets")
    qd = _dtype_code(Q, "Q")
    kvd = _kv_code(K_cache, Q)
    B, dim = Q.shape
    H, D = num_heads, dim // num_heads
    Hkv = K_cache.size(1) // D
    T = cache_indices.numel()
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dev = Q.device
    with _on_device(dev):
        if chunk is None:
            chunk = pick_chunk(B, Hkv, D, T, dev, group=H // Hkv, kv_dtype=kvd)
        need = decode_workspace_bytes(B, H, D, T, chunk)
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        part = torch.empty(B, H, D + 2, dtype=torch.float32, device=dev)
        check(lib.attn_b200_paged_decode_partial(
            Q.data_ptr(), K_cache.data_ptr(), V_cache.data_ptr(), cache_indices.data_ptr(), offsets.data_ptr(),
            part.data_ptr(), workspace.data_ptr(), workspace.numel() * workspace.element_size(), B, H, Hkv, D, T,
            K_cache.size(0), 1, 0, chunk, float(scale), _ptr(k_scale), _ptr(v_scale), qd, kvd, None, _stream()),
            "paged_decode_partial")
    return part


def lse_combine(parts, Q, K=None, V=None, *, num_heads: int, scale: Optional[float] = None) -> torch.Tensor:
    """Fold ``parts`` float32 ``[n_parts, B, H, D+2]`` and, if given, the new token (K, V) into
    the final ``[B, H*D]`` output in Q's dtype."""
    _check_input(parts, "parts")
    _check_input(Q, "Q")
    n_parts, B, H, RS = parts.shape
    D = RS - 2
    if H != num_heads or Q.shape != (B, H * D) or parts.dtype != torch.float32:
        raise RuntimeError("parts must be float32 [n_parts, B, H, D+2] matching Q [B, H*D]")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    O = torch.empty_like(Q)
    Hkv = K.size(1) // D if K is not None else H
    with _on_device(Q.device):
        check(lib.attn_b200_lse_combine(parts.data_ptr(), n_parts, Q.data_ptr(), _ptr(K), _ptr(V), O.data_ptr(),
                                        B, H, Hkv, D, float(scale), _dtype_code(Q, "Q"), _stream()), "lse_combine")
    return O


# ----------------------------------------------------------------------------------------------
# single query over a contiguous cache
# ----------------------------------------------------------------------------------------------
def kv_attention_forward(Q, K, V, K_cache, V_cache, num_heads: int, *, scale: float = 1.0,
                         return_sp: bool = True) -> List[torch.Tensor]:
    """Single-query attention over a contiguous ``[B, ctx, H*D]`` cache plus the new token
    (attention_kernel.cu:231-280).  Scores are NOT scaled, as in the reference kernel (:129,143);
    pass ``scale=`` to change that.  S, P are ``[B, H, ctx+1]`` in the input dtype."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (K_cache, "K_cache"), (V_cache, "V_cache")):
        _check_input(t, n)
    qd = _dtype_code(Q, "Q")
    if any(t.dtype != Q.dtype for t in (K, V, K_cache, V_cache)):
        raise RuntimeError("all tensors must share Q's dtype")
    B, dim = Q.shape
    if dim % num_heads:
        raise RuntimeError("Q.size(1) must be a multiple of num_heads")
    H, D = num_heads, dim // num_heads
    ctx = K_cache.size(1)
    T = B * ctx
    dev = Q.device
    with _on_device(dev):
        chunk = pick_chunk(B, H, D, T, dev)
        need = decode_workspace_bytes(B, H, D, T, chunk)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        O = torch.empty_like(Q)
        if return_sp:
            S64 = torch.zeros(B, H, ctx + 1, dtype=torch.float64, device=dev)
            P64 = torch.zeros_like(S64)
        check(lib.attn_b200_paged_decode(
            Q.data_ptr(), K.data_ptr(), V.data_ptr(), K_cache.data_ptr(), V_cache.data_ptr(), None, None,
            O.data_ptr(), ws.data_ptr(), need, S64.data_ptr() if return_sp else None,
            P64.data_ptr() if return_sp else None, ctx + 1 if return_sp else 0, B, H, H, D, T, max(T, 1), ctx, 1, 0,
            chunk, float(scale), None, None, qd, qd, 3, None, _stream()), "kv_attention_forward")
    if return_sp:
        return [S64.to(Q.dtype), P64.to(Q.dtype), O]
    e = torch.empty(0, dtype=Q.dtype, device=dev)
    return [e, e.clone(), O]


# ----------------------------------------------------------------------------------------------
# packed causal prefill, dense masked attention
# ----------------------------------------------------------------------------------------------
def paged_attention_forward(Q, K, V, offsets, num_heads: int, *, scale: Optional[float] = None,
                            return_sp: bool = True, max_seqlen: Optional[int] = None,
                            out_dtype: Optional[torch.dtype] = None, force_generic: bool = False,
                            err_flag: Optional[torch.Tensor] = None, precise: bool = False) -> List[torch.Tensor]:
    """Causal attention over a packed ``[sum L, H*D]`` token buffer (paged_attention_kernel.cu:189-235).

    ``offsets`` int32 ``[B]`` are inclusive cumulative lengths.  Returns ``[S, P, O]``; S, P are
    ``[B, H, maxL, maxL]`` in the input dtype as in the reference unless ``return_sp=False``
    (empty placeholders; required for the tensor-core path and for any large input).
    ``out_dtype=torch.float32`` makes the tensor-core path store fp32 output.  ``err_flag`` (int32
    device scalar) receives ATTN_B200_FLAG_* bits (bad offsets, an in-kernel wait that ran out).
    ``precise=True`` (tensor-core path) carries P into P·V as two terms on every row, not only on a
    sequence's first 256 rows: bfloat16 inputs then stay within 2e-3 of exact arithmetic everywhere
    (3.4e-3 otherwise), for about a quarter more time.
    """
    for t, n in ((Q, "Q"), (K, "K"), (V, "V")):
        _check_input(t, n)
    _int32(offsets, "offsets")
    dt = _dtype_code(Q, "Q")
    if K.dtype != Q.dtype or V.dtype != Q.dtype or K.shape != Q.shape or V.shape != Q.shape:
        raise RuntimeError("Q, K, V must share shape and dtype")
    n_tokens, dim = Q.shape
    if dim % num_heads:
        raise RuntimeError("Q.size(1) must be a multiple of num_heads")
    H, D = num_heads, dim // num_heads
    B = offsets.numel()
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dev = Q.device
    with _on_device(dev):
        if max_seqlen is None:
            lens = torch.diff(offsets, prepend=offsets.new_zeros(1))
            max_seqlen = int(lens.max().item()) if B > 0 else 0
        out_f32 = out_dtype == torch.float32 and Q.dtype != torch.float32
        # the reference zero-fills O (zeros_like, :209).  The tensor-core path writes every row itself
        # (rows no query tile covers - past offsets[-1], or beyond an understated max_seqlen - are
        # zeroed by a small kernel of the same launch), so it skips the up-front memset
        tc_path = (not return_sp and not force_generic and D == 128 and Q.dtype in (torch.float16, torch.bfloat16))
        O = (torch.empty if tc_path else torch.zeros)(Q.shape, dtype=torch.float32 if out_f32 else Q.dtype,
                                                      device=dev)
        if return_sp:
            S = torch.zeros(B, H, max_seqlen, max_seqlen, dtype=Q.dtype, device=dev)
            P = torch.zeros_like(S)
        else:
            S = torch.empty(0, dtype=Q.dtype, device=dev)
            P = torch.empty(0, dtype=Q.dtype, device=dev)
        check(lib.attn_b200_varlen_prefill(
            Q.data_ptr(), K.data_ptr(), V.data_ptr(), offsets.data_ptr(), O.data_ptr(),
            S.data_ptr() if return_sp else None, P.data_ptr() if return_sp else None, B, n_tokens, max_seqlen, H, D,
            float(scale), dt, int(out_f32) | (2 if precise else 0), int(force_generic), _ptr(err_flag), _stream()),
            "paged_attention_forward")
    return [S, P, O]


def paged_prefill_attention(Q, K_cache, V_cache, cache_indices, kv_offsets, q_offsets, num_heads: int, *,
                            scale: Optional[float] = None, max_q_len: Optional[int] = None,
                            max_kv_len: Optional[int] = None, force_generic: bool = False,
                            err_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Chunked / prefix-cached prefill through the slot table (not in the reference).

    Q ``[sum q_len, H*D]`` holds, per sequence, the query rows of its LAST ``q_len_b`` tokens
    (``q_offsets`` int32 ``[B]``, inclusive cumulative); ``cache_indices`` int32 ``[sum kv_len]`` /
    ``kv_offsets`` address ALL of the sequence's tokens in the pools (prefix and chunk, e.g. appended
    with :func:`rope_and_cache_write`).  Query i of a chunk sees key j iff ``j <= kv_len - q_len + i``.
    With ``q_len == kv_len`` this is the packed causal prefill, with ``q_len == 1`` the paged decode
    without a separate current token.  Returns O ``[sum q_len, H*D]``.
    """
    for t, n in ((Q, "Q"), (K_cache, "K_cache"), (V_cache, "V_cache")):
        _check_input(t, n)
    for t, n in ((cache_indices, "cache_indices"), (kv_offsets, "kv_offsets"), (q_offsets, "q_offsets")):
        _int32(t, n)
    dt = _dtype_code(Q, "Q")
    if K_cache.dtype != Q.dtype or V_cache.dtype != Q.dtype or V_cache.shape != K_cache.shape:
        raise RuntimeError("K_cache and V_cache must share Q's dtype and each other's shape")
    nq, dim = Q.shape
    if dim % num_heads:
        raise RuntimeError("Q.size(1) must be a multiple of num_heads")
    H, D = num_heads, dim // num_heads
    Hkv = K_cache.size(1) // D
    B = q_offsets.numel()
    if K_cache.size(1) % D or H % Hkv or kv_offsets.numel() != B:
        raise RuntimeError("pools must be [slots, Hkv*D] with Hkv dividing num_heads; one offset per sequence")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dev = Q.device
    with _on_device(dev):
        if max_q_len is None:
            max_q_len = int(torch.diff(q_offsets, prepend=q_offsets.new_zeros(1)).max().item()) if B else 0
        if max_kv_len is None:
            max_kv_len = int(torch.diff(kv_offsets, prepend=kv_offsets.new_zeros(1)).max().item()) if B else 0
        tc_path = not force_generic and D == 128 and Q.dtype in (torch.float16, torch.bfloat16)
        O = torch.empty_like(Q) if tc_path else torch.zeros_like(Q)     # the tensor-core path zeroes unused rows itself
        check(lib.attn_b200_paged_prefill(Q.data_ptr(), K_cache.data_ptr(), V_cache.data_ptr(),
                                          cache_indices.data_ptr(), kv_offsets.data_ptr(), q_offsets.data_ptr(),
                                          O.data_ptr(), B, nq, cache_indices.numel(), max_q_len, max_kv_len, H, Hkv, D,
                                          K_cache.size(0), float(scale), dt, int(force_generic), _ptr(err_flag),
                                          _stream()), "paged_prefill_attention")
    return O


def naive_attention_forward(Q, K, V, mask, num_heads: int, *, scale: Optional[float] = None,
                            fill: float = 100000.0, return_sp: bool = True) -> List[torch.Tensor]:
    """Dense masked MHA (attention_kernel.cu:187-229): Q, K, V ``[B, L, H*D]``, mask ``[B, L, L]``
    (1 keeps, 0 masks; scores get ``(mask-1)*fill`` added).  Returns ``[S, P, O]``."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (mask, "mask")):
        _check_input(t, n)
    dt = _dtype_code(Q, "Q")
    if any(t.dtype != Q.dtype for t in (K, V, mask)):
        raise RuntimeError("Q, K, V and mask must share a dtype")
    B, L, dim = Q.shape
    if dim % num_heads:
        raise RuntimeError("Q.size(2) must be a multiple of num_heads")
    H, D = num_heads, dim // num_heads
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dev = Q.device
    with _on_device(dev):
        O = torch.empty_like(Q)
        if return_sp:
            S = torch.zeros(B, H, L, L, dtype=Q.dtype, device=dev)
            P = torch.zeros_like(S)
        else:
            S = torch.empty(0, dtype=Q.dtype, device=dev)
            P = torch.empty(0, dtype=Q.dtype, device=dev)
        check(lib.attn_b200_dense_attention(
            Q.data_ptr(), K.data_ptr(), V.data_ptr(), mask.data_ptr(), O.data_ptr(),
            S.data_ptr() if return_sp else None, P.data_ptr() if return_sp else None, B, L, H, D, float(scale),
            float(fill), dt, _stream()), "naive_attention_forward")
    return [S, P, O]
