"""Generate the golden vectors in this folder from the reference's OWN torch functions.

Run once, on a machine that has the reference checkout (no GPU needed):

    python tests/golden/make_golden.py /path/to/attention-impl

The reference's ground truth lives inside its test modules, which (a) import a
module ``lm_ops`` that the reference does not ship and (b) call ``.cuda()``.
This script registers an empty stand-in for ``lm_ops`` and makes ``.cuda()`` the
identity so the modules import on a CPU-only machine, then calls the reference
functions unchanged on seeded inputs and stores inputs + outputs as ``.npz``.
Half-precision tensors are stored as their uint16 bit patterns so that the
comparison in ``tests/test_oracle_golden.py`` is bit-exact.
"""
import importlib
import os
import sys
import types

import numpy as np
import torch


def _bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def main(ref_root: str, out_dir: str) -> None:
    tests_dir = os.path.join(ref_root, "tests")
    sys.path.insert(0, tests_dir)
    stub = types.ModuleType("lm_ops")
    for name in ("naive_attention_forward", "single_query_attention", "packed_attention",
                 "rotary_embedding_inplace"):
        setattr(stub, name, lambda *a, **k: None)
    # test_kv_paged_attention.py is a script: at import it calls the op and subtracts
    # the results from the torch reference's, so the stand-in returns zeros of those shapes.
    stub.paged_kv_attention_forward = lambda Q, K, V, Kc, Vc, ci, off, nh: (
        torch.zeros(Q.shape[0], nh, 3, dtype=torch.float32),
        torch.zeros(Q.shape[0], nh, 3, dtype=torch.float32),
        torch.zeros_like(Q))
    sys.modules["lm_ops"] = stub
    torch.Tensor.cuda = lambda self, *a, **k: self  # CPU-only import of the reference tests

    t_naive = importlib.import_module("test_naive_attention")
    t_packed = importlib.import_module("test_packed_attention")
    t_single = importlib.import_module("test_single_query_attention")
    t_rope = importlib.import_module("test_rotary_embedding")
    t_paged = importlib.import_module("test_kv_paged_attention")

    g = torch.Generator().manual_seed(20240607)

    def normal(*shape, std=1.0, dtype=torch.float32):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    out = {}

    # ---- naive (tests/test_naive_attention.py:13-25), tril mask as tests/test_util.py:8
    for tag, (B, L, dim, H, dt, std) in {
        "naive_f32": (2, 48, 32, 4, torch.float32, 0.1),
        "naive_f16": (2, 64, 64, 8, torch.float16, 0.1),
        "naive_f32_std1": (1, 40, 64, 2, torch.float32, 1.0),
    }.items():
        Q, K, V = (normal(B, L, dim, std=std, dtype=dt) for _ in range(3))
        mask = torch.tril(torch.ones(L, L)).reshape(1, L, L).repeat(B, 1, 1).to(dt)
        S, P, O = t_naive.reference_MHA(Q, K, V, mask=mask, num_heads=H)
        out[tag] = dict(Q=Q, K=K, V=V, mask=mask, S=S, P=P, O=O, num_heads=torch.tensor(H))

    # ---- packed, equal lengths (tests/test_packed_attention.py:9-22,26-43)
    for tag, (B, L, dim, H, dt, std) in {
        "packed_f16": (4, 32, 64, 4, torch.float16, 0.1),
        "packed_f32": (3, 24, 32, 8, torch.float32, 1.0),
    }.items():
        Q, K, V = (normal(B * L, dim, std=std, dtype=dt) for _ in range(3))
        offsets = torch.tensor([(1 + i) * L for i in range(B)], dtype=torch.int32)
        mask = torch.from_numpy(np.tril(np.ones(L).astype(np.float32))).reshape(1, L, L).repeat(B, 1, 1).to(dt)
        S, P, O = t_packed.reference_MHA(Q.reshape(B, L, dim), K.reshape(B, L, dim), V.reshape(B, L, dim),
                                         mask=mask, num_heads=H)
        out[tag] = dict(Q=Q, K=K, V=V, offsets=offsets, O=O.reshape(B * L, dim), num_heads=torch.tensor(H))

    # ---- single query (tests/test_single_query_attention.py:9-32) with non-zero caches
    for tag, (B, ctx, dim, H, dt, std) in {
        "single_f32": (3, 20, 32, 4, torch.float32, 0.5),
        "single_f16": (2, 33, 64, 8, torch.float16, 0.1),
    }.items():
        Q, K, V = (normal(B, dim, std=std, dtype=dt) for _ in range(3))
        Kc, Vc = (normal(B, ctx, dim, std=std, dtype=dt) for _ in range(2))
        S, P, O = t_single.reference_kv_MHA(Q, K, V, Kc, Vc, num_heads=H)
        out[tag] = dict(Q=Q, K=K, V=V, K_cache=Kc, V_cache=Vc, S=S, P=P, O=O, num_heads=torch.tensor(H))

    # ---- paged decode (tests/test_kv_paged_attention.py:21-43): two cached tokens per
    # sequence, unscaled; the function reads batch_size/dim/num_heads from module globals.
    for tag, (B, dim, H, slots, dt, std) in {
        "paged_ref_shape": (2, 4, 2, 1024, torch.float32, 0.1),   # the reference script's own sizes
        "paged_f32": (5, 64, 4, 256, torch.float32, 1.0),
    }.items():
        t_paged.batch_size, t_paged.dim, t_paged.num_heads = B, dim, H
        Q, K, V = (normal(B, dim, std=std, dtype=dt) for _ in range(3))
        Kc, Vc = (normal(slots, dim, std=std, dtype=dt) for _ in range(2))
        if tag == "paged_ref_shape":
            ci = torch.tensor([16, 24, 1, 2], dtype=torch.int32)      # :18
        else:
            ci = torch.randperm(slots, generator=g)[: 2 * B].to(torch.int32)
        offsets = torch.tensor([2 * (i + 1) for i in range(B)], dtype=torch.int32)  # :19
        S, P, O = t_paged.reference_paged_kv_single_query_attention(Q, K, V, Kc, Vc, ci.long())
        out[tag] = dict(Q=Q, K=K, V=V, K_cache=Kc, V_cache=Vc, cache_indices=ci, offsets=offsets,
                        S=S, P=P, O=O, num_heads=torch.tensor(H))

    # ---- rotary (tests/test_rotary_embedding.py:8-48): the torch module's forward, with
    # its cos/sin buffers set to cat(table, table) of the kernel-side module's table
    # (:65-71), i.e. the same numbers the kernel receives.
    for tag, (N, H, hd, rot, maxpos) in {
        "rope_full": (6, 4, 32, 32, 64),
        "rope_partial": (5, 8, 64, 32, 40),
        "rope_big_pos": (4, 2, 128, 128, 8192),
    }.items():
        q = normal(N, H, hd, std=1.0, dtype=torch.float16)
        k = normal(N, H, hd, std=1.0, dtype=torch.float16)
        pos = torch.randint(0, maxpos, (N,), generator=g).int()
        my = t_rope.MyRotaryEmbedding(head_dim=hd, rot_dim=rot, max_position_embeddings=maxpos, base=10000)
        ref = t_rope.RefRotaryEmbedding(dim=rot, max_position_embeddings=maxpos, base=10000)
        ref.cos_cached = torch.cat((my.cos_cached, my.cos_cached), dim=-1)
        ref.sin_cached = torch.cat((my.sin_cached, my.sin_cached), dim=-1)
        q_rot, k_rot = ref.forward(q[..., :rot], k[..., :rot], pos.long())
        q_out = torch.cat((q_rot, q[..., rot:]), dim=-1).reshape(N, -1)   # :131-135
        k_out = torch.cat((k_rot, k[..., rot:]), dim=-1).reshape(N, -1)
        cos_t, sin_t, pos_t = my.cos_cached, my.sin_cached, pos
        if maxpos > 256:
            # keep the fixture small: store only the table rows that are used, re-indexed
            # 0..N-1, plus the original positions so the table builder can be checked too.
            cos_t, sin_t, pos_t = my.cos_cached[pos.long()], my.sin_cached[pos.long()], torch.arange(N).int()
        out[tag] = dict(q=q.reshape(N, -1), k=k.reshape(N, -1), positions=pos_t, orig_positions=pos,
                        cos=cos_t, sin=sin_t, q_out=q_out, k_out=k_out, head_dim=torch.tensor(hd),
                        max_pos=torch.tensor(maxpos))

    for tag, d in out.items():
        np.savez_compressed(os.path.join(out_dir, tag + ".npz"),
                            **{k: _bits(v) for k, v in d.items()},
                            **{"dtype_" + k: np.array(str(v.dtype)) for k, v in d.items()})
        print(tag, {k: tuple(v.shape) for k, v in d.items()})


if __name__ == "__main__":
    main(sys.argv[1], os.path.dirname(os.path.abspath(__file__)))
