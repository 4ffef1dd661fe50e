"""Seeded synthetic inputs shaped like the workload configurations (CPU tensors)."""
import math

import torch


def decode_inputs(B, H, D, lens, n_slots, dtype, seed, std=1.0):
    """q/k/v ~ N(0, std), slot table = random permutation prefix over an n_slots pool."""
    g = torch.Generator().manual_seed(seed)
    dim = H * D
    Q, K, V = ((torch.randn(B, dim, generator=g) * std).to(dtype) for _ in range(3))
    Kc, Vc = ((torch.randn(n_slots, dim, generator=g) * std).to(dtype) for _ in range(2))
    T = int(sum(lens))
    assert T <= n_slots
    ci = torch.randperm(n_slots, generator=g)[:T].to(torch.int32)
    off = torch.tensor(list(lens), dtype=torch.int64).cumsum(0).to(torch.int32)
    return Q, K, V, Kc, Vc, ci, off


def uniform_lens(B, lo, hi, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (B,), generator=g).tolist()


def prefill_inputs(lens, H, D, dtype, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    T = int(sum(lens))
    Q, K, V = ((torch.randn(T, H * D, generator=g) * std).to(dtype) for _ in range(3))
    off = torch.tensor(list(lens), dtype=torch.int64).cumsum(0).to(torch.int32)
    return Q, K, V, off


def default_scale(D):
    return 1.0 / math.sqrt(D)
