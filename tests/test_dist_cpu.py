"""CPU (gloo, world_size 2 and 3): host logic of the multi-GPU decode sharding.

The CUDA kernels cannot run here; what is tested is the product's partition arithmetic
(`plan_kv_split`, `head_shard`) and its collective step (`gather_partials`) with partial rows
produced by the oracle: gathered partials folded by the oracle's combine must equal the oracle's
one-shot decode.  A rank that fails before the collective is also covered (host-side failure
injection: the other rank's all-gather ends with an error after a short timeout)."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from attention_impl_b200 import dist as adist
from oracle import attention_oracle as orc
from helpers import decode_inputs


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_head_shard_tiles_the_heads():
    for H, G in ((32, 1), (32, 2), (32, 8), (8, 4)):
        got = [adist.head_shard(H, G, r) for r in range(G)]
        assert got[0][0] == 0 and got[-1][1] == H
        assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
    with pytest.raises(ValueError):
        adist.head_shard(30, 4, 0)
    x = torch.arange(2 * 8 * 4).reshape(2, 32)
    assert torch.equal(adist.slice_heads(x, 8, 4, 1), x[:, 8:16])


@pytest.mark.parametrize("G", [1, 2, 3, 8])
def test_plan_kv_split_partitions_every_sequence(G):
    lens = [0, 1, 2, 7, 64, 100, 3]
    T = sum(lens)
    ci = torch.randperm(1000)[:T].int()
    off = torch.tensor(lens).cumsum(0).int()
    begs = [0] + off.tolist()[:-1]
    pieces = [adist.plan_kv_split(ci, off, G, r) for r in range(G)]
    for b, n in enumerate(lens):
        got = []
        for li, lo in pieces:
            lb = [0] + lo.tolist()[:-1]
            got.append(li[lb[b]:lo.tolist()[b]])
        assert torch.equal(torch.cat(got), ci[begs[b]:begs[b] + n])     # contiguous slices, in rank order
        sizes = [g.numel() for g in got]
        assert max(sizes) - min(sizes) <= 1                               # balanced


def _worker(rank, world, port, fail_rank, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        B, H, D = 5, 4, 16
        lens = [9, 0, 33, 1, 20]
        Q, K, V, Kc, Vc, ci, off = decode_inputs(B, H, D, lens, 256, torch.float32, seed=17)
        li, lo = adist.plan_kv_split(ci, off, world, rank)
        part = orc.paged_decode_partial(Q, Kc, Vc, li, lo, H)
        if rank == fail_rank:
            raise RuntimeError("injected host-side failure before the collective")
        parts = adist.gather_partials(part)
        assert parts.shape == (world, B, H, D + 2)
        O = orc.lse_combine(parts, Q, K, V, H)
        _, _, O_ref = orc.paged_decode(Q, K, V, Kc, Vc, ci, off, H)
        q.put((rank, "ok", float((O - O_ref).abs().max())))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error", type(e).__name__ + ": " + str(e)[:80]))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(world, fail_rank=-1):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fail_rank, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    return sorted(res)


@pytest.mark.parametrize("world", [2, 3])
def test_kv_split_gather_and_combine_over_gloo(world):
    for rank, status, err in _run(world):
        assert status == "ok", err
        assert err < 1e-5


def test_rank_failing_before_the_collective_is_seen_by_its_peer():
    res = dict((r, (s, e)) for r, s, e in _run(2, fail_rank=1))
    assert res[1][0] == "error" and "injected" in res[1][1]
    assert res[0][0] == "error"          # the peer's all-gather ended with an error, it did not hang
