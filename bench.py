#!/usr/bin/env python
"""Benchmark of the paged-decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (the configuration the headline metric is quoted on): large-batch KV-paged single-query
decode, fp16 MHA, batch 256, 32 heads, head_dim 128, context lengths uniform in [1024, 32768]
(~71 GB of KV), block_size = 1 slot table = random permutation over the whole pool, q/k/v ~ N(0,1).
At N GPUs the heads are sharded N ways (each rank owns H/N heads of every token: its pool is
[slots, (H/N)*128]); there is no collective in the data path.  Total work is fixed, so this is
strong scaling.

One step = one decode of the whole batch (partial kernel + combine kernel).  `value` is the
aggregate KV-read bandwidth  2*T*H*D*2 bytes / step time  with all inputs resident in HBM, timed
with CUDA events, maximum over ranks.  `e2e` is the same through the public Python operator with
the per-step inputs (q, k, v, slot table, offsets) in pinned HOST memory copied in, and the
output copied back, inside the timed region; the KV pool itself is device-resident state (it is a
cache), as it is for any caller of the reference operator.

`--impl reference` times the reference's torch CPU math (the oracle restatement, since the
reference's test modules cannot be imported without a GPU) on a bounded sample of the same
workload with all host threads.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(batch=256, heads=32, head_dim=128, ctx_lo=1024, ctx_hi=32768, dtype="f16", seed=4)
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


def workload_lengths(cfg):
    g = torch.Generator().manual_seed(cfg["seed"])
    return torch.randint(cfg["ctx_lo"], cfg["ctx_hi"] + 1, (cfg["batch"],), generator=g)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


# ------------------------------------------------------------------------------------------------
# CPU legs (oracle = the reference's torch math)
# ------------------------------------------------------------------------------------------------
def cpu_sample_inputs(cfg, lens, n_seq, heads, seed):
    """The first n_seq sequences of the workload with a compact pool (rows in slot order, so the
    gather stays random within the sample)."""
    from oracle import attention_oracle  # noqa: F401  (CPU baseline leg only)
    g = torch.Generator().manual_seed(seed)
    D = cfg["head_dim"]
    sl = lens[:n_seq]
    T = int(sl.sum())
    dim = heads * D
    Kc = torch.empty(T, dim, dtype=torch.float16)
    Vc = torch.empty(T, dim, dtype=torch.float16)
    for t in (Kc, Vc):                                   # fp32 normal_ is vectorised, fp16 is not
        for r in range(0, T, 8192):
            t[r:r + 8192] = torch.randn(min(8192, T - r), dim, generator=g)
    Q, K, V = (torch.randn(n_seq, dim, generator=g).half() for _ in range(3))
    ci = torch.randperm(T, generator=g).int()
    off = sl.cumsum(0).int()
    return Q, K, V, Kc, Vc, ci, off


def time_cpu_oracle(inputs, heads, steps=1, warmup=0):
    from oracle import attention_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(warmup):
        orc.paged_decode(*inputs, heads)
    t0 = time.perf_counter()
    out = None
    for _ in range(steps):
        out = orc.paged_decode(*inputs, heads)
    return (time.perf_counter() - t0) / steps, out


def pick_cpu_sample(cfg, lens, heads, budget_s, max_tokens):
    """Choose how many leading sequences fit a CPU time budget (and a token cap that bounds host
    memory and set-up time), from a one-sequence probe.  Returns (n_sequences, seconds/token)."""
    probe = cpu_sample_inputs(cfg, lens, 1, heads, seed=99)
    t, _ = time_cpu_oracle(probe, heads, warmup=1)
    per_tok = t / max(1, int(lens[0]))
    n, tok = 1, int(lens[0])
    while n < len(lens) and tok + int(lens[n]) <= max_tokens and (tok + int(lens[n])) * per_tok <= budget_s:
        tok += int(lens[n])
        n += 1
    return n, per_tok


def run_reference(args, cfg, lens):
    """CPU arm: the reference's torch math on the host cores, bounded sample per step."""
    H, D = cfg["heads"], cfg["head_dim"]
    n_seq, _ = pick_cpu_sample(cfg, lens, H, budget_s=max(1.0, 90.0 / max(1, args.steps + args.warmup)),
                               max_tokens=131072)
    inputs = cpu_sample_inputs(cfg, lens, n_seq, H, seed=7)
    T = int(lens[:n_seq].sum())
    sec, _ = time_cpu_oracle(inputs, H, steps=args.steps, warmup=args.warmup)
    kv_bytes = 2 * T * H * D * 2
    value = kv_bytes / sec / 1e12
    cores = torch.get_num_threads()
    sample = f"first {n_seq} of {cfg['batch']} sequences ({T} tokens, {kv_bytes / 1e9:.2f} GB of KV) per step"
    line = {
        "impl": "reference", "metric": "paged_decode_kv_read_bandwidth", "value": value, "unit": "TB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": cfg["dtype"],
        "data": "synthetic", "tokens_per_s": n_seq / sec,
        "config": {"workload": "large_batch_paged_decode", "batch": cfg["batch"], "heads": H, "head_dim": D,
                   "ctx_range": [cfg["ctx_lo"], cfg["ctx_hi"]], "note": "torch CPU path, " + sample},
        "cpu_baseline": {"value": value, "unit": "TB/s", "cores": cores, "kind": "port", "sample": sample,
                         "torch": torch.__version__},
        "e2e": {"value": value, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def fill_normal(t: torch.Tensor, rows_per_chunk: int = 1 << 18):
    for r in range(0, t.size(0), rows_per_chunk):
        t[r:r + rows_per_chunk].normal_()


def run_b200(args, cfg, lens):
    import torch.distributed as dist
    import attention_impl_b200 as A
    from attention_impl_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    H, D, B = cfg["heads"], cfg["head_dim"], cfg["batch"]
    if H % world:
        raise SystemExit("heads must divide by the number of GPUs")
    Hl = H // world
    dim = Hl * D
    T = int(lens.sum())
    torch.manual_seed(1000 * cfg["seed"] + rank)

    # device-resident state: this rank's head shard of the KV pool, slot table, offsets
    Kc = torch.empty(T, dim, dtype=torch.float16, device=dev)
    Vc = torch.empty(T, dim, dtype=torch.float16, device=dev)
    fill_normal(Kc)
    fill_normal(Vc)
    gperm = torch.Generator(device=dev).manual_seed(cfg["seed"])  # same table on every rank
    ci = torch.randperm(T, device=dev, generator=gperm).to(torch.int32)
    off = lens.cumsum(0).to(torch.int32).to(dev)
    Q, K, V = (torch.randn(B, dim, device=dev, dtype=torch.float16) for _ in range(3))
    O = torch.empty_like(Q)
    chunk = A.ops.pick_chunk(B, Hl, D, T, dev)
    ws = torch.empty(A.ops.decode_workspace_bytes(B, Hl, D, T, chunk), dtype=torch.uint8, device=dev)
    kv_bytes_rank = 2 * T * Hl * D * 2
    kv_bytes_total = kv_bytes_rank * world

    def step(stages=3):
        A.paged_kv_attention_forward(Q, K, V, Kc, Vc, ci, off, Hl, return_sp=False, chunk=chunk, workspace=ws,
                                     out=O, stages=stages)

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(3, args.warmup)):
        step()
    sampler = ClockSampler(physical_gpu_index(local))
    fence()
    sampler.start()

    # ---- timed region 1: inputs resident in HBM; events split the two kernels of a step
    K_ = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(K_)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K_):
        ev[i][0].record()
        step(1)            # partial kernel (the one that streams the KV pool)
        ev[i][1].record()
        step(2)            # combine kernel
    e1.record()
    fence()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    kern_ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in ev) / K_)
    ms_per_step = total_ms / K_

    # ---- timed region 2: end to end through the public operator, per-step inputs from pinned host
    hQ, hK, hV = (x.cpu().pin_memory() for x in (Q, K, V))
    hci, hoff = ci.cpu().pin_memory(), off.cpu().pin_memory()
    hO = torch.empty(O.shape, dtype=O.dtype).pin_memory()
    h2d = sum(x.numel() * x.element_size() for x in (hQ, hK, hV, hci, hoff))
    d2h = hO.numel() * hO.element_size()

    def e2e_step():
        dQ, dK, dV = (x.to(dev, non_blocking=True) for x in (hQ, hK, hV))
        dci, doff = hci.to(dev, non_blocking=True), hoff.to(dev, non_blocking=True)
        _, _, o = A.paged_kv_attention_forward(dQ, dK, dV, Kc, Vc, dci, doff, Hl, return_sp=False)
        hO.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()   # the caller reads the result every step

    for _ in range(2):
        e2e_step()
    fence()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(K_):
        e2e_step()
    f1.record()
    fence()
    e2e_ms = max_over_ranks(f0.elapsed_time(f1)) / K_
    sampler.stop()
    sampler.join(timeout=2)

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    achieved = kv_bytes_rank / (kern_ms * 1e-3) / 1e9
    line = {
        "metric": "paged_decode_kv_read_bandwidth", "value": kv_bytes_total / (ms_per_step * 1e-3) / 1e12,
        "unit": "TB/s", "n_gpus": world, "steps": K_, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": cfg["dtype"],
        "data": "synthetic", "tokens_per_s": B / (ms_per_step * 1e-3),
        "config": {"workload": "large_batch_paged_decode", "batch": B, "heads": H, "head_dim": D,
                   "ctx_range": [cfg["ctx_lo"], cfg["ctx_hi"]], "context_tokens": T,
                   "kv_bytes_total": kv_bytes_total, "kv_bytes_per_gpu": kv_bytes_rank,
                   "sharding": f"heads/{world} per GPU, no collective", "chunk": chunk,
                   "l2": f"inputs larger than L2 ({kv_bytes_rank / 1e9:.1f} GB of KV per GPU per step)"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": DECODE_TRAFFIC_RATIO * kv_bytes_rank if DECODE_TRAFFIC_RATIO else None,
                     "kernel": "paged_decode_fast_kernel<half,half,128>", "kernel_ms": kern_ms,
                     "algorithmic_bytes_per_launch": kv_bytes_rank, "peak_source": peak_src},
        "e2e": {"value": kv_bytes_total / (e2e_ms * 1e-3) / 1e12, "unit": "TB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "note": "KV pool is device-resident state; q/k/v/slot table/offsets come from pinned host memory"},
        "gpu_launches": 2 * K_,
        "clocks": sampler.summary(),
    }
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"], line["parity"] = cpu_baseline_and_parity(A, cfg, lens, Q, K, V, Kc, Vc, ci, off, Hl,
                                                                       dev)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum per algorithmic byte of the partial kernel, from the
# ncu capture of a 5.3 GB case of this workload (profiles/paged_decode_fast_kernel_small_case_ncu.md);
# every row is read once, so traffic grows in proportion to the tokens processed.
DECODE_TRAFFIC_RATIO = 1.0017


def cpu_baseline_and_parity(A, cfg, lens, Q, K, V, Kc, Vc, ci, off, H, dev):
    """Oracle on the first sequences of the very tensors the GPU used: CPU timing + parity."""
    from oracle import attention_oracle as orc
    n_seq, per_tok = pick_cpu_sample(cfg, lens, H, budget_s=15.0, max_tokens=262144)
    T = int(lens[:n_seq].sum())
    passes = max(1, min(20, int(round(12.0 / max(1e-3, per_tok * T)))))   # ~12 s of CPU work
    rows = ci[:T].long()
    order = torch.argsort(rows)                       # compact pool in slot order
    rank_of = torch.empty_like(order)
    rank_of[order] = torch.arange(T, device=dev)
    Kc_s, Vc_s = Kc[rows[order]].cpu(), Vc[rows[order]].cpu()
    inputs = (Q[:n_seq].cpu(), K[:n_seq].cpu(), V[:n_seq].cpu(), Kc_s, Vc_s, rank_of.int().cpu(),
              off[:n_seq].cpu())
    sec, _ = time_cpu_oracle(inputs, H, steps=passes)
    _, _, O_gpu = A.paged_kv_attention_forward(Q, K, V, Kc, Vc, ci, off, H, return_sp=False)
    _, _, O32 = orc.paged_decode(*inputs, H, compute_dtype=torch.float32)
    err = (O_gpu[:n_seq].cpu().float() - O32.float()).abs().max().item()
    kv_bytes = 2 * T * H * cfg["head_dim"] * 2
    sample = f"first {n_seq} of {cfg['batch']} sequences ({T} tokens, {kv_bytes / 1e9:.2f} GB of KV), mean of {passes} passes"
    return ({"value": kv_bytes / sec / 1e12, "unit": "TB/s", "cores": torch.get_num_threads(), "kind": "port",
             "sample": sample, "seconds": sec, "torch": torch.__version__},
            {"max_abs_err_vs_fp32_oracle": err, "tolerance": 2e-3, "sequences_checked": n_seq})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="override the batch size (profiling a small case)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    args = ap.parse_args()
    cfg = dict(CFG)
    if args.batch:
        cfg["batch"] = args.batch
    lens = workload_lengths(cfg)
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            run_reference(args, cfg, lens)
        return
    run_b200(args, cfg, lens)


if __name__ == "__main__":
    main()
