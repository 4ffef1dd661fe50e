#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Default workload `large_decode` (the configuration the headline metric is quoted on): large-batch
KV-paged single-query decode, fp16 MHA, batch 256, 32 heads, head_dim 128, context lengths uniform
in [1024, 32768] (~76 GB of KV at the seeded lengths), block_size = 1 slot table = random
permutation over the whole pool, q/k/v ~ N(0,1).  At N GPUs the heads are sharded N ways (each rank
owns H/N heads of every token: its pool is [slots, (H/N)*128]); there is no collective in the data
path.  Total work is fixed, so this is strong scaling.

One step = one pass of the operator over the whole batch.  `value` is the aggregate throughput
with all inputs resident in HBM, timed with CUDA events, maximum over ranks.  `e2e` is the same
through the public Python operator with the per-step inputs in pinned HOST memory copied in, and
the output copied back, inside the timed region; for the decode workloads the KV pool itself is
device-resident state (it is the cache), as it is for any caller of the reference operator.

Other workloads (measurement of the remaining configurations, same JSON shape):
  small_decode  batch 8, ctx U[128,1024], 16384-slot pool (4 pools rotated to defeat L2)
  rope          rotary embedding on q,k [16384, 32*128] fp16, positions U[0,8191]
  prefill       packed causal prefill, bf16, 64 sequences U[256,4096], 32 heads (tensor-core path)
  fp8_split     long-context e4m3-KV decode, batch 64, ctx U[32768,131072]; each sequence's KV is
                split across the N ranks, partial rows all-gathered over NCCL, LSE-combined

The default run (1 GPU, `large_decode`) also measures short legs of `small_decode`, `rope`,
`prefill` and a reduced-batch `fp8_split` after the headline and reports them under the extra key
`secondary` of the same JSON line (each: >= 10 timed steps after warm-up, roofline fraction, parity
against the oracle); `--no-secondary` skips them.

`--impl reference` times the reference's torch CPU math (the oracle restatement: the reference's
test modules cannot be imported without a GPU and its `lm_ops`) on a bounded sample of the same
workload with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
NOMINAL_HBM_GBS = 8000.0          # the HBM3e figure the target is stated against
NOMINAL_BF16_TFLOPS = 2250.0      # dense bf16

# dram__bytes_read.sum + dram__bytes_write.sum per algorithmic byte of the decode partial kernel, from
# the ncu capture of a 5.3 GB case of the large_decode workload
# (profiles/paged_decode_mha_kernel_small_case_ncu.md); every row is read once, so the reads grow in
# proportion to the tokens processed (the partial-row writes grow with tokens / chunk: an upper bound).
DECODE_TRAFFIC_RATIO = 1.0023


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            j = json.load(open(p))
            return float(j["hbm_gbs"]), float(j["bf16_tflops"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback (earlier measurement on this pool)"


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


def seeded_lengths(n, lo, hi, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n,), generator=g)


def quantize_e4m3_per_head(x: torch.Tensor, heads: int, rows_per_chunk: int = 1 << 17):
    """[rows, heads*D] -> (e4m3 codes, float32 scales [heads]) with scale_h = absmax_h / 448, on x's device."""
    rows, dim = x.shape
    D = dim // heads
    amax = torch.zeros(heads, device=x.device)
    for r in range(0, rows, rows_per_chunk):
        amax = torch.maximum(amax, x[r:r + rows_per_chunk].view(-1, heads, D).abs().amax(dim=(0, 2)).float())
    scale = (amax / 448.0).clamp_min(1e-12)
    out = torch.empty(rows, dim, dtype=torch.float8_e4m3fn, device=x.device)
    for r in range(0, rows, rows_per_chunk):
        c = x[r:r + rows_per_chunk].float().view(-1, heads, D)
        out[r:r + rows_per_chunk] = (c / scale.view(1, heads, 1)).to(torch.float8_e4m3fn).view(-1, dim)
    return out, scale


def fill_normal(t: torch.Tensor, rows_per_chunk: int = 1 << 18):
    for r in range(0, t.size(0), rows_per_chunk):
        t[r:r + rows_per_chunk].normal_()


# ================================================================================================
# CPU legs (oracle = the reference's torch math).  The only place bench.py touches oracle/.
# ================================================================================================
def cpu_decode_inputs(lens, n_seq, heads, D, seed):
    """The first n_seq sequences of a decode workload with a compact pool (rows in slot order, so
    the gather stays random within the sample)."""
    g = torch.Generator().manual_seed(seed)
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


def time_cpu(fn, steps=1, warmup=0):
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    return (time.perf_counter() - t0) / steps


def pick_decode_sample(lens, heads, D, budget_s, max_tokens):
    """How many leading sequences fit a CPU time budget and a token cap (bounds host memory and
    set-up time), from a one-sequence probe.  Returns (n_sequences, seconds/token)."""
    from oracle import attention_oracle as orc
    probe = cpu_decode_inputs(lens, 1, heads, D, seed=99)
    t = time_cpu(lambda: orc.paged_decode(*probe, heads), warmup=1)
    per_tok = t / max(1, int(lens[0]))
    n, tok = 1, int(lens[0])
    while n < len(lens) and tok + int(lens[n]) <= max_tokens and (tok + int(lens[n])) * per_tok <= budget_s:
        tok += int(lens[n])
        n += 1
    return n, per_tok


# ================================================================================================
# Workloads
# ================================================================================================
class Workload:
    name = metric = unit = dtype = ""
    scaling = "strong"
    bound = "hbm"

    def __init__(self, args, world, rank, dev):
        self.args, self.world, self.rank, self.dev = args, world, rank, dev

    def step_split(self):               # (dominant kernel, rest) as two callables, or None
        return None

    def traffic(self):
        return None

    def cpu_baseline(self):             # (cpu_baseline dict, parity dict) or (None, None)
        return None, None

    def static_config(self):            # the keys of config() that need no device: shared with the reference arm
        return {"workload": self.name}


class LargeDecode(Workload):
    name, metric, unit, dtype = "large_decode", "paged_decode_kv_read_bandwidth", "TB/s", "f16"
    B, H, D, LO, HI, SEED = 256, 32, 128, 1024, 32768, 4
    kv_bytes_el = 2

    def lens(self):
        return seeded_lengths(self.args.batch or self.B, self.LO, self.HI, self.SEED)

    def setup(self):
        import attention_impl_b200 as A
        self.A = A
        dev, world = self.dev, self.world
        self.lens_ = self.lens()
        self.Bn = len(self.lens_)
        if self.H % world:
            raise SystemExit("heads must divide by the number of GPUs")
        self.Hl = self.H // world
        dim = self.Hl * self.D
        self.T = int(self.lens_.sum())
        torch.manual_seed(1000 * self.SEED + self.rank)
        self.Kc = torch.empty(self.T, dim, dtype=torch.float16, device=dev)
        self.Vc = torch.empty(self.T, dim, dtype=torch.float16, device=dev)
        fill_normal(self.Kc)
        fill_normal(self.Vc)
        gperm = torch.Generator(device=dev).manual_seed(self.SEED)   # same slot table on every rank
        self.ci = torch.randperm(self.T, device=dev, generator=gperm).to(torch.int32)
        self.off = self.lens_.cumsum(0).to(torch.int32).to(dev)
        self.Q, self.K, self.V = (torch.randn(self.Bn, dim, device=dev, dtype=torch.float16) for _ in range(3))
        self.O = torch.empty_like(self.Q)
        self.chunk = A.ops.pick_chunk(self.Bn, self.Hl, self.D, self.T, dev)
        self.ws = torch.empty(A.ops.decode_workspace_bytes(self.Bn, self.Hl, self.D, self.T, self.chunk),
                              dtype=torch.uint8, device=dev)

    def _call(self, stages):
        self.A.paged_kv_attention_forward(self.Q, self.K, self.V, self.Kc, self.Vc, self.ci, self.off, self.Hl,
                                          return_sp=False, chunk=self.chunk, workspace=self.ws, out=self.O,
                                          stages=stages)

    def step(self):
        self._call(3)

    def step_split(self):
        return (lambda: self._call(1)), (lambda: self._call(2))

    def e2e_setup(self):
        self.h_in = [x.cpu().pin_memory() for x in (self.Q, self.K, self.V, self.ci, self.off)]
        self.h_out = torch.empty(self.O.shape, dtype=self.O.dtype).pin_memory()
        # the public host-input operator: uploads overlapped with compute, group by group
        self.staged = self.A.HostStagedDecoder(self.Kc, self.Vc, self.Hl, self.Bn, self.T)
        return sum(x.numel() * x.element_size() for x in self.h_in), self.h_out.numel() * self.h_out.element_size()

    def e2e_step(self):
        # A decode loop knows step s+1's slot table while step s runs (this step's table plus one slot
        # per sequence), so the table of the NEXT step is uploaded during this step's kernels, into
        # the second of two device buffers; q, k, v (which depend on the previous step's output) and
        # the output cross PCIe on the critical path.  Every step still uploads a full table: the
        # copy is overlapped, not dropped.  Two host copies of the table stand for steps s and s+1.
        if not hasattr(self, "h_tables"):
            ci2, off2 = self.h_in[3].clone().pin_memory(), self.h_in[4].clone().pin_memory()
            self.h_tables = [(self.h_in[3], self.h_in[4]), (ci2, off2)]
            self.e2e_i = 0
        ci, off = self.h_tables[self.e2e_i & 1]
        self.staged(self.h_in[0], self.h_in[1], self.h_in[2], ci, off, self.h_out,
                    next_table=self.h_tables[(self.e2e_i + 1) & 1])
        self.e2e_i += 1                              # returns once the last output row is in host memory

    E2E_NOTE = "slot table of step s+1 uploaded during step s (double-buffered); q/k/v in, O out on the critical path"

    def extra_multi_gpu(self, fence, max_over_ranks):
        """Head sharding needs no collective for the attention itself; a caller that wants every rank
        to hold all heads of O adds one all-gather of [B, (H/N)*D] per rank.  Timed apart from the step."""
        import torch.distributed as dist
        if self.world == 1:
            return None
        full = torch.empty(self.world * self.O.size(0), self.O.size(1), dtype=self.O.dtype, device=self.dev)
        for _ in range(3):
            dist.all_gather_into_tensor(full, self.O)
        fence()
        n = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            dist.all_gather_into_tensor(full, self.O)
        e1.record()
        fence()
        return {"o_all_gather_ms": max_over_ranks(e0.elapsed_time(e1)) / n,
                "bytes_per_rank": self.O.numel() * self.O.element_size(),
                "note": "optional NCCL all-gather of O (rank-major head slices), not part of the timed step"}

    def units_per_step_rank(self):
        return 2.0 * self.T * self.Hl * self.D * self.kv_bytes_el

    def sequences_per_step(self):
        return self.Bn

    def launches_per_step(self):
        return 2

    def kernel_name(self):
        return "paged_decode_mha_kernel<half,half,128>"

    def traffic(self):
        return DECODE_TRAFFIC_RATIO * self.units_per_step_rank()

    LABEL = "large_batch_paged_decode"

    def static_config(self):
        return {"workload": self.LABEL, "batch": self.args.batch or self.B, "heads": self.H, "head_dim": self.D,
                "ctx_range": [self.LO, self.HI]}

    def config(self):
        per = self.units_per_step_rank()
        return {"workload": self.LABEL, "batch": self.Bn, "heads": self.H, "head_dim": self.D,
                "ctx_range": [self.LO, self.HI], "context_tokens": self.T, "kv_bytes_total": per * self.world,
                "kv_bytes_per_gpu": per, "sharding": f"heads/{self.world} per GPU, no collective",
                "chunk": self.chunk, "l2": f"inputs larger than L2 ({per / 1e9:.1f} GB of KV per GPU per step)"}

    def cpu_baseline(self):
        """Oracle on the first sequences of the very tensors the GPU used: CPU timing + parity."""
        from oracle import attention_oracle as orc
        H, D, dev = self.Hl, self.D, self.dev
        n_seq, per_tok = pick_decode_sample(self.lens_, H, D, budget_s=15.0, max_tokens=262144)
        T = int(self.lens_[:n_seq].sum())
        passes = max(1, min(20, int(round(12.0 / max(1e-3, per_tok * T)))))   # ~12 s of CPU work
        rows = self.ci[:T].long()
        order = torch.argsort(rows)                       # compact pool in slot order
        rank_of = torch.empty_like(order)
        rank_of[order] = torch.arange(T, device=dev)
        inputs = (self.Q[:n_seq].cpu(), self.K[:n_seq].cpu(), self.V[:n_seq].cpu(), self.Kc[rows[order]].cpu(),
                  self.Vc[rows[order]].cpu(), rank_of.int().cpu(), self.off[:n_seq].cpu())
        sec = time_cpu(lambda: orc.paged_decode(*inputs, H), steps=passes)
        _, _, O_gpu = self.A.paged_kv_attention_forward(self.Q, self.K, self.V, self.Kc, self.Vc, self.ci, self.off,
                                                        H, return_sp=False)
        _, _, O32 = orc.paged_decode(*inputs, H, compute_dtype=torch.float32)
        err = (O_gpu[:n_seq].cpu().float() - O32.float()).abs().max().item()
        kv_bytes = 2 * T * H * D * 2
        sample = (f"first {n_seq} of {self.Bn} sequences ({T} tokens, {kv_bytes / 1e9:.2f} GB of KV), "
                  f"mean of {passes} passes")
        return ({"value": kv_bytes / sec / 1e12, "unit": "TB/s", "cores": torch.get_num_threads(), "kind": "port",
                 "sample": sample, "seconds": sec, "torch": torch.__version__},
                {"max_abs_err_vs_fp32_oracle": err, "tolerance": 2e-3, "sequences_checked": n_seq})

    def reference_run(self, steps, warmup):
        from oracle import attention_oracle as orc
        lens = self.lens()
        n_seq, _ = pick_decode_sample(lens, self.H, self.D, budget_s=max(1.0, 90.0 / max(1, steps + warmup)),
                                      max_tokens=131072)
        inputs = cpu_decode_inputs(lens, n_seq, self.H, self.D, seed=7)
        T = int(lens[:n_seq].sum())
        sec = time_cpu(lambda: orc.paged_decode(*inputs, self.H), steps=steps, warmup=warmup)
        kv_bytes = 2 * T * self.H * self.D * 2
        sample = f"first {n_seq} of {len(lens)} sequences ({T} tokens, {kv_bytes / 1e9:.2f} GB of KV) per step"
        return kv_bytes / sec / 1e12, sec, sample, n_seq


class SmallDecode(LargeDecode):
    name = "small_decode"
    B, LO, HI, SEED = 8, 128, 1024, 1
    POOLS, SLOTS = 4, 16384

    def setup(self):
        import attention_impl_b200 as A
        self.A = A
        dev = self.dev
        self.lens_ = self.lens()
        self.Bn, self.Hl = len(self.lens_), self.H
        dim = self.H * self.D
        self.T = int(self.lens_.sum())
        torch.manual_seed(1000 * self.SEED + self.rank)
        self.pools = [(torch.randn(self.SLOTS, dim, device=dev, dtype=torch.float16),
                       torch.randn(self.SLOTS, dim, device=dev, dtype=torch.float16)) for _ in range(self.POOLS)]
        self.Kc, self.Vc = self.pools[0]
        self.ci = torch.randperm(self.SLOTS, device=dev)[: self.T].to(torch.int32)
        self.off = self.lens_.cumsum(0).to(torch.int32).to(dev)
        self.Q, self.K, self.V = (torch.randn(self.Bn, dim, device=dev, dtype=torch.float16) for _ in range(3))
        self.O = torch.empty_like(self.Q)
        self.chunk = A.ops.pick_chunk(self.Bn, self.H, self.D, self.T, dev)
        self.ws = torch.empty(A.ops.decode_workspace_bytes(self.Bn, self.H, self.D, self.T, self.chunk),
                              dtype=torch.uint8, device=dev)
        self.i = 0
        # The serving form of a step this small is a CUDA-graph launch: launching the kernels from
        # Python costs more than running them.  One single-step graph per rotated pool (used by the
        # parity check and the end-to-end leg); the step's inputs are uploaded to each arena once.
        self.graphs = []
        for Kc, Vc in self.pools:
            g = A.PagedDecodeGraph(Kc, Vc, self.Bn, self.H, self.T)
            g.host_q.copy_(self.Q.cpu()); g.host_k.copy_(self.K.cpu()); g.host_v.copy_(self.V.cpu())
            g.host_cache_indices[: self.T].copy_(self.ci.cpu()); g.host_offsets.copy_(self.off.cpu())
            g.upload()
            self.graphs.append(g)
        # The timed form: INNER decode steps back to back in ONE graph, cycling over the pools.  A
        # step is ~20 us of GPU work while one graph launch from Python costs ~35 us of host time, so
        # single-step replays would time the host, not the kernel.
        def many():
            for i in range(self.INNER):
                Kc, Vc = self.pools[i % self.POOLS]
                A.paged_kv_attention_forward(self.Q, self.K, self.V, Kc, Vc, self.ci, self.off, self.H,
                                             return_sp=False, chunk=self.chunk, workspace=self.ws, out=self.O,
                                             single_launch=False,   # (the warm-up run is eager: same kernels as the capture)
                                             tables_ready=True)     # the slot table and offsets are static
        self.many_graph = A.ops.capture_graph(dev, many)
        torch.cuda.synchronize()

    INNER = 16          # decode steps per timed graph launch
    inner_steps = INNER

    def step(self):
        self.many_graph.replay()

    def step_split(self):       # the two kernels run inside one graph launch: the step is timed as a whole
        return None

    def kernel_name(self):
        return (f"paged_decode_mha_kernel<half,half,128> + lse_combine_kernel<half> (programmatic dependent launch); "
                f"{self.INNER} decode steps per CUDA-graph launch, timed as a whole")

    def launches_per_step(self):
        return 2

    LABEL = "small_batch_paged_decode"
    E2E_NOTE = None

    def config(self):
        c = super().config()
        c.update(workload=self.LABEL, sharding="replicas only",
                 l2=f"{self.POOLS} KV pools of {self.SLOTS} slots rotated: {self.POOLS} x "
                    f"{self.units_per_step_rank() / 1e6:.0f} MB touched cyclically (> 126 MB L2)",
                 steps_per_graph_launch=self.INNER)
        return c

    def e2e_setup(self):
        # the serving-loop form: one CUDA-graph launch per step, inputs copied into its static tensors
        h2d, d2h = super().e2e_setup()
        g = self.graph = self.A.PagedDecodeGraph(self.pools[0][0], self.pools[0][1], self.Bn, self.H, self.T)
        # the step's inputs live in the graph's pinned host mirror (that is where a caller builds them)
        g.host_q.copy_(self.h_in[0]); g.host_k.copy_(self.h_in[1]); g.host_v.copy_(self.h_in[2])
        g.host_cache_indices[: self.T].copy_(self.h_in[3]); g.host_offsets.copy_(self.h_in[4])
        return h2d, d2h

    def e2e_step(self):
        g = self.graph
        g.upload()                                   # one host->device copy of q, k, v, slot table, offsets
        self.h_out.copy_(g.replay(), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def cpu_baseline(self):
        """Oracle on the whole batch (it is small): CPU timing + parity of every rotated pool's output."""
        from oracle import attention_oracle as orc
        worst = 0.0
        host = [t.cpu() for t in (self.Q, self.K, self.V)]
        ci, off = self.ci.cpu(), self.off.cpu()
        for i, (Kc, Vc) in enumerate(self.pools):
            O = self.graphs[i].replay().clone()
            torch.cuda.synchronize()
            _, _, O32 = orc.paged_decode(*host, Kc.cpu(), Vc.cpu(), ci, off, self.H, compute_dtype=torch.float32)
            worst = max(worst, (O.cpu().float() - O32.float()).abs().max().item())
        inputs = (*host, self.pools[0][0].cpu(), self.pools[0][1].cpu(), ci, off)
        sec = time_cpu(lambda: orc.paged_decode(*inputs, self.H), steps=3, warmup=1)
        kv_bytes = 2 * self.T * self.H * self.D * 2
        return ({"value": kv_bytes / sec / 1e12, "unit": "TB/s", "cores": torch.get_num_threads(), "kind": "port",
                 "sample": f"all {self.Bn} sequences ({self.T} tokens), mean of 3 passes", "seconds": sec,
                 "torch": torch.__version__},
                {"max_abs_err_vs_fp32_oracle": worst, "tolerance": 2e-3, "sequences_checked": self.Bn * self.POOLS})


class Rope(Workload):
    name, metric, unit, dtype = "rope", "rope_bandwidth", "TB/s", "f16"
    N, H, D, MAXPOS = 16384, 32, 128, 8192

    def setup(self):
        import attention_impl_b200 as A
        self.A = A
        dev = self.dev
        torch.manual_seed(2000 + self.rank)
        self.q = torch.randn(self.N, self.H * self.D, device=dev, dtype=torch.float16)
        self.k = torch.randn(self.N, self.H * self.D, device=dev, dtype=torch.float16)
        self.pos = torch.randint(0, self.MAXPOS, (self.N,), device=dev, dtype=torch.int32)
        inv = 1.0 / (10000.0 ** (torch.arange(0, self.D, 2, device=dev).float() / self.D))
        fr = torch.outer(torch.arange(self.MAXPOS, device=dev).float(), inv)
        self.cos, self.sin = fr.cos().half(), fr.sin().half()
        # An 80 us kernel between two event records is timed with its launch gap (about 10 us);
        # INNER launches back to back in one CUDA graph time the GPU instead.  The rotation is
        # applied again and again to the same 537 MB, which changes nothing for the memory system.
        self.many_graph = None           # captured at the first step

    INNER = 8
    inner_steps = INNER

    def _once(self):
        self.A.rotary_embedding_inplace(self.q, self.k, self.pos, self.cos, self.sin, self.D)

    def _many(self):
        for _ in range(self.INNER):
            self._once()

    def step(self):
        if self.many_graph is None:
            self.many_graph = self.A.ops.capture_graph(self.dev, self._many)
        self.many_graph.replay()

    def e2e_setup(self):
        self.hq, self.hk, self.hpos = self.q.cpu().pin_memory(), self.k.cpu().pin_memory(), self.pos.cpu().pin_memory()
        b = 2 * self.hq.numel() * 2
        return b + self.hpos.numel() * 4, b

    def e2e_step(self):
        dq, dk = self.hq.to(self.dev, non_blocking=True), self.hk.to(self.dev, non_blocking=True)
        dpos = self.hpos.to(self.dev, non_blocking=True)
        self.A.rotary_embedding_inplace(dq, dk, dpos, self.cos, self.sin, self.D)
        self.hq.copy_(dq, non_blocking=True)
        self.hk.copy_(dk, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def units_per_step_rank(self):
        return 4.0 * self.N * self.H * self.D * 2

    def sequences_per_step(self):
        return self.N

    def launches_per_step(self):
        return 1

    def kernel_name(self):
        return "rope_token_kernel<half2>"

    def static_config(self):
        return {"workload": "rotary_embedding", "tokens": self.N, "heads": self.H, "head_dim": self.D,
                "positions": [0, self.MAXPOS - 1]}

    def config(self):
        return {"workload": "rotary_embedding", "tokens": self.N, "heads": self.H, "head_dim": self.D,
                "positions": [0, self.MAXPOS - 1], "sharding": "replicas only",
                "l2": "537 MB read+written in place per step (> 126 MB L2)", "steps_per_graph_launch": self.INNER}

    def reference_run(self, steps, warmup):
        from oracle import attention_oracle as orc
        g = torch.Generator().manual_seed(2)
        n = 2048
        q = torch.randn(n, self.H * self.D, generator=g).half()
        k = torch.randn(n, self.H * self.D, generator=g).half()
        pos = torch.randint(0, self.MAXPOS, (n,), generator=g).int()
        cos, sin = orc.rope_tables(self.D, self.MAXPOS)
        sec = time_cpu(lambda: orc.rope(q, k, pos, cos, sin, self.D), steps=steps, warmup=warmup)
        return 4.0 * n * self.H * self.D * 2 / sec / 1e12, sec, f"{n} of {self.N} tokens per step", n

    def cpu_baseline(self):
        """Oracle on the first 2048 tokens of fresh inputs with this workload's positions: CPU timing,
        and the kernel's result on the same rows must be bit-identical."""
        from oracle import attention_oracle as orc
        n = 2048
        g = torch.Generator().manual_seed(22)
        q = torch.randn(self.N, self.H * self.D, generator=g).half()
        k = torch.randn(self.N, self.H * self.D, generator=g).half()
        pos = self.pos.cpu()
        cos, sin = self.cos.cpu(), self.sin.cpu()
        sec = time_cpu(lambda: orc.rope(q[:n], k[:n], pos[:n], cos, sin, self.D), steps=3, warmup=1)
        q_ref, k_ref = orc.rope(q[:n], k[:n], pos[:n], cos, sin, self.D)
        qd, kd = q.to(self.dev), k.to(self.dev)
        self.A.rotary_embedding_inplace(qd, kd, self.pos, self.cos, self.sin, self.D)
        same = bool(torch.equal(qd[:n].cpu(), q_ref) and torch.equal(kd[:n].cpu(), k_ref))
        return ({"value": 4.0 * n * self.H * self.D * 2 / sec / 1e12, "unit": "TB/s", "cores": torch.get_num_threads(),
                 "kind": "port", "sample": f"first {n} of {self.N} tokens, mean of 3 passes", "seconds": sec,
                 "torch": torch.__version__},
                {"bit_identical_to_oracle": same, "tokens_checked": n})


class RopeKv(Rope):
    """RoPE on q and k fused with the append of k and v to the KV pools (the step before decode)."""
    name, metric = "rope_kv", "rope_cache_write_bandwidth"

    def setup(self):
        super().setup()
        dev = self.dev
        self.v = torch.randn(self.N, self.H * self.D, device=dev, dtype=torch.float16)
        self.slots = torch.randperm(4 * self.N, device=dev)[: self.N].to(torch.int32)
        self.Kc = torch.empty(4 * self.N, self.H * self.D, device=dev, dtype=torch.float16)
        self.Vc = torch.empty_like(self.Kc)

    def _once(self):
        self.A.rope_and_cache_write(self.q, self.k, self.v, self.pos, self.cos, self.sin, self.slots, self.Kc,
                                    self.Vc, self.D)

    def e2e_setup(self):
        self.hq, self.hk, self.hv = (t.cpu().pin_memory() for t in (self.q, self.k, self.v))
        self.hpos, self.hsl = self.pos.cpu().pin_memory(), self.slots.cpu().pin_memory()
        return 3 * self.hq.numel() * 2 + 2 * self.hpos.numel() * 4, self.hq.numel() * 2

    def e2e_step(self):
        dq, dk, dv = (t.to(self.dev, non_blocking=True) for t in (self.hq, self.hk, self.hv))
        dpos, dsl = self.hpos.to(self.dev, non_blocking=True), self.hsl.to(self.dev, non_blocking=True)
        self.A.rope_and_cache_write(dq, dk, dv, dpos, self.cos, self.sin, dsl, self.Kc, self.Vc, self.D)
        self.hq.copy_(dq, non_blocking=True)          # the rotated q goes on to the attention call; k, v stay in the pools
        torch.cuda.current_stream().synchronize()

    def units_per_step_rank(self):
        # q read + written, k read + rotated k written back + stored, v read + stored
        return 7.0 * self.N * self.H * self.D * 2

    def kernel_name(self):
        return "rope_write_kv_kernel<half>"

    def cpu_baseline(self):
        return None, None

    def static_config(self):
        return dict(super().static_config(), workload="rope_and_kv_cache_append")

    def config(self):
        return dict(self.static_config(), sharding="replicas only", steps_per_graph_launch=self.INNER,
                    l2="940 MB moved per step: q, k, v rows and their pool rows (> 126 MB L2)")

    def reference_run(self, steps, warmup):
        from oracle import attention_oracle as orc
        g = torch.Generator().manual_seed(2)
        n = 2048
        q, k, v = (torch.randn(n, self.H * self.D, generator=g).half() for _ in range(3))
        pos = torch.randint(0, self.MAXPOS, (n,), generator=g).int()
        sl = torch.randperm(4 * n, generator=g)[:n]
        Kc, Vc = torch.empty(4 * n, self.H * self.D).half(), torch.empty(4 * n, self.H * self.D).half()
        cos, sin = orc.rope_tables(self.D, self.MAXPOS)

        def fn():
            q2, k2 = orc.rope(q, k, pos, cos, sin, self.D)
            Kc[sl] = k2
            Vc[sl] = v
        sec = time_cpu(fn, steps=steps, warmup=warmup)
        return 7.0 * n * self.H * self.D * 2 / sec / 1e12, sec, f"{n} of {self.N} tokens per step", n


class Prefill(Workload):
    name, metric, unit, dtype, bound = "prefill", "packed_causal_prefill_throughput", "TFLOP/s", "bf16", "tensor"
    B, H, D, LO, HI, SEED = 64, 32, 128, 256, 4096, 3

    def setup(self):
        import attention_impl_b200 as A
        self.A = A
        dev = self.dev
        self.lens_ = seeded_lengths(self.args.batch or self.B, self.LO, self.HI, self.SEED)
        self.T = int(self.lens_.sum())
        torch.manual_seed(3000 + self.rank)
        self.off = self.lens_.cumsum(0).to(torch.int32).to(dev)
        self.Q, self.K, self.V = (torch.randn(self.T, self.H * self.D, device=dev, dtype=torch.bfloat16)
                                  for _ in range(3))
        self.maxlen = int(self.lens_.max())
        self.flag = torch.zeros(1, dtype=torch.int32, device=dev)

    def step(self):
        self.out = self.A.paged_attention_forward(self.Q, self.K, self.V, self.off, self.H, return_sp=False,
                                                  max_seqlen=self.maxlen, err_flag=self.flag)[2]

    def e2e_setup(self):
        self.h_in = [x.cpu().pin_memory() for x in (self.Q, self.K, self.V, self.off)]
        self.h_out = torch.empty(self.Q.shape, dtype=self.Q.dtype).pin_memory()
        return sum(x.numel() * x.element_size() for x in self.h_in), self.h_out.numel() * 2

    def e2e_step(self):
        dQ, dK, dV, doff = (x.to(self.dev, non_blocking=True) for x in self.h_in)
        o = self.A.paged_attention_forward(dQ, dK, dV, doff, self.H, return_sp=False, max_seqlen=self.maxlen)[2]
        self.h_out.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def units_per_step_rank(self):
        l = self.lens_.double()
        return 4.0 * self.D * self.H * float((l * (l + 1) / 2).sum())

    def sequences_per_step(self):
        return self.T

    def launches_per_step(self):
        return 1

    def kernel_name(self):
        return "prefill_tc2p_kernel<bf16>"

    def static_config(self):
        return {"workload": "packed_varlen_causal_prefill", "sequences": self.args.batch or self.B, "heads": self.H,
                "head_dim": self.D, "len_range": [self.LO, self.HI]}

    def config(self):
        return {"workload": "packed_varlen_causal_prefill", "sequences": len(self.lens_), "heads": self.H,
                "head_dim": self.D, "len_range": [self.LO, self.HI], "tokens": self.T,
                "flops_per_step": self.units_per_step_rank(), "sharding": "replicas only",
                "l2": f"Q,K,V,O = {4 * self.T * self.H * self.D * 2 / 1e9:.1f} GB per step (> 126 MB L2)"}

    def cpu_baseline(self):
        from oracle import attention_oracle as orc
        n_seq = 2
        T = int(self.lens_[:n_seq].sum())
        Q, K, V = (x[:T].cpu() for x in (self.Q, self.K, self.V))
        off = self.off[:n_seq].cpu()
        sec = time_cpu(lambda: orc.packed_prefill(Q, K, V, off, self.H))
        O32 = orc.packed_prefill(Q, K, V, off, self.H, compute_dtype=torch.float32, out_dtype=torch.float32)
        self.step()
        torch.cuda.synchronize()
        err = (self.out[:T].cpu().float() - O32).abs().max().item()
        # the same launch with fp32 output: the kernel's own error without the bf16 rounding of O
        o32 = self.A.paged_attention_forward(self.Q, self.K, self.V, self.off, self.H, return_sp=False,
                                             max_seqlen=self.maxlen, out_dtype=torch.float32, err_flag=self.flag)[2]
        e32 = (o32[:T].cpu() - O32).abs().flatten()
        l = self.lens_[:n_seq].double()
        fl = 4.0 * self.D * self.H * float((l * (l + 1) / 2).sum())
        return ({"value": fl / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                 "sample": f"first {n_seq} of {len(self.lens_)} sequences ({T} tokens), causal flops counted",
                 "seconds": sec, "torch": torch.__version__},
                {"max_abs_err_fp32_out_vs_fp32_oracle": e32.max().item(), "tolerance_fp32_out": 2e-3,
                 "p999_abs_err_fp32_out": torch.quantile(e32[::13], 0.999).item(), "mean_abs_err_fp32_out": e32.mean().item(),
                 "max_abs_err_bf16_out_vs_fp32_oracle": err, "tolerance_bf16_out": 1.6e-2,
                 "sequences_checked": n_seq, "kernel_flag": int(self.flag.item())})

    def reference_run(self, steps, warmup):
        from oracle import attention_oracle as orc
        lens = seeded_lengths(self.B, self.LO, self.HI, self.SEED)[:1].clamp(max=2048)
        T = int(lens.sum())
        g = torch.Generator().manual_seed(3)
        Q, K, V = (torch.randn(T, self.H * self.D, generator=g).bfloat16() for _ in range(3))
        off = lens.cumsum(0).int()
        sec = time_cpu(lambda: orc.packed_prefill(Q, K, V, off, self.H), steps=steps, warmup=warmup)
        l = lens.double()
        fl = 4.0 * self.D * self.H * float((l * (l + 1) / 2).sum())
        return fl / sec / 1e12, sec, f"1 of {self.B} sequences ({T} tokens) per step", T


class PagedPrefill(Prefill):
    """Chunked prefill through the slot table: the last <= 512 tokens of every sequence attend to the
    whole sequence (prefix + chunk), whose K/V rows are scattered over the pools."""
    name, metric = "paged_prefill", "chunked_prefill_throughput"
    CHUNK = 512

    def setup(self):
        import attention_impl_b200 as A
        self.A = A
        dev = self.dev
        self.lens_ = seeded_lengths(self.args.batch or self.B, self.LO, self.HI, self.SEED)
        self.qlens_ = self.lens_.clamp(max=self.CHUNK)
        self.T, self.Tq = int(self.lens_.sum()), int(self.qlens_.sum())
        torch.manual_seed(3100 + self.rank)
        self.Q = torch.randn(self.Tq, self.H * self.D, device=dev, dtype=torch.bfloat16)
        self.K, self.V = (torch.randn(self.T, self.H * self.D, device=dev, dtype=torch.bfloat16) for _ in range(2))
        self.slots = torch.randperm(self.T, device=dev).to(torch.int32)
        self.kvo = self.lens_.cumsum(0).to(torch.int32).to(dev)
        self.qo = self.qlens_.cumsum(0).to(torch.int32).to(dev)
        self.flag = torch.zeros(1, dtype=torch.int32, device=dev)

    def step(self):
        self.out = self.A.paged_prefill_attention(self.Q, self.K, self.V, self.slots, self.kvo, self.qo, self.H,
                                                  max_q_len=int(self.qlens_.max()), max_kv_len=int(self.lens_.max()),
                                                  err_flag=self.flag)

    def e2e_setup(self):
        # the pools are device-resident state (the cache); the chunk's queries and the tables come from the host
        self.h_in = [x.cpu().pin_memory() for x in (self.Q, self.slots, self.kvo, self.qo)]
        self.h_out = torch.empty(self.Q.shape, dtype=self.Q.dtype).pin_memory()
        return sum(x.numel() * x.element_size() for x in self.h_in), self.h_out.numel() * 2

    def e2e_step(self):
        dQ, dsl, dkvo, dqo = (x.to(self.dev, non_blocking=True) for x in self.h_in)
        o = self.A.paged_prefill_attention(dQ, self.K, self.V, dsl, dkvo, dqo, self.H, max_q_len=int(self.qlens_.max()),
                                           max_kv_len=int(self.lens_.max()))
        self.h_out.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def _flops(self, l, q):
        # visible (query, key) pairs: row i of a chunk sees kv_len - q_len + i + 1 keys
        return 4.0 * self.D * self.H * float((q * (l - q) + q * (q + 1) / 2).sum())

    def units_per_step_rank(self):
        return self._flops(self.lens_.double(), self.qlens_.double())

    def sequences_per_step(self):
        return self.Tq

    def kernel_name(self):
        return "paged_prefill_tc_kernel<bf16>"

    def static_config(self):
        return {"workload": "chunked_prefill_through_slot_table", "sequences": self.args.batch or self.B,
                "heads": self.H, "head_dim": self.D, "kv_len_range": [self.LO, self.HI], "chunk": self.CHUNK}

    def config(self):
        return {"workload": "chunked_prefill_through_slot_table", "sequences": len(self.lens_), "heads": self.H,
                "head_dim": self.D, "kv_len_range": [self.LO, self.HI], "chunk": self.CHUNK, "query_tokens": self.Tq,
                "kv_tokens": self.T, "flops_per_step": self.units_per_step_rank(), "sharding": "replicas only",
                "l2": f"K/V pools = {2 * self.T * self.H * self.D * 2 / 1e9:.1f} GB per step (> 126 MB L2)"}

    def cpu_baseline(self):
        from oracle import attention_oracle as orc
        n_seq = 2
        T, Tq = int(self.lens_[:n_seq].sum()), int(self.qlens_[:n_seq].sum())
        Q, K, V, sl = self.Q[:Tq].cpu(), self.K.cpu(), self.V.cpu(), self.slots[:T].cpu()
        kvo, qo = self.kvo[:n_seq].cpu(), self.qo[:n_seq].cpu()
        sec = time_cpu(lambda: orc.paged_prefill(Q, K, V, sl, kvo, qo, self.H))
        O32 = orc.paged_prefill(Q, K, V, sl, kvo, qo, self.H, compute_dtype=torch.float32, out_dtype=torch.float32)
        self.step()
        torch.cuda.synchronize()
        err = (self.out[:Tq].cpu().float() - O32).abs().max().item()
        fl = self._flops(self.lens_[:n_seq].double(), self.qlens_[:n_seq].double())
        return ({"value": fl / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                 "sample": f"first {n_seq} of {len(self.lens_)} sequences ({Tq} query tokens over {T} cached tokens)",
                 "seconds": sec, "torch": torch.__version__},
                {"max_abs_err_vs_fp32_oracle": err, "tolerance": 1.6e-2, "sequences_checked": n_seq,
                 "kernel_flag": int(self.flag.item())})

    def reference_run(self, steps, warmup):
        from oracle import attention_oracle as orc
        lens = seeded_lengths(self.B, self.LO, self.HI, self.SEED)[:1].clamp(max=2048)
        qlens = lens.clamp(max=self.CHUNK)
        T, Tq = int(lens.sum()), int(qlens.sum())
        g = torch.Generator().manual_seed(3)
        Q = torch.randn(Tq, self.H * self.D, generator=g).bfloat16()
        K, V = (torch.randn(T, self.H * self.D, generator=g).bfloat16() for _ in range(2))
        sl = torch.randperm(T, generator=g).int()
        sec = time_cpu(lambda: orc.paged_prefill(Q, K, V, sl, lens.cumsum(0).int(), qlens.cumsum(0).int(), self.H),
                       steps=steps, warmup=warmup)
        return self._flops(lens.double(), qlens.double()) / sec / 1e12, sec, \
            f"1 of {self.B} sequences ({Tq} query tokens over {T} cached tokens) per step", Tq


class GqaDecode(Workload):
    """Grouped-query paged decode (not in the reference): 32 query heads over 32 / group KV heads
    (`--gqa-group`, default 4), fp16 or e4m3 pools (`--gqa-kv`)."""
    name, metric, unit, dtype = "gqa_decode", "paged_decode_kv_read_bandwidth", "TB/s", "f16"
    B, H, HKV, D, LO, HI, SEED = 64, 32, 8, 128, 1024, 32768, 4

    def setup(self):
        import attention_impl_b200 as A
        self.A = A
        dev = self.dev
        self.HKV = self.H // self.args.gqa_group
        self.fp8 = self.args.gqa_kv == "e4m3"
        self.kv_el = 1 if self.fp8 else 2
        self.lens_ = seeded_lengths(self.args.batch or self.B, self.LO, self.HI, self.SEED)
        self.Bn, self.T = len(self.lens_), int(self.lens_.sum())
        torch.manual_seed(4100 + self.rank)
        kvdim = self.HKV * self.D
        self.Kc = torch.empty(self.T, kvdim, dtype=torch.float16, device=dev)
        self.Vc = torch.empty(self.T, kvdim, dtype=torch.float16, device=dev)
        fill_normal(self.Kc)
        fill_normal(self.Vc)
        self.kw = {}
        if self.fp8:       # per-head absmax scales, as in the long-context workload
            self.Kc, ks = quantize_e4m3_per_head(self.Kc, self.HKV)
            self.Vc, vs = quantize_e4m3_per_head(self.Vc, self.HKV)
            self.kw = dict(k_scale=ks, v_scale=vs)
        self.ci = torch.randperm(self.T, device=dev).to(torch.int32)
        self.off = self.lens_.cumsum(0).to(torch.int32).to(dev)
        self.Q = torch.randn(self.Bn, self.H * self.D, device=dev, dtype=torch.float16)
        self.K, self.V = (torch.randn(self.Bn, kvdim, device=dev, dtype=torch.float16) for _ in range(2))
        self.O = torch.empty_like(self.Q)
        self.chunk = A.ops.pick_chunk(self.Bn, self.HKV, self.D, self.T, dev, group=self.H // self.HKV,
                                      kv_dtype=3 if self.fp8 else 0)
        self.ws = torch.empty(A.ops.decode_workspace_bytes(self.Bn, self.H, self.D, self.T, self.chunk),
                              dtype=torch.uint8, device=dev)

    def _call(self, stages):
        self.A.paged_kv_attention_forward(self.Q, self.K, self.V, self.Kc, self.Vc, self.ci, self.off, self.H,
                                          return_sp=False, chunk=self.chunk, workspace=self.ws, out=self.O,
                                          stages=stages, **self.kw)

    def step(self):
        self._call(3)

    def step_split(self):
        return (lambda: self._call(1)), (lambda: self._call(2))

    def e2e_setup(self):
        self.h_in = [x.cpu().pin_memory() for x in (self.Q, self.K, self.V, self.ci, self.off)]
        self.h_out = torch.empty(self.O.shape, dtype=self.O.dtype).pin_memory()
        return sum(x.numel() * x.element_size() for x in self.h_in), self.h_out.numel() * 2

    def e2e_step(self):
        dQ, dK, dV, dci, doff = (x.to(self.dev, non_blocking=True) for x in self.h_in)
        o = self.A.paged_kv_attention_forward(dQ, dK, dV, self.Kc, self.Vc, dci, doff, self.H, return_sp=False,
                                              max_context_len=int(self.lens_.max()), **self.kw)[2]
        self.h_out.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def units_per_step_rank(self):
        return 2.0 * self.T * self.HKV * self.D * self.kv_el

    def sequences_per_step(self):
        return self.Bn

    def launches_per_step(self):
        return 2

    def kernel_name(self):
        g = self.H // self.HKV
        return f"paged_decode_gqa_mma_e4m3_kernel<half,{g}>" if self.fp8 else f"paged_decode_gqa_mma_kernel<half,{g}>"

    def static_config(self):
        return {"workload": "grouped_query_paged_decode", "batch": self.args.batch or self.B, "heads": self.H,
                "kv_heads": self.H // self.args.gqa_group, "kv_dtype": self.args.gqa_kv, "head_dim": self.D,
                "ctx_range": [self.LO, self.HI]}

    def config(self):
        per = self.units_per_step_rank()
        return dict(self.static_config(), context_tokens=self.T, kv_bytes_total=per, sharding="replicas only",
                    chunk=self.chunk, l2=f"inputs larger than L2 ({per / 1e9:.1f} GB of KV per step)")

    def _sample(self, n_seq):
        from oracle import attention_oracle as orc
        T = int(self.lens_[:n_seq].sum())
        rows = self.ci[:T].long()
        order = torch.argsort(rows)
        rank_of = torch.empty_like(order)
        rank_of[order] = torch.arange(T, device=self.dev)
        Kc, Vc = self.Kc[rows[order]].cpu(), self.Vc[rows[order]].cpu()
        Q, K, V = self.Q[:n_seq].cpu(), self.K[:n_seq].cpu(), self.V[:n_seq].cpu()
        if self.fp8:       # the oracle runs on the dequantised pools
            Kc = orc.dequantize_e4m3_per_head(Kc, self.kw["k_scale"].cpu(), self.HKV)
            Vc = orc.dequantize_e4m3_per_head(Vc, self.kw["v_scale"].cpu(), self.HKV)
            Q, K, V = Q.float(), K.float(), V.float()
        return (Q, K, V, Kc, Vc, rank_of.int().cpu(), self.off[:n_seq].cpu()), T

    def cpu_baseline(self):
        from oracle import attention_oracle as orc
        n_seq = 2
        inputs, T = self._sample(n_seq)
        sec = time_cpu(lambda: orc.paged_decode(*inputs, self.H))
        O32 = orc.paged_decode(*inputs, self.H, compute_dtype=torch.float32)[2]
        self.step()
        torch.cuda.synchronize()
        diff = self.O[:n_seq].cpu().float() - O32.float()
        kv_bytes = 2 * T * self.HKV * self.D * self.kv_el
        par = ({"rel_err": (diff.norm() / O32.float().norm()).item(), "tolerance": 2e-2} if self.fp8
               else {"max_abs_err_vs_fp32_oracle": diff.abs().max().item(), "tolerance": 2e-3})
        return ({"value": kv_bytes / sec / 1e12, "unit": "TB/s", "cores": torch.get_num_threads(), "kind": "port",
                 "sample": f"first {n_seq} of {self.Bn} sequences ({T} tokens)", "seconds": sec,
                 "torch": torch.__version__}, dict(par, sequences_checked=n_seq))

    def reference_run(self, steps, warmup):
        from oracle import attention_oracle as orc
        g = torch.Generator().manual_seed(7)
        T = 16384
        Q = torch.randn(1, self.H * self.D, generator=g).half()
        K, V = (torch.randn(1, self.HKV * self.D, generator=g).half() for _ in range(2))
        Kc, Vc = (torch.randn(T, self.HKV * self.D, generator=g).half() for _ in range(2))
        ci, off = torch.randperm(T, generator=g).int(), torch.tensor([T]).int()
        sec = time_cpu(lambda: orc.paged_decode(Q, K, V, Kc, Vc, ci, off, self.H), steps=steps, warmup=warmup)
        return 2.0 * T * self.HKV * self.D * 2 / sec / 1e12, sec, f"1 sequence of {T} tokens per step", 1


class Fp8Split(Workload):
    name, metric, unit, dtype = "fp8_split", "paged_decode_kv_read_bandwidth", "TB/s", "e4m3"
    B, H, D, LO, HI, SEED = 64, 32, 128, 32768, 131072, 5
    GEN_ROWS = 1 << 17          # rows generated per chunk (1 GiB of fp16 at 4096 columns)

    def _gen_chunk(self, which, idx, rows, dim):
        """Chunk `idx` of this rank's K (which=0) or V (which=1) values, ~ N(0,1), reproducible."""
        g = torch.Generator(device=self.dev).manual_seed(((5000 + self.rank) * 2 + which) * 100003 + idx)
        return torch.randn(rows, dim, device=self.dev, dtype=torch.float16, generator=g)

    def _quantised_pool(self, which, dim):
        """K or V ~ N(0,1), quantised to e4m3 with per-head absmax scales (scale_h = absmax_h / 448, the
        absmax taken over the whole cache, i.e. over all ranks' pools): pass 1 finds the absmax, pass 2
        regenerates the same values chunk by chunk and stores rn_e4m3(x / scale_h)."""
        H, D, T = self.H, self.D, self.T
        amax = torch.zeros(H, device=self.dev)
        chunks = [(i, a, min(self.GEN_ROWS, T - a)) for i, a in enumerate(range(0, T, self.GEN_ROWS))]
        for i, a, n in chunks:
            x = self._gen_chunk(which, i, n, dim)
            amax = torch.maximum(amax, x.view(n, H, D).abs().amax(dim=(0, 2)).float())
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        scale = (amax / 448.0).clamp_min(1e-12)
        pool = torch.empty(T, dim, dtype=torch.float8_e4m3fn, device=self.dev)
        for i, a, n in chunks:
            x = self._gen_chunk(which, i, n, dim).float().view(n, H, D)
            pool[a:a + n] = (x / scale.view(1, H, 1)).to(torch.float8_e4m3fn).view(n, dim)
        return pool, scale

    def setup(self):
        import attention_impl_b200 as A
        from attention_impl_b200 import dist as adist
        self.A, self.adist = A, adist
        dev, G, r = self.dev, self.world, self.rank
        self.lens_ = seeded_lengths(self.args.batch or self.B, self.LO, self.HI, self.SEED)
        self.Bn = len(self.lens_)
        lo, hi = adist.kv_split_bounds(self.lens_, G, r)
        self.llens = hi - lo                                   # this rank's slice of every sequence
        self.T = int(self.llens.sum())
        self.T_all = int(self.lens_.sum())
        dim = self.H * self.D
        torch.manual_seed(5000 + r)
        self.Kc, self.ks = self._quantised_pool(0, dim)
        self.Vc, self.vs = self._quantised_pool(1, dim)
        self.ci = torch.randperm(self.T, device=dev).to(torch.int32)
        self.off = self.llens.cumsum(0).to(torch.int32).to(dev)
        g = torch.Generator(device=dev).manual_seed(self.SEED)   # q, k, v replicated on every rank
        self.Q, self.K, self.V = (torch.randn(self.Bn, dim, device=dev, dtype=torch.float16, generator=g)
                                  for _ in range(3))
        self.chunk = A.ops.pick_chunk(self.Bn, self.H, self.D, self.T, dev)
        self.xchg = None
        self.graphed = False
        if self.args.exchange in ("peer", "peer_graph", "peer_unfused") and G > 1:
            # "peer": three launches (the combines push and wait themselves); "peer_unfused": five
            self.xchg = adist.KvSplitExchange(self.Bn, self.H, self.D, dev,
                                              fused=self.args.exchange != "peer_unfused")
            ref = adist.kv_split_decode(self.Q, self.K, self.V, self.Kc, self.Vc, self.ci, self.off, self.H,
                                        k_scale=self.ks, v_scale=self.vs, chunk=self.chunk)
            for _ in range(3):      # both buffer halves and the counter arithmetic
                got = self.xchg.decode(self.Q, self.K, self.V, self.Kc, self.Vc, self.ci, self.off,
                                       k_scale=self.ks, v_scale=self.vs, chunk=self.chunk)
            torch.cuda.synchronize()
            if int(self.xchg.err_flag.item()) != 0 or not torch.equal(got, ref):
                raise SystemExit(f"rank {r}: peer exchange differs from the NCCL path "
                                 f"(flag {int(self.xchg.err_flag.item())}, "
                                 f"max diff {(got.float() - ref.float()).abs().max().item()})")
            if self.args.exchange == "peer_graph":      # the whole step replayed from a CUDA graph per buffer half
                self.xchg.capture(self.Q, self.K, self.V, self.Kc, self.Vc, self.ci, self.off,
                                  k_scale=self.ks, v_scale=self.vs, chunk=self.chunk)
                for _ in range(3):
                    got = self.xchg.replay()
                torch.cuda.synchronize()
                if int(self.xchg.err_flag.item()) != 0 or not torch.equal(got, ref):
                    raise SystemExit(f"rank {r}: graph replay of the peer exchange differs from the NCCL path")
                self.graphed = True

    def step(self):
        if self.graphed:
            self.out = self.xchg.replay()
            return
        if self.xchg is not None:
            self.out = self.xchg.decode(self.Q, self.K, self.V, self.Kc, self.Vc, self.ci, self.off,
                                        k_scale=self.ks, v_scale=self.vs, chunk=self.chunk)
            return
        self.out = self.adist.kv_split_decode(self.Q, self.K, self.V, self.Kc, self.Vc, self.ci, self.off, self.H,
                                              k_scale=self.ks, v_scale=self.vs, chunk=self.chunk)

    E2E_NOTE = ("slot table of step s+1 uploaded during step s on a second stream (double-buffered); q/k/v and the "
                "offsets in, O out on the critical path")

    def e2e_setup(self):
        self.h_in = [x.cpu().pin_memory() for x in (self.Q, self.K, self.V, self.ci, self.off)]
        self.h_out = torch.empty(self.Q.shape, dtype=self.Q.dtype).pin_memory()
        # a decode loop knows the next step's slot table one step ahead: it goes up while this step runs
        self.d_ci = [torch.empty_like(self.ci) for _ in range(2)]
        self.up_stream = torch.cuda.Stream(device=self.dev)
        self.up_done = [torch.cuda.Event() for _ in range(2)]
        self.e2e_i = 0
        self.d_ci[0].copy_(self.h_in[3], non_blocking=True)
        self.up_done[0].record()
        return sum(x.numel() * x.element_size() for x in self.h_in), self.h_out.numel() * 2

    def e2e_step(self):
        cur, nxt = self.e2e_i & 1, (self.e2e_i + 1) & 1
        main = torch.cuda.current_stream()
        dQ, dK, dV = (x.to(self.dev, non_blocking=True) for x in self.h_in[:3])
        doff = self.h_in[4].to(self.dev, non_blocking=True)
        main.wait_event(self.up_done[cur])                 # this step's table, uploaded during the previous step
        self.up_stream.wait_stream(main)                   # buffer `nxt` was read by step s-1, which has completed
        with torch.cuda.stream(self.up_stream):
            self.d_ci[nxt].copy_(self.h_in[3], non_blocking=True)
            self.up_done[nxt].record()
        o = self.adist.kv_split_decode(dQ, dK, dV, self.Kc, self.Vc, self.d_ci[cur], doff, self.H, k_scale=self.ks,
                                       v_scale=self.vs)
        self.h_out.copy_(o, non_blocking=True)
        main.synchronize()
        self.e2e_i += 1

    def units_per_step_rank(self):
        return 2.0 * self.T * self.H * self.D * 1

    def sequences_per_step(self):
        return self.Bn

    def launches_per_step(self):
        if self.xchg is not None:
            return 3 if self.xchg.fused else 5      # partial, combine+push, wait+combine | partial, combine, push, wait, combine
        return 3 + (1 if self.world > 1 else 0)     # partial, local combine, (all-gather), final combine

    def kernel_name(self):
        return "paged_decode_mha_kernel<half,e4m3,128>"

    def static_config(self):
        return {"workload": "long_context_fp8_kv_paged_decode", "batch": self.args.batch or self.B, "heads": self.H,
                "head_dim": self.D, "ctx_range": [self.LO, self.HI]}

    def config(self):
        per = self.units_per_step_rank()
        return {"workload": "long_context_fp8_kv_paged_decode", "batch": self.Bn, "heads": self.H,
                "head_dim": self.D, "ctx_range": [self.LO, self.HI], "context_tokens": self.T_all,
                "kv_bytes_total": 2.0 * self.T_all * self.H * self.D, "kv_bytes_per_gpu": per,
                "sharding": f"each sequence's KV split {self.world} ways; [B,H,D+2] fp32 partials exchanged by "
                            + (("peer stores over NVLink" + (", step replayed from a CUDA graph" if self.graphed else ""))
                               if self.xchg is not None else "NCCL all-gather")
                            + " + LSE combine", "chunk": self.chunk,
                "l2": f"inputs larger than L2 ({per / 1e9:.1f} GB of KV per GPU per step)"}

    collective_cpu_leg = True      # cpu_baseline() is called on every rank (it gathers one sequence to rank 0)

    def extra_multi_gpu(self, fence, max_over_ranks):
        """Every step of the KV split ends with an exchange, so the ranks run in lock step and a step
        lasts as long as the slowest rank's local work.  This times the local part alone (partial
        kernel + local combine, no exchange) on every rank and reports the spread."""
        import torch.distributed as dist
        if self.world == 1:
            return None
        call = lambda: self.A.paged_decode_partial(self.Q, self.Kc, self.Vc, self.ci, self.off, self.H,
                                                   k_scale=self.ks, v_scale=self.vs, chunk=self.chunk)
        for _ in range(3):
            call()
        fence()
        n = 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            call()
        e1.record()
        fence()
        mine = torch.tensor([e0.elapsed_time(e1) / n], device=self.dev)
        allms = [torch.zeros_like(mine) for _ in range(self.world)]
        dist.all_gather(allms, mine)
        ms = [round(float(x), 4) for x in allms]
        return {"local_ms_per_rank": ms, "local_ms_min": min(ms), "local_ms_max": max(ms),
                "note": "partial kernel + local combine only, no exchange; the lock-stepped step cannot be "
                        "shorter than local_ms_max"}

    def cpu_baseline(self):
        """The shortest sequence of the batch, whole (>= 32768 tokens): its e4m3 rows are collected
        from every rank's pool in token order on rank 0, dequantised on the host with the per-head
        scales, and the oracle runs on them (timed: the CPU baseline) -- the pin of this path: <= 2e-2
        relative against the reference math on dequantised KV."""
        from oracle import attention_oracle as orc
        import torch.distributed as dist
        H, D, dev, G = self.H, self.D, self.dev, self.world
        b = int(torch.argmin(self.lens_))
        beg = int(self.off[b - 1]) if b else 0
        end = int(self.off[b])
        rows = self.ci[beg:end].long()
        k8 = self.Kc[rows].view(torch.uint8)
        v8 = self.Vc[rows].view(torch.uint8)
        self.step()
        torch.cuda.synchronize()
        o_gpu = self.out[b:b + 1].cpu().float()
        if G > 1:
            n_loc = torch.tensor([end - beg], device=dev)
            sizes = [torch.zeros_like(n_loc) for _ in range(G)]
            dist.all_gather(sizes, n_loc)
            sizes = [int(x) for x in sizes]
            cap = max(sizes)
            parts = []
            for t in (k8, v8):
                pad = torch.zeros(cap, t.size(1), dtype=torch.uint8, device=dev)
                pad[: t.size(0)] = t
                out = torch.empty(G * cap, t.size(1), dtype=torch.uint8, device=dev)
                dist.all_gather_into_tensor(out, pad)
                parts.append(torch.cat([out[r * cap: r * cap + sizes[r]] for r in range(G)]))   # rank order = token order
            k8, v8 = parts
            if self.rank != 0:
                return None, None
        n = k8.size(0)
        assert n == int(self.lens_[b])
        ks, vs = self.ks.cpu(), self.vs.cpu()
        K8, V8 = k8.cpu().view(torch.float8_e4m3fn), v8.cpu().view(torch.float8_e4m3fn)
        code_max = int(torch.maximum(K8.float().abs().max(), V8.float().abs().max()))
        q, k, v = (t[b:b + 1].cpu().float() for t in (self.Q, self.K, self.V))
        ci, off = torch.arange(n, dtype=torch.int32), torch.tensor([n], dtype=torch.int32)

        def fn():   # dequantisation is part of the CPU path
            Kd = orc.dequantize_e4m3_per_head(K8, ks, H)
            Vd = orc.dequantize_e4m3_per_head(V8, vs, H)
            return orc.paged_decode(q, k, v, Kd, Vd, ci, off, H)[2]
        o_ref = fn()
        sec = time_cpu(fn, steps=2)
        err = o_gpu - o_ref
        kv_bytes = 2.0 * n * H * D
        return ({"value": kv_bytes / sec / 1e12, "unit": "TB/s", "cores": torch.get_num_threads(), "kind": "port",
                 "sample": f"the shortest of {self.Bn} sequences, whole ({n} tokens, {kv_bytes / 1e9:.2f} GB of e4m3 KV, "
                           f"dequantised on the host), mean of 2 passes", "seconds": sec, "torch": torch.__version__},
                {"rel_err": (err.norm() / o_ref.norm()).item(), "max_abs_err_over_max_abs_ref":
                 (err.abs().max() / o_ref.abs().max()).item(), "tolerance": 2e-2, "sequences_checked": 1,
                 "tokens_checked": n, "largest_e4m3_magnitude_in_sample": code_max,
                 "kv": "N(0,1) quantised with per-head absmax scales (absmax / 448)",
                 "gathered_from_ranks": G})

    def reference_run(self, steps, warmup):
        from oracle import attention_oracle as orc
        g = torch.Generator().manual_seed(5)
        T, H, D = 32768, self.H, self.D
        Q, K, V = (torch.randn(1, H * D, generator=g).half() for _ in range(3))
        Kc, Vc = (torch.randn(T, H * D, generator=g) for _ in range(2))
        K8, ks = orc.quantize_e4m3_per_head(Kc, H)
        V8, vs = orc.quantize_e4m3_per_head(Vc, H)
        ci = torch.randperm(T, generator=g).int()
        off = torch.tensor([T]).int()

        def fn():   # oracle on dequantised KV, dequantisation included (it is part of the path)
            Kd = orc.dequantize_e4m3_per_head(K8, ks, H)
            Vd = orc.dequantize_e4m3_per_head(V8, vs, H)
            orc.paged_decode(Q.float(), K.float(), V.float(), Kd, Vd, ci, off, H)
        sec = time_cpu(fn, steps=steps, warmup=warmup)
        return 2.0 * T * H * D / sec / 1e12, sec, f"1 sequence of {T} tokens per step", 1


WORKLOADS = {w.name: w for w in (LargeDecode, SmallDecode, Rope, RopeKv, Prefill, PagedPrefill, GqaDecode, Fp8Split)}


# ================================================================================================
# Drivers
# ================================================================================================
def run_reference(args, W):
    w = W(args, 1, 0, None)
    value, sec, sample, seqs = w.reference_run(args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": W.metric, "value": value, "unit": W.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": W.scaling, "vs_baseline": None, "dtype": W.dtype, "data": "synthetic",
        "tokens_per_s": seqs / sec,
        "config": dict(w.static_config(), note="torch CPU path (oracle restatement of the reference's test-side "
                                                "math), " + sample),
        "cpu_baseline": {"value": value, "unit": W.unit, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample, "torch": torch.__version__},
        "e2e": {"value": value, "unit": W.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def measure(w, W, K_, warm, world, rank, local, fence, max_over_ranks, with_e2e=True):
    """Warm-up, the two timed regions and the roofline arithmetic for one workload; returns the JSON
    pieces (on every rank; the values are maxima over ranks)."""
    for _ in range(warm):
        w.step()
    sampler = ClockSampler(physical_gpu_index(local))
    fence()
    sampler.start()

    # ---- timed region 1: inputs resident in HBM; events isolate the dominant kernel of a step
    split = w.step_split()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(K_)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K_):
        ev[i][0].record()
        if split:
            split[0]()         # the kernel that moves the bytes / does the flops
            ev[i][1].record()
            split[1]()
        else:
            w.step()
            ev[i][1].record()
    e1.record()
    fence()
    inner = getattr(w, "inner_steps", 1)        # decode steps inside one call of w.step()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    kern_ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in ev) / K_) / inner
    ms_per_step = total_ms / (K_ * inner)

    # ---- timed region 2: end to end through the public operator, per-step inputs from pinned host
    e2e = None
    if with_e2e:
        h2d, d2h = w.e2e_setup()
        for _ in range(2):
            w.e2e_step()
        fence()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(K_):
            w.e2e_step()
        f1.record()
        fence()
        e2e_ms = max_over_ranks(f0.elapsed_time(f1)) / K_
    sampler.stop()
    sampler.join(timeout=2)

    hbm, tflops, src = measured_peaks()
    per_rank = w.units_per_step_rank()
    total_units = per_rank * world
    if W.bound == "hbm":
        achieved, peak, nominal, runit = per_rank / (kern_ms * 1e-3) / 1e9, hbm, NOMINAL_HBM_GBS, "GB/s"
    else:
        achieved, peak, nominal, runit = per_rank / (kern_ms * 1e-3) / 1e12, tflops, NOMINAL_BF16_TFLOPS, "TFLOP/s"
    out = {
        "value": total_units / (ms_per_step * 1e-3) / 1e12, "ms_per_step": ms_per_step,
        "tokens_per_s": w.sequences_per_step() / (ms_per_step * 1e-3),
        "roofline": {"bound": W.bound, "achieved": achieved, "peak": peak, "unit": runit,
                     "frac": achieved / peak, "traffic": w.traffic(), "kernel": w.kernel_name(),
                     "kernel_ms": kern_ms, "algorithmic_units_per_launch": per_rank, "peak_source": src,
                     "nominal_peak": nominal, "frac_of_nominal": achieved / nominal},
        "gpu_launches": w.launches_per_step() * K_ * inner,
        "clocks": sampler.summary(),
    }
    if inner > 1:
        out["steps_timed"] = K_ * inner
        out["steps_per_graph_launch"] = inner
    if with_e2e:
        out["e2e"] = {"value": total_units / (e2e_ms * 1e-3) / 1e12, "unit": W.unit, "ms_per_step": e2e_ms,
                      "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        if getattr(w, "E2E_NOTE", None):
            out["e2e"]["overlap"] = w.E2E_NOTE
    return out


# what the default 1-GPU run measures after the headline: (workload, batch override)
SECONDARY = (("small_decode", None), ("rope", None), ("prefill", None), ("fp8_split", 16))


def run_secondary(args, world, rank, local, dev, fence, max_over_ranks):
    """Short legs of the other configurations, for the `secondary` key of the default line."""
    import copy
    import gc
    legs = []
    for name, batch in SECONDARY:
        W = WORKLOADS[name]
        a = copy.copy(args)
        a.batch, a.exchange = batch, "nccl"
        leg = {"workload": name, "metric": W.metric, "unit": W.unit, "dtype": W.dtype}
        try:
            w = W(a, world, rank, dev)
            w.setup()
            K_ = max(10, args.steps)
            m = measure(w, W, K_, max(3, args.warmup), world, rank, local, fence, max_over_ranks, with_e2e=False)
            r = m["roofline"]
            leg.update(config=w.config(), steps=K_, value=m["value"], ms_per_step=m["ms_per_step"],
                       tokens_per_s=m["tokens_per_s"], kernel=r["kernel"], kernel_ms=r["kernel_ms"],
                       roofline={k: r[k] for k in ("bound", "achieved", "peak", "unit", "frac", "frac_of_nominal")},
                       gpu_launches=m["gpu_launches"], clocks=m["clocks"])
            if not args.no_cpu:
                cb, par = w.cpu_baseline()
                if cb:
                    leg["cpu_baseline"], leg["parity"] = cb, par
        except Exception as e:          # a failed leg must not cost the headline its line
            leg["error"] = f"{type(e).__name__}: {e}"
        legs.append(leg)
        w = None
        gc.collect()
        torch.cuda.empty_cache()
    return legs


def run_b200(args, W):
    import gc
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w = W(args, world, rank, dev)
    w.setup()

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

    warm = max(3, args.warmup)
    m = measure(w, W, args.steps, warm, world, rank, local, fence, max_over_ranks)
    line = {
        "metric": W.metric, "value": m["value"], "unit": W.unit, "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": W.scaling, "vs_baseline": None,
        "dtype": W.dtype, "data": "synthetic", "tokens_per_s": m["tokens_per_s"], "config": w.config(),
        "roofline": m["roofline"], "e2e": m["e2e"], "gpu_launches": m["gpu_launches"], "clocks": m["clocks"],
    }
    if world > 1 and hasattr(w, "extra_multi_gpu"):
        x = w.extra_multi_gpu(fence, max_over_ranks)
        if x:
            line["o_all_gather" if "o_all_gather_ms" in x else "rank_skew"] = x
    # CPU leg: rank 0 at N = 1; workloads whose sample is spread over the ranks run it collectively
    if not args.no_cpu and (world == 1 or getattr(w, "collective_cpu_leg", False)):
        cb, par = w.cpu_baseline()
        if cb and rank == 0:
            if world == 1:
                line["cpu_baseline"] = cb
            line["parity"] = par
    if world == 1 and args.workload == "large_decode" and not args.no_secondary and not args.batch:
        w = None
        gc.collect()
        torch.cuda.empty_cache()
        line["secondary"] = run_secondary(args, world, rank, local, dev, fence, max_over_ranks)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="large_decode", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=None, help="override the batch size (profiling a small case)")
    ap.add_argument("--exchange", default="nccl", choices=["nccl", "peer", "peer_graph", "peer_unfused"],
                    help="fp8_split: how the partial rows travel between ranks")
    ap.add_argument("--gqa-group", type=int, default=4, choices=[2, 4, 8], help="gqa_decode: query heads per KV head")
    ap.add_argument("--gqa-kv", default="f16", choices=["f16", "e4m3"], help="gqa_decode: type of the KV pools")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--no-secondary", action="store_true",
                    help="default workload at 1 GPU: skip the short legs of the other configurations")
    args = ap.parse_args()
    W = WORKLOADS[args.workload]
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            run_reference(args, W)
        return
    run_b200(args, W)


if __name__ == "__main__":
    main()
