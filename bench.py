#!/usr/bin/env python
"""Benchmark of the fused-BMM hot path on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5] [--impl reference]

Prints ONE JSON line (rank 0). The five benchmark configurations:
  c1 min_bmm  A[1,16384,64]    B[1,64,16384]            rows sharded
  c2 bmm      A[128,1024,128]  B[128,128,1024]          batches sharded
  c3 mbmm     A[128,1024,64]   B[128,64,1024] + mask    batches sharded
  c4 min_bmm  A[1,1048576,128] B[1,128,65536]           rows sharded
  c5 topk_bmm A[1,1048576,256] B[1,256,1048576], k=64   B columns sharded + all-gather + merge
The headline (`value`, `ms_per_step`, `roofline`, `e2e`) is the workload named by --workload,
by default c5: the largest configuration that fits one GPU, and the one whose multi-GPU runs
carry the data-path collective. The other four are measured in the same invocation and
reported under `per_config`, each with its own step time, roofline, end-to-end figure, result
check and (at one GPU) CPU baseline.

A step is one pass of the op over the whole configuration (strong scaling: the configuration
is fixed, each rank takes its shard). Inputs are seeded synthetic tensors generated on the
host. `value` is timed with the shard resident in HBM; `e2e` runs the same step through the
Python wrapper from pinned host buffers, host<->device copies inside the timed region.
`check` compares a seeded sample of the timed outputs with the CPU oracle, outside the timed
region. `--impl reference` times the reference's semantics on the host cores (torch.bmm +
min / topk / masked_fill, the reference's own test expressions) on a bounded sample of the
same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024

SHAPES = {  # l, m, k, n
    "c1": (1, 16384, 64, 16384),
    "c2": (128, 1024, 128, 1024),
    "c3": (128, 1024, 64, 1024),
    "c4": (1, 1048576, 128, 65536),
    "c5": (1, 1048576, 256, 1048576),
}
SEEDS = {"c1": 1001, "c2": 1002, "c3": 1003, "c4": 1004, "c5": 1005}
OPS = {"c1": "min_bmm", "c2": "bmm", "c3": "mbmm", "c4": "min_bmm", "c5": "topk_bmm"}
UNIT = {"c1": "rows/s", "c2": "batches/s", "c3": "batches/s", "c4": "rows/s", "c5": "rows/s"}
TOPK = 64
# Which measured cuBLAS figure a tensor-bound workload is held against: the sub-millisecond
# kernels are timed one at a time with an L2 flush in between (burst); c4 and c5 run back to
# back for seconds under the power cap (sustained). One yardstick per workload at every N;
# both fractions are printed.
SUSTAINED = {"c1": False, "c2": False, "c3": False, "c4": True, "c5": True}
ARITHMETIC = "3xTF32 tensor-core products (tcgen05.mma kind::tf32), fp32 accumulation in TMEM"


def env_int(name, default):
    return int(os.environ.get(name, default))


# ---------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 7:
                continue
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for nm, val in zip(names, p[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------
# inputs
# ---------------------------------------------------------------------------------------
def host_inputs(name, rank, world):
    """Seeded host tensors of this rank's shard (generated whole, then cut, so that every
    world size sees the same configuration). Rank 0 also keeps what its result check needs."""
    from custom_matmul_kernels_b200.sharding import shard_range, shard_stride
    l, m, k, n = SHAPES[name]
    g = torch.Generator().manual_seed(SEEDS[name])
    out = {}
    if name in ("c2", "c3"):
        b0, b1 = shard_range(l, world, rank)
        if name == "c2":
            A = torch.rand(l, m, k, generator=g) * 2 - 1
            B = torch.rand(l, k, n, generator=g) * 2 - 1
        else:
            A = torch.randn(l, m, k, generator=g)
            B = torch.randn(l, k, n, generator=g)
            half = l // 2
            mask = torch.zeros(l, m, n, dtype=torch.bool)
            mask[:half] = torch.tril(torch.ones(m, n, dtype=torch.bool))
            tiles = torch.rand(l - half, m // 64, n // 64, generator=g) < 0.3
            mask[half:] = tiles.repeat_interleave(64, 1).repeat_interleave(64, 2)
            out["mask"] = mask[b0:b1].contiguous()
        out["A"], out["B"] = A[b0:b1].contiguous(), B[b0:b1].contiguous()
        out["units"] = b1 - b0
        return out
    if name in ("c1", "c4"):
        r0, r1 = shard_range(m, world, rank, 128)
        A = torch.randn(l, m, k, generator=g)
        B = torch.randn(l, k, n, generator=g)
        out["A"], out["B"] = A[:, r0:r1].contiguous(), B
        out["units"] = r1 - r0
        return out
    # c5: a grid of ranks: columns of B cut `cs` ways (the exchange stays inside each group of ranks that
    # share rows), rows of A cut across the `rg` groups. B is generated in 64Ki-column pieces, every rank alike.
    from custom_matmul_kernels_b200.sharding import topk_grid
    rg, cs = topk_grid(world)
    r0, r1 = shard_range(m, rg, rank // cs, 256)
    c0, c1 = shard_range(n, cs, rank % cs, 128)
    A = torch.randn(l, m, k, generator=g)
    B = torch.empty(l, k, c1 - c0)
    sample_rows = check_rows("c5", r1 - r0) + r0
    prod = torch.zeros(len(sample_rows), n, dtype=torch.float64) if rank == 0 else None
    As = A[0, sample_rows].double() if rank == 0 else None
    piece = 65536
    for p0 in range(0, n, piece):
        blk = torch.randn(l, k, min(piece, n - p0), generator=g)
        lo, hi = max(p0, c0), min(p0 + blk.shape[2], c1)
        if lo < hi:
            B[:, :, lo - c0:hi - c0] = blk[:, :, lo - p0:hi - p0]
        if rank == 0:  # the oracle's fp64 product of the sampled rows against ALL columns, piece by piece
            prod[:, p0:p0 + blk.shape[2]] = As @ blk[0].double()
    out["A"], out["B"], out["col0"] = A[:, r0:r1].contiguous(), B, c0
    out["cols_per_rank"] = shard_stride(n, cs, 128)
    out["units"] = r1 - r0
    out["grid"] = (rg, cs)
    out["check_product"] = prod
    return out


def check_rows(name, m):
    """Seeded sample of output rows the result check looks at."""
    count = {"c1": 512, "c4": 256, "c5": 48}[name]
    g = torch.Generator().manual_seed(SEEDS[name] + 77)
    return torch.randperm(m, generator=g)[:min(count, m)].sort().values


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------
class Workload:
    def __init__(self, name, rank, world, dev):
        from custom_matmul_kernels_b200 import BMMCUDA, MBMMCUDA, MinBMMCUDA, TopkBMMCUDA, make_masks
        from custom_matmul_kernels_b200 import sharding
        self.name, self.rank, self.world, self.dev = name, rank, world, dev
        self.sharding = sharding
        h = host_inputs(name, rank, world)
        self.h = h
        self.A_pin = h["A"].pin_memory()
        self.B_pin = h["B"].pin_memory()
        self.A = self.A_pin.to(dev)
        self.B = self.B_pin.to(dev)
        self.in_bytes = self.A.numel() * 4 + self.B.numel() * 4
        self.kernels_per_step = 1
        self.phase_events = []
        l_, m_, k_ = self.A.shape
        n_ = self.B.shape[2]
        if name == "c3":
            self.masks = make_masks(h["mask"].to(dev))
            self.masks_pin = tuple(t.cpu().pin_memory() for t in self.masks)
            self.in_bytes += sum(t.numel() for t in self.masks)
            self.op = MBMMCUDA()
        elif name == "c2":
            self.op = BMMCUDA()
        elif name in ("c1", "c4"):
            self.op = MinBMMCUDA()
            self.kernels_per_step = 2   # fused GEMM+min kernel, key-unpack kernel
            if self.op.lib.fbmm_presplit_workspace_bytes(l_, m_, n_, k_, 2, ord("n"), k_, m_ * k_, ord("n"), n_, k_ * n_):
                self.kernels_per_step += 1  # lo-plane pass over B (A is split in shared memory)
        else:
            self.op = TopkBMMCUDA()
            self.group = sharding.make_column_groups(world, h["grid"][1], rank) if world > 1 else None
            self.kernels_per_step = 1 + (1 if world > 1 else 0)  # + candidate merge
            if n_ > 0 and self.op.lib.fbmm_presplit_workspace_bytes(l_, m_, n_, k_, 2, ord("n"), k_, m_ * k_, ord("n"), n_,
                                                                    k_ * n_):
                self.kernels_per_step += 2 if k_ > 128 else 1  # plane passes over B and, when it streams, A
        self.out_host = None
        self.last = None

    def run(self, A, B, masks=None, timings=None):
        n = self.name
        if n == "c2":
            return (self.op(A, B),)
        if n == "c3":
            return (self.op(A, B, *(masks or self.masks)),)
        if n in ("c1", "c4"):
            return self.op(A, B, dim=2)
        if self.world == 1:
            return self.op(A, B, k=TOPK, dim=2)
        return self.sharding.topk_bmm_column_sharded(
            A, B, self.h["cols_per_rank"], TOPK, lambda a, b, k: self.op.packed(a, b, k=k, dim=2), group=self.group,
            timings=timings)

    def step(self):
        timings = {} if (self.name == "c5" and self.world > 1) else None
        self.last = self.run(self.A, self.B, timings=timings)
        if timings:
            self.phase_events.append(timings["events"])
        return self.last

    def e2e_step(self):
        self.A.copy_(self.A_pin, non_blocking=True)
        self.B.copy_(self.B_pin, non_blocking=True)
        masks = None
        if self.name == "c3":
            masks = self.masks
            for d, s in zip(self.masks, self.masks_pin):
                d.copy_(s, non_blocking=True)
        outs = self.run(self.A, self.B, masks)
        if self.out_host is None:
            self.out_host = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
        for hbuf, o in zip(self.out_host, outs):
            hbuf.copy_(o, non_blocking=True)
        return outs

    def out_bytes(self):
        return sum(h.numel() * h.element_size() for h in (self.out_host or []))

    # ---- result check against the CPU oracle (outside every timed region)
    def check(self):
        """Compares a seeded sample of this rank's last timed output with the oracle's fp64
        product. Returns counts; `unexplained` > 0 means a value outside rel 1e-5 / abs 1e-4
        or an index that does not point at a (near-)extremal entry."""
        from oracle import ref_semantics as R
        n = self.name
        outs = [o.detach() for o in self.last]
        res = {"max_abs_err": 0.0, "max_err_over_tol": 0.0, "index_mismatches": 0, "unexplained": 0, "checked": ""}
        try:
            if n in ("c2", "c3"):
                C = outs[0]
                picks = sorted({0, C.shape[0] // 2, C.shape[0] - 1}) if C.shape[0] else []
                for b in picks:
                    want = torch.mm(self.h["A"][b].double(), self.h["B"][b].double())
                    if n == "c3":
                        want.masked_fill_(~self.h["mask"][b], 0)
                        if bool((C[b].cpu()[~self.h["mask"][b]] != 0).any()):
                            res["unexplained"] += 1
                    err = (C[b].cpu().double() - want).abs()
                    tol = R.ATOL + R.RTOL * want.abs()
                    res["max_abs_err"] = max(res["max_abs_err"], float(err.max()))
                    res["max_err_over_tol"] = max(res["max_err_over_tol"], float((err / tol).max()))
                    res["unexplained"] += int((err > tol).sum())
                res["checked"] = f"{len(picks)} batches of this rank's shard, every element"
            elif n in ("c1", "c4"):
                v, i = outs
                rows = check_rows(n, v.shape[1])
                C = self.h["A"][0, rows].double() @ self.h["B"][0].double()
                wv, wi = C.min(dim=1)
                gv, gi = v[0].cpu()[rows].double(), i[0].cpu()[rows]
                tol = R.ATOL + R.RTOL * wv.abs()
                err = (gv - wv).abs()
                at = C.gather(1, gi.clamp(0, C.shape[1] - 1)[:, None])[:, 0]
                res["max_abs_err"] = float(err.max())
                res["max_err_over_tol"] = float((err / tol).max())
                res["index_mismatches"] = int((gi != wi).sum())
                res["unexplained"] = int((err > tol).sum()) + int(((at - wv).abs() > tol).sum()) + int(
                    ((gi < 0) | (gi >= C.shape[1])).sum())
                res["checked"] = f"{len(rows)} rows of this rank's shard against all {C.shape[1]} columns"
            else:
                if self.rank != 0:
                    return res
                v, i = outs
                rows = check_rows("c5", v.shape[1])
                C = self.h["check_product"]
                wv, wi = C.topk(TOPK, dim=1)
                gv, gi = v[0].cpu()[rows].double(), i[0].cpu()[rows]
                tol = R.ATOL + R.RTOL * wv.abs()
                err = (gv - wv).abs()
                inr = (gi >= 0) & (gi < C.shape[1])
                at = C.gather(1, gi.clamp(0, C.shape[1] - 1))
                dup = (gi.sort(dim=1).values[:, 1:] == gi.sort(dim=1).values[:, :-1])
                res["max_abs_err"] = float(err.max())
                res["max_err_over_tol"] = float((err / tol).max())
                res["index_mismatches"] = int((gi != wi).sum())
                res["unexplained"] = int((err > tol).sum()) + int(((at - gv).abs() > tol).sum()) + int((~inr).sum()) + int(
                    dup.sum()) + int((gv[:, :-1] < gv[:, 1:]).sum())
                res["checked"] = (f"{len(rows)} rows of the {'merged ' if self.world > 1 else ''}result against all "
                                  f"{C.shape[1]} columns, all {TOPK} entries")
        except Exception as e:  # noqa: BLE001 -- a broken check must show up in the line, not kill the bench
            res["unexplained"] += 1
            res["error"] = repr(e)
        return res


def timed_steps(fn, steps, flush):
    """K steps, each bracketed by CUDA events on the current stream; an L2 flush (outside
    the events) between steps when the inputs fit in L2. Returns per-step ms."""
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s in range(steps):
        if flush is not None:
            flush.add_(1.0)
        ev[s][0].record()
        fn()
        ev[s][1].record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in ev]


def back_to_back_ms(fn, steps):
    """K enqueues under ONE event pair (no flush in between): launch latency amortised."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def sync_each_ms(fn, steps):
    """Wall clock with a device synchronisation after every call, as the reference's harness
    times (colab/test_minbmm.ipynb:2123-2134)."""
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
        torch.cuda.synchronize()
    return (time.perf_counter() - t0) / steps * 1e3


_tf32_live = None


def measure_tf32_cublas():
    """cuBLAS TF32 throughput (fp32 torch.matmul with TF32 allowed, 8192^3, best of 10)."""
    global _tf32_live
    if _tf32_live is not None:
        return _tf32_live
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(8192, 8192, device="cuda")
        b = torch.randn(8192, 8192, device="cuda")
        best = float("inf")
        for i in range(13):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                best = min(best, e0.elapsed_time(e1))
        _tf32_live = 2 * 8192 ** 3 / best / 1e9
        return _tf32_live
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def algorithmic_bytes(name, units, n_cols):
    """Compulsory HBM bytes of one launch over `units` rows/batches (and n_cols columns) of this rank."""
    l, m, k, n = SHAPES[name]
    if name == "c2":
        return units * (m * k + k * n + m * n) * 4
    if name == "c3":
        return units * ((m * k + k * n + m * n) * 4 + (m // 128) * (n // 128) + (m // 8) * (n // 8))
    if name in ("c1", "c4"):
        return units * k * 4 + k * n_cols * 4 + units * 12
    return units * k * 4 + k * n_cols * 4 + units * TOPK * 12


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the fused kernel, from
# the ncu captures summarised in profiles/: (units captured, bytes that do not grow with the
# units, bytes that do).
#   c1-c3: the full workload was captured; everything is scaled by the rows / batches.
#   c4: 262 144 rows; B's hi and lo planes (67.1 MB) are read once per launch, the rest (A, once
#       per column range, and the keys) grows with the rows.
#   c5: 37 888 rows = two waves of 74 CTA pairs; every wave streams B's planes (2 x 1 GiB) from
#       DRAM once, so the traffic grows with the number of waves: bytes per row = capture / rows.
TRAFFIC_CAPTURES = {
    "c1": (16384, 0.0, 12771840.0 + 0.0),
    "c2": (128, 0.0, 142640640.0 + 477262080.0),
    "c3": (128, 0.0, 202073344.0 + 478761728.0),
    "c4": (262144, 2.0 * 128 * 65536 * 4, 356611840.0 + 5492992.0 - 2.0 * 128 * 65536 * 4),
    "c5": (37888, 0.0, 4635089152.0 + 292627200.0),
}


def measured_traffic(name, units, n_cols):
    """DRAM bytes per launch of the fused kernel, scaled from the capture by the units this rank
    processes; None for a column shard (no capture of that shape was taken)."""
    if n_cols != SHAPES[name][3]:
        return None
    cap_units, fixed, growing = TRAFFIC_CAPTURES[name]
    return fixed + growing * units / cap_units


def cpu_baseline(name, budget_s):
    """Reference semantics on the host cores over a bounded sample (rank 0, N=1)."""
    from oracle import ref_semantics as R
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    l, m, k, n = SHAPES[name]
    if name in ("c1", "c4"):
        rows = 8192 if name == "c4" else 16384
        d = R.make_inputs(name, rows=rows)
        fn = lambda: torch.bmm(d["A"], d["B"]).min(dim=-1)  # noqa: E731
        fn()
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < budget_s:
            fn()
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return {"value": rows / dt, "unit": "rows/s", "cores": cores, "kind": "port",
                "sample": f"{rows} rows x all {n} columns, torch.bmm + min on CPU, mean of {reps} passes"}
    if name == "c5":
        rows = 256
        d = R.make_inputs("c5", rows=rows, cols=n)
        t0 = time.perf_counter()
        R.cpu_topk_bmm_chunked(d["A"], d["B"], TOPK)
        dt = time.perf_counter() - t0
        return {"value": rows / dt, "unit": "rows/s", "cores": cores, "kind": "port",
                "sample": f"{rows} rows x all {n} columns in 131072-column chunks with a running top-64, one pass"}
    batches = 8
    d = R.make_inputs(name, batches=batches)
    if name == "c2":
        fn = lambda: torch.bmm(d["A"], d["B"])  # noqa: E731
    else:
        fn = lambda: torch.bmm(d["A"], d["B"]).masked_fill_(~d["mask"], 0)  # noqa: E731
    fn()
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < budget_s:
        fn()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": batches / dt, "unit": "batches/s", "cores": cores, "kind": "port",
            "sample": f"{batches} of {l} batches, torch.bmm{' + masked_fill' if name == 'c3' else ''} on CPU, mean of {reps} passes"}


def config_dict(name, world):
    """The same for both arms: what is computed, on what, cut how."""
    l, m, k, n = SHAPES[name]
    part = {"c1": "A rows", "c4": "A rows", "c2": "batches", "c3": "batches", "c5": "B columns + all-gather"}[name]
    how = f"{part} over {world} GPU(s)"
    if name == "c5" and world > 1:
        from custom_matmul_kernels_b200.sharding import topk_grid
        rg, cs = topk_grid(world)
        how = f"B columns over {cs} GPUs (packed all-gather + merge)" + (f" x A rows over {rg} such groups" if rg > 1 else "")
    return {"workload": f"{name}: {OPS[name]} A[{l},{m},{k}] B[{l},{k},{n}]" + (f" k={TOPK}" if name == "c5" else ""),
            "sharding": how, "precision": "fp32 in, fp32 out",
            "l2": "flushed between steps" if name in ("c1", "c2", "c3") else "inputs exceed L2"}


def roofline(name, wl, ms_mean, peaks, world):
    """Roofline record of the dominant kernel (the fused GEMM) of this rank's launch."""
    l, m, k, n = SHAPES[name]
    n_cols = wl.B.shape[2]
    units = wl.h["units"]
    if name in ("c2", "c3"):
        flops = 2.0 * units * m * n * k
    else:
        flops = 2.0 * units * n_cols * k
    nbytes = algorithmic_bytes(name, units, n_cols)
    burst = peaks["bf16"] / 2 / 3
    sustained = peaks["bf16_sustained"] / 2 / 3
    tensor_time = flops / (burst * 1e12)
    hbm_time = nbytes / (peaks["hbm_gbs"] * 1e9)
    achieved_tflops = flops / (ms_mean / 1e3) / 1e12 if ms_mean > 0 else 0.0
    achieved_gbs = nbytes / (ms_mean / 1e3) / 1e9 if ms_mean > 0 else 0.0
    roof = {}
    if hbm_time > tensor_time:
        roof.update({"bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "peak_note": f"{peaks['source']} STREAM-style copy"})
    else:
        use_sustained = SUSTAINED[name]
        roof.update({"bound": "tensor", "achieved": achieved_tflops, "peak": sustained if use_sustained else burst,
                     "unit": "TFLOP/s",
                     "peak_note": f"{peaks['source']} cuBLAS bf16 {'sustained' if use_sustained else 'burst'} / 2 (tf32) / 3 "
                                  "(three tf32 MMAs per fp32 product)"})
    roof["frac"] = roof["achieved"] / roof["peak"] if roof["peak"] else None
    roof["tensor"] = {"achieved_tflops": achieved_tflops, "frac_burst": achieved_tflops / burst,
                      "frac_sustained": achieved_tflops / sustained, "frac_mma_issue_ceiling": achieved_tflops / 341.0}
    roof["hbm"] = {"achieved_gbs": achieved_gbs, "frac": achieved_gbs / peaks["hbm_gbs"], "algorithmic_bytes": nbytes}
    roof["ideal_ms"] = {"tensor_burst": tensor_time * 1e3, "hbm": hbm_time * 1e3}
    roof["traffic"] = measured_traffic(name, units, n_cols)
    roof["kernel"] = "fbmm_gemm_kernel"
    return roof


def measure(name, args, rank, local_rank, world, dev, headline):
    """One workload: warm-up, K device-timed steps, the end-to-end leg, the result check."""
    import torch.distributed as dist
    wl = Workload(name, rank, world, dev)
    small = name in ("c1", "c2", "c3")
    flush = torch.zeros(L2_BYTES * 2 // 4, device=dev) if small else None
    steps = args.steps if (headline or not small) else max(args.steps, 50)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        wl.step()
    barrier()
    wl.phase_events = []
    sampler = None
    if rank == 0 and headline:
        sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else
                               os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank])
        sampler.start()
    ms = timed_steps(wl.step, steps, flush)
    barrier()
    phases = None
    if wl.phase_events:
        acc = [0.0, 0.0, 0.0]
        for ev in wl.phase_events:
            for j in range(3):
                acc[j] += ev[j].elapsed_time(ev[j + 1])
        phases = {"local_topk_ms": acc[0] / len(wl.phase_events), "all_gather_ms": acc[1] / len(wl.phase_events),
                  "merge_ms": acc[2] / len(wl.phase_events)}
    check = wl.check()
    extra = {}
    if small and not args.no_e2e:
        extra["ms_back_to_back"] = back_to_back_ms(wl.step, steps)
        extra["ms_sync_each"] = sync_each_ms(wl.step, steps)
        barrier()
    # end to end: pinned host -> device -> op -> pinned host, every step
    if args.no_e2e:
        ms_e2e = [float("nan")] * steps
    else:
        for _ in range(2):
            wl.e2e_step()
        barrier()
        ms_e2e = timed_steps(wl.e2e_step, steps, None)
        barrier()
    clocks = sampler.stop() if sampler is not None else None

    tot = torch.tensor([sum(ms), sum(ms_e2e), check["max_abs_err"], check["max_err_over_tol"]], device=dev,
                       dtype=torch.float64)
    cnt = torch.tensor([check["index_mismatches"], check["unexplained"]], device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(tot, op=dist.ReduceOp.MAX)
        dist.all_reduce(cnt, op=dist.ReduceOp.SUM)
    total_ms, total_e2e_ms = float(tot[0]), float(tot[1])
    l, m, k, n = SHAPES[name]
    units_total = l if name in ("c2", "c3") else m
    rec = None
    if rank == 0:
        ms_per_step = total_ms / steps
        peaks = load_peaks()
        roof = roofline(name, wl, statistics.mean(ms), peaks, world)
        if world == 1:
            roof["tf32_cublas_tflops_live"] = measure_tf32_cublas()
            roof["tensor"]["frac_live_tf32"] = roof["tensor"]["achieved_tflops"] / (roof["tf32_cublas_tflops_live"] / 3)
        check_out = dict(check)
        check_out.update({"max_abs_err": float(tot[2]), "max_err_over_tol": float(tot[3]),
                          "index_mismatches": int(cnt[0]), "unexplained": int(cnt[1]),
                          "ok": int(cnt[1]) == 0, "ranks": world,
                          "tolerance": "rel 1e-5 / abs 1e-4 against the fp64 product of the CPU oracle"})
        rec = {
            "metric": f"fused {OPS[name]} throughput ({name})", "value": units_total / (ms_per_step / 1e3),
            "unit": UNIT[name], "steps": steps, "ms_per_step": ms_per_step,
            "ms_per_step_median": statistics.median(ms), "ms_per_step_best": min(ms),
            "tflops": 2.0 * l * m * n * k / (ms_per_step / 1e3) / 1e12,
            "config": config_dict(name, world),
            "e2e": {"value": units_total / (total_e2e_ms / steps / 1e3), "unit": UNIT[name],
                    "h2d_bytes_per_step": wl.in_bytes, "d2h_bytes_per_step": wl.out_bytes(),
                    "note": "bytes are this rank's; every rank copies its own shard"},
            "gpu_launches": wl.kernels_per_step * steps * world,
            "roofline": roof, "check": check_out,
        }
        rec.update(extra)
        if phases:
            rec["phases_rank0"] = phases
        if clocks is not None:
            rec["clocks"] = clocks
        if world == 1 and not args.no_cpu:
            rec["cpu_baseline"] = cpu_baseline(name, 10.0 if headline else 4.0)
    del wl, flush
    torch.cuda.empty_cache()
    return rec


def measure_softmax_consumer(args, dev):
    """The consumer behind mbmm (row softmax over the kept entries, scores never written) on
    configuration 3's operands and masks: device-timed steps with an L2 flush in between, and
    a check of three batches against the fp64 oracle. One GPU only (an extra, not a headline)."""
    from custom_matmul_kernels_b200 import MBMMSoftmaxCUDA, make_masks
    from oracle import ref_semantics as R
    h = host_inputs("c3", 0, 1)
    A, B = h["A"].to(dev), h["B"].to(dev)
    masks = make_masks(h["mask"].to(dev))
    op = MBMMSoftmaxCUDA()
    scale = 0.125
    flush = torch.zeros(L2_BYTES * 2 // 4, device=dev)
    steps = args.steps if args.consumer_only else max(args.steps, 30)
    for _ in range(max(args.warmup, 3)):
        P = op(A, B, *masks, scale=scale)
    ms = timed_steps(lambda: op(A, B, *masks, scale=scale), steps, flush)
    P = op(A, B, *masks, scale=scale)
    # the same result from separate steps: the masked product written out by MBMMCUDA, then
    # torch's where + softmax over it (what a caller of the reference's mbmm would run next)
    from custom_matmul_kernels_b200 import MBMMCUDA
    mbmm, keep = MBMMCUDA(), h["mask"].to(dev)
    neg = torch.full((), float("-inf"), device=dev)

    def unfused():
        return torch.softmax(torch.where(keep, mbmm(A, B, *masks) * scale, neg), dim=-1)
    for _ in range(3):
        unfused()
    ms_unfused = timed_steps(unfused, min(steps, 10), flush)
    del keep
    worst, bad = 0.0, 0
    for b in sorted({0, SHAPES["c3"][0] // 2, SHAPES["c3"][0] - 1}):
        want = R.mbmm_softmax(h["A"][b], h["B"][b], *(t[b].cpu() for t in masks), scale=scale)
        err = (P[b].cpu().double() - want).abs()
        worst = max(worst, float(err.max()))
        bad += int((err > 2e-6 + 1e-4 * want.abs()).sum()) + int((P[b].cpu()[~h["mask"][b]] != 0).sum())
    l, m, k, n = SHAPES["c3"]
    nbytes = algorithmic_bytes("c3", l, n) + l * m * n  # + the element mask, which this op reads in full
    mean = statistics.mean(ms)
    peaks = load_peaks()
    del A, B, masks, P, flush
    torch.cuda.empty_cache()
    return {"op": "mbmm + row softmax (MBMMSoftmaxCUDA) on the c3 operands and masks", "steps": steps,
            "ms_per_step": mean, "ms_per_step_best": min(ms), "batches_per_s": l / (mean / 1e3),
            "ms_per_step_unfused": statistics.mean(ms_unfused),
            "unfused": "MBMMCUDA, then torch.where(mask, C * scale, -inf) and torch.softmax",
            "achieved_gbs": nbytes / (mean / 1e3) / 1e9, "hbm_frac": nbytes / (mean / 1e3) / 1e9 / peaks["hbm_gbs"],
            "algorithmic_bytes": nbytes,
            "check": {"max_abs_err": worst, "unexplained": bad, "ok": bad == 0,
                      "tolerance": "abs 2e-6 + rel 1e-4 on the probabilities, 3 batches, fp64 oracle"}}


def measure_l1_mode(args, dev):
    """distance="l1" (the SIMT kernel) on configuration 1's operands: min and top-64 over
    sum_k |a - b|, device-timed with an L2 flush between steps, 64 sampled rows checked against the
    fp64 formula. One GPU only (an extra, not a headline). The roofline is the fp32 issue rate:
    two instructions per term on 128 lanes per SM at the sampled SM clock's maximum."""
    from custom_matmul_kernels_b200 import MinBMMCUDA, TopkBMMCUDA
    from oracle import ref_semantics as R
    h = host_inputs("c1", 0, 1)
    A, B = h["A"].to(dev), h["B"].to(dev)
    l, m, k, n = SHAPES["c1"]
    mn, tk = MinBMMCUDA(distance="l1"), TopkBMMCUDA(distance="l1")
    flush = torch.zeros(L2_BYTES * 2 // 4, device=dev)
    steps = args.steps if args.consumer_only else max(min(args.steps, 20), 10)
    out = {"op": "min_bmm / topk_bmm with distance='l1' on the c1 operands", "steps": steps}
    rows = check_rows("c1", m)[:64]
    want = (h["A"][0, rows].double()[:, None, :] - h["B"][0].double().t()[None, :, :]).abs().sum(-1)  # [64, n]
    for tag, fn in (("min", lambda: mn(A, B, dim=2)), ("top64", lambda: tk(A, B, k=TOPK, dim=2))):
        for _ in range(max(args.warmup, 3)):
            fn()
        ms = timed_steps(fn, steps, flush)
        v, i = fn()
        gv, gi = v[0].cpu()[rows].double(), i[0].cpu()[rows]
        if tag == "min":
            wv = want.min(dim=1).values
            at = want.gather(1, gi[:, None])[:, 0]
            bad = int(((gv - wv).abs() > R.ATOL + R.RTOL * wv.abs()).sum()) + int(((at - wv).abs() > R.ATOL + R.RTOL * wv.abs()).sum())
        else:
            wv = want.topk(TOPK, dim=1).values
            at = want.gather(1, gi)
            bad = int(((gv - wv).abs() > R.ATOL + R.RTOL * wv.abs()).sum()) + int(((at - gv).abs() > R.ATOL + R.RTOL * gv.abs()).sum())
        mean = statistics.mean(ms)
        terms = float(l) * m * n * k
        peak = 148 * 128 * 1.965e9 / 2.0  # terms/s if every fp32 issue slot did useful work at the maximum clock
        out[tag] = {"ms_per_step": mean, "ms_per_step_best": min(ms), "rows_per_s": m / (mean / 1e3),
                    "terms_per_s": terms / (mean / 1e3), "frac_of_fp32_issue_rate": terms / (mean / 1e3) / peak,
                    "unexplained": bad, "ok": bad == 0}
    out["checked"] = "64 rows against all 16384 columns, fp64 formula, rel 1e-5 / abs 1e-4"
    del A, B, flush
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    rank, local_rank, world = env_int("RANK", 0), env_int("LOCAL_RANK", 0), env_int("WORLD_SIZE", 1)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    name = args.workload
    head = measure(name, args, rank, local_rank, world, dev, True)
    per = {}
    if not args.no_per_config:
        for other in sorted(SHAPES):
            if other != name:
                per[other] = measure(other, args, rank, local_rank, world, dev, False)
    consumers = None
    if world == 1 and not args.no_per_config:
        consumers = {"c3_softmax": measure_softmax_consumer(args, dev), "c1_l1": measure_l1_mode(args, dev)}
    if rank == 0:
        line = {
            "metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "arithmetic": ARITHMETIC,
        }
        for key in ("config", "tflops", "e2e", "gpu_launches", "clocks", "roofline", "check", "phases_rank0",
                    "ms_per_step_median", "ms_per_step_best", "ms_back_to_back", "ms_sync_each", "cpu_baseline"):
            if key in head:
                line[key] = head[key]
        if per:
            line["per_config"] = per
            line["gpu_launches"] += sum(p["gpu_launches"] for p in per.values())
        if consumers:
            line["consumers"] = consumers
            line["gpu_launches"] += consumers["c3_softmax"]["steps"] + 2 * consumers["c1_l1"]["steps"]
        if args.rows is not None or args.batches is not None:
            line["reduced"] = True
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------
# reference arm: the reference's semantics on the host cores
# ---------------------------------------------------------------------------------------
def reference_kernels_on_gpu():
    """The reference's OWN kernels (kernels/bmm.cu, mbmm.cu, minbmm.cu compiled as its wrappers
    compile them into oracle/_ref/ and launched with its grids) timed on this GPU on c1, c2 and
    c3: the direct kernel-against-kernel figure beside the CPU arm. c4 and c5 cannot be launched
    (gridDim.y overflows, minbmm.py:127-129), and kernels/topkbmm.cu is not run at all (it takes
    a global spin mutex). Output buffers are created by the launch helper as the reference's
    wrappers create them (zeros / +inf), inside the timed call."""
    try:
        from oracle import ref_kernels as K
        from oracle import ref_semantics as R
        from custom_matmul_kernels_b200 import make_masks
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"}
    if not torch.cuda.is_available():
        return {"unavailable": "no GPU"}
    if not K.available():
        return {"unavailable": "oracle/_ref holds no cubins (python -m oracle.build_ref <reference root>)"}
    dev = torch.device("cuda", 0)
    out = {}
    for name in ("c1", "c2", "c3"):
        h = R.make_inputs(name)
        A, B = h["A"].to(dev), h["B"].to(dev)
        if name == "c1":
            fn = lambda: K.min_bmm(A, B, 2)  # noqa: E731
        elif name == "c2":
            fn = lambda: K.bmm(A, B)  # noqa: E731
        else:
            masks = make_masks(h["mask"].to(dev))
            fn = lambda: K.mbmm(A, B, *masks)  # noqa: E731
        for _ in range(2):
            fn()
        ms = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        l, m, k, n = SHAPES[name]
        units = m if name == "c1" else l
        out[name] = {"ms_per_call": statistics.mean(ms), "ms_best": min(ms), "value": units / (statistics.mean(ms) / 1e3),
                     "unit": UNIT[name], "kernel": {"c1": "min_bmm_nn", "c2": "bmm_nn", "c3": "mbmm_nn"}[name]}
        del A, B
        torch.cuda.empty_cache()
    out["note"] = ("the reference's SIMT fp32 kernels recompiled for sm_100a, one call = output fill + kernel; "
                   "c4 and c5 are beyond the reference's grid limits")
    return out


def run_reference(args):
    rank, world = env_int("RANK", 0), env_int("WORLD_SIZE", 1)
    if rank != 0:
        return
    from oracle import ref_semantics as R
    name = args.workload
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    l, m, k, n = SHAPES[name]
    if name in ("c1", "c4"):
        rows = 8192 if name == "c4" else 16384
        d = R.make_inputs(name, rows=rows)
        step = lambda: torch.bmm(d["A"], d["B"]).min(dim=-1)  # noqa: E731
        units, sample = rows, f"{rows} rows x all {n} columns per step"
    elif name == "c5":
        rows = 128
        d = R.make_inputs("c5", rows=rows, cols=n)
        step = lambda: R.cpu_topk_bmm_chunked(d["A"], d["B"], TOPK)  # noqa: E731
        units, sample = rows, f"{rows} rows x all {n} columns per step, running top-64 over 131072-column chunks"
    else:
        batches = 8
        d = R.make_inputs(name, batches=batches)
        if name == "c2":
            step = lambda: torch.bmm(d["A"], d["B"])  # noqa: E731
        else:
            step = lambda: torch.bmm(d["A"], d["B"]).masked_fill_(~d["mask"], 0)  # noqa: E731
        units, sample = batches, f"{batches} of {l} batches per step"
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = units / dt
    line = {
        "impl": "reference", "metric": f"fused {OPS[name]} throughput ({name})", "value": value, "unit": UNIT[name],
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "arithmetic": "fp32 on the host cores (torch CPU)",
        "config": config_dict(name, world),
        "cpu_baseline": {"value": value, "unit": UNIT[name], "cores": cores, "kind": "port",
                         "sample": sample + "; torch CPU restatement of the reference's test expressions "
                                            "(the reference's kernels need CuPy and a GPU)"},
        "e2e": {"value": value, "unit": UNIT[name], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if world == 1 and not args.no_per_config:
        line["reference_kernels_on_this_gpu"] = reference_kernels_on_gpu()
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c5", choices=sorted(SHAPES))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--no-per-config", action="store_true", help="measure the headline workload only")
    ap.add_argument("--rows", type=int, default=None,
                    help="profiling only: cut c1/c4/c5 to this many rows of A (the line is marked reduced)")
    ap.add_argument("--batches", type=int, default=None,
                    help="profiling only: cut c2/c3 to this many batches (the line is marked reduced)")
    ap.add_argument("--no-e2e", action="store_true", help="profiling only: skip the end-to-end legs")
    ap.add_argument("--consumer-only", nargs="?", const="softmax", default=None, choices=["softmax", "l1"],
                    help="profiling only: run just the masked row softmax on the c3 operands (honours --batches), or "
                         "just the l1 mode on the c1 operands, and print its record")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = {"c1": 50, "c2": 30, "c3": 30, "c4": 10, "c5": 4}[args.workload]
    if args.rows is not None and args.workload in ("c1", "c4", "c5"):
        l, m, k, n = SHAPES[args.workload]
        SHAPES[args.workload] = (l, args.rows, k, n)
    if args.batches is not None and args.workload in ("c2", "c3"):
        l, m, k, n = SHAPES[args.workload]
        SHAPES[args.workload] = (args.batches, m, k, n)
    if args.rows is not None or args.batches is not None:
        args.no_per_config = True
    if args.consumer_only:
        torch.cuda.set_device(0)
        dev0 = torch.device("cuda", 0)
        rec = {"c1_l1": measure_l1_mode(args, dev0)} if args.consumer_only == "l1" else {"c3_softmax": measure_softmax_consumer(args, dev0)}
        print(json.dumps({"consumers": rec}))
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
