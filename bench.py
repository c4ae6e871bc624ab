#!/usr/bin/env python
"""Benchmark of the LEGO hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload softmax] [--impl reference]

A step is one pass of one kernel over one batch of seeded synthetic input.  The
headline workload is the row-wise softmax (fp16, 16384 x 8192); the other four
configurations (tiled transpose, LayerNorm, GEMM 8192^3, grouped GEMM) are
measured in the same run and reported under "workloads".  One JSON line is
printed by rank 0.  With --impl reference the reference's CPU path (index maps
in numpy as lego_python prints them + torch CPU ops) is timed on the host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import inputs  # noqa: E402  (tests/inputs.py: the seeded builders of the five configurations)

L2_BYTES = 126 * 1024 * 1024


# --------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------

class Workload:
    name = ""
    unit = "GB/s"
    bound = "hbm"
    dtype = "f16"
    kernels_per_step = 1
    description = ""
    graph_ok = False   # the step can be captured in a CUDA graph (no host-to-device copy inside)

    def work(self) -> float:
        """Algorithmic bytes (or flops) of one step."""
        raise NotImplementedError

    def metric(self) -> str:
        kind = "HBM GB/s" if self.unit == "GB/s" else "TFLOP/s"
        return f"{getattr(self, 'short', self.name.split('_f')[0])} {kind}"

    def setup(self, dev):
        raise NotImplementedError

    def step(self, i: int):
        raise NotImplementedError

    def e2e_setup(self):
        raise NotImplementedError

    def e2e_step(self, i: int):
        raise NotImplementedError

    def cpu_sample(self, threads: int, budget: float = 4.0):
        """(work done, seconds, what was run) for a bounded sample (about `budget` seconds) on the host cores."""
        raise NotImplementedError


def _rate(work: float, seconds: float, unit: str) -> float:
    return work / seconds / (1e9 if unit == "GB/s" else 1e12)


class Softmax(Workload):
    graph_ok = True
    name = "softmax_f16_16384x8192"
    description = ("row-wise softmax, fp16 16384 x 8192 ~ N(0, 2^2) seed 1, fp32 arithmetic, rows mapped by "
                   "OrderBy(Row(16384)).TileBy([4096],[4]); inputs (256 MiB) larger than L2")
    rows, cols = 16384, 8192

    def work(self):
        return 2.0 * self.rows * self.cols * 2

    def setup(self, dev):
        from lego_b200 import ops
        self.ops = ops
        self.x_host = inputs.softmax_input(self.rows, self.cols)
        self.x = self.x_host.to(dev)
        self.row_map = ops.row_tiling_layout(self.rows, 4)
        self.y = None

    def step(self, i):
        self.y = self.ops.softmax(self.x, self.row_map)

    def check(self):
        from oracle import lego_oracle as O
        sel = torch.arange(0, self.rows, 257)
        err = (self.y[sel.to(self.y.device)].cpu().float() - O.softmax(self.x_host[sel]).float()).abs().max().item()
        return err <= 1e-3, f"max-abs {err:.2e} on {len(sel)} rows vs oracle (tol 1e-3)"

    def e2e_setup(self):
        self.x_pinned = self.x_host.pin_memory()
        return self.x_pinned.numel() * 2, self.x_pinned.numel() * 2

    def e2e_step(self, i):
        return self.ops.softmax(self.x_pinned, self.row_map)

    def cpu_sample(self, threads, budget=4.0):
        rows = 2048
        x = self.x_host[:rows]
        t0 = time.perf_counter()
        n = 0
        while time.perf_counter() - t0 < budget:
            torch.softmax(x.float(), dim=-1).half()
            n += 1
        dt = time.perf_counter() - t0
        return 2.0 * rows * self.cols * 2 * n, dt, f"{n} x torch.softmax(x.float(),-1).half() on {rows} of {self.rows} rows"


class LayerNorm(Workload):
    graph_ok = True
    name = "layernorm_fwd_f16_16384x8192"
    description = ("LayerNorm forward, fp16 16384 x 8192 seed 2, eps 1e-5, fp32 statistics, fp16 y + fp32 mean/rstd; "
                   "inputs (256 MiB) larger than L2")
    rows, cols = 16384, 8192

    def work(self):
        return 2.0 * self.rows * self.cols * 2

    def setup(self, dev):
        from lego_b200 import ops
        self.ops = ops
        self.x_host, self.g_host, self.b_host = inputs.layernorm_input(self.rows, self.cols)
        self.x, self.g, self.b = self.x_host.to(dev), self.g_host.to(dev), self.b_host.to(dev)
        self.row_map = ops.row_tiling_layout(self.rows, 4)

    def step(self, i):
        self.out = self.ops.layer_norm_fwd(self.x, self.g, self.b, 1e-5, self.row_map)

    def check(self):
        from oracle import lego_oracle as O
        sel = torch.arange(0, self.rows, 257)
        ref = O.layernorm_fwd(self.x_host[sel], self.g_host, self.b_host, 1e-5, round_output=False)[0]
        err = (self.out[0][sel.to(self.x.device)].cpu().float() - ref).abs()
        ok = bool((err <= 1e-3 + ref.abs() * 2.0 ** -11).all())
        small = err[ref.abs() < 2].max().item()
        return ok, (f"max-abs {small:.2e} where |y| < 2 on {len(sel)} rows vs fp32 oracle (tol 1e-3; beyond, "
                    f"1e-3 + half an fp16 ulp of y)")

    def e2e_setup(self):
        self.xp = self.x_host.pin_memory()
        return self.xp.numel() * 2 + 2 * self.cols * 2, self.xp.numel() * 2 + 2 * self.rows * 4

    def e2e_step(self, i):
        return self.ops.layer_norm_fwd(self.xp, self.g_host, self.b_host, 1e-5, self.row_map)

    def cpu_sample(self, threads, budget=4.0):
        rows = 2048
        x = self.x_host[:rows]
        t0 = time.perf_counter()
        n = 0
        while time.perf_counter() - t0 < budget:
            torch.nn.functional.layer_norm(x.float(), (self.cols,), self.g_host.float(), self.b_host.float(), 1e-5).half()
            n += 1
        dt = time.perf_counter() - t0
        return 2.0 * rows * self.cols * 2 * n, dt, f"{n} x F.layer_norm fp32 on {rows} of {self.rows} rows"


class LayerNormBwd(Workload):
    graph_ok = True
    name = "layernorm_bwd_f16_16384x8192"
    short = "layernorm_bwd"
    kernels_per_step = 2   # dx + column partials, then the column reduction
    description = ("LayerNorm backward (dx, dgamma, dbeta), fp16 16384 x 8192 seed 2 with dy ~ N(0, 0.1^2) from the same "
                   "generator, fp32 arithmetic, fixed-order two-stage column reduction; x and dy (512 MiB) larger than L2")
    rows, cols = 16384, 8192

    def work(self):
        return 3.0 * self.rows * self.cols * 2   # x and dy read, dx written (the reference's formula)

    def setup(self, dev):
        from lego_b200 import ops
        from oracle import lego_oracle as O
        self.ops = ops
        self.x_host, self.g_host, self.b_host = inputs.layernorm_input(self.rows, self.cols)
        self.dy_host = (0.1 * torch.randn(self.rows, self.cols, generator=torch.Generator().manual_seed(22))).half()
        self.x, self.g, self.dy = self.x_host.to(dev), self.g_host.to(dev), self.dy_host.to(dev)
        _, self.mean, self.rstd = ops.layer_norm_fwd(self.x, self.g, self.b_host.to(dev), 1e-5)

    def step(self, i):
        self.out = self.ops.layer_norm_bwd(self.dy, self.x, self.g, self.mean, self.rstd)

    def check(self):
        from oracle import lego_oracle as O
        sel = torch.arange(0, self.rows, 257)
        _, mean, rstd = O.layernorm_fwd(self.x_host[sel], self.g_host, self.b_host, 1e-5)
        rdx, _, _ = O.layernorm_bwd(self.dy_host[sel], self.x_host[sel], self.g_host, mean, rstd)
        err = (self.out[0][sel.to(self.x.device)].cpu().float() - rdx.float()).abs().max().item()
        # column sums over all rows, against fp64 sums of a strided sample of columns
        cols = torch.arange(0, self.cols, 263)
        xs, dys = self.x_host[:, cols].double(), self.dy_host[:, cols].double()
        m, r = self.mean.cpu().double()[:, None], self.rstd.cpu().double()[:, None]
        dw_ref, db_ref = (dys * (xs - m) * r).sum(0), dys.sum(0)
        dw, db = self.out[1].cpu().double()[cols], self.out[2].cpu().double()[cols]
        ew = ((dw - dw_ref).abs().max() / dw_ref.abs().max()).item()
        eb = ((db - db_ref).abs().max() / db_ref.abs().max()).item()
        ok = err <= 1e-3 and ew <= 2e-3 and eb <= 2e-3
        return ok, (f"dx max-abs {err:.2e} on {len(sel)} rows vs oracle (tol 1e-3); dgamma / dbeta rel-to-max "
                    f"{ew:.1e} / {eb:.1e} on {len(cols)} columns vs fp64 sums (tol 2e-3)")

    def e2e_setup(self):
        self.xp, self.dyp = self.x_host.pin_memory(), self.dy_host.pin_memory()
        self.mp, self.rp = self.mean.cpu().pin_memory(), self.rstd.cpu().pin_memory()
        return 2 * self.xp.numel() * 2 + self.cols * 2 + 2 * self.rows * 4, self.xp.numel() * 2 + 2 * self.cols * 2

    def e2e_step(self, i):
        return self.ops.layer_norm_bwd(self.dyp, self.xp, self.g_host, self.mp, self.rp)

    def cpu_sample(self, threads, budget=4.0):
        from oracle import lego_oracle as O
        rows = 2048
        x, dy = self.x_host[:rows], self.dy_host[:rows]
        mean, rstd = self.mean[:rows].cpu(), self.rstd[:rows].cpu()
        t0 = time.perf_counter()
        n = 0
        while time.perf_counter() - t0 < budget:
            O.layernorm_bwd(dy, x, self.g_host, mean, rstd)
            n += 1
        dt = time.perf_counter() - t0
        return 3.0 * rows * self.cols * 2 * n, dt, f"{n} x oracle layernorm_bwd (torch fp32) on {rows} of {self.rows} rows"


class Transpose(Workload):
    graph_ok = True
    name = "tiled_transpose_f32_4096"
    dtype = "f32"
    description = ("LEGO 2-level tiled transpose, fp32 4096 x 4096 uniform[-1,1) seed 0, 32 x 32 tiles, tiles in "
                   "column-major order; 4 rotating buffer pairs (512 MiB) so no step finds its data in L2")
    n = 4096
    sets = 4

    def work(self):
        return 2.0 * self.n * self.n * 4

    def setup(self, dev):
        import lego_b200 as L
        from lego_b200 import ops
        self.ops = ops
        n = self.n
        self.a_host = inputs.transpose_input(n)
        self.src = L.OrderBy(L.Row(n, n)).TileBy([n // 32, n // 32], [32, 32])
        self.dst = L.OrderBy(L.Col(n, n)).TileBy([n // 32, n // 32], [32, 32])
        self.order = L.OrderBy(L.Col(n // 32, n // 32)).TileBy([n // 32, n // 32])
        self.ins = [self.a_host.to(dev) for _ in range(self.sets)]
        self.outs = [torch.empty_like(self.ins[0]) for _ in range(self.sets)]

    def step(self, i):
        k = i % self.sets
        self.ops.permute(self.ins[k], self.src, self.dst, self.order, out=self.outs[k])

    def check(self):
        ok = torch.equal(self.outs[0].cpu().reshape(self.n, self.n), self.a_host.t().contiguous())
        return ok, "bit-exact vs A.T"

    def e2e_setup(self):
        self.ap = self.a_host.pin_memory()
        return self.ap.numel() * 4, self.ap.numel() * 4

    def e2e_step(self, i):
        return self.ops.permute(self.ap, self.src, self.dst, self.order)

    def cpu_sample(self, threads, budget=4.0):
        from oracle import lego_oracle as O
        from helpers import spec_of
        x = self.a_host.reshape(-1).numpy()
        t0 = time.perf_counter()
        O.permute(x, spec_of(self.src), spec_of(self.dst))
        dt = time.perf_counter() - t0
        return self.work(), dt, "1 x numpy index maps of both layouts over 4096^2 ids + gather/scatter (single thread)"


class Gemm(Workload):
    graph_ok = True
    name = "gemm_f16_8192"
    unit = "TFLOP/s"
    bound = "tensor"
    description = ("C = A.B, fp16 8192^3 ~ N(0, 1/sqrt(8192)) seed 3, fp32 accumulate, fp16 C, 128 x 256 tiles, "
                   "tile order = LEGO grouped swizzle GROUP_M = 8; operands (384 MiB) larger than L2")
    m = n = k = 8192

    def work(self):
        return 2.0 * self.m * self.n * self.k

    def setup(self, dev):
        from lego_b200 import ops
        self.ops = ops
        self.a_host, self.b_host = inputs.gemm_input(self.m, self.n, self.k)
        self.a, self.b = self.a_host.to(dev), self.b_host.to(dev)
        self.order = ops.grouped_swizzle_layout(self.m // 128, self.n // 256, 8)

    def step(self, i):
        self.c = self.ops.matmul(self.a, self.b, tile_order=self.order)

    def check(self):
        self.ops.device_status()
        rows = torch.tensor([0, 129, self.m // 2 + 1, self.m - 1])
        ref = self.a_host[rows].float() @ self.b_host.float()
        got = self.c[rows.to(self.c.device)].cpu().float()
        err = ((got - ref).norm() / ref.norm()).item()
        return err <= 1e-3, f"rel-Frobenius {err:.2e} on 4 rows vs oracle (tol 1e-3)"

    def e2e_setup(self):
        self.ap, self.bp = self.a_host.pin_memory(), self.b_host.pin_memory()
        return (self.ap.numel() + self.bp.numel()) * 2, self.m * self.n * 2

    def e2e_step(self, i):
        return self.ops.matmul(self.ap, self.bp)  # default tile order = the same swizzle, per row block

    def cpu_sample(self, threads, budget=4.0):
        m = 1024
        a = self.a_host[:m].float()
        b = self.b_host.float()
        t0 = time.perf_counter()
        n = 0
        while time.perf_counter() - t0 < budget:
            a @ b
            n += 1
        dt = time.perf_counter() - t0
        return 2.0 * m * self.n * self.k * n, dt, f"{n} x (A[:{m}].float() @ B.float()) of the 8192^3 problem"


class GemmE5M2(Gemm):
    name = "gemm_e5m2_8192"
    short = "gemm_e5m2"
    dtype = "f8e5m2"
    peak_scale = 2.0   # no measured fp8 peak on file: twice the measured bf16 figure (the tensor cores' nominal ratio)
    description = ("C = A.B, e5m2 operands 8192^3 (the fp16 inputs of the GEMM workload scaled by 64 and rounded to e5m2), "
                   "fp32 accumulate (tcgen05 kind::f8f6f4), fp16 C, 128 x 256 tiles, tile order = LEGO grouped swizzle "
                   "GROUP_M = 8; operands (256 MiB) larger than L2")

    def setup(self, dev):
        super().setup(dev)
        self.a_host = (self.a_host * 64).to(torch.float8_e5m2)
        self.b_host = (self.b_host * 64).to(torch.float8_e5m2)
        self.a, self.b = self.a_host.to(dev), self.b_host.to(dev)

    def check(self):
        self.ops.device_status()
        rows = torch.tensor([0, 129, self.m // 2 + 1, self.m - 1])
        ref = self.a_host[rows].float() @ self.b_host.float()
        got = self.c[rows.to(self.c.device)].cpu().float()
        err = ((got - ref).norm() / ref.norm()).item()
        return err <= 1e-3, f"rel-Frobenius {err:.2e} on 4 rows vs fp32 product of the e5m2 values (tol 1e-3)"

    def e2e_setup(self):
        self.ap, self.bp = self.a_host.pin_memory(), self.b_host.pin_memory()
        return self.ap.numel() + self.bp.numel(), self.m * self.n * 2

    def cpu_sample(self, threads, budget=4.0):
        m = 1024
        a = self.a_host[:m].float()
        b = self.b_host.float()
        t0 = time.perf_counter()
        n = 0
        while time.perf_counter() - t0 < budget:
            a @ b
            n += 1
        dt = time.perf_counter() - t0
        return 2.0 * m * self.n * self.k * n, dt, f"{n} x (e5m2 -> fp32) a @ b on {m} of {self.m} rows of A"


class GroupedGemm(Workload):
    name = "grouped_gemm_f16_16groups"
    unit = "TFLOP/s"
    bound = "tensor"
    description = ("16 independent fp16 GEMMs, M,N drawn from {1024,2048,4096} seed 4, K = 4096, inputs ~ N(0,1/64), "
                   "fp32 accumulate; persistent CTAs walk (group, tile_m, tile_n), per-group order OrderBy(Row(M/128, N/256)) as in the reference; operands larger than L2")

    def work(self):
        return float(sum(2 * m * n * k for m, n, k in self.sizes))

    def setup(self, dev):
        import lego_b200 as L
        from lego_b200 import ops
        self.ops = ops
        self.sizes, _ = inputs.grouped_sizes()
        self.A_host, self.B_host = inputs.grouped_input()
        self.A = [t.to(dev) for t in self.A_host]
        self.B = [t.to(dev) for t in self.B_host]
        self.orders = [L.OrderBy(L.Row(m // 128, n // 256)).TileBy([m // 128, n // 256]) for m, n, _ in self.sizes]

    def step(self, i):
        self.C = self.ops.lego_group_gemm_fn(self.A, self.B, self.orders)

    def check(self):
        self.ops.device_status()
        worst = 0.0
        for g in (0, 4, 13):
            ref = self.A_host[g][:64].float() @ self.B_host[g].float()
            got = self.C[g][:64].cpu().float()
            worst = max(worst, ((got - ref).norm() / ref.norm()).item())
        return worst <= 1e-3, f"rel-Frobenius {worst:.2e} on 64 rows of 3 groups vs oracle (tol 1e-3)"

    def e2e_setup(self):
        self.Ap = [t.pin_memory() for t in self.A_host]
        self.Bp = [t.pin_memory() for t in self.B_host]
        h2d = sum(t.numel() for t in self.Ap + self.Bp) * 2
        d2h = sum(m * n for m, n, _ in self.sizes) * 2
        return h2d, d2h

    def e2e_step(self, i):
        return self.ops.lego_group_gemm_fn(self.Ap, self.Bp, self.orders)

    def cpu_sample(self, threads, budget=4.0):
        a = self.A_host[4].float()
        b = self.B_host[4].float()
        t0 = time.perf_counter()
        n = 0
        while time.perf_counter() - t0 < budget:
            a @ b
            n += 1
        dt = time.perf_counter() - t0
        m, nn, k = self.sizes[4]
        return 2.0 * m * nn * k * n, dt, f"{n} x group 4 ({m}x{nn}x{k}) as a.float() @ b.float()"


class IndexMap(Workload):
    graph_ok = True
    name = "index_map_range_i64_4096x4096"
    short = "index_map"
    dtype = "int64"
    description = ("index-map evaluator: layout.apply over all 2^24 logical ids of OrderBy(Col(4096,4096))"
                   ".TileBy([128,128],[32,32]) (the transpose's destination layout), int64 results (128 MiB, larger than L2)")

    def work(self):
        return 8.0 * (1 << 24)

    def setup(self, dev):
        import lego_b200 as L
        from lego_b200 import ops
        self.ops = ops
        self.layout = L.OrderBy(L.Col(4096, 4096)).TileBy([128, 128], [32, 32])

    def step(self, i):
        self.flat = self.ops.eval_range(self.layout)

    def check(self):
        from oracle import lego_oracle as O
        from helpers import spec_of
        ids = torch.arange(0, 1 << 24, 4099)
        idx = [v.numpy() for v in torch.unravel_index(ids, self.layout.dims())]
        ref = O.groupby_apply(spec_of(self.layout), idx)
        ok = bool((self.flat[ids.to(self.flat.device)].cpu().numpy() == ref).all())
        return ok, f"bit-exact on {len(ids)} sampled ids vs oracle"

    def e2e_setup(self):
        return 0, 8 * (1 << 24)

    def e2e_step(self, i):
        return self.ops.eval_range(self.layout, host=True)

    def cpu_sample(self, threads, budget=4.0):
        from oracle import lego_oracle as O
        from helpers import spec_of
        n = 1 << 22
        t0 = time.perf_counter()
        ids = np.arange(n, dtype=np.int64)
        O.groupby_apply(spec_of(self.layout), O.unflatten_index(ids, list(self.layout.dims())))
        dt = time.perf_counter() - t0
        return 8.0 * n, dt, "1 x numpy GroupBy.apply over 2^22 of the 2^24 ids (single thread)"


WORKLOADS = {"softmax": Softmax, "layernorm": LayerNorm, "layernorm_bwd": LayerNormBwd, "transpose": Transpose, "gemm": Gemm, "gemm_e5m2": GemmE5M2,
             "grouped_gemm": GroupedGemm, "index_map": IndexMap}


# --------------------------------------------------------------------------------------
# measurement helpers
# --------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm": p["hbm_gbs"], "tensor_burst": p["bf16_tflops"], "tensor_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm": 6650.0, "tensor_burst": 1590.0, "tensor_sustained": 1400.0, "source": "fallback"}


def recorded_traffic(name):
    """DRAM bytes per launch of a workload's kernel from the committed ncu summary, if any."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get(name)
    return None


def time_steps(fn, steps, warmup, dist_ctx, graph=False):
    """Device time of `steps` calls of fn(i): CUDA events on the launching stream,
    barrier + synchronize on both sides, max over ranks.  Returns seconds.  With
    graph=True the `steps` launches are captured once in a CUDA graph and the
    timed region is its replay, so host launch overhead is not in the number."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    g = None
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(steps):
                fn(warmup + i)
        g.replay()
        torch.cuda.synchronize()
    if dist_ctx:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    if g is not None:
        g.replay()
    else:
        for i in range(steps):
            fn(warmup + i)
    end.record()
    torch.cuda.synchronize()
    if dist_ctx:
        torch.distributed.barrier()
    ms = start.elapsed_time(end)
    if dist_ctx:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    return ms / 1e3


def run_workload(w: Workload, args, dev, n_gpus, rank, dist_ctx, peaks, with_cpu, with_e2e):
    w.setup(dev)
    w.step(0)
    torch.cuda.synchronize()
    ok, parity = w.check()
    sec = time_steps(w.step, args.steps, args.warmup, dist_ctx, graph=(w.graph_ok and not args.no_graph))
    per_step = sec / args.steps
    value = _rate(w.work() * n_gpus, per_step, w.unit)
    # One kernel per step everywhere except LayerNorm backward, whose short column reduction
    # is charged to the dominant (dx) kernel: the algorithmic bytes over the whole step.
    achieved = _rate(w.work(), per_step, w.unit)
    if w.bound == "hbm":
        peak, which = peaks["hbm"], "copy bandwidth"
    else:
        peak, which = peaks["tensor_sustained"], "cuBLAS bf16 sustained (kernel timed inside a seconds-long loop)"
        if getattr(w, "peak_scale", 1.0) != 1.0:
            peak, which = peak * w.peak_scale, which + f" x {w.peak_scale:g} for 8-bit operands"
    res = {
        "workload": w.name, "metric": w.metric(), "value": value, "unit": w.unit,
        "ms_per_step": per_step * 1e3, "dtype": w.dtype, "parity": parity, "parity_ok": bool(ok),
        "roofline": {"bound": w.bound, "achieved": achieved, "peak": peak, "unit": w.unit, "frac": achieved / peak,
                     "traffic": recorded_traffic(w.name), "peak_source": f"{peaks['source']}: {which}"},
        "gpu_launches": args.steps * w.kernels_per_step,
        "timed_as": "cuda graph replay" if (w.graph_ok and not args.no_graph) else "stream launches",
        "description": w.description,
    }
    if w.bound == "tensor":
        res["roofline"]["frac_of_burst"] = achieved / (peaks["tensor_burst"] * getattr(w, "peak_scale", 1.0))
    if with_e2e:
        h2d, d2h = w.e2e_setup()
        e_steps = max(3, min(args.steps, 10))
        sec_e = time_steps(w.e2e_step, e_steps, 3, dist_ctx)
        res["e2e"] = {"value": _rate(w.work() * n_gpus, sec_e / e_steps, w.unit), "unit": w.unit,
                      "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                      "ms_per_step": sec_e / e_steps * 1e3}
    if with_cpu and rank == 0:
        threads = torch.get_num_threads()
        work, dt, what = w.cpu_sample(threads)
        res["cpu_baseline"] = {"value": _rate(work, dt, w.unit), "unit": w.unit, "cores": threads, "kind": "port",
                               "sample": what}
    return res


def reference_arm(args, rank):
    """The reference's CPU path on the host cores, same metric and config."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    w = WORKLOADS[args.workload]()
    w.setup(torch.device("cpu"))
    threads = torch.get_num_threads()
    rates = []
    what = ""
    budget = min(4.0, 150.0 / (args.warmup + args.steps))
    for i in range(args.warmup + args.steps):
        work, dt, what = w.cpu_sample(threads, budget)
        if i >= args.warmup:
            rates.append((work, dt))
    work = sum(r[0] for r in rates)
    dt = sum(r[1] for r in rates)
    value = _rate(work, dt, w.unit)
    line = {"impl": "reference", "metric": w.metric(), "value": value, "unit": w.unit,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / max(1, args.steps) * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": {"workload": w.name, "description": w.description},
            "cpu_baseline": {"value": value, "unit": w.unit, "cores": threads, "kind": "port", "sample": what},
            "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="softmax", choices=sorted(WORKLOADS))
    ap.add_argument("--only", action="store_true", help="measure the headline workload only")
    ap.add_argument("--no-graph", action="store_true", help="time plain stream launches instead of a graph replay")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--small", action="store_true",
                    help="halve the row / matrix sizes (for profiler captures; not a bench configuration)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        reference_arm(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist_ctx = world > 1
    if dist_ctx:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=dev)
    n_gpus = world

    peaks = measured_peaks()
    if args.small:
        Softmax.rows = LayerNorm.rows = LayerNormBwd.rows = 8192
        Gemm.m = Gemm.n = Gemm.k = 4096
    head = WORKLOADS[args.workload]()
    with ClockSampler(local_rank) as clocks:
        res = run_workload(head, args, dev, n_gpus, rank, dist_ctx, peaks,
                           with_cpu=(n_gpus == 1 and not args.no_cpu), with_e2e=not args.no_e2e)
    clock_summary = clocks.summary()
    others = {}
    if not args.only:
        for name, cls in WORKLOADS.items():
            if name == args.workload:
                continue
            del head
            head = None
            torch.cuda.empty_cache()
            w = cls()
            with ClockSampler(local_rank) as c2:
                r = run_workload(w, args, dev, n_gpus, rank, dist_ctx, peaks,
                                 with_cpu=(n_gpus == 1 and not args.no_cpu), with_e2e=not args.no_e2e)
            r["clocks"] = c2.summary()
            others[name] = r
            del w

    if rank == 0:
        line = {
            "metric": res["metric"], "value": res["value"], "unit": res["unit"], "n_gpus": n_gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": res["dtype"],
            "data": "synthetic",
            "config": {"workload": res["workload"], "description": res["description"],
                       "l2_policy": "inputs larger than L2 (transpose rotates 4 buffer pairs)",
                       "sharding": "each rank runs the full named shape on its own GPU (independent rows / tiles; "
                                   "no data-path collective)"},
            "roofline": res["roofline"], "e2e": res.get("e2e"), "gpu_launches": res["gpu_launches"],
            "timed_as": res["timed_as"],
            "clocks": clock_summary, "parity": res["parity"], "parity_ok": res["parity_ok"],
            "workloads": others,
        }
        if "cpu_baseline" in res:
            line["cpu_baseline"] = res["cpu_baseline"]
        print(json.dumps(line), flush=True)
    if dist_ctx:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
