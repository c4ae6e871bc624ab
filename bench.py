#!/usr/bin/env python
"""Benchmark of the LEGO hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload softmax] [--impl reference]

A step is one pass of one kernel over one batch of seeded synthetic input.  The
headline workload is the row-wise softmax (fp16, 16384 x 8192); the other four
configurations (tiled transpose, LayerNorm, GEMM 8192^3, grouped GEMM), LayerNorm
backward, the e5m2 GEMM and the index-map evaluator are measured in the same run and
reported under "workloads".

With N > 1 (one process per GPU, launched by torch.distributed.run) every named shape is
SPLIT across the ranks -- rows for the row-wise kernels, output-row slabs for the
transpose, M for the GEMM with B replicated, 512-row blocks of the groups packed by weight
for the grouped GEMM, id ranges for the index map -- with no data-path collective: "scaling": "strong", value =
the named shape's work / the slowest rank's device time.  After the timed region the
shards are gathered over NCCL and rank 0 checks the assembled result against the oracle.
The replica figure (every rank the full shape, "weak") is reported beside it.

Timing: R replays (default 10) of a CUDA graph of L = max(K, 100) launches, one CUDA-event
pair per replay on the launching stream, barrier + synchronize before each replay, max
over ranks per replay, then the median over replays.  Rank 0 prints ONE JSON line on
stdout; a detailed record per workload goes to stderr.  With --impl reference the
reference's CPU path (index maps in numpy as lego_python prints them + torch CPU ops) is
timed on the host cores at the full named shape.
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

from lego_b200 import configs as inputs  # noqa: E402  (seeded builders of the five configurations)
from lego_b200 import shard  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
MIN_LAUNCHES = 100
REPLAYS = 10


def log(*a):
    print(*a, file=sys.stderr, flush=True)


# --------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------

class Workload:
    name = ""
    unit = "GB/s"
    bound = "hbm"
    dtype = "f16"
    kernels_per_step = 1
    graph_ok = True    # the step can be captured in a CUDA graph (no host-to-device copy inside)
    peak_scale = 1.0

    def work(self) -> float:
        """Algorithmic bytes (or flops) of one pass over the whole named shape."""
        raise NotImplementedError

    def metric(self) -> str:
        kind = "HBM GB/s" if self.unit == "GB/s" else "TFLOP/s"
        return f"{getattr(self, 'short', self.name.split('_f')[0])} {kind}"

    def setup(self, dev, rank, world):
        """Create this rank's shard of the inputs (the whole shape when world == 1)."""
        raise NotImplementedError

    def step(self, i: int):
        raise NotImplementedError

    def shard_result(self):
        """This rank's part of the result as one contiguous tensor (equal sizes on every rank)."""
        raise NotImplementedError

    def check(self, full):
        """Rank 0: the assembled result against the oracle -> (ok, text)."""
        raise NotImplementedError

    def e2e_setup(self):
        raise NotImplementedError

    def e2e_step(self, i: int):
        raise NotImplementedError

    def cpu_pass(self):
        """One pass of the reference's CPU path over the whole named shape: (work, seconds, what)."""
        raise NotImplementedError

    def comparators(self):
        """name -> callable(i) of same-box library kernels doing the same work (never a product path)."""
        return {}

    @staticmethod
    def n_sets(bytes_per_set):
        """Rotating buffer sets so that consecutive launches never find their data in L2."""
        return max(1, min(64, math.ceil(3 * L2_BYTES / max(1, bytes_per_set))))


def _rate(work: float, seconds: float, unit: str) -> float:
    return work / seconds / (1e9 if unit == "GB/s" else 1e12)


def _timed(fn):
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


class _Rows(Workload):
    rows, cols = 16384, 8192

    def _rows_setup(self, rank, world):
        self.rank, self.world = rank, world
        self.r0, self.r1 = shard.shard_rows(self.rows, rank, world)
        self.sets = self.n_sets(2 * (self.r1 - self.r0) * self.cols * 2)
        self.keep = [None] * (self.sets + 1)


class Softmax(_Rows):
    name = "softmax_f16_16384x8192"

    def work(self):
        return 2.0 * self.rows * self.cols * 2

    def setup(self, dev, rank, world):
        from lego_b200 import ops
        self.ops = ops
        self._rows_setup(rank, world)
        self.x_host = inputs.softmax_input(self.rows, self.cols)
        xs = self.x_host[self.r0:self.r1]
        self.x = [xs.to(dev) for _ in range(self.sets)]
        self.row_map = ops.row_tiling_layout(self.r1 - self.r0, 4)

    def step(self, i):
        k = i % self.sets
        self.keep[i % len(self.keep)] = self.y = self.ops.softmax(self.x[k], self.row_map)

    def shard_result(self):
        return self.y

    def check(self, full):
        from oracle import lego_oracle as O
        sel = torch.arange(0, self.rows, 257)
        err = (full[sel.to(full.device)].cpu().float() - O.softmax(self.x_host[sel]).float()).abs().max().item()
        return err <= 1e-3, f"max-abs {err:.2e} on {len(sel)} rows vs oracle (tol 1e-3)"

    def e2e_setup(self):
        self.x_pinned = self.x_host[self.r0:self.r1].contiguous().pin_memory()
        return self.x_pinned.numel() * 2, self.x_pinned.numel() * 2

    def e2e_step(self, i):
        return self.ops.softmax(self.x_pinned, self.row_map)

    def cpu_pass(self):
        x = self.x_host
        dt = _timed(lambda: torch.softmax(x.float(), dim=-1).half())
        return self.work(), dt, f"torch.softmax(x.float(),-1).half() on all {self.rows} rows"

    def comparators(self):
        return {"torch.softmax": lambda i: torch.softmax(self.x[i % self.sets], dim=-1),
                "d2d_copy": _copy_comparator(self.x[0], self.sets)}


class SoftmaxF32(Softmax):
    """The precision the reference's own softmax table was measured in (softmax.py:238,271); used by --sweep."""
    name = "softmax_f32"
    short = "softmax_f32"
    dtype = "f32"

    def work(self):
        return 2.0 * self.rows * self.cols * 4

    def setup(self, dev, rank, world):
        from lego_b200 import ops
        self.ops = ops
        self._rows_setup(rank, world)
        self.sets = self.n_sets(2 * (self.r1 - self.r0) * self.cols * 4)
        self.keep = [None] * (self.sets + 1)
        self.x_host = inputs.softmax_input(self.rows, self.cols).float()
        xs = self.x_host[self.r0:self.r1]
        self.x = [xs.to(dev) for _ in range(self.sets)]
        self.row_map = ops.row_tiling_layout(self.r1 - self.r0, 4)

    def check(self, full):
        sel = torch.arange(0, self.rows, 257)
        err = (full[sel.to(full.device)].cpu() - torch.softmax(self.x_host[sel], dim=-1)).abs().max().item()
        return err <= 1e-6, f"max-abs {err:.2e} on {len(sel)} rows vs torch CPU fp32 (tol 1e-6)"


def _copy_comparator(like, sets):
    src = [torch.empty_like(like) for _ in range(sets)]
    dst = [torch.empty_like(like) for _ in range(sets)]
    return lambda i: dst[i % sets].copy_(src[i % sets])


class LayerNorm(_Rows):
    name = "layernorm_fwd_f16_16384x8192"

    def work(self):
        return 2.0 * self.rows * self.cols * 2

    def setup(self, dev, rank, world):
        from lego_b200 import ops
        self.ops = ops
        self._rows_setup(rank, world)
        self.x_host, self.g_host, self.b_host = inputs.layernorm_input(self.rows, self.cols)
        xs = self.x_host[self.r0:self.r1]
        self.x = [xs.to(dev) for _ in range(self.sets)]
        self.g, self.b = self.g_host.to(dev), self.b_host.to(dev)
        self.row_map = ops.row_tiling_layout(self.r1 - self.r0, 4)

    def step(self, i):
        self.keep[i % len(self.keep)] = self.out = self.ops.layer_norm_fwd(self.x[i % self.sets], self.g, self.b,
                                                                           1e-5, self.row_map)

    def shard_result(self):
        return self.out[0]

    def check(self, full):
        from oracle import lego_oracle as O
        sel = torch.arange(0, self.rows, 257)
        ref = O.layernorm_fwd(self.x_host[sel], self.g_host, self.b_host, 1e-5, round_output=False)[0]
        err = (full[sel.to(full.device)].cpu().float() - ref).abs()
        ok = bool((err <= 1e-3 + ref.abs() * 2.0 ** -11).all())
        small = err[ref.abs() < 2].max().item()
        return ok, (f"max-abs {small:.2e} where |y| < 2 on {len(sel)} rows vs fp32 oracle (tol 1e-3; beyond, "
                    f"1e-3 + half an fp16 ulp of y)")

    def e2e_setup(self):
        self.xp = self.x_host[self.r0:self.r1].contiguous().pin_memory()
        return self.xp.numel() * 2 + 2 * self.cols * 2, self.xp.numel() * 2 + 2 * (self.r1 - self.r0) * 4

    def e2e_step(self, i):
        return self.ops.layer_norm_fwd(self.xp, self.g_host, self.b_host, 1e-5, self.row_map)

    def cpu_pass(self):
        x, g, b = self.x_host, self.g_host.float(), self.b_host.float()
        dt = _timed(lambda: torch.nn.functional.layer_norm(x.float(), (self.cols,), g, b, 1e-5).half())
        return self.work(), dt, f"F.layer_norm fp32 on all {self.rows} rows"

    def comparators(self):
        F = torch.nn.functional
        return {"F.layer_norm": lambda i: F.layer_norm(self.x[i % self.sets], (self.cols,), self.g, self.b, 1e-5),
                "d2d_copy": _copy_comparator(self.x[0], self.sets)}


class LayerNormBwd(_Rows):
    name = "layernorm_bwd_f16_16384x8192"
    short = "layernorm_bwd"
    kernels_per_step = 2   # dx + column partials, then the column reduction

    def work(self):
        return 3.0 * self.rows * self.cols * 2   # x and dy read, dx written (the reference's formula)

    def setup(self, dev, rank, world):
        from lego_b200 import ops
        self.ops = ops
        self._rows_setup(rank, world)
        self.sets = self.n_sets(3 * (self.r1 - self.r0) * self.cols * 2)
        self.keep = [None] * (self.sets + 1)
        self.x_host, self.g_host, self.b_host = inputs.layernorm_input(self.rows, self.cols)
        self.dy_host = (0.1 * torch.randn(self.rows, self.cols, generator=torch.Generator().manual_seed(22))).half()
        xs, dys = self.x_host[self.r0:self.r1], self.dy_host[self.r0:self.r1]
        self.x = [xs.to(dev) for _ in range(self.sets)]
        self.dy = [dys.to(dev) for _ in range(self.sets)]
        self.g = self.g_host.to(dev)
        self.bdev = self.b_host.to(dev)
        _, self.mean, self.rstd = ops.layer_norm_fwd(self.x[0], self.g, self.bdev, 1e-5)

    def step(self, i):
        k = i % self.sets
        self.keep[i % len(self.keep)] = self.out = self.ops.layer_norm_bwd(self.dy[k], self.x[k], self.g, self.mean,
                                                                           self.rstd)

    def shard_result(self):
        # dx rows, then this rank's partial dgamma / dbeta as two more rows (summed over ranks by the check)
        return torch.cat([self.out[0], self.out[1][None], self.out[2][None]])

    def check(self, full):
        from oracle import lego_oracle as O
        per = (self.r1 - self.r0) + 2
        parts = full.reshape(self.world, per, self.cols)
        dx = parts[:, :per - 2].reshape(-1, self.cols)
        dw = parts[:, per - 2].float().sum(0).cpu().double()
        db = parts[:, per - 1].float().sum(0).cpu().double()
        sel = torch.arange(0, self.rows, 257)
        _, mean, rstd = O.layernorm_fwd(self.x_host[sel], self.g_host, self.b_host, 1e-5)
        rdx, _, _ = O.layernorm_bwd(self.dy_host[sel], self.x_host[sel], self.g_host, mean, rstd)
        err = (dx[sel.to(dx.device)].cpu().float() - rdx.float()).abs().max().item()
        # column sums over all rows, against fp64 sums of a strided sample of columns
        cols = torch.arange(0, self.cols, 263)
        _, mean_all, rstd_all = O.layernorm_fwd(self.x_host, self.g_host, self.b_host, 1e-5)
        xs, dys = self.x_host[:, cols].double(), self.dy_host[:, cols].double()
        m, r = mean_all.double()[:, None], rstd_all.double()[:, None]
        dw_ref, db_ref = (dys * (xs - m) * r).sum(0), dys.sum(0)
        ew = ((dw[cols] - dw_ref).abs().max() / dw_ref.abs().max()).item()
        eb = ((db[cols] - db_ref).abs().max() / db_ref.abs().max()).item()
        ok = err <= 1e-3 and ew <= 2e-3 and eb <= 2e-3
        return ok, (f"dx max-abs {err:.2e} on {len(sel)} rows vs oracle (tol 1e-3); dgamma / dbeta rel-to-max "
                    f"{ew:.1e} / {eb:.1e} on {len(cols)} columns vs fp64 sums (tol 2e-3)")

    def e2e_setup(self):
        n = self.r1 - self.r0
        self.xp = self.x_host[self.r0:self.r1].contiguous().pin_memory()
        self.dyp = self.dy_host[self.r0:self.r1].contiguous().pin_memory()
        self.mp, self.rp = self.mean.cpu().pin_memory(), self.rstd.cpu().pin_memory()
        return 2 * self.xp.numel() * 2 + self.cols * 2 + 2 * n * 4, self.xp.numel() * 2 + 2 * self.cols * 2

    def e2e_step(self, i):
        return self.ops.layer_norm_bwd(self.dyp, self.xp, self.g_host, self.mp, self.rp)

    def cpu_pass(self):
        from oracle import lego_oracle as O
        _, mean, rstd = O.layernorm_fwd(self.x_host, self.g_host, self.b_host, 1e-5)
        dt = _timed(lambda: O.layernorm_bwd(self.dy_host, self.x_host, self.g_host, mean, rstd))
        return self.work(), dt, f"oracle layernorm_bwd (torch fp32) on all {self.rows} rows"

    def comparators(self):
        def torch_bwd(i):
            k = i % self.sets
            return torch.ops.aten.native_layer_norm_backward(self.dy[k], self.x[k], [self.cols], self.mean[:, None],
                                                             self.rstd[:, None], self.g, self.bdev, [True, True, True])
        return {"aten.native_layer_norm_backward": torch_bwd}


class Transpose(Workload):
    name = "tiled_transpose_f32_4096"
    dtype = "f32"
    n = 4096

    def work(self):
        return 2.0 * self.n * self.n * 4

    def setup(self, dev, rank, world):
        import lego_b200 as L
        from lego_b200 import ops
        self.ops = ops
        self.rank, self.world = rank, world
        n, nt = self.n, self.n // 32
        self.a_host = inputs.transpose_input(n)
        self.src = L.OrderBy(L.Row(n, n)).TileBy([nt, nt], [32, 32])
        self.dst = L.OrderBy(L.Col(n, n)).TileBy([nt, nt], [32, 32])
        self.order = L.OrderBy(L.Col(nt, nt)).TileBy([nt, nt])
        # this rank's slab of OUTPUT rows = a range of ids of the column-major tile order
        self.r0, self.r1 = shard.shard_transpose(n, n, rank, world, 32)
        self.tiles = (self.r0 // 32 * nt, (self.r1 - self.r0) // 32 * nt)
        self.sets = self.n_sets(2 * (self.r1 - self.r0) * n * 4)
        self.ins = [self.a_host.to(dev) for _ in range(self.sets)]
        self.outs = [torch.empty_like(self.ins[0]) for _ in range(self.sets)]

    def step(self, i):
        k = i % self.sets
        self.ops.permute(self.ins[k], self.src, self.dst, self.order, out=self.outs[k],
                         tiles=None if self.world == 1 else self.tiles)

    def shard_result(self):
        return self.outs[0].reshape(self.n, self.n)[self.r0:self.r1].contiguous()

    def check(self, full):
        ok = torch.equal(full.cpu().reshape(self.n, self.n), self.a_host.t().contiguous())
        return ok, "bit-exact vs A.T"

    def e2e_setup(self):
        if self.world == 1:
            self.ap = self.a_host.pin_memory()
            return self.ap.numel() * 4, self.ap.numel() * 4
        # a rank's slab of output rows is a slab of input columns: a matrix of its own
        self.ap = self.a_host[:, self.r0:self.r1].contiguous().pin_memory()
        return self.ap.numel() * 4, self.ap.numel() * 4

    def e2e_step(self, i):
        return self.ops.transpose(self.ap)      # the same layouts and tile order, built by the op from the shape

    def cpu_pass(self):
        from oracle import lego_oracle as O
        x = self.a_host.reshape(-1).numpy()
        dt = _timed(lambda: O.permute(x, O.spec_of(self.src), O.spec_of(self.dst)))
        return self.work(), dt, "numpy index maps of both layouts over 4096^2 ids + gather/scatter (single thread)"

    def comparators(self):
        return {"x.t().contiguous()": lambda i: self.ins[i % self.sets].t().contiguous(),
                "d2d_copy": _copy_comparator(self.ins[0], self.sets)}


class Bricks(Workload):
    """The reference's brick re-layout (benchmarks/cuda/bricks_f3d.py:10-13): a 384^3 fp32 volume from
    row-major order into 8^3 bricks, one permute call.  Ranks split the slowest axis."""
    name = "bricks_relayout_f32_384"
    short = "bricks"
    dtype = "f32"
    n, b = 384, 8

    def work(self):
        return 2.0 * self.n ** 3 * 4

    def setup(self, dev, rank, world):
        import lego_b200 as L
        from lego_b200 import ops
        self.ops = ops
        self.rank, self.world = rank, world
        n, b = self.n, self.b
        self.r0, self.r1 = shard.split_range(n, rank, world, b)
        m = self.r1 - self.r0                                  # this rank's slab of planes is a volume of its own
        self.x_host = torch.rand(n, n, n, generator=torch.Generator().manual_seed(8))
        self.src = L.OrderBy(L.Row(m, n, n)).TileBy([m // b, n // b, n // b], [b, b, b])
        self.dst = L.OrderBy(L.Row(m // b, n // b, n // b), L.Row(b, b, b)).TileBy([m // b, n // b, n // b], [b, b, b])
        self.sets = self.n_sets(2 * m * n * n * 4)
        self.ins = [self.x_host[self.r0:self.r1].to(dev) for _ in range(self.sets)]
        self.outs = [torch.empty_like(self.ins[0]) for _ in range(self.sets)]

    def step(self, i):
        k = i % self.sets
        self.ops.permute(self.ins[k], self.src, self.dst, out=self.outs[k])

    def shard_result(self):
        return self.outs[0]

    def check(self, full):
        n, b = self.n, self.b
        want = self.x_host.reshape(n // b, b, n // b, b, n // b, b).permute(0, 2, 4, 1, 3, 5).contiguous()
        ok = torch.equal(full.cpu().reshape(-1), want.reshape(-1))
        return ok, "bit-exact vs reshape(48,8,48,8,48,8).permute(0,2,4,1,3,5)"

    def e2e_setup(self):
        self.xp = self.x_host[self.r0:self.r1].contiguous().pin_memory()
        return self.xp.numel() * 4, self.xp.numel() * 4

    def e2e_step(self, i):
        return self.ops.permute(self.xp, self.src, self.dst)

    def cpu_pass(self):
        from oracle import lego_oracle as O
        import lego_b200 as L
        n, b = self.n, self.b
        src = L.OrderBy(L.Row(n, n, n)).TileBy([n // b] * 3, [b] * 3)
        dst = L.OrderBy(L.Row(n // b, n // b, n // b), L.Row(b, b, b)).TileBy([n // b] * 3, [b] * 3)
        x = self.x_host.reshape(-1).numpy()
        dt = _timed(lambda: O.permute(x, O.spec_of(src), O.spec_of(dst)))
        return self.work(), dt, "numpy index maps of both layouts over 384^3 ids + gather/scatter (single thread)"

    def comparators(self):
        n, b = self.n, self.b

        def torch_relayout(i):
            return self.ins[i % self.sets].reshape(n // b, b, n // b, b, n // b, b).permute(0, 2, 4, 1, 3, 5).contiguous()
        return {"reshape.permute.contiguous": torch_relayout, "d2d_copy": _copy_comparator(self.ins[0], self.sets)}


class Gemm(Workload):
    name = "gemm_f16_8192"
    unit = "TFLOP/s"
    bound = "tensor"
    m = n = k = 8192

    def work(self):
        return 2.0 * self.m * self.n * self.k

    def _cast(self, t):
        return t

    def setup(self, dev, rank, world):
        from lego_b200 import ops
        self.ops = ops
        self.rank, self.world = rank, world
        self.a_host, self.b_host = inputs.gemm_input(self.m, self.n, self.k)
        self.a_host, self.b_host = self._cast(self.a_host), self._cast(self.b_host)
        self.r0, self.r1 = shard.shard_gemm_m(self.m, rank, world)
        self.a, self.b = self.a_host[self.r0:self.r1].to(dev), self.b_host.to(dev)
        self.order = ops.default_tile_order(self.r1 - self.r0, self.n, self.k, self.a.element_size())
        self.keep = [None] * 3

    def step(self, i):
        self.keep[i % 3] = self.c = self.ops.matmul(self.a, self.b, tile_order=self.order)

    def shard_result(self):
        return self.c

    def check(self, full):
        self.ops.device_status()
        rows = torch.tensor([0, 129, self.m // 2 + 1, self.m - 1])
        ref = self.a_host[rows].float() @ self.b_host.float()
        got = full[rows.to(full.device)].cpu().float()
        err = ((got - ref).norm() / ref.norm()).item()
        return err <= 1e-3, f"rel-Frobenius {err:.2e} on 4 rows vs oracle (tol 1e-3)"

    def e2e_setup(self):
        self.ap, self.bp = self.a_host[self.r0:self.r1].contiguous().pin_memory(), self.b_host.pin_memory()
        eb = self.ap.element_size()
        return (self.ap.numel() + self.bp.numel()) * eb, (self.r1 - self.r0) * self.n * 2

    def e2e_step(self, i):
        return self.ops.matmul(self.ap, self.bp)  # default tile order = the same swizzle, per row block

    def cpu_pass(self):
        a, b = self.a_host.float(), self.b_host.float()
        dt = _timed(lambda: a @ b)
        return self.work(), dt, "A.float() @ B.float() of the whole 8192^3 problem"

    def comparators(self):
        if self.a.dtype != torch.float16:
            return {}
        return {"torch.matmul(fp16)": lambda i: torch.matmul(self.a, self.b)}


class GemmE5M2(Gemm):
    name = "gemm_e5m2_8192"
    short = "gemm_e5m2"
    dtype = "f8e5m2"
    peak_scale = 2.0   # no measured fp8 peak on file: twice the measured bf16 figure (the tensor cores' nominal ratio)

    def _cast(self, t):
        return (t * 64).to(torch.float8_e5m2)

    def check(self, full):
        ok, text = super().check(full)
        return ok, text.replace("vs oracle", "vs fp32 product of the e5m2 values")


class GroupedGemm(Workload):
    name = "grouped_gemm_f16_16groups"
    unit = "TFLOP/s"
    bound = "tensor"
    graph_ok = False   # the call uploads its problem table from host memory
    groups, k = 16, 4096

    def work(self):
        return float(sum(2 * m * n * k for m, n, k in self.sizes))

    def setup(self, dev, rank, world):
        import lego_b200 as L
        from lego_b200 import ops
        self.ops = ops
        self.rank, self.world = rank, world
        self.sizes, _ = inputs.grouped_sizes(self.groups, self.k)
        self.A_host, self.B_host = inputs.grouped_input(self.groups, self.k)
        # one rank: the 16 groups as they are.  Several: 512-row blocks of the groups, packed by weight.
        self.packing = ([[(g, 0, m) for g, (m, _n, _k) in enumerate(self.sizes)]] if world == 1
                        else shard.pack_grouped_gemm_blocks(self.sizes, world, 512))
        self.mine = self.packing[rank]
        self.A = [self.A_host[g][b:e].to(dev) for g, b, e in self.mine]
        b_dev = {g: self.B_host[g].to(dev) for g in sorted({g for g, _, _ in self.mine})}
        self.B = [b_dev[g] for g, _, _ in self.mine]
        # in-group tile order: column-major LEGO layout over the (M/128, N/256) tile grid
        self.orders = [L.OrderBy(L.Col(-(-(e - b) // 128), self.sizes[g][1] // 256)).TileBy(
            [-(-(e - b) // 128), self.sizes[g][1] // 256]) for g, b, e in self.mine]
        self.slot = max(sum((e - b) * self.sizes[g][1] for g, b, e in p) for p in self.packing)
        self.keep = [None] * 3

    def step(self, i):
        self.keep[i % 3] = self.C = self.ops.lego_group_gemm_fn(self.A, self.B, self.orders)

    def shard_result(self):
        flat = torch.cat([c.reshape(-1) for c in self.C])
        out = torch.zeros(self.slot, dtype=flat.dtype, device=flat.device)   # ranks' results differ in size
        out[:flat.numel()] = flat
        return out

    def check(self, full):
        self.ops.device_status()
        where = {}                                   # (group, row_begin) -> offset of that block in `full`
        for r, blocks in enumerate(self.packing):
            off = r * self.slot
            for g, b, e in blocks:
                where[(g, b)] = (off, e)
                off += (e - b) * self.sizes[g][1]
        worst = 0.0
        for g, (m, n, _k) in enumerate(self.sizes):  # 64 rows of EVERY group
            pick = torch.arange(0, m, max(1, m // 64))[:64]
            rows = []
            for r in pick.tolist():
                b0 = max(b for (gg, b) in where if gg == g and b <= r)
                off, _e = where[(g, b0)]
                rows.append(full[off + (r - b0) * n: off + (r - b0 + 1) * n])
            got = torch.stack(rows).cpu().float()
            ref = self.A_host[g][pick].float() @ self.B_host[g].float()
            worst = max(worst, ((got - ref).norm() / ref.norm()).item())
        return worst <= 1e-3, (f"rel-Frobenius {worst:.2e} (worst group) on 64 rows of each of the "
                               f"{len(self.sizes)} groups vs oracle (tol 1e-3)")

    def e2e_setup(self):
        self.Ap = [self.A_host[g][b:e].contiguous().pin_memory() for g, b, e in self.mine]
        b_pin = {g: self.B_host[g].pin_memory() for g in sorted({g for g, _, _ in self.mine})}
        self.Bp = [b_pin[g] for g, _, _ in self.mine]
        h2d = sum(t.numel() for t in self.Ap + self.Bp) * 2
        d2h = sum((e - b) * self.sizes[g][1] for g, b, e in self.mine) * 2
        return h2d, d2h

    def e2e_step(self, i):
        return self.ops.lego_group_gemm_fn(self.Ap, self.Bp, self.orders)

    def cpu_pass(self):
        A = [t.float() for t in self.A_host]
        B = [t.float() for t in self.B_host]
        dt = _timed(lambda: [a @ b for a, b in zip(A, B)])
        return self.work(), dt, "a.float() @ b.float() for each of the 16 groups"

    def comparators(self):
        return {"torch.matmul loop": lambda i: [torch.matmul(a, b) for a, b in zip(self.A, self.B)]}


class IndexMap(Workload):
    name = "index_map_range_i64_4096x4096"
    short = "index_map"
    dtype = "int64"
    size = 1 << 24

    def work(self):
        return 8.0 * self.size

    def setup(self, dev, rank, world):
        import lego_b200 as L
        from lego_b200 import ops
        self.ops = ops
        self.rank, self.world = rank, world
        self.layout = L.OrderBy(L.Col(4096, 4096)).TileBy([128, 128], [32, 32])
        self.b0, self.b1 = shard.split_range(self.size, rank, world, 1024)
        self.keep = [None] * (self.n_sets(8 * (self.b1 - self.b0)) + 1)

    def step(self, i):
        self.keep[i % len(self.keep)] = self.flat = self.ops.eval_range(self.layout, self.b0, self.b1 - self.b0)

    def shard_result(self):
        return self.flat

    def check(self, full):
        from oracle import lego_oracle as O
        ids = torch.arange(0, self.size, 4099)
        idx = [v.numpy() for v in torch.unravel_index(ids, self.layout.dims())]
        ref = O.groupby_apply(O.spec_of(self.layout), idx)
        ok = bool((full[ids.to(full.device)].cpu().numpy() == ref).all())
        return ok, f"bit-exact on {len(ids)} sampled ids vs oracle"

    def e2e_setup(self):
        return 0, 8 * (self.b1 - self.b0)

    def e2e_step(self, i):
        return self.ops.eval_range(self.layout, self.b0, self.b1 - self.b0, host=True)

    def cpu_pass(self):
        from oracle import lego_oracle as O
        spec = O.spec_of(self.layout)

        def run():
            ids = np.arange(self.size, dtype=np.int64)
            O.groupby_apply(spec, O.unflatten_index(ids, list(self.layout.dims())))
        return self.work(), _timed(run), "numpy GroupBy.apply over all 2^24 ids (single thread)"

    def comparators(self):
        n = self.b1 - self.b0
        bufs = [torch.empty(n, dtype=torch.int64, device="cuda") for _ in range(len(self.keep))]
        return {"fill_i64": lambda i: bufs[i % len(bufs)].fill_(i)}


class IndexInv(Workload):
    """layout.inv over flat positions: the multi-index of every element (lego_eval_inv)."""
    name = "index_inv_i64_4096x4096"
    short = "index_inv"
    dtype = "int64"
    size = 1 << 24

    def work(self):
        return 8.0 * (1 + 4) * self.size        # one int64 read, rank (4) int64 written per id

    def setup(self, dev, rank, world):
        import lego_b200 as L
        from lego_b200 import ops
        self.ops = ops
        self.rank, self.world = rank, world
        self.layout = L.OrderBy(L.Col(4096, 4096)).TileBy([128, 128], [32, 32])
        self.b0, self.b1 = shard.split_range(self.size, rank, world, 1024)
        n = self.b1 - self.b0
        self.sets = self.n_sets(40 * n)
        g = torch.Generator().manual_seed(6)
        self.flat_host = torch.randperm(self.size, generator=g)[self.b0:self.b1].contiguous()
        self.flat = [self.flat_host.to(dev) for _ in range(self.sets)]
        self.keep = [None] * (self.sets + 1)

    def step(self, i):
        self.keep[i % len(self.keep)] = self.idx = self.ops.eval_inv(self.layout, self.flat[i % self.sets])

    def shard_result(self):
        return self.idx

    def check(self, full):
        from oracle import lego_oracle as O
        g = torch.Generator().manual_seed(6)
        flat = torch.randperm(self.size, generator=g)
        pick = torch.arange(0, self.size, 4099)
        ref = O.groupby_inv(O.spec_of(self.layout), flat[pick].numpy())
        got = full[pick.to(full.device)].cpu().numpy()
        ok = all(bool((got[:, k] == ref[k]).all()) for k in range(4))
        return ok, f"bit-exact on {len(pick)} sampled positions vs oracle"

    def e2e_setup(self):
        self.fp = self.flat_host.pin_memory()
        n = self.b1 - self.b0
        return 8 * n, 32 * n

    def e2e_step(self, i):
        return self.ops.eval_inv(self.layout, self.fp)

    def cpu_pass(self):
        from oracle import lego_oracle as O
        spec = O.spec_of(self.layout)
        flat = torch.randperm(self.size, generator=torch.Generator().manual_seed(6)).numpy()
        return self.work(), _timed(lambda: O.groupby_inv(spec, flat)), "numpy GroupBy.inv over all 2^24 positions (single thread)"


WORKLOADS = {"softmax": Softmax, "layernorm": LayerNorm, "layernorm_bwd": LayerNormBwd, "transpose": Transpose,
             "gemm": Gemm, "gemm_e5m2": GemmE5M2, "grouped_gemm": GroupedGemm, "index_map": IndexMap, "index_inv": IndexInv,
             "bricks": Bricks}


# --------------------------------------------------------------------------------------
# measurement helpers
# --------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clocks, power and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

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
        sm, mx, power, reasons = [], [], [], set()
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
            if len(s) > 6:
                try:
                    power.append(float(s[6]))
                except ValueError:
                    pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        if power:
            out["power_w_max"] = max(power)
        return out


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


class Timer:
    """Device time of `replays` runs of `launches` calls of fn(i).  The launches are captured
    once in a CUDA graph (host launch overhead stays out of the number) when the step allows
    it, else issued on the stream.  Every replay is bracketed by its own CUDA-event pair on
    the launching stream, preceded by a barrier + synchronize; per replay the MAX over ranks
    is kept.  Returns the list of replay times in seconds."""

    def __init__(self, dist_ctx):
        self.dist = dist_ctx
        self.stream = torch.cuda.Stream()

    def run(self, fn, launches, replays, warmup, graph=True):
        s = self.stream
        s.wait_stream(torch.cuda.current_stream())
        times = []
        with torch.cuda.stream(s):
            for i in range(warmup):
                fn(i)
            s.synchronize()
            g = None
            if graph:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=s):
                    for i in range(launches):
                        fn(warmup + i)
                g.replay()
                s.synchronize()
            for _ in range(replays):
                if self.dist:
                    torch.distributed.barrier()
                torch.cuda.synchronize()
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record(s)
                if g is not None:
                    g.replay()
                else:
                    for i in range(launches):
                        fn(warmup + i)
                end.record(s)
                s.synchronize()
                times.append(start.elapsed_time(end))
            del g
        torch.cuda.current_stream().wait_stream(s)
        t = torch.tensor(times, dtype=torch.float64, device="cuda")
        if self.dist:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return [float(v) / 1e3 for v in t.tolist()]

    def sustained(self, fn, launches, seconds, warmup):
        """One event pair around back-to-back graph replays lasting at least `seconds`."""
        s = self.stream
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for i in range(warmup):
                fn(i)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                for i in range(launches):
                    fn(warmup + i)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(s)
            g.replay()
            end.record(s)
            s.synchronize()
            n = max(2, math.ceil(seconds * 1e3 / max(1e-3, start.elapsed_time(end))))
            if self.dist:
                torch.distributed.barrier()
            torch.cuda.synchronize()
            start.record(s)
            for _ in range(n):
                g.replay()
            end.record(s)
            s.synchronize()
            ms = start.elapsed_time(end)
            del g
        torch.cuda.current_stream().wait_stream(s)
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        if self.dist:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item()) / 1e3, n * launches


def host_ceiling(world, dist_ctx, seconds=0.5):
    """What the host side allows: every rank copies pinned memory to its GPU and back on two
    streams at once, no kernel in between.  Returns the whole-box rate in GB/s counted like the
    bandwidth workloads' e2e figure (bytes in + bytes out over the slowest rank's time)."""
    n = 64 << 20
    h_in = torch.empty(n, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(n, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(n, dtype=torch.uint8, device="cuda")
    d_out = torch.empty(n, dtype=torch.uint8, device="cuda")
    up, down = torch.cuda.Stream(), torch.cuda.Stream()

    def burst(reps):
        for _ in range(reps):
            with torch.cuda.stream(up):
                d_in.copy_(h_in, non_blocking=True)
            with torch.cuda.stream(down):
                h_out.copy_(d_out, non_blocking=True)
    burst(2)
    torch.cuda.synchronize()
    reps = 8
    if dist_ctx:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    burst(reps)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    t = torch.tensor([dt], dtype=torch.float64, device="cuda")
    if dist_ctx:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return 2.0 * n * reps * world / float(t.item()) / 1e9


def gather(t, world):
    """All ranks' equal-sized shards, concatenated along the first axis (NCCL over NVLink)."""
    if world == 1:
        return t
    t = t.contiguous()
    out = torch.empty((world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    if t.dtype in (torch.float8_e5m2,):
        torch.distributed.all_gather_into_tensor(out.view(torch.uint8), t.view(torch.uint8))
    else:
        torch.distributed.all_gather_into_tensor(out, t)
    return out


def run_workload(cls, args, dev, world, rank, timer, peaks, local_rank, headline=True):
    w = cls()
    launches = args.steps if args.profile else max(args.steps, MIN_LAUNCHES)
    w.setup(dev, rank, world)
    w.step(0)
    torch.cuda.synchronize()
    ok, parity = (True, "")
    if args.as_rank0_of:
        parity = f"not checked: one GPU running rank 0's shard of a world of {world}"
    else:
        full = gather(w.shard_result(), world)
        if rank == 0:
            ok, parity = w.check(full)
        del full
    graph = w.graph_ok and not args.no_graph
    with ClockSampler(local_rank) as clocks:
        times = timer.run(w.step, launches, args.replays, args.warmup, graph=graph)
    med = statistics.median(times)
    per_step = med / launches
    value = _rate(w.work(), per_step, w.unit)            # whole named shape / slowest rank's time
    per_gpu = value / world                              # what one GPU achieves on its shard
    if w.bound == "hbm":
        peak, which = peaks["hbm"], "copy bandwidth"
    else:
        peak = peaks["tensor_burst"] * w.peak_scale
        which = "cuBLAS bf16 burst (best single launch); the timed replays are shorter than a second each"
        if w.peak_scale != 1.0:
            which += f", x {w.peak_scale:g} for 8-bit operands"
    res = {
        "workload": w.name, "metric": w.metric(), "value": value, "unit": w.unit, "ms_per_step": per_step * 1e3,
        "dtype": w.dtype, "parity": parity, "parity_ok": bool(ok),
        "timed": {"launches_per_replay": launches, "replays": len(times), "median_ms": med * 1e3,
                  "min_ms": min(times) * 1e3, "max_ms": max(times) * 1e3,
                  "as": "cuda graph replay" if graph else "stream launches"},
        "roofline": {"bound": w.bound, "achieved": per_gpu, "peak": peak, "unit": w.unit, "frac": per_gpu / peak,
                     "traffic": recorded_traffic(w.name) if world == 1 and not args.shape else None,
                     "peak_source": f"{peaks['source']}: {which}"},
        "gpu_launches": launches * len(times) * w.kernels_per_step,
        "clocks": clocks.summary(),
    }
    if w.bound == "tensor" and graph and not args.no_sustained:
        with ClockSampler(local_rank) as c2:
            sec, n = timer.sustained(w.step, launches, 2.0, 2)
        v = _rate(w.work() * n / world, sec, w.unit)     # per GPU
        res["sustained"] = {"value": v * world, "per_gpu": v, "seconds": sec, "launches": n,
                            "peak": peaks["tensor_sustained"] * w.peak_scale,
                            "frac": v / (peaks["tensor_sustained"] * w.peak_scale),
                            "peak_source": f"{peaks['source']}: cuBLAS bf16 back to back for seconds under the power cap",
                            "clocks": c2.summary()}
    if args.as_rank0_of:
        del w
        torch.cuda.empty_cache()
        return res
    if not args.no_e2e and (world == 1 or headline):   # N ranks' host staging shares one box: headline only
        h2d, d2h = w.e2e_setup()
        e_launches = 5
        te = timer.run(w.e2e_step, e_launches, 3, 3, graph=False)
        sec_e = statistics.median(te) / e_launches
        res["e2e"] = {"value": _rate(w.work(), sec_e, w.unit), "unit": w.unit, "h2d_bytes_per_step": int(h2d),
                      "d2h_bytes_per_step": int(d2h), "ms_per_step": sec_e * 1e3}
    if world == 1 and not args.no_cmp:
        cmp_res = {}
        for name, fn in w.comparators().items():
            ring = [None] * 4   # results stay alive for a few launches: no output block is rewritten while in L2

            def call(i, fn=fn, ring=ring):
                ring[i % 4] = fn(i)
            tc = timer.run(call, launches, max(3, args.replays // 2), args.warmup, graph=True)
            del ring[:]
            cmp_res[name] = _rate(w.work(), statistics.median(tc) / launches, w.unit)
        res["comparators"] = cmp_res
    if world == 1 and rank == 0 and not args.no_cpu:
        threads = torch.get_num_threads()
        work, dt, what = w.cpu_pass()
        res["cpu_baseline"] = {"value": _rate(work, dt, w.unit), "unit": w.unit, "cores": threads, "kind": "port",
                               "sample": "1 x " + what}
    if world > 1 and not args.no_weak:
        # replicas: every rank the full named shape (per-GPU work fixed as N grows)
        del w
        torch.cuda.empty_cache()
        w = cls()
        w.setup(dev, 0, 1)
        tw = timer.run(w.step, launches, max(3, args.replays // 2), args.warmup, graph=graph)
        res["weak"] = {"value": _rate(w.work() * world, statistics.median(tw) / launches, w.unit), "unit": w.unit,
                       "scaling": "weak", "what": "every rank runs the full named shape"}
    del w
    torch.cuda.empty_cache()
    return res


def sweep(args, dev, timer, peaks):
    """The shapes of the reference's own result tables (result/triton/softmax.txt,
    result/triton/layernorm.txt: 4096 rows, fp16, the widths below), one GPU: our kernel and the
    library kernel for the same work, GB/s by the reference's byte count, buffer sets rotating
    past L2.  One JSON line on stdout, a row per shape on stderr."""
    rows = 4096
    table = []
    for cls, widths in ((SoftmaxF32, (512, 1024, 2048, 4096, 8192)),        # result/triton/softmax.txt:4-8 (fp32, as there)
                        (Softmax, (512, 1024, 2048, 4096, 8192)),           # the same widths in fp16
                        (LayerNorm, (1024, 2048, 4096, 8192)),              # result/triton/layernorm.txt:7-10
                        (LayerNormBwd, (1024, 2048, 4096, 8192))):          # result/triton/layernorm.txt:16-19
        for cols in widths:
            w = cls()
            w.rows, w.cols = rows, cols
            w.setup(dev, 0, 1)
            w.step(0)
            torch.cuda.synchronize()
            ok, _ = w.check(w.shard_result())
            launches = max(args.steps, MIN_LAUNCHES)
            t = statistics.median(timer.run(w.step, launches, args.replays, args.warmup, graph=True)) / launches
            rec = {"op": getattr(w, "short", w.name.split("_f")[0]), "rows": rows, "cols": cols,
                   "GB/s": round(_rate(w.work(), t, "GB/s"), 1), "us": round(t * 1e6, 2), "ok": bool(ok),
                   "frac": round(_rate(w.work(), t, "GB/s") / peaks["hbm"], 3)}
            for name, fn in w.comparators().items():
                if name == "d2d_copy":
                    continue
                ring = [None] * 4

                def call(i, fn=fn, ring=ring):
                    ring[i % 4] = fn(i)
                tc = statistics.median(timer.run(call, launches, 3, args.warmup, graph=True)) / launches
                rec[name] = round(_rate(w.work(), tc, "GB/s"), 1)
            table.append(rec)
            log(json.dumps(rec))
            del w
            inputs.clear_cache()
            torch.cuda.empty_cache()
    print(json.dumps({"sweep": "reference result tables, 4096 rows fp16", "rows": table}), flush=True)


def _rounded(x):
    """Floats to six significant digits: the one-line record stays under 3 KB."""
    if isinstance(x, float):
        return float(f"{x:.6g}")
    if isinstance(x, dict):
        return {k: _rounded(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_rounded(v) for v in x]
    return x


def brief(r):
    """The few numbers of a workload that go on the one-line record."""
    out = {"v": round(r["value"], 1), "u": r["unit"], "frac": round(r["roofline"]["frac"], 3),
           "ok": r["parity_ok"]}
    if "sustained" in r:
        out["sus"] = round(r["sustained"]["value"], 1)
        out["sus_frac"] = round(r["sustained"]["frac"], 3)
    if "e2e" in r:
        out["e2e"] = round(r["e2e"]["value"], 1)
    if "cpu_baseline" in r:
        out["cpu"] = round(r["cpu_baseline"]["value"], 2)
    if "comparators" in r:
        out["cmp"] = {k: round(v, 1) for k, v in r["comparators"].items()}
    if "weak" in r:
        out["weak"] = round(r["weak"]["value"], 1)
    return out


def reference_arm(args, rank):
    """The reference's CPU path on the host cores, same metric and config, whole named shape per step."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    w = WORKLOADS[args.workload]()
    _cpu_setup(w)
    threads = torch.get_num_threads()
    done = []
    what = ""
    t_begin = time.perf_counter()
    budget = 150.0
    for i in range(args.warmup + args.steps):
        work, dt, what = w.cpu_pass()
        if i >= args.warmup or not done:
            done.append((work, dt))
        if time.perf_counter() - t_begin > budget and done:
            break
    timed = done[-args.steps:]
    work = sum(r[0] for r in timed)
    dt = sum(r[1] for r in timed)
    value = _rate(work, dt, w.unit)
    line = {"impl": "reference", "metric": w.metric(), "value": value, "unit": w.unit,
            "n_gpus": args.gpus, "steps": len(timed), "warmup": args.warmup, "ms_per_step": dt / len(timed) * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": {"workload": w.name},
            "cpu_baseline": {"value": value, "unit": w.unit, "cores": threads, "kind": "port",
                             "sample": f"{len(timed)} x " + what},
            "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def _cpu_setup(w):
    """Host inputs of a workload without touching a GPU (the reference arm runs where there may be none)."""
    import lego_b200 as L
    if isinstance(w, Softmax):
        w.x_host = inputs.softmax_input(w.rows, w.cols)
    elif isinstance(w, LayerNormBwd):
        w.x_host, w.g_host, w.b_host = inputs.layernorm_input(w.rows, w.cols)
        w.dy_host = (0.1 * torch.randn(w.rows, w.cols, generator=torch.Generator().manual_seed(22))).half()
    elif isinstance(w, LayerNorm):
        w.x_host, w.g_host, w.b_host = inputs.layernorm_input(w.rows, w.cols)
    elif isinstance(w, Bricks):
        w.x_host = torch.rand(w.n, w.n, w.n, generator=torch.Generator().manual_seed(8))
    elif isinstance(w, Transpose):
        n, nt = w.n, w.n // 32
        w.a_host = inputs.transpose_input(n)
        w.src = L.OrderBy(L.Row(n, n)).TileBy([nt, nt], [32, 32])
        w.dst = L.OrderBy(L.Col(n, n)).TileBy([nt, nt], [32, 32])
    elif isinstance(w, Gemm):
        a, b = inputs.gemm_input(w.m, w.n, w.k)
        w.a_host, w.b_host = w._cast(a), w._cast(b)
    elif isinstance(w, GroupedGemm):
        w.sizes, _ = inputs.grouped_sizes(w.groups, w.k)
        w.A_host, w.B_host = inputs.grouped_input(w.groups, w.k)
    elif isinstance(w, (IndexMap, IndexInv)):
        w.layout = L.OrderBy(L.Col(4096, 4096)).TileBy([128, 128], [32, 32])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--replays", type=int, default=REPLAYS)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="softmax", choices=sorted(WORKLOADS))
    ap.add_argument("--only", action="store_true", help="measure the headline workload only")
    ap.add_argument("--no-graph", action="store_true", help="time plain stream launches instead of a graph replay")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-cmp", action="store_true", help="skip the same-box library comparators")
    ap.add_argument("--no-weak", action="store_true", help="skip the replica (weak-scaling) leg at N > 1")
    ap.add_argument("--no-sustained", action="store_true", help="skip the seconds-long leg of the GEMMs")
    ap.add_argument("--profile", action="store_true",
                    help="for profiler captures: exactly --steps launches in one replay, kernel legs only")
    ap.add_argument("--as-rank0-of", type=int, default=0, metavar="N",
                    help="one GPU, no process group: time rank 0's shard of a world of N (what a launch costs "
                         "when the named shape is split N ways); kernel legs only, nothing is gathered or checked")
    ap.add_argument("--sweep", action="store_true",
                    help="one GPU: the shapes of the reference's result tables (4096 rows, widths 512 .. 8192)")
    ap.add_argument("--shape", default="", metavar="ROWSxCOLS",
                    help="row-wise workloads only: another matrix shape than the named one (for profiler captures "
                         "and width studies; not a bench configuration)")
    ap.add_argument("--small", action="store_true",
                    help="halve the row / matrix sizes (for profiler captures; not a bench configuration)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.profile:
        args.replays = 1
        args.no_e2e = args.no_cpu = args.no_cmp = args.no_weak = args.no_sustained = True

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.as_rank0_of:
        if world != 1:
            raise SystemExit("--as-rank0-of is a one-GPU mode")
        args.no_e2e = args.no_cpu = args.no_cmp = args.no_weak = args.no_sustained = True

    if args.impl == "reference":
        reference_arm(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist_ctx = world > 1
    if args.as_rank0_of:
        world = args.as_rank0_of          # shard arithmetic only; this process is rank 0 and alone
    if dist_ctx:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=dev)

    if world > 1:   # the ranks of one box share its cores (input generation, parity checks)
        torch.set_num_threads(max(1, (os.cpu_count() or world) // world))
    peaks = measured_peaks()
    if args.shape:
        _Rows.rows, _Rows.cols = (int(v) for v in args.shape.lower().split("x"))
    if args.small:
        _Rows.rows = 8192
        Gemm.m = Gemm.n = Gemm.k = 4096
        Bricks.n = 192
    timer = Timer(dist_ctx)
    if args.sweep:
        if world != 1:
            raise SystemExit("--sweep is a one-GPU mode")
        sweep(args, dev, timer, peaks)
        return
    names = [args.workload] + ([] if args.only else [n for n in WORKLOADS if n != args.workload])
    results = {}
    for name in names:
        r = run_workload(WORKLOADS[name], args, dev, world, rank, timer, peaks, local_rank,
                         headline=(name == args.workload))
        inputs.clear_cache()
        results[name] = r
        if rank == 0:
            log(json.dumps({"detail": name, **r}))
    ceiling = None if args.no_e2e else host_ceiling(world, dist_ctx)
    if rank == 0:
        res = results[args.workload]
        line = {
            "metric": res["metric"], "value": res["value"], "unit": res["unit"], "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": res["dtype"],
            "data": "synthetic",
            "config": {"workload": res["workload"],
                       "l2_policy": "inputs larger than L2; rotating buffer sets where a shard is smaller",
                       "sharding": "named shape split across ranks, no data-path collective"},
            "roofline": res["roofline"], "e2e": res.get("e2e"), "gpu_launches": res["gpu_launches"],
            "timed": res["timed"], "clocks": res["clocks"], "parity": res["parity"], "parity_ok": res["parity_ok"],
        }
        for key in ("cpu_baseline", "comparators", "weak"):
            if key in res:
                line[key] = res[key]
        if ceiling is not None:
            line["host_ceiling"] = {"value": ceiling, "unit": "GB/s", "what": "pinned H2D + D2H at once, no kernel"}
            if res.get("e2e") and res["unit"] == "GB/s":
                line["e2e"]["frac_of_host_ceiling"] = res["e2e"]["value"] / ceiling
        line["workloads"] = {n: brief(r) for n, r in results.items() if n != args.workload}
        if args.shape:
            line["config"]["shape_override"] = args.shape + " (row-wise workloads; not the named configuration)"
        if args.as_rank0_of:
            line["n_gpus"] = 1
            line["as_rank0_of"] = {"world": world, "what": "one GPU timing rank 0's shard; value = the named shape's "
                                   "work / that time, i.e. what the world would deliver if every rank took as long"}
        print(json.dumps(_rounded(line)), flush=True)
    if dist_ctx:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
