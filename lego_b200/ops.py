"""Kernel-level callables: the Python side of the C ABI.

The names and argument meaning follow the callables the reference generates:
``matmul(a, b, activation="")`` (``triton_generated/matmul/matmul_NTA_NTB.py:129-145``),
``softmax(x)`` (``triton_generated/softmax/softmax.py:97-160``),
``LEGOLayerNorm.apply(x, normalized_shape, weight, bias, eps)``
(``triton_generated/layernorm/layernorm.py:279-340``),
``lego_group_gemm_fn(group_A, group_B)``
(``triton_generated/grouped_gemm/grouped_gemm.py:120-162``), plus ``permute`` /
``transpose`` for the MLIR transpose programs and the index-map evaluator.

Tensors are torch tensors; torch only owns memory and streams here.  A CUDA
tensor is processed in place on the current stream.  A CPU tensor is staged
through the device (large ones in row blocks, so that copy-in, kernel and copy-out
overlap) and a CPU tensor comes back: that is the end-to-end path.  Without a GPU or without the built library every
op raises; there is no CPU implementation behind them.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _abi
from .layout import Col, GroupBy, OrderBy, Row
from .lowering import lower, lower_optional

__all__ = [
    "eval_apply", "eval_inv", "eval_range", "permute", "permute_plan", "permute_dma_plan", "permute_slabs", "permute_slab_info", "transpose", "softmax",
    "LEGOLayerNorm", "lego_layer_norm", "layer_norm_fwd", "layer_norm_bwd", "matmul", "lego_group_gemm_fn",
    "grouped_swizzle_layout", "default_group_m", "default_tile_order", "row_tiling_layout", "device_status", "tune", "selftest_bounded_wait",
]


def _device() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("lego_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _to_device(t: torch.Tensor) -> torch.Tensor:
    if t.is_cuda:
        return t
    return t.to(_device(), non_blocking=True)


def _to_host(result: torch.Tensor) -> torch.Tensor:
    """A device result as a pinned host tensor (synchronises the current stream)."""
    out = torch.empty(result.shape, dtype=result.dtype, device="cpu", pin_memory=True)
    out.copy_(result, non_blocking=True)
    torch.cuda.current_stream().synchronize()
    return out


def _like_input(result: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Results follow the residence of the input: CPU in, CPU out."""
    return result if ref.is_cuda else _to_host(result)


# Host-resident operands.  A host tensor is staged through the device in row blocks on
# three streams: block i + 1 is copied in while block i is computed and block i - 1 is
# copied out, so that a call on host buffers costs about one PCIe direction's time, not
# the sum of both.  Pinned inputs overlap; pageable ones still work, serialised by the
# driver's own staging.
_HOST_BLOCK_BYTES = 16 << 20   # measured best on PCIe 5 x16 (8 and 32 MiB are within 4 %)
_side_streams = {}


def _copy_streams(dev: torch.device):
    key = (dev.index, torch.cuda.current_stream().cuda_stream)
    if key not in _side_streams:
        _side_streams[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _side_streams[key]


class _HostPipeline:
    """Copy-in / compute / copy-out over row blocks.  ``feed(dst, src)`` copies a host
    block to the device on the inbound stream, ``ready()`` makes the compute stream wait
    for everything fed so far, ``drain(dst, src)`` sends a device block back once the
    compute stream has reached this point, ``finish()`` waits for the last block."""

    def __init__(self):
        self.dev = _device()
        self.main = torch.cuda.current_stream()
        self.inbound, self.outbound = _copy_streams(self.dev)
        self.inbound.wait_stream(self.main)
        self.outbound.wait_stream(self.main)

    def feed(self, dst: torch.Tensor, src: torch.Tensor) -> None:
        with torch.cuda.stream(self.inbound):
            dst.copy_(src, non_blocking=True)

    def ready(self) -> None:
        ev = torch.cuda.Event()
        ev.record(self.inbound)
        self.main.wait_event(ev)

    def drain(self, dst: torch.Tensor, src: torch.Tensor) -> None:
        ev = torch.cuda.Event()
        ev.record(self.main)
        self.outbound.wait_event(ev)
        with torch.cuda.stream(self.outbound):
            dst.copy_(src, non_blocking=True)

    def finish(self) -> None:
        # device blocks were allocated on the compute stream: order their reuse after both copy streams
        self.main.wait_stream(self.inbound)
        self.main.wait_stream(self.outbound)
        self.outbound.synchronize()


def _row_blocks(rows: int, row_bytes: int, multiple: int = 1):
    """Consecutive row ranges of about ``_HOST_BLOCK_BYTES`` each (whole multiples of ``multiple``
    rows except the last).  Blocks of equal size: starting and ending a long input with blocks of
    an eighth, a quarter and a half of the size -- to shorten the first copy-in and the last
    copy-out, the only transfers nothing overlaps -- measured no gain (softmax 16384 x 8192 from
    pinned memory 6.15 against 6.08 ms): a copy of 2 MiB runs at 20 GB/s, one of 4 MiB at 29,
    so the small blocks give back what they save."""
    step = max(1, _HOST_BLOCK_BYTES // max(1, row_bytes))
    step = max(multiple, step // multiple * multiple)
    return [(r0, min(rows, r0 + step)) for r0 in range(0, rows, step)]


def _pinned_like(shape, dtype) -> torch.Tensor:
    return torch.empty(tuple(shape), dtype=dtype, device="cpu", pin_memory=True)


def device_status() -> int:
    """Synchronise the current stream and return the device status word's verdict;
    raises if a bounded wait inside a kernel ran out."""
    detail = C.c_uint32(0)
    st = _abi.lib().lego_device_status(_stream(), C.byref(detail))
    if st != 0:
        for ws in _gemm_workspaces.values():   # a kernel that gave up may have left split-K flags set
            ws[:8192].zero_()
        raise _abi.LegoError(st, f"device status word 0x{detail.value:x}")
    return 0


def selftest_bounded_wait(limit_cycles: int = 1_000_000) -> None:
    """Launch the one-CTA kernel whose wait nothing completes: it gives up after
    ``limit_cycles`` SM cycles and records its code; ``device_status()`` then raises once."""
    _device()
    _abi.check(_abi.lib().lego_selftest_bounded_wait(int(limit_cycles), _stream()), "lego_selftest_bounded_wait")


def tune(gemm_blocks: Optional[int] = None, gemm_streamk: Optional[bool] = None,
         gemm_lag: Optional[int] = None, permute_dma_tile: Optional[int] = None,
         permute_dma_ctas: Optional[int] = None, permute_tile_vecs: Optional[int] = None,
         pdl_last_wave: Optional[int] = None, permute_dma_long: Optional[int] = None,
         lnbwd_min_rows: Optional[int] = None, lnbwd_fold_warp: Optional[int] = None) -> None:
    """Process-wide knobs.  GEMM: ``gemm_blocks`` 0 library's choice / 1 (256 x 256 per SM
    pair) / 2 (512 x 256 per SM pair); ``gemm_streamk`` 0 / False keeps every tile whole,
    1 / True splits a poorly filled last wave along K, 2 splits any partial wave;
    ``gemm_lag`` 0..4, the lead of the first accumulator block of a 512 x 256 tile.
    Permute: ``permute_dma_tile`` most bytes per box of the DMA kernel (0: the chunk-tiled
    kernel takes those layouts), ``permute_dma_ctas`` its CTAs per SM, ``permute_tile_vecs``
    most 16-byte vectors per tile of the chunk-tiled kernel, ``permute_dma_long`` 0: pairs whose
    common run is a whole line or more stay with the vector copy.  ``pdl_last_wave`` 1: only the last
    wave of an index-map grid lets the next grid of the stream become resident.
    ``lnbwd_min_rows``: fewest rows for which LayerNorm backward uses its ring-fed kernels
    (default 1; below, the kernel that holds a row in registers); ``lnbwd_fold_warp``: most
    consumer groups for which its grouped kernel runs a folding warp per group (0 .. 3, default 3)."""
    lib = _abi.lib()
    if lnbwd_fold_warp is not None:
        _abi.check(lib.lego_tune(_abi.TUNE_LNBWD_FOLD_WARP, int(lnbwd_fold_warp)), "lego_tune")
    if lnbwd_min_rows is not None:
        _abi.check(lib.lego_tune(_abi.TUNE_LNBWD_MIN_ROWS, int(lnbwd_min_rows)), "lego_tune")
    if permute_dma_tile is not None:
        _abi.check(lib.lego_tune(_abi.TUNE_PERMUTE_DMA_TILE, int(permute_dma_tile)), "lego_tune")
    if permute_dma_ctas is not None:
        _abi.check(lib.lego_tune(_abi.TUNE_PERMUTE_DMA_CTAS, int(permute_dma_ctas)), "lego_tune")
    if permute_tile_vecs is not None:
        _abi.check(lib.lego_tune(_abi.TUNE_PERMUTE_TILE_VECS, int(permute_tile_vecs)), "lego_tune")
    if permute_dma_long is not None:
        _abi.check(lib.lego_tune(_abi.TUNE_PERMUTE_DMA_LONG, int(permute_dma_long)), "lego_tune")
    if pdl_last_wave is not None:
        _abi.check(lib.lego_tune(_abi.TUNE_PDL_LAST_WAVE, int(pdl_last_wave)), "lego_tune")
    if gemm_blocks is not None:
        _abi.check(lib.lego_tune(_abi.TUNE_GEMM_BLOCKS, int(gemm_blocks)), "lego_tune")
    if gemm_streamk is not None:
        _abi.check(lib.lego_tune(_abi.TUNE_GEMM_STREAMK, int(gemm_streamk)), "lego_tune")
    if gemm_lag is not None:
        _abi.check(lib.lego_tune(_abi.TUNE_GEMM_LAG, int(gemm_lag)), "lego_tune")


# One split-K scratch buffer per (device, stream): calls on one stream are ordered, calls on
# different streams must not share a buffer.  Flags (first 8 KiB) start at zero and every
# completed call leaves them zero.
_gemm_workspaces = {}


def _gemm_workspace(dev: torch.device) -> torch.Tensor:
    key = (dev.index, torch.cuda.current_stream().cuda_stream)
    ws = _gemm_workspaces.get(key)
    if ws is None:
        nbytes = _abi.lib().lego_gemm_workspace_bytes()
        if nbytes <= 0:
            raise RuntimeError("lego_gemm_workspace_bytes failed")
        if torch.cuda.is_current_stream_capturing():
            # memory allocated while capturing belongs to the graph: use it for this call only
            ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            ws[:8192].zero_()
            return ws
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        _gemm_workspaces[key] = ws
    return ws


# ---- layouts used by the ops --------------------------------------------------------

def grouped_swizzle_layout(num_pid_m: int, num_pid_n: int, group_m: int = 8) -> GroupBy:
    """Tile order of the reference GEMM (``benchmarks/triton/matmul_sympy.py:57-65``):
    ``inv(pid)`` gives ``(pid_m, pid_n)`` walking ``group_m`` tile rows at a time."""
    return OrderBy(Col(max(num_pid_m // group_m, 1), 1),
                   Col(min(num_pid_m, group_m), num_pid_n)).TileBy([num_pid_m, num_pid_n])


def row_tiling_layout(n_rows: int, rows_per_tile: int = 1) -> GroupBy:
    """1-D tiling of rows, ``OrderBy(Row(n_rows)).TileBy([n_rows / R], [R])``."""
    if rows_per_tile <= 1 or n_rows % rows_per_tile:
        return OrderBy(Row(n_rows)).TileBy([n_rows])
    return OrderBy(Row(n_rows)).TileBy([n_rows // rows_per_tile], [rows_per_tile])


# ---- index-map evaluator ------------------------------------------------------------

def eval_apply(layout: GroupBy, idx: torch.Tensor) -> torch.Tensor:
    """``layout.apply`` over rows of ``idx`` (int64 ``[n, rank]``) -> int64 ``[n]``."""
    desc = lower(layout)
    if idx.dtype != torch.int64 or idx.dim() != 2 or idx.shape[1] != desc.rank:
        raise ValueError(f"idx must be int64 [n, {desc.rank}]")
    d = _to_device(idx).contiguous()
    out = torch.empty(d.shape[0], dtype=torch.int64, device=d.device)
    _abi.check(_abi.lib().lego_eval_apply(C.byref(desc), d.data_ptr(), out.data_ptr(), d.shape[0], _stream()),
               "lego_eval_apply")
    return _like_input(out, idx)


def eval_inv(layout: GroupBy, flat: torch.Tensor) -> torch.Tensor:
    """``layout.inv`` over ``flat`` (int64 ``[n]``) -> int64 ``[n, rank]``."""
    desc = lower(layout)
    if flat.dtype != torch.int64 or flat.dim() != 1:
        raise ValueError("flat must be int64 [n]")
    d = _to_device(flat).contiguous()
    out = torch.empty((d.shape[0], desc.rank), dtype=torch.int64, device=d.device)
    _abi.check(_abi.lib().lego_eval_inv(C.byref(desc), d.data_ptr(), out.data_ptr(), d.shape[0], _stream()),
               "lego_eval_inv")
    return _like_input(out, flat)


def eval_range(layout: GroupBy, begin: int = 0, count: Optional[int] = None, host: bool = False) -> torch.Tensor:
    """``layout.apply`` over logical flat ids ``begin .. begin+count`` -> int64, on the
    device, or with ``host=True`` in pinned host memory (evaluated block by block, each
    block leaving the device while the next is computed)."""
    desc = lower(layout)
    size = layout.size()
    if count is None:
        count = size - begin
    call = _abi.lib().lego_eval_range
    if host and count * 8 > 2 * _HOST_BLOCK_BYTES:
        pipe = _HostPipeline()
        res = _pinned_like((count,), torch.int64)
        bufs = [torch.empty(_HOST_BLOCK_BYTES // 8, dtype=torch.int64, device=pipe.dev) for _ in range(2)]
        done = [None, None]  # the copy-out that last read each buffer
        for i, (r0, r1) in enumerate(_row_blocks(count, 8)):
            buf = bufs[i & 1][: r1 - r0]
            if done[i & 1] is not None:
                pipe.main.wait_event(done[i & 1])
            _abi.check(call(C.byref(desc), begin + r0, r1 - r0, buf.data_ptr(), _stream()), "lego_eval_range")
            pipe.drain(res[r0:r1], buf)
            done[i & 1] = torch.cuda.Event()
            done[i & 1].record(pipe.outbound)
        pipe.finish()
        return res
    out = torch.empty(count, dtype=torch.int64, device=_device())
    _abi.check(call(C.byref(desc), begin, count, out.data_ptr(), _stream()), "lego_eval_range")
    return _to_host(out) if host else out


# ---- layout reorganisation ----------------------------------------------------------

def permute_plan(elem_bytes: int, src: GroupBy, dst: GroupBy, tile_order: Optional[GroupBy] = None):
    """Which kernel ``permute`` would run: ``(kind, tile_in, tile_out)`` with kind
    0 staged, 1 gather, 2 shared-memory tiled transpose, 3 TMA-fed tiled transpose,
    4 chunk-tiled permute, 5 DMA permute.  Host-only; needs no GPU."""
    kind, ti, to = C.c_int32(0), C.c_int64(0), C.c_int64(0)
    _abi.check(_abi.lib().lego_permute_plan(elem_bytes, C.byref(lower(src)), C.byref(lower(dst)),
                                            lower_optional(tile_order), C.byref(kind), C.byref(ti), C.byref(to)),
               "lego_permute_plan")
    return kind.value, ti.value, to.value


def permute_dma_plan(elem_bytes: int, src: GroupBy, dst: GroupBy, slabs: int = -1) -> dict:
    """The DMA permute's plan for a pair of layouts: both tensor maps (``size``, ``stride``,
    ``box`` per dimension, innermost first, in elements of ``elem_bytes``) and the digits of
    the tile id; ``slabs >= 0``: the plan of that many slabs (``permute_slabs``).  Raises
    ``ValueError`` when the pair is not moved that way.  Host-only."""
    plan = _abi.DmaPlan()
    _abi.check(_abi.lib().lego_permute_dma_plan(elem_bytes, C.byref(lower(src)), C.byref(lower(dst)), int(slabs),
                                                C.byref(plan)), "lego_permute_dma_plan")

    def side(sd):
        return {k: [int(getattr(sd, k)[i]) for i in range(sd.rank)] for k in ("size", "stride", "box")}

    return {"elem_bytes": plan.elem_bytes, "n_tiles": plan.n_tiles, "tile_bytes": plan.tile_bytes,
            "load": side(plan.load), "store": side(plan.store),
            "outer": [{"radix": int(o.radix), "ld": (o.ld_dim, o.ld_mul), "st": (o.st_dim, o.st_mul)}
                      for o in plan.outer[:plan.n_outer]]}


def permute_slab_info(elem_bytes: int, src: GroupBy, dst: GroupBy):
    """``(n_slabs, slab_elems)`` when the slowest digit of the flat index is the same logical
    digit in both layouts -- the re-layout then is ``n_slabs`` independent pieces, each
    contiguous in both buffers -- else ``None``.  Host-only."""
    n, e = C.c_int64(0), C.c_int64(0)
    st = _abi.lib().lego_permute_slab_info(elem_bytes, C.byref(lower(src)), C.byref(lower(dst)), C.byref(n),
                                           C.byref(e))
    if st == _abi.ERR_UNSUPPORTED:
        return None
    _abi.check(st, "lego_permute_slab_info")
    return n.value, e.value


def permute_slabs(x: torch.Tensor, src: GroupBy, dst: GroupBy, count: int,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The re-layout ``src -> dst`` restricted to ``count`` consecutive slabs (see
    ``permute_slab_info``): ``x`` and the result hold those slabs only."""
    d = _to_device(x).contiguous()
    res = out if out is not None else torch.empty_like(d)
    if not res.is_cuda or not res.is_contiguous() or res.numel() != d.numel() or res.dtype != d.dtype:
        raise ValueError("out must be a contiguous CUDA tensor of x's size and dtype")
    info = permute_slab_info(d.element_size(), src, dst)
    if info is None:
        raise ValueError("this pair of layouts does not split into slabs")
    if count < 0 or count > info[0] or d.numel() != count * info[1]:
        raise ValueError(f"{count} slabs of {info[1]} elements do not match a tensor of {d.numel()}")
    _abi.check(_abi.lib().lego_permute_slabs(d.data_ptr(), res.data_ptr(), d.element_size(), C.byref(lower(src)),
                                             C.byref(lower(dst)), int(count), _stream()), "lego_permute_slabs")
    return _like_input(res, x)


def _permute_from_host(x, src, dst, n_slabs, slab_elems):
    """A re-layout that splits into slabs, on a host buffer: groups of slabs of about 16 MiB go
    through the device on three streams (copy in / move / copy out), so the call costs about
    one PCIe direction instead of copy-in + kernel + copy-out."""
    eb = x.element_size()
    pipe = _HostPipeline()
    lib = _abi.lib()
    flat = x.reshape(-1)
    out = _pinned_like((x.numel(),), x.dtype)
    d_in = torch.empty(x.numel(), dtype=x.dtype, device=pipe.dev)
    d_out = torch.empty_like(d_in)
    s_desc, d_desc = lower(src), lower(dst)
    for k0, k1 in _row_blocks(n_slabs, slab_elems * eb):
        e0, e1 = k0 * slab_elems, k1 * slab_elems
        pipe.feed(d_in[e0:e1], flat[e0:e1])
        pipe.ready()
        _abi.check(lib.lego_permute_slabs(d_in[e0:e1].data_ptr(), d_out[e0:e1].data_ptr(), eb, C.byref(s_desc),
                                          C.byref(d_desc), k1 - k0, _stream()), "lego_permute_slabs")
        pipe.drain(out[e0:e1], d_out[e0:e1])
    pipe.finish()
    return out.reshape(x.shape)


def permute(x: torch.Tensor, src: GroupBy, dst: GroupBy, tile_order: Optional[GroupBy] = None,
            out: Optional[torch.Tensor] = None, tiles: Optional[Sequence[int]] = None) -> torch.Tensor:
    """``out_flat[dst(idx)] = x_flat[src(idx)]`` over the layouts' common logical
    domain.  ``x`` is read as a flat contiguous buffer; the result has x's shape.
    ``tiles=(begin, count)`` moves only that range of ``tile_order`` ids (one GPU's
    slab of a reorganisation split across several) and leaves the rest of ``out`` alone."""
    if src.size() != x.numel():
        raise ValueError(f"layout covers {src.size()} elements, tensor has {x.numel()}")
    if (not x.is_cuda and out is None and tiles is None and tile_order is None and x.is_contiguous()
            and x.numel() * x.element_size() > 2 * _HOST_BLOCK_BYTES):
        info = permute_slab_info(x.element_size(), src, dst)
        if info is not None and info[0] * info[1] == x.numel() and info[1] * x.element_size() <= _HOST_BLOCK_BYTES:
            return _permute_from_host(x, src, dst, *info)
    d = _to_device(x).contiguous()
    res = out if out is not None else torch.empty_like(d)
    if not res.is_cuda or not res.is_contiguous() or res.numel() != d.numel() or res.dtype != d.dtype:
        raise ValueError("out must be a contiguous CUDA tensor of x's size and dtype")
    if tiles is not None:
        begin, count = tiles
        _abi.check(_abi.lib().lego_permute_tiles(d.data_ptr(), res.data_ptr(), d.element_size(), C.byref(lower(src)),
                                                 C.byref(lower(dst)), lower_optional(tile_order), int(begin),
                                                 int(count), _stream()), "lego_permute_tiles")
        return _like_input(res, x)
    _abi.check(_abi.lib().lego_permute(d.data_ptr(), res.data_ptr(), d.element_size(), C.byref(lower(src)),
                                       C.byref(lower(dst)), lower_optional(tile_order), _stream()),
               "lego_permute")
    return _like_input(res, x)


def transpose(x: torch.Tensor, tile: int = 32, tile_order: Optional[GroupBy] = None) -> torch.Tensor:
    """2-D transpose through the tiled layouts of the reference's MLIR programs
    (``benchmarks/mlir/transpose_smem.py:33-37``): source viewed row-major in
    ``tile x tile`` tiles, destination column-major, tiles visited in ``tile_order``
    (default: column-major over tiles)."""
    if x.dim() != 2:
        raise ValueError("transpose expects a matrix")
    r, c = x.shape
    if r % tile or c % tile:
        raise ValueError(f"matrix {r}x{c} is not a multiple of the {tile}x{tile} tile")
    src = OrderBy(Row(r, c)).TileBy([r // tile, c // tile], [tile, tile])
    dst = OrderBy(Col(r, c)).TileBy([r // tile, c // tile], [tile, tile])
    default_order = tile_order is None
    if default_order:
        tile_order = OrderBy(Col(r // tile, c // tile)).TileBy([r // tile, c // tile])
    nbytes = x.numel() * x.element_size()
    if (not x.is_cuda and x.is_contiguous() and default_order and nbytes > 2 * _HOST_BLOCK_BYTES
            and permute_plan(x.element_size(), src, dst, tile_order)[0] in (2, 3)):
        return _transpose_from_host(x, tile, src, dst, tile_order)
    return permute(x, src, dst, tile_order).reshape(c, r)


def _transpose_from_host(x, tile, src, dst, tile_order):
    """Host matrix: slabs of output rows.  A slab's input is a band of columns, copied in with
    one strided copy; its tiles are a contiguous range of the column-major tile order; its
    output rows are contiguous.  Slab i + 1 arrives while slab i is transposed and slab i - 1
    leaves, so the call costs about one PCIe direction instead of copy-in + kernel + copy-out."""
    r, c = x.shape
    eb = x.element_size()
    pipe = _HostPipeline()
    lib = _abi.lib()
    d_in = torch.empty((r, c), dtype=x.dtype, device=pipe.dev)
    d_out = torch.empty((c, r), dtype=x.dtype, device=pipe.dev)
    out = _pinned_like((c, r), x.dtype)
    tiles_down = r // tile
    for c0, c1 in _row_blocks(c, r * eb, multiple=tile):        # bands of columns
        _abi.check(lib.lego_copy_2d(d_in.data_ptr() + c0 * eb, c * eb, x.data_ptr() + c0 * eb, c * eb,
                                    (c1 - c0) * eb, r, pipe.inbound.cuda_stream), "lego_copy_2d")
        pipe.ready()
        permute(d_in, src, dst, tile_order, out=d_out.reshape(r, c),
                tiles=(c0 // tile * tiles_down, (c1 - c0) // tile * tiles_down))
        pipe.drain(out[c0:c1], d_out[c0:c1])
    pipe.finish()
    return out


# ---- row-wise kernels ---------------------------------------------------------------

def softmax(x: torch.Tensor, row_map: Optional[GroupBy] = None) -> torch.Tensor:
    """Row-wise softmax of a 2-D fp16 or fp32 tensor (fp32 arithmetic)."""
    if x.dim() != 2:
        raise ValueError("softmax expects a 2-D tensor")
    fn = {torch.float16: "lego_softmax_f16", torch.float32: "lego_softmax_f32"}.get(x.dtype)
    if fn is None:
        raise ValueError(f"softmax supports float16 and float32, got {x.dtype}")
    call = getattr(_abi.lib(), fn)
    if not x.is_cuda and x.is_contiguous() and x.numel() * x.element_size() > 2 * _HOST_BLOCK_BYTES:
        # Host rows: staged block by block.  A row map only decides which CTA takes which
        # row, never the result, so the blocks run in arrival order without it.
        lower_optional(row_map)
        pipe = _HostPipeline()
        d = torch.empty(x.shape, dtype=x.dtype, device=pipe.dev)
        y = torch.empty_like(d)
        out = _pinned_like(x.shape, x.dtype)
        for r0, r1 in _row_blocks(x.shape[0], x.shape[1] * x.element_size()):
            pipe.feed(d[r0:r1], x[r0:r1])
            pipe.ready()
            _abi.check(call(d[r0:r1].data_ptr(), y[r0:r1].data_ptr(), r1 - r0, x.shape[1], None, _stream()), fn)
            pipe.drain(out[r0:r1], y[r0:r1])
        pipe.finish()
        return out
    d = _to_device(x).contiguous()
    y = torch.empty_like(d)
    n_rows, n_cols = d.shape
    _abi.check(call(d.data_ptr(), y.data_ptr(), n_rows, n_cols, lower_optional(row_map), _stream()), fn)
    return _like_input(y, x)


def layer_norm_fwd(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float,
                   row_map: Optional[GroupBy] = None):
    """LayerNorm forward over the last axis: ``(y, mean, rstd)``, statistics fp32."""
    if x.dtype != torch.float16 or weight.dtype != torch.float16 or bias.dtype != torch.float16:
        raise ValueError("layer norm supports float16 tensors")
    n = x.shape[-1]
    if weight.numel() != n or bias.numel() != n:
        raise ValueError("weight / bias must have the size of the last axis")
    if n * x.element_size() > 65536:
        raise RuntimeError("This layer norm doesn't support feature dim >= 64KB.")
    call = _abi.lib().lego_layernorm_fwd_f16
    if not x.is_cuda and x.is_contiguous() and x.numel() * x.element_size() > 2 * _HOST_BLOCK_BYTES:
        # host rows: staged block by block (a row map never changes the result, see softmax)
        lower_optional(row_map)
        pipe = _HostPipeline()
        xh = x.reshape(-1, n)
        m = xh.shape[0]
        w, b = _to_device(weight).contiguous(), _to_device(bias).contiguous()
        d = torch.empty(xh.shape, dtype=x.dtype, device=pipe.dev)
        y = torch.empty_like(d)
        mean = torch.empty(m, dtype=torch.float32, device=pipe.dev)
        rstd = torch.empty(m, dtype=torch.float32, device=pipe.dev)
        y_h, mean_h, rstd_h = _pinned_like(xh.shape, x.dtype), _pinned_like((m,), torch.float32), _pinned_like((m,), torch.float32)
        for r0, r1 in _row_blocks(m, n * x.element_size()):
            pipe.feed(d[r0:r1], xh[r0:r1])
            pipe.ready()
            _abi.check(call(d[r0:r1].data_ptr(), w.data_ptr(), b.data_ptr(), y[r0:r1].data_ptr(),
                            mean[r0:r1].data_ptr(), rstd[r0:r1].data_ptr(), r1 - r0, n, float(eps), None, _stream()),
                       "lego_layernorm_fwd_f16")
            pipe.drain(y_h[r0:r1], y[r0:r1])
        pipe.drain(mean_h, mean)
        pipe.drain(rstd_h, rstd)
        pipe.finish()
        return y_h.reshape(x.shape), mean_h, rstd_h
    d = _to_device(x).contiguous()
    x2 = d.reshape(-1, n)
    w, b = _to_device(weight).contiguous(), _to_device(bias).contiguous()
    m = x2.shape[0]
    y = torch.empty_like(d)
    mean = torch.empty(m, dtype=torch.float32, device=d.device)
    rstd = torch.empty(m, dtype=torch.float32, device=d.device)
    _abi.check(_abi.lib().lego_layernorm_fwd_f16(x2.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(),
                                                 mean.data_ptr(), rstd.data_ptr(), m, n, float(eps),
                                                 lower_optional(row_map), _stream()),
               "lego_layernorm_fwd_f16")
    return _like_input(y, x), _like_input(mean, x), _like_input(rstd, x)


class LEGOLayerNorm(torch.autograd.Function):
    """``LEGOLayerNorm.apply(x, normalized_shape, weight, bias, eps)``."""

    @staticmethod
    def forward(ctx, x, normalized_shape, weight, bias, eps):
        y, mean, rstd = layer_norm_fwd(x, weight, bias, eps)
        ctx.save_for_backward(x, weight, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        dx, dw, db = layer_norm_bwd(dy, x, w, mean, rstd)
        return dx, None, dw, db, None


def layer_norm_bwd(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, mean: torch.Tensor, rstd: torch.Tensor):
    """LayerNorm backward over the last axis: ``(dx, dweight, dbias)`` from the saved
    row statistics; dweight / dbias come from a fixed-order two-stage column reduction
    (same bits on every run)."""
    n = x.shape[-1]
    if (not x.is_cuda and not dy.is_cuda and x.is_contiguous() and dy.is_contiguous() and x.shape == dy.shape
            and x.dtype == torch.float16 and dy.dtype == torch.float16 and weight.dtype == torch.float16
            and x.numel() * 2 > 2 * _HOST_BLOCK_BYTES):
        return _layer_norm_bwd_from_host(dy, x, weight, mean, rstd)
    xd = _to_device(x).contiguous().reshape(-1, n)
    dyd = _to_device(dy).contiguous().reshape(-1, n)
    wd = _to_device(weight).contiguous()
    md, rd = _to_device(mean).contiguous(), _to_device(rstd).contiguous()
    m = xd.shape[0]
    if dyd.shape != xd.shape or wd.numel() != n or md.numel() != m or rd.numel() != m:
        raise ValueError("layer norm backward: shapes of dy, x, weight, mean, rstd do not agree")
    if xd.dtype != torch.float16 or dyd.dtype != torch.float16 or wd.dtype != torch.float16:
        raise ValueError("layer norm supports float16 tensors")
    lib = _abi.lib()
    prow = lib.lego_layernorm_bwd_partial_rows(m, n)
    partial = torch.empty((2, prow, n), dtype=torch.float32, device=xd.device)
    dx = torch.empty_like(xd)
    dw = torch.empty_like(wd)
    db = torch.empty_like(wd)
    _abi.check(lib.lego_layernorm_bwd_f16(dyd.data_ptr(), xd.data_ptr(), wd.data_ptr(), md.data_ptr(),
                                          rd.data_ptr(), dx.data_ptr(), dw.data_ptr(), db.data_ptr(),
                                          partial.data_ptr(), m, n, _stream()),
               "lego_layernorm_bwd_f16")
    return _like_input(dx.reshape(x.shape), x), _like_input(dw, weight), _like_input(db, weight)


def _layer_norm_bwd_from_host(dy, x, weight, mean, rstd):
    """Host rows of x and dy: staged block by block (copy-in / compute / copy-out overlap).  Every
    block yields its own dweight / dbias (fp16, as the entry point rounds them); they are summed
    in fp32 on the device and rounded once more at the end, so these two results may differ in
    the last bit from one call on device-resident rows."""
    n = x.shape[-1]
    xh, dyh = x.reshape(-1, n), dy.reshape(-1, n)
    m = xh.shape[0]
    if weight.numel() != n or mean.numel() != m or rstd.numel() != m:
        raise ValueError("layer norm backward: shapes of dy, x, weight, mean, rstd do not agree")
    pipe = _HostPipeline()
    lib = _abi.lib()
    wd = _to_device(weight).contiguous()
    md, rd = _to_device(mean).contiguous(), _to_device(rstd).contiguous()
    xd = torch.empty(xh.shape, dtype=x.dtype, device=pipe.dev)
    dyd = torch.empty_like(xd)
    dx = torch.empty_like(xd)
    dx_h = _pinned_like(xh.shape, x.dtype)
    dw32 = torch.zeros(n, dtype=torch.float32, device=pipe.dev)
    db32 = torch.zeros(n, dtype=torch.float32, device=pipe.dev)
    dw_b, db_b = torch.empty_like(wd), torch.empty_like(wd)
    blocks = _row_blocks(m, n * 2, multiple=4)
    prow = lib.lego_layernorm_bwd_partial_rows(max(r1 - r0 for r0, r1 in blocks), n)
    partial = torch.empty((2, prow, n), dtype=torch.float32, device=pipe.dev)
    for r0, r1 in blocks:
        pipe.feed(xd[r0:r1], xh[r0:r1])
        pipe.feed(dyd[r0:r1], dyh[r0:r1])
        pipe.ready()
        _abi.check(lib.lego_layernorm_bwd_f16(dyd[r0:r1].data_ptr(), xd[r0:r1].data_ptr(), wd.data_ptr(),
                                              md[r0:r1].data_ptr(), rd[r0:r1].data_ptr(), dx[r0:r1].data_ptr(),
                                              dw_b.data_ptr(), db_b.data_ptr(), partial.data_ptr(), r1 - r0, n, _stream()),
                   "lego_layernorm_bwd_f16")
        dw32 += dw_b
        db32 += db_b
        pipe.drain(dx_h[r0:r1], dx[r0:r1])
    dw, db = dw32.to(torch.float16), db32.to(torch.float16)
    pipe.finish()
    return dx_h.reshape(x.shape), _like_input(dw, weight), _like_input(db, weight)


lego_layer_norm = LEGOLayerNorm.apply


# ---- GEMM ---------------------------------------------------------------------------

def _operand(t: torch.Tensor):
    """(contiguous storage, transposed?) of a 2-D operand that is either
    contiguous or the ``.T`` view of a contiguous matrix."""
    if t.is_contiguous():
        return t, 0
    if t.t().is_contiguous():
        return t.t(), 1
    return t.contiguous(), 0


# Rows of 128 x 256 tiles walked together by the default tile order.  One wave of the
# persistent kernel covers 74 tiles of 512 x 256: with GROUP_M tile rows per group it reads a
# GROUP_M * 128-row panel of A and 74 * 512 / (GROUP_M * 128) tile columns of B.  GROUP_M = 8
# (the value the reference tunes for its own kernel) makes a wave read every column of an
# 8192-wide B; 32 makes the wave nearly square (A panel 64 MiB + B 36 MiB for K = 8192 in
# fp16) and the A panel stays in the 126 MB L2 from wave to wave: 8192^3 fp16 sustained
# 1 224 -> 1 271 TFLOP/s on one box, DRAM reads per launch 1.17 GB -> about a third.
_A_PANEL_BYTES = 72 << 20


def default_group_m(num_pid_m: int, k: int, elem_bytes: int) -> int:
    """GROUP_M of the default tile order: the largest of 32, 16, 8 that tiles ``num_pid_m``
    and whose A panel (GROUP_M * 128 rows x K) stays within about half of L2."""
    for gm in (32, 16, 8):
        if (num_pid_m % gm == 0 or num_pid_m <= gm) and (gm == 8 or min(gm, num_pid_m) * 128 * k * elem_bytes <= _A_PANEL_BYTES):
            return gm
    return 8


def default_tile_order(m: int, n: int, k: int, elem_bytes: int = 2, group_m: Optional[int] = None) -> Optional[GroupBy]:
    """The tile order ``matmul`` uses when the caller passes none: the reference's grouped
    swizzle over the grid of 128 x 256 tiles, or None (row-major) when GROUP_M does not tile it."""
    npm, npn = -(-m // 128), -(-n // 256)
    gm = default_group_m(npm, k, elem_bytes) if group_m is None else group_m
    if npm % gm == 0 or npm <= gm:
        return grouped_swizzle_layout(npm, npn, gm)
    return None


def matmul(a: torch.Tensor, b: torch.Tensor, activation: str = "", tile_order: Optional[GroupBy] = None,
           group_m: Optional[int] = None) -> torch.Tensor:
    """``C = act(A @ B)``: fp16 in, fp32 accumulate, fp16 out.  Either operand may
    be a ``.T`` view.  Tile order defaults to the reference's grouped swizzle with
    ``GROUP_M = group_m`` (chosen by ``default_group_m`` when None) when it is a bijection
    for the tile grid, row-major otherwise."""
    if a.dtype != b.dtype or a.dtype not in (torch.float16, torch.float8_e5m2):
        raise ValueError("matmul supports float16 operands, or float8_e5m2 operands (fp16 result)")
    fn = "lego_gemm_f16" if a.dtype == torch.float16 else "lego_gemm_e5m2"
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError("Incompatible dimensions")
    act = {"": _abi.ACT_NONE, "leaky_relu": _abi.ACT_LEAKY_RELU}.get(activation)
    if act is None:
        raise ValueError(f"unknown activation {activation!r}")
    m, k = a.shape
    n = b.shape[1]
    lib = _abi.lib()
    if (not a.is_cuda and not b.is_cuda and a.is_contiguous() and tile_order is None
            and a.numel() * a.element_size() > 2 * _HOST_BLOCK_BYTES and m % 256 == 0):
        # Host operands: B goes in first, then A in blocks of rows; each block's rows of C
        # leave while the next block arrives.  Every block is its own GEMM with its own
        # default tile order.
        pipe = _HostPipeline()
        if not b.is_contiguous() and b.t().is_contiguous():  # a .T view: copy the storage, keep the view
            store = torch.empty(b.t().shape, dtype=b.dtype, device=pipe.dev)
            pipe.feed(store, b.t())
            bd = store.t()
        else:
            bd = torch.empty(b.shape, dtype=b.dtype, device=pipe.dev)
            pipe.feed(bd, b)
        b_st, tb = _operand(bd)
        ad = torch.empty(a.shape, dtype=a.dtype, device=pipe.dev)
        c = torch.empty((m, n), dtype=torch.float16, device=pipe.dev)
        c_h = _pinned_like((m, n), torch.float16)
        call = getattr(lib, fn + "_ws")
        ws = _gemm_workspace(pipe.dev)
        for r0, r1 in _row_blocks(m, max(k * a.element_size(), n * 2), multiple=256):
            pipe.feed(ad[r0:r1], a[r0:r1])
            pipe.ready()
            order = default_tile_order(r1 - r0, n, k, a.element_size(), group_m)
            _abi.check(call(ad[r0:r1].data_ptr(), b_st.data_ptr(), c[r0:r1].data_ptr(), r1 - r0, n, k,
                            0, tb, act, lower_optional(order), ws.data_ptr(), ws.numel(), _stream()), fn)
            pipe.drain(c_h[r0:r1], c[r0:r1])
        pipe.finish()
        return c_h
    ad, bd = _to_device(a), _to_device(b)
    a_st, ta = _operand(ad)
    b_st, tb = _operand(bd)
    c = torch.empty((m, n), dtype=torch.float16, device=ad.device)
    if tile_order is None:
        tile_order = default_tile_order(m, n, k, a.element_size(), group_m)
    ws = _gemm_workspace(ad.device)
    _abi.check(getattr(lib, fn + "_ws")(a_st.data_ptr(), b_st.data_ptr(), c.data_ptr(), m, n, k, ta, tb, act,
                                        lower_optional(tile_order), ws.data_ptr(), ws.numel(), _stream()), fn)
    return _like_input(c, a)


def lego_group_gemm_fn(group_A: Sequence[torch.Tensor], group_B: Sequence[torch.Tensor],
                       tile_orders: Optional[Sequence[Optional[GroupBy]]] = None) -> List[torch.Tensor]:
    """Grouped GEMM: ``[A_g @ B_g for g]`` in one persistent launch."""
    assert len(group_A) == len(group_B)
    g = len(group_A)
    if g == 0:
        return []
    if g > _abi.MAX_GROUPS:
        raise ValueError(f"at most {_abi.MAX_GROUPS} groups per call")
    for A, B in zip(group_A, group_B):
        if A.dtype != torch.float16 or B.dtype != torch.float16:
            raise ValueError("grouped GEMM supports float16 operands")
        assert A.shape[1] == B.shape[0]
    if all(not t.is_cuda for t in list(group_A) + list(group_B)) and g > 1:
        return _group_gemm_from_host(group_A, group_B, tile_orders)
    a_dev, b_dev, c_dev, mnk = [], [], [], []
    for A, B in zip(group_A, group_B):
        ad, bd = _to_device(A).contiguous(), _to_device(B).contiguous()
        a_dev.append(ad)
        b_dev.append(bd)
        c_dev.append(torch.empty((A.shape[0], B.shape[1]), dtype=torch.float16, device=ad.device))
        mnk += [A.shape[0], B.shape[1], A.shape[1]]
    PtrArr = C.c_void_p * g
    ap = PtrArr(*[t.data_ptr() for t in a_dev])
    bp = PtrArr(*[t.data_ptr() for t in b_dev])
    cp = PtrArr(*[t.data_ptr() for t in c_dev])
    sizes = (C.c_int64 * (3 * g))(*mnk)
    orders = None
    if tile_orders is not None:
        keep = [None if o is None else lower(o) for o in tile_orders]
        orders = (_abi.LayoutP * g)(*[C.cast(None, _abi.LayoutP) if o is None else C.pointer(o) for o in keep])
    _abi.check(_abi.lib().lego_grouped_gemm_f16(ap, bp, cp, sizes, g, orders, _stream()),
               "lego_grouped_gemm_f16")
    return [_like_input(c, A) for c, A in zip(c_dev, group_A)]


def _group_gemm_from_host(group_A, group_B, tile_orders) -> List[torch.Tensor]:
    """Grouped GEMM on host operands: group g + 1 is copied in while group g is computed
    (one single-problem launch each) and group g - 1 is copied out."""
    pipe = _HostPipeline()
    lib = _abi.lib()
    outs, keep = [], []
    for i, (A, B) in enumerate(zip(group_A, group_B)):
        ad = torch.empty(A.shape, dtype=A.dtype, device=pipe.dev)
        bd = torch.empty(B.shape, dtype=B.dtype, device=pipe.dev)
        cd = torch.empty((A.shape[0], B.shape[1]), dtype=torch.float16, device=pipe.dev)
        keep += [ad, bd, cd]
        pipe.feed(ad, A)
        pipe.feed(bd, B)
        pipe.ready()
        order = None if tile_orders is None or tile_orders[i] is None else lower(tile_orders[i])
        orders = None if order is None else (_abi.LayoutP * 1)(C.pointer(order))
        _abi.check(lib.lego_grouped_gemm_f16((C.c_void_p * 1)(ad.data_ptr()), (C.c_void_p * 1)(bd.data_ptr()),
                                             (C.c_void_p * 1)(cd.data_ptr()),
                                             (C.c_int64 * 3)(A.shape[0], B.shape[1], A.shape[1]), 1, orders, _stream()),
                   "lego_grouped_gemm_f16")
        out = _pinned_like(cd.shape, torch.float16)
        pipe.drain(out, cd)
        outs.append(out)
    pipe.finish()
    return outs
