"""Build ``liblego_b200.so`` in-tree with nvcc for sm_100a.

    python -m lego_b200.build [--force] [--verbose]

Each source under ``csrc/`` is compiled to an object (in parallel, only when it
or a header changed) and linked into ``lego_b200/liblego_b200.so``.  nvcc
cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
OUT = os.path.join(HERE, "liblego_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
          "-Xcompiler", "-Wall", "-Xcompiler", "-Wno-unused-function"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: lego_b200 needs the CUDA toolkit (sm_100a) to build")
    return exe


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _headers_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    paths.append(os.path.join(HERE, "..", "include", "lego_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    extra = os.environ.get("LEGO_B200_NVCC_FLAGS", "").split()   # e.g. -DNAME for an instrumented build
    cmd = [_nvcc(), *ARCH, *CFLAGS, *extra, "-x", "cu", "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr = _headers_mtime()
    todo, objs = [], []
    for src in _sources():
        obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        stale = (force or not os.path.exists(obj)
                 or os.path.getmtime(obj) < max(hdr, os.path.getmtime(os.path.join(CSRC, src))))
        if stale:
            todo.append(src)
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as pool:
            list(pool.map(lambda s: _compile(s, verbose), todo))
    if todo or not os.path.exists(OUT):
        cmd = [_nvcc(), *ARCH, "-shared", "-cudart", "static", "-o", OUT, *objs]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return OUT


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / shared-memory usage")
    args = ap.parse_args()
    print(build(args.force, args.verbose))


if __name__ == "__main__":
    main()
