"""Seeded synthetic inputs of the five benchmark configurations (shapes, dtypes
and value distributions as the benchmark description names them), shared by
bench.py, the smoke run and the tests.  All generation happens on the CPU
generator so the values do not depend on the GPU."""
import functools
import math

import torch

GROUPED_CHOICES = (1024, 2048, 4096)

# Generating a 16384 x 8192 tensor on the CPU generator takes seconds, and a benchmark run asks
# for the same tensor more than once (sharded and replicated legs): results are kept, read-only,
# until clear_cache() is called.
_cached = functools.lru_cache(maxsize=None)


def clear_cache():
    for fn in (transpose_input, softmax_input, layernorm_input, gemm_input, grouped_input):
        fn.cache_clear()



@_cached
def transpose_input(n=4096, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(n, n, generator=g, dtype=torch.float32) * 2 - 1


@_cached
def softmax_input(rows=16384, cols=8192, seed=1):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * 2).half()


@_cached
def layernorm_input(rows=16384, cols=8192, seed=2):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g).half()
    gamma = (1 + 0.1 * torch.randn(cols, generator=g)).half()
    beta = (0.1 * torch.randn(cols, generator=g)).half()
    return x, gamma, beta


@_cached
def gemm_input(m=8192, n=8192, k=8192, seed=3):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(m, k, generator=g) / math.sqrt(k)).half()
    b = (torch.randn(k, n, generator=g) / math.sqrt(k)).half()
    return a, b


def grouped_sizes(groups=16, k=4096, seed=4):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, 3, (groups, 2), generator=g)
    return [(GROUPED_CHOICES[int(i)], GROUPED_CHOICES[int(j)], k) for i, j in idx], g


@_cached
def grouped_input(groups=16, k=4096, seed=4, scale_rows=1):
    """A_g [M_g / scale_rows, K], B_g [K, N_g]; scale_rows shrinks M for quick tests."""
    sizes, g = grouped_sizes(groups, k, seed)
    A, B = [], []
    for m, n, kk in sizes:
        A.append((torch.randn(m // scale_rows, kk, generator=g) / 64).half())
        B.append((torch.randn(kk, n, generator=g) / 64).half())
    return A, B
