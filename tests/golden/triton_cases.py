"""Seeded inputs of the golden vectors produced by the reference's own Triton kernels
(make_golden_gpu.py writes the outputs; the pin tests regenerate the inputs from here)."""
import numpy as np

ROW_SHAPES = [(4, 4096), (16, 128), (2, 5000)]   # the C4 widths, and a ragged width
EPS = 1e-6


def row_case(shape, seed=3):
    """x ~ N(0,3), dy ~ N(0,1), gamma ~ N(1,0.02): the C4 value distributions."""
    rng = np.random.default_rng(seed * 1000 + shape[1])
    x = (3.0 * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
    dy = rng.standard_normal(shape, dtype=np.float32)
    gamma = (1 + 0.02 * rng.standard_normal(shape[1])).astype(np.float32)
    return x, dy, gamma


def index_case(seed=2, V=512, D=256, N=1024):
    """A C2-shaped table with uniform indices (gather) and Zipf(1.1) indices (scatter_add)."""
    rng = np.random.default_rng(seed)
    table = rng.standard_normal((V, D), dtype=np.float32)
    idx_u = rng.integers(0, V, N).astype(np.int64)
    p = np.arange(1, V + 1, dtype=np.float64) ** -1.1
    ranks = np.searchsorted(np.cumsum(p / p.sum()), rng.random(N))
    idx_z = rng.permutation(V)[np.minimum(ranks, V - 1)].astype(np.int64)
    upd = rng.standard_normal((N, D), dtype=np.float32)
    return table, idx_u, idx_z, upd
