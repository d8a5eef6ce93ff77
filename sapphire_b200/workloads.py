"""Seeded synthetic inputs for the five workload configurations.

All generators are numpy (PCG64 through ``default_rng``) so that the CPU
checker and the CUDA path see the same bits on any machine, and so that the
result does not depend on how many GPUs the work is later sharded over: a
batched tensor is drawn one batch at a time from ``default_rng([seed, tag,
batch])``, hence a rank can draw only the batches it owns.

Values are drawn in float64 and cast to float32.
"""
from __future__ import annotations

import numpy as np

_TAG = {"a": 1, "b": 2, "c": 3, "dy": 4, "x": 5, "w": 6}


def _rng(seed: int, tag: str, batch: int = 0):
    return np.random.default_rng([seed, _TAG[tag], batch])


def uniform_pm1(seed, tag, shape, batch=0):
    return _rng(seed, tag, batch).uniform(-1.0, 1.0, size=shape).astype(np.float32)


def normal(seed, tag, shape, std=1.0, batch=0):
    return (_rng(seed, tag, batch).standard_normal(size=shape) * std).astype(np.float32)


def dense_batched(seed, batch_ids, M, N, K, dist="uniform"):
    """a [b,M,K], b [b,K,N], c [b,M,N] for the listed batch indices.

    dist="uniform": a, b, c ~ U[-1,1)            (4 x 256^3 case)
    dist="normal":  a, b ~ N(0,1), c ~ U[-1,1)   (8 x 4096^3 / 4000^3 case)
    """
    a = np.empty((len(batch_ids), M, K), np.float32)
    b = np.empty((len(batch_ids), K, N), np.float32)
    c = np.empty((len(batch_ids), M, N), np.float32)
    for i, bi in enumerate(batch_ids):
        if dist == "uniform":
            a[i] = uniform_pm1(seed, "a", (M, K), bi)
            b[i] = uniform_pm1(seed, "b", (K, N), bi)
        else:
            a[i] = normal(seed, "a", (M, K), 1.0, bi)
            b[i] = normal(seed, "b", (K, N), 1.0, bi)
        c[i] = uniform_pm1(seed, "c", (M, N), bi)
    return a, b, c


ROW_BLOCK = 1024  # rows drawn per generator call for the Linear-backward case


def linear_backward(seed, row_lo, row_hi, n_in=4096, n_out=4096, std=0.02):
    """dY [rows, out], X [rows, in] for global rows [row_lo, row_hi) and the full
    W [in, out] (Sapphire stores the weight [in, out]), all N(0, std).

    Rows are drawn in blocks of ROW_BLOCK so that any row range aligned to it
    reproduces the same values as the full tensor.
    """
    assert row_lo % ROW_BLOCK == 0 and (row_hi % ROW_BLOCK == 0)
    dy = np.empty((row_hi - row_lo, n_out), np.float32)
    x = np.empty((row_hi - row_lo, n_in), np.float32)
    for blk in range(row_lo // ROW_BLOCK, row_hi // ROW_BLOCK):
        o = blk * ROW_BLOCK - row_lo
        dy[o:o + ROW_BLOCK] = normal(seed, "dy", (ROW_BLOCK, n_out), std, blk)
        x[o:o + ROW_BLOCK] = normal(seed, "x", (ROW_BLOCK, n_in), std, blk)
    w = normal(seed, "w", (n_in, n_out), std, 0)
    return dy, x, w


# ------------------------------------------------------------------ MLP

MLP_WIDTHS = (784, 512, 256, 10)


def mlp_init(seed, widths=MLP_WIDTHS):
    """He-uniform W_l ~ U(+-sqrt(6/in)) stored [in, out]; biases zero."""
    rng = np.random.default_rng(seed)
    Ws, bs = [], []
    for fan_in, fan_out in zip(widths[:-1], widths[1:]):
        lim = np.sqrt(6.0 / fan_in)
        Ws.append(rng.uniform(-lim, lim, size=(fan_in, fan_out)).astype(np.float32))
        bs.append(np.zeros(fan_out, np.float32))
    return Ws, bs


def mlp_batch(step, batch=64, widths=MLP_WIDTHS):
    """x ~ U[0,1) [batch, in]; labels uniform over the classes, one-hot fp32."""
    rng = np.random.default_rng(1000 + step)
    x = rng.uniform(0.0, 1.0, size=(batch, widths[0])).astype(np.float32)
    lab = rng.integers(0, widths[-1], size=batch)
    onehot = np.zeros((batch, widths[-1]), np.float32)
    onehot[np.arange(batch), lab] = 1.0
    return x, onehot


# ------------------------------------------------------------------ CSR

def _sorted_unique(keys):
    keys = np.sort(keys)
    if keys.size == 0:
        return keys
    keep = np.empty(keys.size, bool)
    keep[0] = True
    np.not_equal(keys[1:], keys[:-1], out=keep[1:])
    return keys[keep]


def _distinct_cols(rng, counts, N):
    """For every row i, counts[i] distinct columns uniform over [0, N).

    Draw with replacement, drop duplicates, redraw the deficit until none is
    left (rejection sampling of distinct sets).  Returns int64 keys row*N+col,
    sorted, i.e. ascending column inside every row.
    """
    M = counts.size
    ridx = np.arange(M, dtype=np.int64)
    rows = np.repeat(ridx, counts)
    keys = _sorted_unique(rows * N + rng.integers(0, N, size=rows.size))
    while True:
        have = np.bincount(keys // N, minlength=M)
        deficit = counts - have
        if not deficit.any():
            return keys
        rows = np.repeat(ridx, deficit)
        keys = _sorted_unique(np.concatenate([keys, rows * N + rng.integers(0, N, size=rows.size)]))


def zipf_counts(rng, M, s=1.5, cap=4096):
    """Truncated Zipf(s) on {1..cap} by inverse CDF of the explicit pmf."""
    k = np.arange(1, cap + 1, dtype=np.float64)
    cdf = np.cumsum(k ** (-s))
    cdf /= cdf[-1]
    return (np.searchsorted(cdf, rng.uniform(size=M), side="left") + 1).astype(np.int64)


def csr_random(seed, M, N, density=None, row_dist="poisson", zipf_s=1.5, zipf_cap=4096):
    """(ROW uint32[M+1], COL uint32[nnz], V float32[nnz]).

    row_dist="poisson": nnz per row ~ Poisson(density*N), clipped to [0, N]
    row_dist="zipf":    nnz per row ~ truncated Zipf(zipf_s) on {1..min(zipf_cap, N)}
    Column positions uniform without replacement, ascending; values U[-1,1).
    """
    rng = np.random.default_rng(seed)
    if row_dist == "poisson":
        counts = np.clip(rng.poisson(density * N, size=M), 0, N).astype(np.int64)
    elif row_dist == "zipf":
        counts = zipf_counts(rng, M, zipf_s, min(zipf_cap, N))
    else:
        raise ValueError(row_dist)
    keys = _distinct_cols(rng, counts, N)
    row = np.zeros(M + 1, np.int64)
    np.cumsum(counts, out=row[1:])
    col = (keys % N).astype(np.uint32)
    val = rng.uniform(-1.0, 1.0, size=col.size).astype(np.float32)
    return row.astype(np.uint32), col, val


def csr_products(rowA, colA, rowB):
    """Scalar products of C = A.B per row of A (int64[M])."""
    nnzB = np.diff(rowB.astype(np.int64))
    per_nz = nnzB[colA]
    cs = np.concatenate([[0], np.cumsum(per_nz)])
    return cs[rowA[1:].astype(np.int64)] - cs[rowA[:-1].astype(np.int64)]
