"""The multi-GPU partitions, exercised on one GPU: each shard is computed by a
separate call exactly as a rank would, and the stitched / reduced result must
equal the unsharded one."""
import numpy as np
import pytest
import torch

from sapphire_b200 import _lib as L
from sapphire_b200 import ops, runner
from sapphire_b200 import workloads as W

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_spgemm_row_blocks_stitch_to_the_full_product(ctx):
    """A row-blocked by scalar products over 4 'ranks', B replicated, no exchange:
    concatenating the blocks' CSR arrays gives the full C bit for bit (ROW, COL)."""
    M = N = 8192
    rA, cA, vA = W.csr_random(0, M, N, row_dist="zipf", zipf_cap=1024)
    rB, cB, vB = W.csr_random(1, N, N, row_dist="zipf", zipf_cap=1024)
    B = ops.CsrMatrix.from_numpy(rB, cB, vB, N, N, DEV)
    full = ops.spgemm(ctx, ops.CsrMatrix.from_numpy(rA, cA, vA, M, N, DEV), B)
    fr, fc, fv = full.to_numpy()
    work = W.csr_products(rA, cA, rB)
    blocks = runner.balanced_row_blocks(work, 4)
    rows, cols, vals, base = [np.zeros(1, np.int64)], [], [], 0
    for blk in blocks:
        rb, cb, vb = runner.csr_row_block(rA, cA, vA, blk)
        part = ops.spgemm(ctx, ops.CsrMatrix.from_numpy(rb, cb, vb, len(blk), N, DEV), B)
        pr, pc, pv = part.to_numpy()
        rows.append(pr[1:].astype(np.int64) + base)     # global offsets: prefix over the blocks
        base += int(pr[-1])
        cols.append(pc)
        vals.append(pv)
    row = np.concatenate(rows)
    assert np.array_equal(row.astype(np.uint32), fr)
    assert np.array_equal(np.concatenate(cols), fc)
    assert np.abs(np.concatenate(vals) - fv).max() <= 1e-5 * max(np.abs(fv).max(), 1.0)
    # the blocks are balanced by work, not by rows
    sums = np.array([work[b.start:b.stop].sum() for b in blocks])
    assert sums.max() <= work.sum() / 4 + work.max()


def test_linear_backward_row_shards_reduce_to_the_full_gradients(ctx):
    """Rows of dY / X split over 4 'ranks': dX rows are final, dW is the SUM of
    the partial products, dB the MEAN of the partial column means."""
    rows, n_in, n_out, world = 1024, 256, 384, 4
    g = torch.Generator(device=DEV); g.manual_seed(5)
    dy = torch.randn(rows, n_out, device=DEV, generator=g) * 0.02
    x = torch.randn(rows, n_in, device=DEV, generator=g) * 0.02
    w = torch.randn(n_in, n_out, device=DEV, generator=g) * 0.02
    mode = L.MODE_TF32X3
    dx_full = ops.gemm(ctx, dy, w, trans_b=True, mode=mode)
    db_full = torch.empty(n_out, device=DEV)
    dw_full = ops.gemm(ctx, x, dy, trans_a=True, mode=mode, colsum_out=db_full, colsum_scale=1.0 / rows)
    dw_sum = torch.zeros_like(dw_full)
    db_sum = torch.zeros_like(db_full)
    dx_parts = []
    for r in range(world):
        blk = runner.row_shard(rows, world, r, align=128)
        sl = slice(blk.start, blk.stop)
        dx_parts.append(ops.gemm(ctx, dy[sl], w, trans_b=True, mode=mode))
        db = torch.empty(n_out, device=DEV)
        dw = ops.gemm(ctx, x[sl], dy[sl], trans_a=True, mode=mode, colsum_out=db,
                      colsum_scale=1.0 / len(blk))
        dw_sum += dw                 # what the allreduce-SUM does
        db_sum += db
    db_mean = db_sum / world         # allreduce-SUM then 1 / world
    rel = lambda a, b: float((a.double() - b.double()).norm() / b.double().norm())
    assert torch.equal(torch.cat(dx_parts), dx_full)
    assert rel(dw_sum, dw_full) <= 1e-5
    assert rel(db_mean, db_full) <= 1e-5
