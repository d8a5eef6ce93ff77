"""GPU test of sb200_colsum_noalloc, the entry point for callers that must not
allocate device memory (they live under another allocator's share of the device memory, or
on a latency path where cudaMalloc would synchronise the device).

It is compared with the column sums the regular entry point
(sb200_gemm_batched with colsum_out) produces, on two calls in a row that share
the library's fixed scratch array.  The file name makes pytest collect it last.
"""
import numpy as np
import pytest
import torch

from sapphire_b200 import _lib as L
from sapphire_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def existing_colsum(ctx, dy, scale):
    """Column sums through the existing entry point: dW = x^T.dy with colsum_out."""
    x = torch.zeros(dy.shape[0], 4, device=DEV)
    out = torch.empty(dy.shape[1], device=DEV)
    ops.gemm(ctx, x, dy, trans_a=True, colsum_out=out, colsum_scale=scale)
    return out


def noalloc_colsum(dy, scale, trans=False):
    rows, cols = dy.shape
    K, N = (cols, rows) if trans else (rows, cols)
    out = torch.full((N,), float("nan"), device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    rc = L.lib().sb200_colsum_noalloc(dy.data_ptr(), int(trans), K, N, dy.stride(0), out.data_ptr(),
                                      scale, st)
    assert rc == L.OK, L.status_string(rc)
    return out


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def test_noalloc_colsum_matches_existing_entry_point_twice(ctx):
    torch.cuda.set_device(0)
    g = torch.Generator(device=DEV)
    g.manual_seed(3)
    # first call: a Linear-backward sized dy; second call: fewer rows and columns,
    # so stale partial sums of the first call sit right next to the cells it uses
    for rows, cols in ((8192, 4096), (1000, 520)):
        dy = torch.randn(rows, cols, device=DEV, generator=g) * 0.02
        want = existing_colsum(ctx, dy, 1.0 / rows)
        got = noalloc_colsum(dy, 1.0 / rows)
        torch.cuda.synchronize()
        assert bool(torch.isfinite(got).all())
        assert rel(got, want) <= 1e-5
        exact = dy.double().sum(0) / rows
        assert rel(got, exact) <= 1e-5
    # transposed operand: op(B)[k, n] = B[n, k]
    b = torch.randn(300, 2048, device=DEV, generator=g)
    got = noalloc_colsum(b, 0.5, trans=True)
    assert rel(got, b.double().sum(1) * 0.5) <= 1e-5


def test_noalloc_colsum_allocates_nothing_and_clamps_slices(ctx):
    """What the entry point is for: after a first call (which looks up the scratch
    array's address) further calls leave the device's free memory unchanged.  The
    second shape, few columns and many rows, asks for more row slices than the
    array has (64): the clamp and the empty trailing slices are exercised."""
    torch.cuda.set_device(0)
    g = torch.Generator(device=DEV)
    g.manual_seed(5)
    dy = torch.randn(4096, 1024, device=DEV, generator=g)
    tall = torch.randn(16384, 64, device=DEV, generator=g)
    out = torch.empty(1024, device=DEV)
    out2 = torch.empty(64, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    lib = L.lib()
    assert lib.sb200_colsum_noalloc(dy.data_ptr(), 0, 4096, 1024, 1024, out.data_ptr(), 1.0, st) == L.OK
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(0)[0]
    assert lib.sb200_colsum_noalloc(dy.data_ptr(), 0, 4096, 1024, 1024, out.data_ptr(), 0.25, st) == L.OK
    assert lib.sb200_colsum_noalloc(tall.data_ptr(), 0, 16384, 64, 64, out2.data_ptr(), 1.0, st) == L.OK
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(0)[0] == free_before
    assert rel(out, dy.double().sum(0) * 0.25) <= 1e-5
    assert rel(out2, tall.double().sum(0)) <= 1e-5


def test_noalloc_colsum_limits():
    torch.cuda.set_device(0)
    lib = L.lib()
    st = torch.cuda.current_stream().cuda_stream
    big_n = 16384 + 4
    b = torch.zeros(2, big_n, device=DEV)
    out = torch.zeros(big_n, device=DEV)
    assert lib.sb200_colsum_noalloc(b.data_ptr(), 0, 2, big_n, big_n, out.data_ptr(), 1.0, st) \
        == L.ERR_TOO_LARGE
    assert lib.sb200_colsum_noalloc(b.data_ptr(), 0, 2, 8, 4, out.data_ptr(), 1.0, st) \
        == L.ERR_INVALID_ARG                      # ld < columns
    assert lib.sb200_colsum_noalloc(None, 0, 2, 8, 8, out.data_ptr(), 1.0, st) == L.ERR_INVALID_ARG
    assert lib.sb200_colsum_noalloc(b.data_ptr(), 0, 0, 8, 8, out.data_ptr(), 1.0, st) == L.OK
    torch.cuda.synchronize()
    assert float(out[:8].abs().max()) == 0.0      # K == 0: sums are zero
