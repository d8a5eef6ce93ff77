"""GPU parity tests of the convolution lowering (im2col / col2im kernels and the
Conv2D forward / backward composed from them and the batched GEMM) against the
CPU restatement of Sapphire's host path.  Data movement is bit-exact; the GEMMs
carry the dense tolerances (3xTF32 1e-5, TF32 2e-3 relative Frobenius)."""
import ctypes as C

import numpy as np
import pytest
import torch

from sapphire_b200 import _lib as L
from sapphire_b200 import conv, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CASES = [
    # N, C, H, W, Cout, kh, kw, stride, pad, dil
    (2, 3, 8, 9, 4, 3, 3, (1, 1), (1, 1), (1, 1)),
    (1, 2, 11, 7, 5, 3, 2, (2, 1), (0, 1), (1, 2)),
    (3, 1, 6, 6, 2, 1, 1, (1, 1), (0, 0), (1, 1)),
    (2, 4, 10, 10, 3, 5, 5, (2, 2), (2, 2), (1, 1)),
    (1, 2, 9, 12, 2, 2, 3, (3, 2), (1, 0), (2, 1)),
    (4, 16, 32, 32, 32, 3, 3, (1, 1), (1, 1), (1, 1)),      # P = 1024: the tensor-core path
]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def rel_fro(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)


@pytest.mark.parametrize("case", CASES)
def test_im2col_and_col2im_are_bit_exact(ctx, oracle, case):
    N, Cc, H, W, _, kh, kw, stride, pad, dil = case
    rng = np.random.default_rng(sum(case[:7]))
    x = rng.standard_normal((N, Cc, H, W)).astype(np.float32)
    want = oracle.im2col(x, kh, kw, stride, pad, dil, pad_value=0.5)
    got = conv.im2col(ctx, dev(x), kh, kw, stride, pad, dil, pad_value=0.5).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    m = rng.standard_normal(want.shape).astype(np.float32)
    dx0 = rng.standard_normal(x.shape).astype(np.float32)
    wdx = oracle.col2im(dx0.copy(), m, kh, kw, stride, pad, dil)
    gdx = conv.col2im(ctx, dev(dx0), dev(m), kh, kw, stride, pad, dil).cpu().numpy()
    assert np.array_equal(gdx.view(np.uint32), wdx.view(np.uint32))


@pytest.mark.parametrize("mode,tol", [(L.MODE_TF32X3, 1e-5), (L.MODE_TF32, 2e-3)])
@pytest.mark.parametrize("case", CASES)
def test_conv2d_forward_and_backward_match_the_host_path(ctx, oracle, case, mode, tol):
    N, Cc, H, W, Cout, kh, kw, stride, pad, dil = case
    rng = np.random.default_rng(sum(case[:7]) + 1)
    x = rng.standard_normal((N, Cc, H, W)).astype(np.float32)
    f = rng.standard_normal((Cout, Cc, kh, kw)).astype(np.float32)
    outR = conv.out_size(H, pad[0], dil[0], kh, stride[0])
    outC = conv.out_size(W, pad[1], dil[1], kw, stride[1])
    y0 = rng.standard_normal((N, Cout, outR, outC)).astype(np.float32)
    want = oracle.conv2d(y0, x, f, stride, pad, dil)
    got = conv.conv2d_forward(ctx, dev(y0), dev(x), dev(f), stride, pad, dil, mode=mode).cpu().numpy()
    assert rel_fro(got, want) <= tol
    dy = rng.standard_normal(y0.shape).astype(np.float32)
    dx0 = rng.standard_normal(x.shape).astype(np.float32)
    df0 = rng.standard_normal(f.shape).astype(np.float32)
    wdx, wdf = oracle.conv2d_backward(dx0, df0, dy, x, f, stride, pad, dil)
    gdx, gdf = conv.conv2d_backward(ctx, dev(dx0), dev(df0), dev(dy), dev(x), dev(f), stride, pad, dil,
                                    mode=mode)
    assert rel_fro(gdx.cpu().numpy(), wdx) <= tol
    assert rel_fro(gdf.cpu().numpy(), wdf) <= tol
    ctx.check_device_status()


def test_conv_geometry_validation(ctx):
    x = torch.zeros(1, 1, 4, 4, device=DEV)
    bad = [dict(kh=0), dict(strideR=0), dict(dilC=0), dict(padR=-1), dict(kh=7)]   # 7x7 taps do not fit 4x4
    for change in bad:
        g = dict(N=1, C=1, H=4, W=4, kh=3, kw=3, strideR=1, strideC=1, padR=0, padC=0, dilR=1, dilC=1)
        g.update(change)
        geom = L.ConvGeometry(**g)
        rc = L.lib().sb200_im2col(ctx.handle, x.data_ptr(), x.data_ptr(), C.byref(geom), 0.0, None)
        assert rc == L.ERR_INVALID_ARG, change


def test_empty_batch_is_a_no_op(ctx):
    x = torch.zeros(0, 3, 8, 8, device=DEV)
    cols = conv.im2col(ctx, x, 3, 3, (1, 1), (1, 1), (1, 1))
    assert cols.shape == (0, 27, 64)
