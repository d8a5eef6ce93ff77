"""Conv2D on the batched GEMM: the device version of Sapphire's host lowering
(Sources/Sapphire/compute/dense/naive/Convolution.cpp:217-316).  The reference runs this path
on the host only and hands the GPU case to cuDNN; here the lowering kernels and
the GEMMs all run on the B200 library:

forward    cols = im2col(x);  y[N, Cout, P] += filter[Cout, C*kh*kw] . cols[N, C*kh*kw, P]
           (one batched GEMM, the filter matrix shared by every image: the
           broadcast-A case of ``Compute::Gemm``)
backward   drX[N, C*kh*kw, P] = filter^T . dY      (transposed operand by descriptor)
           dFilter += dY_n . cols_n^T, n = 0 .. N-1 in ascending order, each
           accumulating in place like the reference's batch-1 output
           dx += col2im(drX)
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib as L
from . import ops

Pair = Tuple[int, int]


def out_size(size: int, pad: int, dil: int, k: int, stride: int) -> int:
    return (size + 2 * pad - dil * (k - 1) - 1) // stride + 1


def _geometry(x_shape, kh: int, kw: int, stride: Pair, pad: Pair, dil: Pair) -> L.ConvGeometry:
    N, Cc, H, W = x_shape
    return L.ConvGeometry(N, Cc, H, W, kh, kw, stride[0], stride[1], pad[0], pad[1], dil[0], dil[1])


def im2col(ctx: ops.Context, x: torch.Tensor, kh: int, kw: int, stride: Pair = (1, 1),
           pad: Pair = (0, 0), dil: Pair = (1, 1), pad_value: float = 0.0,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [N, C, H, W] (contiguous) -> cols [N, C*kh*kw, outR*outC] (``out`` if given:
    contiguous, that shape)."""
    N, Cc, H, W = x.shape
    P = out_size(H, pad[0], dil[0], kh, stride[0]) * out_size(W, pad[1], dil[1], kw, stride[1])
    shape = (N, Cc * kh * kw, P)
    if out is None:
        cols = torch.empty(shape, dtype=torch.float32, device=x.device)
    else:
        if tuple(out.shape) != shape or not out.is_contiguous() or out.dtype != torch.float32:
            raise ValueError(f"out must be a contiguous fp32 tensor of shape {shape}")
        cols = out
    g = _geometry(x.shape, kh, kw, stride, pad, dil)
    L.check("sb200_im2col", L.lib().sb200_im2col(ctx.handle, cols.data_ptr(), x.contiguous().data_ptr(),
                                                  C.byref(g), float(pad_value), ops._stream_ptr(ctx.device)))
    return cols


def col2im(ctx: ops.Context, dx: torch.Tensor, cols: torch.Tensor, kh: int, kw: int,
           stride: Pair = (1, 1), pad: Pair = (0, 0), dil: Pair = (1, 1)) -> torch.Tensor:
    """dx [N, C, H, W] (contiguous) += adjoint of im2col applied to cols."""
    g = _geometry(dx.shape, kh, kw, stride, pad, dil)
    L.check("sb200_col2im", L.lib().sb200_col2im(ctx.handle, dx.data_ptr(), cols.data_ptr(), C.byref(g),
                                                  ops._stream_ptr(ctx.device)))
    return dx


def conv2d_forward(ctx: ops.Context, y: torch.Tensor, x: torch.Tensor, filt: torch.Tensor,
                   stride: Pair = (1, 1), pad: Pair = (0, 0), dil: Pair = (1, 1),
                   mode: int = L.MODE_TF32) -> torch.Tensor:
    """y [N, Cout, outR, outC] += conv(x [N, C, H, W], filt [Cout, C, kh, kw]), in place."""
    N, Cout = y.shape[:2]
    kh, kw = filt.shape[-2:]
    cols = im2col(ctx, x, kh, kw, stride, pad, dil)
    y3 = y.view(N, Cout, -1)
    ops.gemm(ctx, filt.reshape(Cout, -1), cols, y3, y3, mode=mode)
    return y


def conv2d_backward(ctx: ops.Context, dx: torch.Tensor, dfilt: torch.Tensor, dy: torch.Tensor,
                    x: torch.Tensor, filt: torch.Tensor, stride: Pair = (1, 1), pad: Pair = (0, 0),
                    dil: Pair = (1, 1), mode: int = L.MODE_TF32):
    """dx += input gradient, dfilt += filter gradient, both in place."""
    N, Cout = dy.shape[:2]
    kh, kw = filt.shape[-2:]
    cols = im2col(ctx, x, kh, kw, stride, pad, dil)
    f2 = filt.reshape(Cout, -1)
    dy3 = dy.reshape(N, Cout, -1)
    drx = ops.gemm(ctx, f2, dy3, mode=mode, trans_a=True)
    df2 = dfilt.view(Cout, -1)
    for n in range(N):
        ops.gemm(ctx, dy3[n], cols[n], df2, df2, mode=mode, trans_b=True)
    col2im(ctx, dx, drx, kh, kw, stride, pad, dil)
    return dx, dfilt
