"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

ctypes front end of the two CPU checkers:

* ``port``  -- ``oracle/sapphire_oracle.c``, the restatement of Sapphire's CPU
  arithmetic (built on demand with gcc into ``oracle/_build``);
* ``ref``   -- ``oracle/_ref/libsapphire_ref.so``, the reference's own CPU leaf
  files compiled by ``oracle/Makefile`` from the reference tree.  It exists
  only where that tree was present at build time (or the prebuilt ``.so`` was
  shipped along); ``have_ref()`` says which.  ``ref_conv`` is the same for the
  reference's host convolution (``oracle/_ref/libsapphire_ref_ops.so``).

Only tests, the smoke check and the CPU-baseline legs of the benchmark import
this module.  The product package never does.

Dense parity is pinned (port == ref bit-for-bit, plus fixtures made from ref
under ``tests/golden``), the convolution lowering and its composition included.
Sparse parity is UNPINNED: the reference ships no
sparse GEMM implementation, see the header of ``sapphire_oracle.c``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT_SO = os.path.join(_HERE, "_build", "libsapphire_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libsapphire_ref.so")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")


def build(with_ref: bool = True) -> None:
    """Run oracle/Makefile (port always; ref when the reference tree is there)."""
    target = "all" if with_ref else os.path.join(_HERE, "_build", "libsapphire_oracle.so")
    subprocess.run(["make", "-s", "-C", _HERE, "-f", os.path.join(_HERE, "Makefile"), target],
                   check=True)


_port = None
_ref = None


def port():
    global _port
    if _port is None:
        src = os.path.join(_HERE, "sapphire_oracle.c")
        if (not os.path.exists(_PORT_SO)
                or os.path.getmtime(_PORT_SO) < os.path.getmtime(src)):
            build(with_ref=False)
        lib = C.CDLL(_PORT_SO)
        lib.orc_gemm.argtypes = [C.c_uint, _f32p, _f32p, _f32p, C.c_uint, C.c_uint, C.c_uint]
        lib.orc_gemm.restype = None
        lib.orc_gemm_ex.argtypes = [C.c_int, C.c_int, C.c_long, C.c_long, C.c_long,
                                    C.c_void_p, C.c_long, C.c_long,
                                    C.c_void_p, C.c_long, C.c_long,
                                    C.c_void_p, C.c_long, C.c_long,
                                    C.c_void_p, C.c_long, C.c_long,
                                    C.c_void_p, C.c_long]
        lib.orc_gemm_ex.restype = None
        lib.orc_colsum.argtypes = [_f32p, C.c_void_p, C.c_long, C.c_long, C.c_long, C.c_float]
        lib.orc_colsum.restype = None
        lib.orc_transpose.argtypes = [_f32p, _f32p, C.c_uint, C.c_uint, C.c_uint, C.c_int]
        lib.orc_scale.argtypes = [_f32p, _f32p, C.c_float, C.c_uint]
        lib.orc_sub.argtypes = [_f32p, _f32p, _f32p, C.c_uint]
        lib.orc_relu.argtypes = [_f32p, _f32p, C.c_uint]
        lib.orc_relu_backward.argtypes = [_f32p, _f32p, _f32p, C.c_uint]
        lib.orc_softmax.argtypes = [_f32p, _f32p, C.c_uint, C.c_uint]
        lib.orc_softmax_backward.argtypes = [_f32p, _f32p, _f32p, C.c_uint, C.c_uint]
        lib.orc_cross_entropy.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]
        lib.orc_cross_entropy_backward.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]
        for n in ("orc_transpose", "orc_scale", "orc_sub", "orc_relu", "orc_relu_backward",
                  "orc_softmax", "orc_softmax_backward", "orc_cross_entropy",
                  "orc_cross_entropy_backward"):
            getattr(lib, n).restype = None
        conv_geom = [C.c_int] * 12
        lib.orc_im2col.argtypes = [_f32p, _f32p] + conv_geom + [C.c_float]
        lib.orc_col2im.argtypes = [_f32p, _f32p] + conv_geom
        lib.orc_spgemm_symbolic.argtypes = [C.c_uint32, C.c_uint32, _u32p, _u32p, _u32p, _u32p,
                                            _u32p, C.POINTER(C.c_long)]
        lib.orc_spgemm_symbolic.restype = C.c_long
        lib.orc_spgemm_numeric.argtypes = [C.c_uint32, C.c_uint32, _u32p, _u32p, _f32p,
                                           _u32p, _u32p, _f32p, _u32p, _u32p, _f32p]
        lib.orc_spgemm_numeric.restype = C.c_int
        _port = lib
    return _port


def have_ref() -> bool:
    return os.path.exists(_REF_SO)


def ref():
    global _ref
    if _ref is None:
        if not have_ref():
            raise FileNotFoundError(
                f"{_REF_SO} is missing: run `make -C oracle` where the reference tree is mounted")
        lib = C.CDLL(_REF_SO)
        lib.ref_gemm.argtypes = [C.c_uint, _f32p, _f32p, _f32p, C.c_uint, C.c_uint, C.c_uint]
        lib.ref_transpose.argtypes = [_f32p, _f32p, C.c_uint, C.c_uint, C.c_uint, C.c_int]
        lib.ref_scale.argtypes = [_f32p, _f32p, C.c_float, C.c_uint]
        lib.ref_sub.argtypes = [C.c_uint, _f32p, _f32p, _f32p, C.c_uint, C.c_int, C.c_int]
        lib.ref_relu.argtypes = [_f32p, _f32p, C.c_uint]
        lib.ref_relu_backward.argtypes = [_f32p, _f32p, _f32p, C.c_uint]
        lib.ref_softmax.argtypes = [_f32p, _f32p, C.c_uint, C.c_uint]
        lib.ref_softmax_backward.argtypes = [_f32p, _f32p, _f32p, C.c_uint, C.c_uint]
        lib.ref_cross_entropy.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]
        lib.ref_cross_entropy_backward.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]
        for n in ("ref_gemm", "ref_transpose", "ref_scale", "ref_sub", "ref_relu",
                  "ref_relu_backward", "ref_softmax", "ref_softmax_backward",
                  "ref_cross_entropy", "ref_cross_entropy_backward"):
            getattr(lib, n).restype = None
        _ref = lib
    return _ref


_REF_OPS_SO = os.path.join(os.path.dirname(_REF_SO), "libsapphire_ref_ops.so")
_ref_ops = None


def have_ref_ops() -> bool:
    return os.path.exists(_REF_OPS_SO)


def ref_ops():
    """The reference's own host convolution and Linear backward unit (Convolution.cpp,
    LinearBackward.cpp, SGD.cpp compiled unmodified against stand-in TensorData /
    CudaDevice / Model headers: oracle/ref_ops_shim.cpp)."""
    global _ref_ops
    if _ref_ops is None:
        if not have_ref_ops():
            raise FileNotFoundError(
                f"{_REF_OPS_SO} is missing: run `make -C oracle` where the reference tree is mounted")
        lib = C.CDLL(_REF_OPS_SO)
        ints = [C.c_int] * 14
        lib.ref_im2col.argtypes = [_f32p, _f32p] + ints + [C.c_float]
        lib.ref_col2im.argtypes = [_f32p, _f32p] + ints
        lib.ref_conv2d.argtypes = [_f32p] * 3 + [C.c_int] * 15
        lib.ref_conv2d_backward.argtypes = [_f32p] * 5 + [C.c_int] * 15
        i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
        lib.ref_compute_gemm.argtypes = [_f32p, i32p, C.c_int, _f32p, i32p, C.c_int, _f32p, i32p, C.c_int]
        lib.ref_linear_backprop.argtypes = [_f32p] * 5 + [C.c_int] * 3 + [C.c_float]
        lib.ref_mul_backprop.argtypes = [_f32p] * 5 + [C.c_int] * 4
        for n in ("ref_im2col", "ref_col2im", "ref_conv2d", "ref_conv2d_backward", "ref_compute_gemm",
                  "ref_linear_backprop", "ref_mul_backprop"):
            getattr(lib, n).restype = None
        _ref_ops = lib
    return _ref_ops


def ref_linear_backprop(dx, dy, weight, bias, x, lr):
    """The reference's LinearBackProp unit with SGD inside
    (Sources/Sapphire/operations/Backward/LinearBackward.cpp:27-99,
    Sources/Sapphire/operations/optimizers/SGD.cpp:22-28), run by the reference build.
    Returns (dx + dy.W^T, updated weight, updated bias) as copies."""
    B, n_in = x.shape
    n_out = dy.shape[1]
    dxo = np.ascontiguousarray(dx, dtype=np.float32).copy()
    w = np.ascontiguousarray(weight, dtype=np.float32).copy()
    b = np.ascontiguousarray(bias, dtype=np.float32).reshape(-1).copy()
    ref_ops().ref_linear_backprop(dxo.reshape(-1), _c(dy).reshape(-1), w.reshape(-1), b, _c(x).reshape(-1),
                                  B, n_in, n_out, float(lr))
    return dxo, w, b


def matmul_backward(da, db, dy, a, b, impl: str = "port"):
    """The MatMul backward unit (Sources/Sapphire/operations/Backward/MathBackward.cpp:39-51):
    da [batch, M, K] + dy . b^T and db [batch, K, N] + a^T . dy, each a Transpose into a
    fresh buffer followed by an accumulating Gemm.  impl "ref" runs the reference's own
    MulBackProp.  Returns copies (da, db)."""
    batch, M, K = a.shape
    N = b.shape[2]
    dao = np.ascontiguousarray(da, dtype=np.float32).copy()
    dbo = np.ascontiguousarray(db, dtype=np.float32).copy()
    if impl == "ref":
        ref_ops().ref_mul_backprop(dao.reshape(-1), dbo.reshape(-1), _c(dy).reshape(-1), _c(a).reshape(-1),
                                   _c(b).reshape(-1), batch, M, K, N)
        return dao, dbo
    return gemm(dao, dy, transpose(b)), gemm(dbo, transpose(a), dy)


def ref_compute_gemm(y, a, b):
    """y + a.b by the reference's Compute::Gemm host path (shape expansion and
    BroadcastWith2Inputs of the reference, Sources/Sapphire/compute/BasicOps.cpp:183-248,
    Includes/Sapphire/compute/Broadcast.hpp:82-133, over Dense::Naive::Gemm); returns a copy."""
    out = np.ascontiguousarray(y, dtype=np.float32).copy()
    sh = lambda t: np.asarray(t.shape, dtype=np.int32)
    ref_ops().ref_compute_gemm(out.reshape(-1), sh(out), out.ndim, _c(a).reshape(-1), sh(a), a.ndim,
                                _c(b).reshape(-1), sh(b), b.ndim)
    return out


# ---------------------------------------------------------------- dense helpers

def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def gemm(c, a, b, impl: str = "port"):
    """y = c + a.b over [batch, M, K] x [batch, K, N]; returns a new array.

    The reference entry point accumulates into y (Compute::Gemm,
    Sources/Sapphire/compute/BasicOps.cpp:183-248), so "c" is the initial y.
    """
    a, b = _c(a), _c(b)
    y = _c(c).copy()
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-1]
    fn = port().orc_gemm if impl == "port" else ref().ref_gemm
    fn(y.size, y.reshape(-1), a.reshape(-1), b.reshape(-1), M, N, K)
    return y


def gemm_ex(transA, transB, M, N, K, A, lda, strideA, B, ldb, strideB,
            C_, ldc, strideC, ldd, strideD, bias, batch, d_size):
    """General strided form on flat fp32 buffers; returns the flat D buffer.

    C_ may be None.  D starts as a copy of C_ when the two have the same
    geometry (the in-place case), else zeros.
    """
    A, B = _c(A).reshape(-1), _c(B).reshape(-1)
    D = np.zeros(d_size, dtype=np.float32)
    cptr = None
    if C_ is not None:
        C_ = _c(C_).reshape(-1)
        cptr = C_.ctypes.data
    bptr = None
    if bias is not None:
        bias = _c(bias).reshape(-1)
        bptr = bias.ctypes.data
    port().orc_gemm_ex(int(transA), int(transB), M, N, K,
                       A.ctypes.data, lda, strideA, B.ctypes.data, ldb, strideB,
                       cptr, ldc, strideC, D.ctypes.data, ldd, strideD, bptr, batch)
    return D


def colsum(dy, scale: float, ld=None):
    dy = _c(dy)
    rows, cols = dy.shape
    out = np.zeros(cols, dtype=np.float32)
    port().orc_colsum(out, dy.ctypes.data, rows, cols, ld or cols, scale)
    return out


def transpose(x, impl: str = "port"):
    x = _c(x)
    x3 = x.reshape((-1,) + x.shape[-2:])
    out = np.empty((x3.shape[0], x3.shape[2], x3.shape[1]), dtype=np.float32)
    fn = port().orc_transpose if impl == "port" else ref().ref_transpose
    fn(out.reshape(-1), x3.reshape(-1), x3.shape[1], x3.shape[2], x3.shape[0], 0)
    return out.reshape(x.shape[:-2] + (x.shape[-1], x.shape[-2]))


# ------------------------------------------------------------- convolution

def conv_out(size, pad, dil, k, stride):
    return (size + 2 * pad - dil * (k - 1) - 1) // stride + 1


def im2col(x, kh, kw, stride=(1, 1), pad=(0, 0), dil=(1, 1), pad_value=0.0, impl: str = "port"):
    """x [N, C, H, W] -> cols [N, C*kh*kw, outR*outC] (taps stored in reverse).
    impl "ref" runs the reference's own Im2Col
    (Sources/Sapphire/compute/dense/naive/Convolution.cpp:15-115)."""
    x = _c(x)
    N, Cc, H, W = x.shape
    oR, oC = conv_out(H, pad[0], dil[0], kh, stride[0]), conv_out(W, pad[1], dil[1], kw, stride[1])
    cols = np.empty((N, Cc * kh * kw, oR * oC), dtype=np.float32)
    if impl == "ref":
        ref_ops().ref_im2col(cols.reshape(-1), x.reshape(-1), N, Cc, H, W, kh, kw, stride[0], stride[1],
                              pad[0], pad[1], dil[0], dil[1], oR, oC, pad_value)
    else:
        port().orc_im2col(cols.reshape(-1), x.reshape(-1), N, Cc, H, W, kh, kw, stride[0], stride[1],
                          pad[0], pad[1], dil[0], dil[1], pad_value)
    return cols


def col2im(dx, cols, kh, kw, stride=(1, 1), pad=(0, 0), dil=(1, 1), impl: str = "port"):
    """dx [N, C, H, W] += adjoint of im2col applied to cols; returns dx.
    impl "ref": the reference's own Col2Im (Convolution.cpp:117-211)."""
    assert dx.dtype == np.float32 and dx.flags.c_contiguous
    cols = _c(cols)
    N, Cc, H, W = dx.shape
    if impl == "ref":
        oR, oC = conv_out(H, pad[0], dil[0], kh, stride[0]), conv_out(W, pad[1], dil[1], kw, stride[1])
        ref_ops().ref_col2im(dx.reshape(-1), cols.reshape(-1), N, Cc, H, W, kh, kw, stride[0], stride[1],
                              pad[0], pad[1], dil[0], dil[1], oR, oC)
    else:
        port().orc_col2im(dx.reshape(-1), cols.reshape(-1), N, Cc, H, W, kh, kw, stride[0], stride[1],
                          pad[0], pad[1], dil[0], dil[1])
    return dx


def _conv_geometry(x, filt, stride, pad, dil):
    N, Cc, H, W = x.shape
    Cout, _, kh, kw = filt.shape
    oR, oC = conv_out(H, pad[0], dil[0], kh, stride[0]), conv_out(W, pad[1], dil[1], kw, stride[1])
    return (N, Cc, H, W, Cout, kh, kw, stride[0], stride[1], pad[0], pad[1], dil[0], dil[1], oR, oC)


def conv2d(y, x, filt, stride=(1, 1), pad=(0, 0), dil=(1, 1), impl: str = "port"):
    """y [N, Cout, outR, outC] += conv(x, filt) the way the reference's host path
    composes it: Im2Col, then Gemm(rY[N,Cout,P], rFilter[1,Cout,C*kh*kw], rX)
    (Sources/Sapphire/compute/dense/naive/Convolution.cpp:217-253).  impl "ref" runs
    that function itself."""
    N, Cout = y.shape[:2]
    kh, kw = filt.shape[-2:]
    if impl == "ref":
        out = np.ascontiguousarray(y, dtype=np.float32).copy()
        ref_ops().ref_conv2d(out.reshape(-1), _c(x).reshape(-1), _c(filt).reshape(-1),
                              *_conv_geometry(x, filt, stride, pad, dil))
        return out
    cols = im2col(x, kh, kw, stride, pad, dil)
    f2 = np.repeat(_c(filt).reshape(1, Cout, -1), N, 0)
    return gemm(_c(y).reshape(N, Cout, -1), f2, cols).reshape(y.shape)


def conv2d_backward(dx, dfilt, dy, x, filt, stride=(1, 1), pad=(0, 0), dil=(1, 1), impl: str = "port"):
    """dx += ..., dfilt += ... as Conv2DBackward composes them
    (Convolution.cpp:255-316): drX = filter^T . dY per batch, dFilter += dY_n . rX_n^T
    over the batches in ascending order, Col2Im(dx, drX).  Returns (dx, dfilt).
    impl "ref" runs that function itself."""
    N, Cout = dy.shape[:2]
    kh, kw = filt.shape[-2:]
    if impl == "ref":
        dxo = np.ascontiguousarray(dx, dtype=np.float32).copy()
        dfo = np.ascontiguousarray(dfilt, dtype=np.float32).copy()
        ref_ops().ref_conv2d_backward(dxo.reshape(-1), dfo.reshape(-1), _c(dy).reshape(-1), _c(x).reshape(-1),
                                       _c(filt).reshape(-1), *_conv_geometry(x, filt, stride, pad, dil))
        return dxo, dfo
    cols = im2col(x, kh, kw, stride, pad, dil)
    f2 = _c(filt).reshape(1, Cout, -1)
    dy3 = _c(dy).reshape(N, Cout, -1)
    drx = gemm(np.zeros_like(cols), np.repeat(transpose(f2), N, 0), dy3)
    colsT = transpose(cols)
    df = _c(dfilt).reshape(1, Cout, -1).copy()
    for n in range(N):                      # y's batch is 1: the N products accumulate in place
        df = gemm(df, dy3[n:n + 1], colsT[n:n + 1])
    dx = col2im(np.ascontiguousarray(dx, dtype=np.float32).copy(), drx, kh, kw, stride, pad, dil)
    return dx, df.reshape(dfilt.shape)


# --------------------------------------------------------------- sparse helpers

def spgemm(rowA, colA, valA, rowB, colB, valB, M, N):
    """CSR x CSR (parity unpinned).  Returns (rowC, colC, valC, products)."""
    rowA, colA, rowB, colB = (np.ascontiguousarray(x, dtype=np.uint32)
                              for x in (rowA, colA, rowB, colB))
    valA, valB = _c(valA), _c(valB)
    # zero-length arrays still need a valid pointer for ndpointer
    pad_u = lambda x: x if x.size else np.zeros(1, np.uint32)
    pad_f = lambda x: x if x.size else np.zeros(1, np.float32)
    rowC = np.zeros(M + 1, dtype=np.uint32)
    prods = C.c_long(0)
    nnz = port().orc_spgemm_symbolic(M, N, rowA, pad_u(colA), rowB, pad_u(colB), rowC,
                                     C.byref(prods))
    if nnz < 0:
        raise MemoryError("oracle spgemm symbolic")
    colC = np.zeros(max(nnz, 1), dtype=np.uint32)
    valC = np.zeros(max(nnz, 1), dtype=np.float32)
    rc = port().orc_spgemm_numeric(M, N, rowA, pad_u(colA), pad_f(valA), rowB, pad_u(colB),
                                   pad_f(valB), rowC, colC, valC)
    if rc != 0:
        raise RuntimeError(f"oracle spgemm numeric failed: {rc}")
    return rowC, colC[:nnz], valC[:nnz], prods.value


# ------------------------------------------------------------------- MLP step

class MlpOracle:
    """One SGD step of Linear->ReLU->Linear->ReLU->Linear->SoftMax->CrossEntropy,
    restated call by call from the reference's units:

    forward   Sources/Sapphire/operations/Forward/Linear.cpp:134-136 (bias rank-1 Gemm,
              then y += x.W with W stored [in, out]); NaiveBasic.cpp:159-165 (ReLU),
              :235-255 (SoftMax); NaiveCrossEntropy.cpp:15-31
    backward  NaiveCrossEntropy.cpp:33-51 (dx -= label/x), NaiveBasic.cpp:257-281,
              :167-174; Sources/Sapphire/operations/Backward/LinearBackward.cpp:27-99
              (dx with the pre-update W, dW unscaled, dB scaled by 1/batch,
              optimizer inside backward)
    SGD       Sources/Sapphire/operations/optimizers/SGD.cpp:22-28 (temp = lr*dz; z = z - temp)
    """

    def __init__(self, weights, biases, lr: float, impl: str = "port"):
        self.W = [_c(w).copy() for w in weights]
        self.b = [_c(b).copy() for b in biases]
        self.lr = np.float32(lr)
        self.impl = impl
        # per layer: sum over the steps of lr * mean_i |dy[i, :]|, the distance a bias
        # would have travelled had its per-sample gradients not cancelled (float64);
        # the scale against which a bias error is a relative error of the gradients
        self.bias_travel = [np.zeros(b.size, np.float64) for b in biases]

    # leaf dispatch: identical results either way; `ref` proves it
    def _gemm_acc(self, y, a, b):
        M, K = a.shape
        N = b.shape[1]
        fn = port().orc_gemm if self.impl == "port" else ref().ref_gemm
        fn(y.size, y.reshape(-1), _c(a).reshape(-1), _c(b).reshape(-1), M, N, K)

    def _leaves(self):
        """Elementwise leaves by name; with impl="ref" they are the reference's own."""
        if self.impl == "port":
            p = port()
            return dict(scale=p.orc_scale, sub=p.orc_sub, relu=p.orc_relu,
                        relu_bwd=p.orc_relu_backward, softmax=p.orc_softmax,
                        softmax_bwd=p.orc_softmax_backward, ce=p.orc_cross_entropy,
                        ce_bwd=p.orc_cross_entropy_backward)
        r = ref()
        return dict(scale=r.ref_scale,
                    sub=lambda out, a, b, n: r.ref_sub(n, out, a, b, 0, 0, 0),
                    relu=r.ref_relu, relu_bwd=r.ref_relu_backward, softmax=r.ref_softmax,
                    softmax_bwd=r.ref_softmax_backward, ce=r.ref_cross_entropy,
                    ce_bwd=r.ref_cross_entropy_backward)

    def _sgd(self, z, dz):
        f = self._leaves()
        tmp = np.empty_like(dz)
        f["scale"](tmp.reshape(-1), dz.reshape(-1), self.lr, dz.size)
        out = np.empty_like(z)
        f["sub"](out.reshape(-1), z.reshape(-1), tmp.reshape(-1), z.size)
        z[...] = out

    def linear_backward(self, l, xin, dy):
        """Layer l's backward unit (LinearBackward.cpp:27-99): returns dx = dy.W^T with the
        pre-update weight, then updates W by SGD with dW = x^T.dy (unscaled) and the bias
        with dB = (1/B) ones.dy."""
        f = self._leaves()
        B = xin.shape[0]
        dx = np.zeros_like(xin)
        self._gemm_acc(dx, dy, transpose(self.W[l], self.impl))
        dw = np.zeros_like(self.W[l])
        self._gemm_acc(dw, transpose(xin, self.impl), dy)
        self._sgd(self.W[l], dw)
        db = np.zeros((1, self.b[l].size), dtype=np.float32)
        self._gemm_acc(db, np.ones((1, B), np.float32), dy)
        dbs = np.empty_like(db)
        f["scale"](dbs.reshape(-1), db.reshape(-1), np.float32(1.0 / B), db.size)
        bl = self.b[l].reshape(1, -1)
        self.bias_travel[l] += float(self.lr) * np.abs(dy.astype(np.float64)).sum(0) / B
        self._sgd(bl, dbs)
        self.b[l] = bl.reshape(-1)
        return dx

    def step(self, x, onehot):
        f = self._leaves()
        B = x.shape[0]
        acts = [_c(x)]
        pre = []
        nl = len(self.W)
        for l in range(nl):
            y = np.zeros((B, self.W[l].shape[1]), dtype=np.float32)
            self._gemm_acc(y, np.ones((B, 1), np.float32), self.b[l].reshape(1, -1))
            self._gemm_acc(y, acts[-1], self.W[l])
            pre.append(y)
            if l < nl - 1:
                h = np.empty_like(y)
                f["relu"](h.reshape(-1), y.reshape(-1), y.size)
                acts.append(h)
        logits = pre[-1]
        unit = logits.shape[1]
        prob = np.empty_like(logits)
        f["softmax"](prob.reshape(-1), logits.reshape(-1), logits.size, unit)
        loss = np.zeros(B, dtype=np.float32)
        onehot = _c(onehot)
        f["ce"](loss, prob.reshape(-1), onehot.reshape(-1), B, unit)
        # backward
        dprob = np.zeros_like(prob)
        f["ce_bwd"](dprob.reshape(-1), prob.reshape(-1), onehot.reshape(-1), B, unit)
        dy = np.zeros_like(logits)
        f["softmax_bwd"](dy.reshape(-1), dprob.reshape(-1), prob.reshape(-1), prob.size, unit)
        for l in reversed(range(nl)):
            dx = self.linear_backward(l, acts[l], dy)
            if l > 0:
                dpre = np.zeros_like(pre[l - 1])
                f["relu_bwd"](dpre.reshape(-1), dx.reshape(-1), pre[l - 1].reshape(-1), dx.size)
                dy = dpre
        return loss

    def gradients(self, x, onehot):
        """(loss, dWs, dBs) of one batch without touching the parameters: step()
        with the SGD calls intercepted (dB carries the 1/batch scale).  The
        backward pass visits the layers last to first and hands first the weight
        gradient, then the bias gradient, of each layer to the optimizer."""
        n = len(self.W)
        saved = ([w.copy() for w in self.W], [b.copy() for b in self.b])
        dWs, dBs, calls = [None] * n, [None] * n, [0]

        def capture(z, dz):
            layer = n - 1 - calls[0] // 2
            if calls[0] % 2 == 0:
                dWs[layer] = dz.copy()
            else:
                dBs[layer] = dz.reshape(-1).copy()
            calls[0] += 1

        orig = self._sgd
        self._sgd = capture
        try:
            loss = self.step(x, onehot)
        finally:
            self._sgd = orig
            self.W, self.b = saved
        return loss, dWs, dBs
