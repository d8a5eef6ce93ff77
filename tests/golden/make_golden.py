"""Generates the golden fixtures of tests/golden from the REFERENCE's own CPU
code (oracle/_ref/libsapphire_ref.so and libsapphire_ref_ops.so, compiled from the
reference tree by oracle/Makefile).  Run where the reference tree is mounted:

    make -C oracle && python tests/golden/make_golden.py

Inputs are not stored: they are regenerated from seeds by
sapphire_b200.workloads / the small generators below.  Outputs are stored in
full for small cases and as a strided sample plus a float64 checksum for the
4 x 256^3 case.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as O  # noqa: E402
from sapphire_b200 import workloads as W  # noqa: E402

# (batch, M, N, K): the reference's Gemm1 test family draws M, N, K from [1, 100]
# (Tests/UnitTests/Sources/FunctionTest/GemmTest.cpp:20-84)
SMALL_SHAPES = [(1, 1, 1, 1), (2, 3, 5, 7), (3, 17, 9, 33), (1, 64, 10, 256), (2, 100, 99, 98),
                (4, 32, 32, 32), (1, 128, 128, 128), (1, 130, 70, 40)]


def small_case(idx):
    b, M, N, K = SMALL_SHAPES[idx]
    rng = np.random.default_rng(100 + idx)
    a = rng.normal(10.0, 5.0, size=(b, M, K)).astype(np.float32)   # N(10,5) as in Gemm1
    bm = rng.normal(10.0, 5.0, size=(b, K, N)).astype(np.float32)
    c = rng.uniform(-1, 1, size=(b, M, N)).astype(np.float32)
    return a, bm, c


# N, C, H, W, Cout, kh, kw, stride, pad, dil: the geometries of the convolution tests
CONV_CASES = [
    (2, 3, 8, 9, 4, 3, 3, (1, 1), (1, 1), (1, 1)),
    (1, 2, 11, 7, 5, 3, 2, (2, 1), (0, 1), (1, 2)),
    (3, 1, 6, 6, 2, 1, 1, (1, 1), (0, 0), (1, 1)),
    (2, 4, 10, 10, 3, 5, 5, (2, 2), (2, 2), (1, 1)),
    (1, 2, 9, 12, 2, 2, 3, (3, 2), (1, 0), (2, 1)),
]


def conv_case(idx):
    """Seeded inputs of convolution case idx: x, filter, y0 (accumulated into), dy, dx0, dfilter0."""
    N, Cc, H, Wd, Cout, kh, kw, stride, pad, dil = CONV_CASES[idx]
    rng = np.random.default_rng(500 + idx)
    oR, oC = O.conv_out(H, pad[0], dil[0], kh, stride[0]), O.conv_out(Wd, pad[1], dil[1], kw, stride[1])
    x = rng.standard_normal((N, Cc, H, Wd)).astype(np.float32)
    f = rng.standard_normal((Cout, Cc, kh, kw)).astype(np.float32)
    y0 = rng.standard_normal((N, Cout, oR, oC)).astype(np.float32)
    dy = rng.standard_normal((N, Cout, oR, oC)).astype(np.float32)
    dx0 = rng.standard_normal(x.shape).astype(np.float32)
    df0 = rng.standard_normal(f.shape).astype(np.float32)
    return x, f, y0, dy, dx0, df0


def conv_outputs(idx, impl):
    """im2col(x), col2im(dx0, dy-shaped columns), Conv2D and Conv2DBackward of case idx."""
    _, _, _, _, _, kh, kw, stride, pad, dil = CONV_CASES[idx]
    x, f, y0, dy, dx0, df0 = conv_case(idx)
    cols = O.im2col(x, kh, kw, stride, pad, dil, pad_value=0.5, impl=impl)
    back = O.col2im(dx0.copy(), np.cos(cols), kh, kw, stride, pad, dil, impl=impl)
    y = O.conv2d(y0, x, f, stride, pad, dil, impl=impl)
    dx, df = O.conv2d_backward(dx0, df0, dy, x, f, stride, pad, dil, impl=impl)
    return {"cols": cols, "col2im": back, "y": y, "dx": dx, "df": df}


# (y, a, b) shapes for Compute::Gemm's batch / broadcast rules: the families of the reference's
# broadcast tests (Tests/UnitTests/Sources/FunctionTest/BroadcastTest.cpp:20-202) and a few more
BROADCAST_CASES = [
    ([4, 6, 5], [4, 6, 3], [4, 3, 5]),                   # equal batch: one call
    ([3, 4, 4, 5], [3, 1, 4, 2], [3, 4, 2, 5]),          # [b,1,M,K].[b,M,K,N]: not numpy's pairing
    ([4, 4, 5], [4, 2], [4, 2, 5]),                      # [M,K].[M,K,N]: missing dimension
    ([5, 4, 4, 5], [4, 2], [5, 4, 2, 5]),                # [M,K].[N,M,K,N]
    ([6, 5], [6, 3], [3, 5]),                            # plain 2-D
    ([2, 3, 6, 5], [2, 3, 6, 3], [1, 1, 3, 5]),          # shared B
    ([2, 3, 6, 5], [1, 3, 6, 3], [2, 1, 3, 5]),          # each operand shared along another dimension
    ([7, 1, 5], [7, 1, 9], [9, 5]),                      # a row vector per batch
    ([3, 4, 4, 8], [3, 1, 4, 12], [3, 4, 12, 8]),        # the three shapes of the GPU test
    ([4, 4, 8], [4, 12], [4, 12, 8]),
    ([5, 4, 4, 8], [4, 12], [5, 4, 12, 8]),
]


def broadcast_case(idx):
    ys, as_, bs = BROADCAST_CASES[idx]
    rng = np.random.default_rng(700 + idx)
    return (rng.standard_normal(ys).astype(np.float32), rng.standard_normal(as_).astype(np.float32),
            rng.standard_normal(bs).astype(np.float32))


# (batch, in, out) of the Linear backward unit fixtures
LINEAR_CASES = [(7, 13, 5), (1, 3, 4), (16, 40, 24), (64, 256, 10)]


def linear_case(idx):
    B, n_in, n_out = LINEAR_CASES[idx]
    rng = np.random.default_rng(900 + idx)
    x = rng.uniform(0, 1, (B, n_in)).astype(np.float32)
    dy = rng.standard_normal((B, n_out)).astype(np.float32)
    w = rng.standard_normal((n_in, n_out)).astype(np.float32)
    b = rng.standard_normal(n_out).astype(np.float32)
    return x, dy, w, b


# (batch, M, K, N) of the MatMul backward unit fixtures
MATMUL_CASES = [(1, 5, 7, 3), (3, 16, 12, 20), (2, 33, 8, 40)]


def matmul_case(idx):
    """da0, db0, dy, a, b of MatMul backward case idx."""
    batch, M, K, N = MATMUL_CASES[idx]
    rng = np.random.default_rng(1100 + idx)
    a = rng.standard_normal((batch, M, K)).astype(np.float32)
    b = rng.standard_normal((batch, K, N)).astype(np.float32)
    dy = rng.standard_normal((batch, M, N)).astype(np.float32)
    da0 = rng.standard_normal((batch, M, K)).astype(np.float32)
    db0 = rng.standard_normal((batch, K, N)).astype(np.float32)
    return da0, db0, dy, a, b


def mlp_reference(steps, impl):
    Ws, bs = W.mlp_init(0)
    net = O.MlpOracle(Ws, bs, 0.01, impl=impl)
    losses = []
    for t in range(steps):
        x, onehot = W.mlp_batch(t)
        losses.append(net.step(x, onehot))
    return np.stack(losses), net


def main():
    assert O.have_ref(), "build oracle/_ref first (make -C oracle)"
    out = {}
    for i in range(len(SMALL_SHAPES)):
        a, b, c = small_case(i)
        out[f"small{i}"] = O.gemm(c, a, b, impl="ref")
    a, b, c = W.dense_batched(0, range(4), 256, 256, 256, "uniform")
    y = O.gemm(c, a, b, impl="ref")
    out["c1_sample"] = y.reshape(-1)[::16].copy()
    out["c1_sum64"] = np.array([y.astype(np.float64).sum()])
    # transpose leaf
    rng = np.random.default_rng(7)
    t_in = rng.uniform(-1, 1, size=(3, 5, 8)).astype(np.float32)
    out["transpose"] = O.transpose(t_in, impl="ref")
    # 3 MLP steps through the reference leaves (Gemm via ref; elementwise leaves via ref below)
    losses, net = mlp_reference(3, "ref")
    out["mlp_loss3"] = losses
    out["mlp_w2_after3"] = net.W[2]
    out["mlp_b0_after3"] = net.b[0]
    np.savez_compressed(os.path.join(HERE, "dense_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "dense_golden.npz"),
          {k: v.shape for k, v in out.items()})
    # the reference's own host convolution (Convolution.cpp:15-316)
    assert O.have_ref_ops(), "build oracle/_ref first (make -C oracle)"
    conv = {}
    for i in range(len(CONV_CASES)):
        for k, v in conv_outputs(i, "ref").items():
            conv[f"case{i}_{k}"] = v
    np.savez_compressed(os.path.join(HERE, "conv_golden.npz"), **conv)
    print("wrote", os.path.join(HERE, "conv_golden.npz"), {k: v.shape for k, v in conv.items()})
    # Compute::Gemm's batch / broadcast rules (BasicOps.cpp:183-248 over the reference's
    # BroadcastWith2Inputs and CPU GEMM)
    bc = {f"case{i}": O.ref_compute_gemm(*broadcast_case(i)) for i in range(len(BROADCAST_CASES))}
    # LinearBackProp with SGD inside (LinearBackward.cpp:27-99, SGD.cpp:22-28)
    for i in range(len(LINEAR_CASES)):
        x, dy, w, b = linear_case(i)
        dx, w1, b1 = O.ref_linear_backprop(np.zeros_like(x), dy, w, b, x, 0.01)
        bc[f"linear{i}_dx"], bc[f"linear{i}_w"], bc[f"linear{i}_b"] = dx, w1, b1
    # MulBackProp (MathBackward.cpp:13-51)
    for i in range(len(MATMUL_CASES)):
        da, db = O.matmul_backward(*matmul_case(i), impl="ref")
        bc[f"matmul{i}_da"], bc[f"matmul{i}_db"] = da, db
    np.savez_compressed(os.path.join(HERE, "compute_units_golden.npz"), **bc)
    print("wrote", os.path.join(HERE, "compute_units_golden.npz"), {k: v.shape for k, v in bc.items()})


if __name__ == "__main__":
    main()
