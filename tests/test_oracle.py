"""CPU tests: the oracle restatement against the golden fixtures made from the
reference's own CPU code, and against that code itself where its build is
present (oracle/_ref)."""
import os

import numpy as np
import pytest

from sapphire_b200 import workloads as W

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "dense_golden.npz"))


def _bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)


def _small_case(idx):
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.small_case(idx), mod.SMALL_SHAPES


@pytest.mark.parametrize("idx", range(8))
def test_port_matches_golden_small(oracle, idx):
    (a, b, c), _ = _small_case(idx)
    y = oracle.gemm(c, a, b, impl="port")
    assert np.array_equal(_bits(y), _bits(GOLD[f"small{idx}"]))     # bit-exact


def test_port_matches_golden_c1(oracle):
    a, b, c = W.dense_batched(0, range(4), 256, 256, 256, "uniform")
    y = oracle.gemm(c, a, b, impl="port")
    assert np.array_equal(_bits(y.reshape(-1)[::16]), _bits(GOLD["c1_sample"]))
    assert y.astype(np.float64).sum() == GOLD["c1_sum64"][0]


def test_port_transpose_matches_golden(oracle):
    rng = np.random.default_rng(7)
    t_in = rng.uniform(-1, 1, size=(3, 5, 8)).astype(np.float32)
    assert np.array_equal(oracle.transpose(t_in), GOLD["transpose"])


def test_port_mlp_matches_golden(oracle):
    Ws, bs = W.mlp_init(0)
    net = oracle.MlpOracle(Ws, bs, 0.01, impl="port")
    losses = np.stack([net.step(*W.mlp_batch(t)) for t in range(3)])
    assert np.array_equal(_bits(losses), _bits(GOLD["mlp_loss3"]))
    assert np.array_equal(_bits(net.W[2]), _bits(GOLD["mlp_w2_after3"]))
    assert np.array_equal(_bits(net.b[0]), _bits(GOLD["mlp_b0_after3"]))


def test_port_equals_reference_build(oracle):
    """Where the reference's CPU files were compiled (oracle/_ref), the
    restatement must agree with them bit for bit on fresh seeded inputs."""
    if not oracle.have_ref():
        pytest.skip("oracle/_ref not built on this machine")
    rng = np.random.default_rng(42)
    for (b, M, N, K) in [(1, 1, 1, 1), (2, 7, 13, 29), (1, 96, 100, 64), (3, 33, 2, 150)]:
        a = rng.standard_normal((b, M, K)).astype(np.float32)
        bm = rng.standard_normal((b, K, N)).astype(np.float32)
        c = rng.standard_normal((b, M, N)).astype(np.float32)
        assert np.array_equal(_bits(oracle.gemm(c, a, bm, "port")), _bits(oracle.gemm(c, a, bm, "ref")))
    x = rng.standard_normal((2, 9, 4)).astype(np.float32)
    assert np.array_equal(oracle.transpose(x, "port"), oracle.transpose(x, "ref"))


def test_gemm_ex_restates_transpose_then_gemm(oracle):
    """The strided/transposed form equals what the reference does: explicit
    Transpose into a temporary, then the plain Gemm (LinearBackward.cpp:49-50,70-72)."""
    rng = np.random.default_rng(3)
    M, N, K = 19, 23, 31
    at = rng.standard_normal((K, M)).astype(np.float32)      # stored transposed
    bt = rng.standard_normal((N, K)).astype(np.float32)
    c = rng.standard_normal((M, N)).astype(np.float32)
    want = oracle.gemm(c[None], oracle.transpose(at)[None], oracle.transpose(bt)[None])[0]
    got = oracle.gemm_ex(1, 1, M, N, K, at, M, 0, bt, K, 0, c, N, 0, N, 0, None, 1, M * N)
    assert np.array_equal(_bits(got.reshape(M, N)), _bits(want))


def test_gemm_ex_bias_is_rank1_gemm_first(oracle):
    """bias: y starts at zero, y += ones.bias, y += x.W (Linear.cpp:134-136)."""
    rng = np.random.default_rng(4)
    B, I, Oo = 8, 12, 5
    x = rng.standard_normal((B, I)).astype(np.float32)
    w = rng.standard_normal((I, Oo)).astype(np.float32)
    bias = rng.standard_normal(Oo).astype(np.float32)
    y = np.zeros((1, B, Oo), np.float32)
    y = oracle.gemm(y, np.ones((1, B, 1), np.float32), bias.reshape(1, 1, Oo))
    y = oracle.gemm(y, x[None], w[None])[0]
    got = oracle.gemm_ex(0, 0, B, Oo, I, x, I, 0, w, Oo, 0, None, Oo, 0, Oo, 0, bias, 1, B * Oo)
    assert np.array_equal(_bits(got.reshape(B, Oo)), _bits(y))


def test_colsum_is_ones_gemm_then_scale(oracle):
    rng = np.random.default_rng(5)
    dy = rng.standard_normal((37, 11)).astype(np.float32)
    db = oracle.gemm(np.zeros((1, 1, 11), np.float32), np.ones((1, 1, 37), np.float32), dy[None])[0]
    want = (db * np.float32(1.0 / 37)).reshape(-1)
    assert np.array_equal(_bits(oracle.colsum(dy, 1.0 / 37)), _bits(want))


# ------------------------------------------------------------------ sparse

def _scipy_product(rA, cA, vA, rB, cB, vB, M, K, N):
    import scipy.sparse as sp
    A = sp.csr_matrix((vA.astype(np.float64), cA.astype(np.int64), rA.astype(np.int64)), shape=(M, K))
    B = sp.csr_matrix((vB.astype(np.float64), cB.astype(np.int64), rB.astype(np.int64)), shape=(K, N))
    C = A @ B
    C.sort_indices()
    return C


@pytest.mark.parametrize("M,N,dens,dist", [(64, 64, 0.05, "poisson"), (512, 700, 0.01, "poisson"),
                                           (300, 300, None, "zipf"), (5, 9, 0.0, "poisson")])
def test_spgemm_oracle_against_scipy(oracle, M, N, dens, dist):
    """The sparse restatement is unpinned by the reference (it ships no sparse
    GEMM); this checks it against an independent implementation."""
    rA, cA, vA = W.csr_random(0, M, N, dens, dist, zipf_cap=64)
    rB, cB, vB = W.csr_random(1, N, N, dens, dist, zipf_cap=64)
    rc, cc, vc, prods = oracle.spgemm(rA, cA, vA, rB, cB, vB, M, N)
    assert prods == int(W.csr_products(rA, cA, rB).sum())
    C = _scipy_product(rA, cA, vA, rB, cB, vB, M, N, N)
    # scipy drops nothing either: structural pattern
    assert np.array_equal(rc, C.indptr.astype(np.uint32))
    assert np.array_equal(cc, C.indices.astype(np.uint32))
    assert np.allclose(vc, C.data, rtol=1e-5, atol=1e-6)
    for i in range(M):                                 # ascending columns
        seg = cc[rc[i]:rc[i + 1]].astype(np.int64)
        assert np.all(np.diff(seg) > 0)


def test_csr_generators():
    r, c, v = W.csr_random(0, 1000, 1000, 0.01)
    assert r[0] == 0 and r[-1] == c.size == v.size
    for i in range(0, 1000, 37):
        seg = c[r[i]:r[i + 1]].astype(np.int64)
        assert np.all(np.diff(seg) > 0) and (seg < 1000).all()
    r2, c2, _ = W.csr_random(0, 1000, 1000, 0.01)
    assert np.array_equal(c, c2) and np.array_equal(r, r2)          # seeded
    rz, cz, _ = W.csr_random(2, 2000, 4096, row_dist="zipf", zipf_cap=512)
    d = np.diff(rz.astype(np.int64))
    assert d.min() >= 1 and d.max() <= 512


CONV_CASES = [
    # N, C, H, W, Cout, kh, kw, stride, pad, dil
    (2, 3, 8, 9, 4, 3, 3, (1, 1), (1, 1), (1, 1)),
    (1, 2, 11, 7, 5, 3, 2, (2, 1), (0, 1), (1, 2)),
    (3, 1, 6, 6, 2, 1, 1, (1, 1), (0, 0), (1, 1)),
    (2, 4, 10, 10, 3, 5, 5, (2, 2), (2, 2), (1, 1)),
    (1, 2, 9, 12, 2, 2, 3, (3, 2), (1, 0), (2, 1)),
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_lowering_is_a_true_convolution(oracle, case):
    """The restated Im2Col + Gemm and Conv2DBackward (im2col, two Gemms, Col2Im)
    against an independent formulation: torch's cross-correlation with the kernel
    flipped in both spatial axes (a true convolution, the mode the reference asks
    of cuDNN), and its autograd gradients.  fp32 with different summation orders:
    1e-5 relative."""
    import torch
    import torch.nn.functional as F
    N, Cc, H, Wd, Cout, kh, kw, stride, pad, dil = case
    rng = np.random.default_rng(sum(case[:7]))
    x = rng.standard_normal((N, Cc, H, Wd)).astype(np.float32)
    f = rng.standard_normal((Cout, Cc, kh, kw)).astype(np.float32)
    outR = oracle.conv_out(H, pad[0], dil[0], kh, stride[0])
    outC = oracle.conv_out(Wd, pad[1], dil[1], kw, stride[1])
    y0 = rng.standard_normal((N, Cout, outR, outC)).astype(np.float32)
    got = oracle.conv2d(y0, x, f, stride, pad, dil)
    xt = torch.from_numpy(x).requires_grad_(True)
    ft = torch.from_numpy(f).requires_grad_(True)
    want = F.conv2d(xt, ft.flip(2, 3), stride=stride, padding=pad, dilation=dil)
    assert np.abs(got - (y0 + want.detach().numpy())).max() <= 1e-5 * max(1.0, np.abs(got).max())
    dy = rng.standard_normal(want.shape).astype(np.float32)
    want.backward(torch.from_numpy(dy))
    dx0 = rng.standard_normal(x.shape).astype(np.float32)
    df0 = rng.standard_normal(f.shape).astype(np.float32)
    dx, df = oracle.conv2d_backward(dx0, df0, dy, x, f, stride, pad, dil)
    assert np.abs(dx - (dx0 + xt.grad.numpy())).max() <= 1e-5 * max(1.0, np.abs(dx).max())
    assert np.abs(df - (df0 + ft.grad.numpy())).max() <= 2e-5 * max(1.0, np.abs(df).max())


def _golden_module():
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("idx", range(5))
def test_conv_port_matches_golden_from_the_reference(oracle, idx):
    """The restated lowering and composition against fixtures written by the reference's
    own Im2Col, Col2Im, Conv2D and Conv2DBackward
    (Sources/Sapphire/compute/dense/naive/Convolution.cpp:15-316, compiled unmodified):
    every element bit for bit, asymmetric strides, paddings and dilations included."""
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "conv_golden.npz"))
    got = _golden_module().conv_outputs(idx, "port")
    for k, v in got.items():
        assert np.array_equal(_bits(v), _bits(gold[f"case{idx}_{k}"])), k


def test_conv_port_equals_reference_build(oracle):
    """Where the reference build is present: the same comparison live, plus a case of the
    benchmark's geometry class (3 x 3 taps, padding 1) too large for a fixture."""
    if not oracle.have_ref_ops():
        pytest.skip("oracle/_ref/libsapphire_ref_ops.so not built (reference tree absent)")
    mod = _golden_module()
    for idx in range(len(mod.CONV_CASES)):
        ref, port = mod.conv_outputs(idx, "ref"), mod.conv_outputs(idx, "port")
        for k in ref:
            assert np.array_equal(_bits(ref[k]), _bits(port[k])), (idx, k)
    rng = np.random.default_rng(9)
    x = rng.standard_normal((2, 16, 32, 32)).astype(np.float32)
    f = rng.standard_normal((32, 16, 3, 3)).astype(np.float32)
    y0 = rng.standard_normal((2, 32, 32, 32)).astype(np.float32)
    args = ((1, 1), (1, 1), (1, 1))
    assert np.array_equal(_bits(oracle.conv2d(y0, x, f, *args)), _bits(oracle.conv2d(y0, x, f, *args, impl="ref")))
    dy = rng.standard_normal(y0.shape).astype(np.float32)
    dx0, df0 = np.zeros_like(x), np.zeros_like(f)
    a = oracle.conv2d_backward(dx0, df0, dy, x, f, *args)
    b = oracle.conv2d_backward(dx0, df0, dy, x, f, *args, impl="ref")
    assert np.array_equal(_bits(a[0]), _bits(b[0])) and np.array_equal(_bits(a[1]), _bits(b[1]))


@pytest.mark.parametrize("idx", range(4))
def test_linear_backward_unit_matches_the_reference(oracle, idx):
    """The MLP oracle's layer backward + SGD against the reference's own LinearBackProp
    unit with its optimizer (Sources/Sapphire/operations/Backward/LinearBackward.cpp:27-99,
    Sources/Sapphire/operations/optimizers/SGD.cpp:22-28, compiled unmodified): dx with the
    pre-update weight, dW unscaled, dB scaled by 1/batch, z -= lr dz -- bit for bit
    against fixtures written by the reference build, and live where it is present."""
    mod = _golden_module()
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "compute_units_golden.npz"))
    x, dy, w, b = mod.linear_case(idx)
    net = oracle.MlpOracle([w], [b], 0.01)
    dx = net.linear_backward(0, x, dy)
    assert np.array_equal(_bits(dx), _bits(gold[f"linear{idx}_dx"]))
    assert np.array_equal(_bits(net.W[0]), _bits(gold[f"linear{idx}_w"]))
    assert np.array_equal(_bits(net.b[0]), _bits(gold[f"linear{idx}_b"]))
    if oracle.have_ref_ops():
        rdx, rw, rb = oracle.ref_linear_backprop(np.zeros_like(x), dy, w, b, x, 0.01)
        assert np.array_equal(_bits(dx), _bits(rdx)) and np.array_equal(_bits(net.W[0]), _bits(rw))
        assert np.array_equal(_bits(net.b[0]), _bits(rb))


@pytest.mark.parametrize("idx", range(3))
def test_matmul_backward_unit_matches_the_reference(oracle, idx):
    """da += dy.b^T and db += a^T.dy as the GPU tests state them (transposed operand,
    accumulate in place) against the reference's own MulBackProp
    (Sources/Sapphire/operations/Backward/MathBackward.cpp:13-51, compiled unmodified):
    bit for bit against fixtures written by the reference build, and live where it is
    present."""
    mod = _golden_module()
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "compute_units_golden.npz"))
    args = mod.matmul_case(idx)
    da, db = oracle.matmul_backward(*args)
    assert np.array_equal(_bits(da), _bits(gold[f"matmul{idx}_da"]))
    assert np.array_equal(_bits(db), _bits(gold[f"matmul{idx}_db"]))
    if oracle.have_ref_ops():
        rda, rdb = oracle.matmul_backward(*args, impl="ref")
        assert np.array_equal(_bits(da), _bits(rda)) and np.array_equal(_bits(db), _bits(rdb))


def test_im2col_tap_order_and_padding(oracle):
    """Row c*kh*kw + (kh*kw - 1 - tap) holds tap (fr, fc); outside pixels read the pad value."""
    x = np.arange(1, 1 + 2 * 3 * 3, dtype=np.float32).reshape(1, 2, 3, 3)
    cols = oracle.im2col(x, 2, 2, (1, 1), (1, 1), (1, 1), pad_value=-7.0)
    assert cols.shape == (1, 8, 16)
    # output pixel (0, 0): tap (1, 1) reads x[0, 0, 0, 0], the other three are padding
    assert cols[0, 0, 0] == x[0, 0, 0, 0] and (cols[0, 1:4, 0] == -7.0).all()
    # output pixel (1, 1): taps (0,0),(0,1),(1,0),(1,1) read x[..,0,0],[0,1],[1,0],[1,1], stored in reverse
    assert list(cols[0, 0:4, 5]) == [x[0, 0, 1, 1], x[0, 0, 1, 0], x[0, 0, 0, 1], x[0, 0, 0, 0]]
    assert list(cols[0, 4:8, 5]) == [x[0, 1, 1, 1], x[0, 1, 1, 0], x[0, 1, 0, 1], x[0, 1, 0, 0]]
