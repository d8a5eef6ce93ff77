"""GPU parity tests of the dense path, through the C ABI, against the CPU
oracle (bit-exact restatement of Sapphire's CPU loop) on the same seeded inputs.

Tolerances (relative Frobenius error against Sapphire's own CPU result):
    TF32 mode    <= 2e-3
    TF32X3 mode  <= 1e-5
    SIMT path    bit-exact
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from sapphire_b200 import _lib as L
from sapphire_b200 import ops
from sapphire_b200 import workloads as W

pytestmark = pytest.mark.gpu

TOL = {L.MODE_TF32: 2e-3, L.MODE_TF32X3: 1e-5}
DEV = "cuda:0"
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "dense_golden.npz"))


def rel_fro(got, want):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def bits(x):
    return np.ascontiguousarray(x, np.float32).view(np.uint32)


# ------------------------------------------------------------------ config 1
@pytest.mark.parametrize("mode", [L.MODE_TF32, L.MODE_TF32X3])
@pytest.mark.parametrize("pad", [0, 8])
def test_config1_4x256(ctx, oracle, mode, pad):
    """batch 4, M=N=K=256, U[-1,1) seed 0, y <- c + a.b, every element compared;
    ld = cols (Sapphire's layout) and ld = cols + 8 (padded rows)."""
    a, b, c = W.dense_batched(0, range(4), 256, 256, 256, "uniform")
    want = oracle.gemm(c, a, b)
    ld = 256 + pad
    ta = torch.zeros(4, 256, ld, device=DEV); ta[:, :, :256] = dev(a)
    tb = torch.zeros(4, 256, ld, device=DEV); tb[:, :, :256] = dev(b)
    ty = torch.zeros(4, 256, ld, device=DEV); ty[:, :, :256] = dev(c)
    y = ty[:, :, :256]
    ops.gemm(ctx, ta[:, :, :256], tb[:, :, :256], y, y, mode=mode)       # in place: C aliases D
    ctx.check_device_status()
    assert ctx.last_path() == L.PATH_TCGEN05
    assert rel_fro(y.cpu().numpy(), want) <= TOL[mode]
    if pad:
        assert float(ty[:, :, 256:].abs().max()) == 0.0                  # padding untouched


def test_config1_matches_reference_fixture(ctx):
    """Against the fixture written by the reference's own CPU build."""
    a, b, c = W.dense_batched(0, range(4), 256, 256, 256, "uniform")
    y = ops.gemm(ctx, dev(a), dev(b), dev(c), mode=L.MODE_TF32X3).cpu().numpy()
    assert rel_fro(y.reshape(-1)[::16], GOLD["c1_sample"]) <= 1e-5
    assert abs(y.astype(np.float64).sum() - GOLD["c1_sum64"][0]) <= 1e-5 * np.abs(y).sum()


# ------------------------------------------------------------ SIMT: bit-exact
@pytest.mark.parametrize("idx", range(8))
def test_simt_bit_exact_small_shapes(ctx, idx):
    """The reference's Gemm1 family (M, N, K in [1,100], N(10,5) inputs,
    GemmTest.cpp:20-84): the CUDA-core kernel reproduces the CPU loop bit for bit."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    a, b, c = mod.small_case(idx)
    y = ops.gemm(ctx, dev(a), dev(b), dev(c), path=L.PATH_SIMT).cpu().numpy()
    assert ctx.last_path() == L.PATH_SIMT
    assert np.array_equal(bits(y), bits(GOLD[f"small{idx}"]))


def test_auto_path_falls_to_simt_for_tma_hostile_rows(ctx, oracle):
    """[64,256].[256,10]: a 40-byte row pitch breaks TMA's 16-byte rule."""
    rng = np.random.default_rng(1)
    a = rng.standard_normal((1, 64, 256)).astype(np.float32)
    b = rng.standard_normal((1, 256, 10)).astype(np.float32)
    c = np.zeros((1, 64, 10), np.float32)
    y = ops.gemm(ctx, dev(a), dev(b), dev(c)).cpu().numpy()
    assert ctx.last_path() == L.PATH_SIMT
    assert np.array_equal(bits(y), bits(oracle.gemm(c, a, b)))
    with pytest.raises(L.Sb200Error) as e:
        ops.gemm(ctx, dev(a), dev(b), dev(c), path=L.PATH_TCGEN05)
    assert e.value.status == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("M,N,K,batch,ta,tb", [
    (64, 10, 256, 1, 0, 0),        # 16 x 16 tiles (few CTAs even with 16-column tiles), k steps of 64
    (3200, 10, 100, 1, 0, 0),      # 64 x 16 tiles, 50 CTAs: k steps of 64
    (64, 256, 10, 1, 0, 1),        # the dx GEMM of the 10-class layer (B read transposed)
    (256, 10, 64, 1, 1, 0),        # its dW GEMM (A read transposed)
    (19200, 10, 40, 1, 0, 0),      # 16-column tiles, 300 CTAs: steps of 16
    (100, 100, 70, 3, 0, 0),       # 64-column tiles, few CTAs: steps of 64
    (1500, 1500, 24, 1, 1, 1),     # 64-column tiles, 576 CTAs: steps of 16
    (33, 32, 130, 2, 0, 0),        # 32 columns = two 16-column tiles
])
def test_simt_tile_variants_are_bit_exact(ctx, oracle, M, N, K, batch, ta, tb):
    """The CUDA-core kernel has five instances (tiles of 64 x 64, 64 x 16 or 16 x 16, k
    steps of 16 or 64); none changes the order of the additions, so each equals the
    CPU loop bit for bit."""
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    a = rng.standard_normal((batch, K, M) if ta else (batch, M, K)).astype(np.float32)
    b = rng.standard_normal((batch, N, K) if tb else (batch, K, N)).astype(np.float32)
    c = rng.uniform(-1, 1, (batch, M, N)).astype(np.float32)
    want = np.stack([oracle.gemm_ex(ta, tb, M, N, K, a[i], a.shape[2], 0, b[i], b.shape[2], 0, c[i], N, 0,
                                    N, 0, None, 1, M * N).reshape(M, N) for i in range(batch)])
    y = ops.gemm(ctx, dev(a), dev(b), dev(c), trans_a=bool(ta), trans_b=bool(tb), path=L.PATH_SIMT)
    assert ctx.last_path() == L.PATH_SIMT
    assert np.array_equal(bits(y.cpu().numpy()), bits(want))


def test_k_zero_and_empty(ctx):
    c = torch.randn(2, 5, 8, device=DEV)
    a = torch.empty(2, 5, 0, device=DEV)
    b = torch.empty(2, 0, 8, device=DEV)
    bias = torch.randn(8, device=DEV)
    y = ops.gemm(ctx, a, b, c, bias=bias)
    assert torch.equal(y, c + bias)
    # M == 0 is a no-op
    ops.gemm(ctx, torch.empty(0, 4, device=DEV), torch.empty(4, 8, device=DEV),
             out=torch.empty(0, 8, device=DEV))


# ------------------------------------------- layouts, tails, strides, epilogue
@pytest.mark.parametrize("mode", [L.MODE_TF32, L.MODE_TF32X3])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K,batch", [(128, 128, 32, 1), (200, 328, 100, 2), (1, 4, 4, 1),
                                         (130, 260, 36, 3), (384, 512, 1000, 1)])
def test_layouts_and_tails(ctx, oracle, mode, ta, tb, M, N, K, batch):
    rng = np.random.default_rng(M * 7 + N * 3 + K + ta * 2 + tb)
    a = rng.standard_normal((batch, K, M) if ta else (batch, M, K)).astype(np.float32)
    b = rng.standard_normal((batch, N, K) if tb else (batch, K, N)).astype(np.float32)
    c = rng.uniform(-1, 1, (batch, M, N)).astype(np.float32)
    want = oracle.gemm_ex(ta, tb, M, N, K, a, a.shape[2], a.shape[1] * a.shape[2],
                          b, b.shape[2], b.shape[1] * b.shape[2], c, N, M * N, N, M * N,
                          None, batch, batch * M * N).reshape(batch, M, N)
    tma_ok = a.shape[2] % 4 == 0 and b.shape[2] % 4 == 0
    y = ops.gemm(ctx, dev(a), dev(b), dev(c), mode=mode, trans_a=bool(ta), trans_b=bool(tb),
                 path=L.PATH_TCGEN05 if tma_ok else L.PATH_AUTO)
    ctx.check_device_status()
    assert ctx.last_path() == (L.PATH_TCGEN05 if tma_ok else L.PATH_SIMT)
    assert rel_fro(y.cpu().numpy(), want) <= TOL[mode]


def test_random_small_shapes_on_the_tensor_core_path(ctx, oracle):
    """The reference's Gemm1 family (M, N, K in [1, 100], batch up to 30, inputs
    N(10, 5), GemmTest.cpp:20-84) with rows padded to a multiple of 4 floats so
    that TMA can fetch them: 40 seeded random cases over all four operand
    orientations and both arithmetic modes, every output element compared."""
    rng = np.random.default_rng(2024)
    for case in range(40):
        M, N, K = (int(x) for x in rng.integers(1, 131, 3))
        batch = int(rng.integers(1, 6))
        ta, tb = int(rng.integers(0, 2)), int(rng.integers(0, 2))
        mode = L.MODE_TF32X3 if case % 2 else L.MODE_TF32
        pad4 = lambda n: (n + 3) // 4 * 4
        ar, ac = (K, M) if ta else (M, K)
        br, bc = (N, K) if tb else (K, N)
        a = rng.normal(10.0, 5.0, (batch, ar, ac)).astype(np.float32)
        b = rng.normal(10.0, 5.0, (batch, br, bc)).astype(np.float32)
        c = rng.uniform(-1, 1, (batch, M, N)).astype(np.float32)
        want = oracle.gemm_ex(ta, tb, M, N, K, a, ac, ar * ac, b, bc, br * bc, c, N, M * N, N, M * N,
                              None, batch, batch * M * N).reshape(batch, M, N)
        pa = torch.zeros(batch, ar, pad4(ac), device=DEV); pa[:, :, :ac] = dev(a)
        pb = torch.zeros(batch, br, pad4(bc), device=DEV); pb[:, :, :bc] = dev(b)
        py = torch.zeros(batch, M, pad4(N), device=DEV); py[:, :, :N] = dev(c)
        y = py[:, :, :N]
        ops.gemm(ctx, pa[:, :, :ac], pb[:, :, :bc], y, y, mode=mode, trans_a=bool(ta),
                 trans_b=bool(tb), path=L.PATH_TCGEN05)
        ctx.check_device_status()
        err = rel_fro(y.cpu().numpy(), want)
        assert err <= TOL[mode], (case, M, N, K, batch, ta, tb, mode, err)
        assert float(py[:, :, N:].abs().max()) == 0.0 if pad4(N) > N else True


def test_long_k_accumulation_tf32x3(ctx, oracle):
    """K = 4096: the split mode must stay fp32-accurate over a long reduction."""
    rng = np.random.default_rng(11)
    a = rng.standard_normal((1, 128, 4096)).astype(np.float32)
    b = rng.standard_normal((1, 4096, 256)).astype(np.float32)
    c = rng.uniform(-1, 1, (1, 128, 256)).astype(np.float32)
    want = oracle.gemm(c, a, b)
    y = ops.gemm(ctx, dev(a), dev(b), dev(c), mode=L.MODE_TF32X3).cpu().numpy()
    assert rel_fro(y, want) <= 1e-5
    y64 = c.astype(np.float64) + a.astype(np.float64) @ b.astype(np.float64)
    assert rel_fro(y, y64) <= 1e-5


def test_broadcast_strides(ctx, oracle):
    """stride 0 re-reads one matrix for every batch (GemmMatrixWiseBroadcast)."""
    rng = np.random.default_rng(5)
    a = rng.standard_normal((1, 64, 96)).astype(np.float32)
    b = rng.standard_normal((6, 96, 128)).astype(np.float32)
    c = rng.standard_normal((6, 64, 128)).astype(np.float32)
    want = oracle.gemm(c, np.repeat(a, 6, 0), b)
    y = ops.gemm(ctx, dev(a), dev(b), dev(c), mode=L.MODE_TF32X3, path=L.PATH_TCGEN05)
    assert rel_fro(y.cpu().numpy(), want) <= 1e-5
    a2 = rng.standard_normal((6, 64, 96)).astype(np.float32)
    b2 = rng.standard_normal((1, 96, 128)).astype(np.float32)
    want = oracle.gemm(c, a2, np.repeat(b2, 6, 0))
    y = ops.gemm(ctx, dev(a2), dev(b2), dev(c), mode=L.MODE_TF32X3, path=L.PATH_TCGEN05)
    assert rel_fro(y.cpu().numpy(), want) <= 1e-5


@pytest.mark.parametrize("path", [L.PATH_TCGEN05, L.PATH_SIMT])
def test_bias_epilogue_is_linear_forward(ctx, oracle, path):
    """y = bias + x.W with W stored [in, out] (Linear.cpp:134-136)."""
    rng = np.random.default_rng(6)
    x = rng.uniform(0, 1, (64, 784)).astype(np.float32)
    w = rng.uniform(-0.1, 0.1, (784, 512)).astype(np.float32)
    bias = rng.uniform(-1, 1, 512).astype(np.float32)
    want = oracle.gemm_ex(0, 0, 64, 512, 784, x, 784, 0, w, 512, 0, None, 512, 0, 512, 0, bias, 1,
                          64 * 512).reshape(64, 512)
    y = ops.gemm(ctx, dev(x), dev(w), bias=dev(bias), mode=L.MODE_TF32X3, path=path).cpu().numpy()
    if path == L.PATH_SIMT:
        assert np.array_equal(bits(y), bits(want))
    else:
        assert rel_fro(y, want) <= 1e-5


@pytest.mark.parametrize("mode", [L.MODE_TF32, L.MODE_TF32X3])
def test_linear_backward_gemms_with_fused_bias_grad(ctx, oracle, mode):
    """dx = dy.W^T, dW = x^T.dy, dB = colsum(dy)/B with transposes done by
    descriptors (LinearBackward.cpp:27-99 does Transpose + Gemm + ones-Gemm)."""
    rng = np.random.default_rng(8)
    B, I, Oo = 256, 192, 320
    dy = (rng.standard_normal((B, Oo)) * 0.02).astype(np.float32)
    x = (rng.standard_normal((B, I)) * 0.02).astype(np.float32)
    w = (rng.standard_normal((I, Oo)) * 0.02).astype(np.float32)
    z = np.zeros
    want_dx = oracle.gemm(z((1, B, I), np.float32), dy[None], oracle.transpose(w)[None])[0]
    want_dw = oracle.gemm(z((1, I, Oo), np.float32), oracle.transpose(x)[None], dy[None])[0]
    want_db = oracle.colsum(dy, 1.0 / B)
    dx = ops.gemm(ctx, dev(dy), dev(w), trans_b=True, mode=mode)
    db = torch.empty(Oo, device=DEV)
    dw = ops.gemm(ctx, dev(x), dev(dy), trans_a=True, mode=mode, colsum_out=db,
                  colsum_scale=1.0 / B)
    ctx.check_device_status()
    assert rel_fro(dx.cpu().numpy(), want_dx) <= TOL[mode]
    assert rel_fro(dw.cpu().numpy(), want_dw) <= TOL[mode]
    assert rel_fro(db.cpu().numpy(), want_db) <= 1e-5


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K,batch", [(1024, 512, 256, 40), (1000, 520, 100, 38), (512, 256, 64, 80)])
def test_two_cta_kernel_matches_one_cta_and_oracle(ctx, oracle, ta, tb, M, N, K, batch):
    """Problems with enough 256 x 256 tiles run on pairs of SMs (cta_group::2);
    the same request with pairs switched off runs on the one-CTA kernel.  Both
    must meet the TF32 bar against the CPU loop (checked on one batch) and agree
    with each other on all batches."""
    rng = np.random.default_rng(M + N + K + ta * 2 + tb)
    a = rng.standard_normal((batch, K, M) if ta else (batch, M, K)).astype(np.float32)
    b = rng.standard_normal((batch, N, K) if tb else (batch, K, N)).astype(np.float32)
    c = rng.uniform(-1, 1, (batch, M, N)).astype(np.float32)
    ta_, tb_, tc_ = dev(a), dev(b), dev(c)
    outs = []
    for pairs in (1, 0):
        ctx.set_option(L.OPT_CTA_PAIRS, pairs)
        outs.append(ops.gemm(ctx, ta_, tb_, tc_, trans_a=bool(ta), trans_b=bool(tb)))
        ctx.check_device_status()
    ctx.set_option(L.OPT_CTA_PAIRS, 1)
    bi = batch - 1
    want = oracle.gemm_ex(ta, tb, M, N, K, a[bi], a.shape[2], 0, b[bi], b.shape[2], 0, c[bi], N, 0,
                          N, 0, None, 1, M * N).reshape(M, N)
    assert rel_fro(outs[0][bi].cpu().numpy(), want) <= 2e-3
    assert rel_fro(outs[1][bi].cpu().numpy(), want) <= 2e-3
    # same products, same k order per output: the two kernels agree to rounding of the accumulation
    assert rel_fro(outs[0].cpu().numpy(), outs[1].cpu().numpy()) <= 1e-5


# ------------------------------------------------- full-size property checks
@pytest.mark.parametrize("n", [4096, 4000])
def test_config3_full_size_row_sample_and_linearity(ctx, oracle, n):
    """8 x n^3 is an hour of scalar CPU work, so at full size: (1) a sample of
    output rows of two batches against the CPU loop, (2) linearity
    gemm(a, b, c) - gemm(a, b, 0) == c, (3) every batch of a batched call equals
    the same matrices run alone."""
    batch = 8
    ids = [0, 7]
    a2, b2, c2 = W.dense_batched(0, ids, n, n, n, "normal")
    ta = torch.randn(batch, n, n, device=DEV)
    tb = torch.randn(batch, n, n, device=DEV)
    tc = torch.rand(batch, n, n, device=DEV) * 2 - 1
    for j, bi in enumerate(ids):
        ta[bi] = dev(a2[j]); tb[bi] = dev(b2[j]); tc[bi] = dev(c2[j])
    rows = [0, 1, 127, 128, n // 2 + 3, n - 1]
    for mode in (L.MODE_TF32, L.MODE_TF32X3):
        y = ops.gemm(ctx, ta, tb, tc, mode=mode)
        ctx.check_device_status()
        for j, bi in enumerate(ids):
            want = oracle.gemm(c2[j][rows][None], a2[j][rows][None], b2[j][None])[0]
            assert rel_fro(y[bi][rows].cpu().numpy(), want) <= TOL[mode]
        y0 = ops.gemm(ctx, ta, tb, None, mode=mode)
        assert float((y - y0 - tc).abs().max()) <= 1e-3
        alone = ops.gemm(ctx, ta[7], tb[7], tc[7], mode=mode)
        assert torch.equal(alone, y[7])
        del y, y0, alone


@pytest.mark.parametrize("mode", [L.MODE_TF32, L.MODE_TF32X3])
def test_config4_full_size_linear_backward(ctx, oracle, mode):
    """dY [8192 x 4096], X [8192 x 4096], W [4096 x 4096] ~ N(0, 0.02): dx = dy.W^T
    and dW = x^T.dy with the fused bias gradient, at the size the benchmark runs
    (other kernel instances than the small case: the K = 8192 chain, the column-sum
    warps over 32 row tiles, the panel tile order).  A sample of rows of dx and of
    dW against the CPU loop, every element of dB."""
    rows_total, width = 8192, 4096
    dy, x, w = W.linear_backward(0, 0, rows_total, width, width)
    tdy, tx, tw = dev(dy), dev(x), dev(w)
    dx = ops.gemm(ctx, tdy, tw, trans_b=True, mode=mode)
    db = torch.empty(width, device=DEV)
    dw = ops.gemm(ctx, tx, tdy, trans_a=True, mode=mode, colsum_out=db,
                  colsum_scale=1.0 / rows_total)
    ctx.check_device_status()
    assert ctx.last_path() == L.PATH_TCGEN05
    rows = [0, 127, 128, 4095, 4096, 8191]
    wt = np.ascontiguousarray(w.T)
    want_dx = oracle.gemm(np.zeros((1, len(rows), width), np.float32), dy[rows][None], wt[None])[0]
    assert rel_fro(dx[rows].cpu().numpy(), want_dx) <= TOL[mode]
    wrows = [0, 1, 255, 256, 2049, 4095]                 # rows of dW = columns of x
    xt = np.ascontiguousarray(x[:, wrows].T)
    want_dw = oracle.gemm(np.zeros((1, len(wrows), width), np.float32), xt[None], dy[None])[0]
    assert rel_fro(dw[wrows].cpu().numpy(), want_dw) <= TOL[mode]
    assert rel_fro(db.cpu().numpy(), oracle.colsum(dy, 1.0 / rows_total)) <= 1e-5
    assert rel_fro(db.cpu().numpy(), dy.astype(np.float64).sum(0) / rows_total) <= 1e-5


@pytest.mark.parametrize("n", [4096, 4000])
def test_single_product_tail_wave_split(ctx, oracle, n):
    """One n^3 product is 256 pair tiles on 74 pairs of SMs; with the tail-wave
    option on, the bottom rows go to a second launch of the one-CTA kernel.  The
    split result must meet the TF32 bar on rows of both parts and agree with the
    single launch (the default) to accumulation rounding."""
    a, b, c = W.dense_batched(0, [0], n, n, n, "normal")
    ta, tb, tc = dev(a[0]), dev(b[0]), dev(c[0])
    before = ctx.launch_count()
    y1 = ops.gemm(ctx, ta, tb, tc)
    whole_launches = ctx.launch_count() - before
    ctx.set_option(L.OPT_SPLIT_TAIL_WAVE, 1)
    before = ctx.launch_count()
    y = ops.gemm(ctx, ta, tb, tc)
    split_launches = ctx.launch_count() - before
    ctx.check_device_status()
    assert (split_launches, whole_launches) == (2, 1)
    rows = [0, 255, 3327, 3328, 3329, n - 129, n - 1]    # both sides of the cut at row 3328
    want = oracle.gemm(c[0][rows][None], a[0][rows][None], b[0][None])[0]
    assert rel_fro(y[rows].cpu().numpy(), want) <= 2e-3
    assert rel_fro(y.cpu().numpy(), y1.cpu().numpy()) <= 1e-5
    # in place (C aliases D) and with transposed A: the second launch shifts every base
    yt = tc.clone()
    ops.gemm(ctx, ta.t().contiguous(), tb, yt, yt, trans_a=True)
    ctx.set_option(L.OPT_SPLIT_TAIL_WAVE, 0)
    assert rel_fro(yt.cpu().numpy(), y1.cpu().numpy()) <= 1e-5


def _split_k_case(ctx, oracle, M, N, K, batch, ta, tb, on, off):
    """`on()` selects the kernel under test, `off()` one CTA per tile.  Checked against the
    CPU loop with every epilogue (in-place C, bias + ReLU, ReLU gate), against the
    one-CTA-per-tile launch, and for run-to-run bit-reproducibility."""
    rng = np.random.default_rng(M + N + K)
    a = rng.standard_normal((batch, K, M) if ta else (batch, M, K)).astype(np.float32)
    b = rng.standard_normal((batch, N, K) if tb else (batch, K, N)).astype(np.float32)
    c = rng.uniform(-1, 1, (batch, M, N)).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    gate = rng.standard_normal((batch, M, N)).astype(np.float32)
    ta_, tb_, tg = dev(a), dev(b), dev(gate)
    want = np.stack([oracle.gemm_ex(ta, tb, M, N, K, a[i], a.shape[2], 0, b[i], b.shape[2], 0, c[i], N, 0,
                                    N, 0, None, 1, M * N).reshape(M, N) for i in range(batch)])
    on()
    launches = ctx.launch_count()
    y = dev(c)
    ops.gemm(ctx, ta_, tb_, y, y, trans_a=bool(ta), trans_b=bool(tb))                 # y <- y + a.b
    assert ctx.launch_count() - launches == 1 and ctx.last_path() == L.PATH_TCGEN05
    ctx.check_device_status()
    assert rel_fro(y.cpu().numpy(), want) <= 2e-3
    # the same request with one CTA per tile
    off()
    y1 = dev(c)
    ops.gemm(ctx, ta_, tb_, y1, y1, trans_a=bool(ta), trans_b=bool(tb))
    on()
    assert rel_fro(y.cpu().numpy(), y1.cpu().numpy()) <= 1e-5
    assert not torch.equal(y, y1) or K <= 32          # other summation order: it did run the other kernel
    # bias + ReLU, then the ReLU gate; reproducible bit for bit
    r1 = ops.gemm(ctx, ta_, tb_, trans_a=bool(ta), trans_b=bool(tb), bias=dev(bias), relu=True)
    r2 = ops.gemm(ctx, ta_, tb_, trans_a=bool(ta), trans_b=bool(tb), bias=dev(bias), relu=True)
    assert torch.equal(r1, r2)
    lin = want - c + bias[None, None, :]
    assert rel_fro(r1.cpu().numpy(), np.maximum(lin, 0)) <= 2e-3
    g1 = ops.gemm(ctx, ta_, tb_, trans_a=bool(ta), trans_b=bool(tb), relu_gate=tg)
    assert rel_fro(g1.cpu().numpy(), np.where(gate > 0, want - c, 0)) <= 2e-3
    ctx.check_device_status()


def _options(ctx, slices):
    def f():
        ctx.set_option(L.OPT_K_SLICES, slices)
    return f


@pytest.mark.parametrize("M,N,K,batch,ta,tb,slices", [
    (64, 512, 784, 1, 0, 0, 1),       # the MLP's first layer at batch 64 (the policy's own choice)
    (64, 256, 512, 1, 0, 0, 2),       # its second layer (the policy leaves K = 512 whole: forced)
    (64, 784, 512, 1, 0, 1, 4),       # the dx GEMM of the first layer (W read transposed)
    (64, 512, 1536, 1, 0, 0, 1),      # a wider layer
    (256, 256, 1024, 4, 0, 0, 1),     # 32 tiles
    (64, 512, 784, 1, 0, 0, 2),
    (64, 512, 784, 1, 0, 0, 5),       # 25 k-blocks in 5 slices of 5
    (64, 512, 784, 1, 0, 0, 7),       # ... in slices of 4, 4, 4, 4, 4, 4, 1
    (64, 512, 784, 1, 0, 0, 16),      # more slices asked for than k-blocks allow: 13 of 2, 2, ..., 1
    (100, 132, 1100, 2, 1, 0, 3),     # ragged everything, K not a multiple of 32, A stored [K, M]
    (128, 64, 1024, 3, 1, 1, 8),      # both operands in the transposed orientation
    (300, 200, 96, 1, 0, 0, 3),       # one k-block per slice
])
def test_k_slices(ctx, oracle, M, N, K, batch, ta, tb, slices):
    """Few output tiles: S CTAs per tile on separate SMs, each a slice of k; the CTA
    that finishes last adds the partial tiles in slice order and runs the ordinary
    epilogue.  The ticket counters return to zero by themselves: the calls of this
    test (and of every later one) follow each other on one context."""
    try:
        _split_k_case(ctx, oracle, M, N, K, batch, ta, tb, _options(ctx, slices), _options(ctx, 0))
    finally:
        _options(ctx, 1)()


@pytest.mark.parametrize("M,N,K,batch,tb", [(256, 256, 256, 4, 0), (200, 136, 100, 3, 0),
                                            (384, 260, 1056, 2, 1), (128, 128, 32, 1, 0),
                                            (1024, 1024, 2048, 2, 0)])
def test_tf32x3_parts_of_a_in_tensor_memory(ctx, M, N, K, batch, tb):
    """fp32-accurate mode, A stored [M, K]: the high and low parts of A's tiles are
    written to tensor memory and read from there by the tensor core (the default)
    or both low parts go to shared memory (option off).  The same products in the
    same order: bit-identical results, and within 1e-5 of the fp64 product."""
    g = torch.Generator(device=DEV); g.manual_seed(M + N + K)
    a = torch.randn(batch, M, K, device=DEV, generator=g)
    b = torch.randn(batch, N, K, device=DEV, generator=g) if tb else \
        torch.randn(batch, K, N, device=DEV, generator=g)
    c = torch.rand(batch, M, N, device=DEV, generator=g)
    bias = torch.randn(N, device=DEV, generator=g)
    res = []
    for opt in (1, 0):
        ctx.set_option(L.OPT_SPLIT_A_TMEM, opt)
        res.append(ops.gemm(ctx, a, b, c, trans_b=bool(tb), bias=bias, mode=L.MODE_TF32X3))
        assert ctx.last_path() == L.PATH_TCGEN05
    ctx.set_option(L.OPT_SPLIT_A_TMEM, 1)
    ctx.check_device_status()
    bm = b.transpose(1, 2) if tb else b
    want = (c.double() + bias.double() + a.double() @ bm.double()).cpu().numpy()
    assert rel_fro(res[0].cpu().numpy(), want) <= 1e-5
    assert torch.equal(res[0], res[1])


def test_tensor_map_cache(ctx):
    """A GEMM on operands the context has seen encodes no TMA descriptor."""
    a = torch.randn(512, 256, device=DEV)
    b = torch.randn(256, 384, device=DEV)
    out = torch.empty(512, 384, device=DEV)
    ops.gemm(ctx, a, b, None, out)
    h0, m0 = ctx.counter(L.COUNTER_TENSOR_MAP_HITS), ctx.counter(L.COUNTER_TENSOR_MAP_MISSES)
    for _ in range(5):
        ops.gemm(ctx, a, b, None, out)
    assert ctx.counter(L.COUNTER_TENSOR_MAP_MISSES) == m0
    assert ctx.counter(L.COUNTER_TENSOR_MAP_HITS) == h0 + 10
    # another shape at the same address is another descriptor
    ops.gemm(ctx, a[:256], b, None, out[:256])
    assert ctx.counter(L.COUNTER_TENSOR_MAP_MISSES) == m0 + 1       # A's; B's is reused
    # more live descriptors than slots: the oldest are replaced, results stay right
    outs = []
    for i in range(70):
        ai = torch.randn(128, 64 + 4 * i, device=DEV)
        bi = torch.randn(64 + 4 * i, 128, device=DEV)
        outs.append((ai, bi, ops.gemm(ctx, ai, bi, mode=L.MODE_TF32X3)))
    for ai, bi, y in outs[::23]:
        assert rel_fro(y.cpu().numpy(), ai.double().cpu().numpy() @ bi.double().cpu().numpy()) <= 1e-5
    ctx.check_device_status()


@pytest.mark.parametrize("shape", ["one_cta", "pair", "split_mode", "split_mode_transposed_a",
                                   "k_slices"])
def test_bounded_wait_runs_out_and_context_survives(ctx, shape):
    """The TMA producers stop after 3 k-blocks (test hook) with the wait limit at
    2 ms: the MMA issuer's and the epilogue's waits run out, every role leaves
    through the common exit, TMEM is released, and the host reads
    SB200_ERR_DEVICE_TIMEOUT -- the error convention in place of the reference's
    CHECK_CUBLAS.  The same context then runs a normal GEMM."""
    if shape == "pair":
        M, N, K, batch, mode = 1024, 512, 256, 40, L.MODE_TF32
    elif shape == "k_slices":
        M, N, K, batch, mode = 64, 512, 1536, 1, L.MODE_TF32      # (from K = 2048 on, slices of k run as batches)
    elif shape == "one_cta":
        M, N, K, batch, mode = 256, 256, 256, 4, L.MODE_TF32
    else:
        M, N, K, batch, mode = 256, 256, 512, 2, L.MODE_TF32X3
    ta = shape == "split_mode_transposed_a"     # the low parts of A in shared memory, not TMEM
    a = torch.randn(batch, K, M, device=DEV) if ta else torch.randn(batch, M, K, device=DEV)
    b = torch.randn(batch, K, N, device=DEV)
    good = ops.gemm(ctx, a, b, mode=mode, trans_a=ta)
    ctx.check_device_status()
    ctx.set_option(L.OPT_WAIT_LIMIT_US, 2000)
    ctx.set_option(L.OPT_TEST_STALL_KBLOCKS, 3)
    try:
        ops.gemm(ctx, a, b, mode=mode, trans_a=ta)
        with pytest.raises(L.Sb200Error) as e:
            ctx.check_device_status()
        assert e.value.status == L.ERR_DEVICE_TIMEOUT
    finally:
        ctx.set_option(L.OPT_TEST_STALL_KBLOCKS, -1)
        ctx.set_option(L.OPT_WAIT_LIMIT_US, 2000000)
    ctx.check_device_status()                            # the word was cleared
    # (k-slices: every CTA drew its ticket although its waits ran out, so the counters are
    # back at zero and the next product is complete)
    again = ops.gemm(ctx, a, b, mode=mode, trans_a=ta)
    ctx.check_device_status()
    assert torch.equal(again, good)


# ------------------------------------------------ Sapphire-signature shims
def test_compat_dense_gemm_signature(ctx, oracle):
    """Sapphire::Compute::Dense::Cuda::Gemm(totalSize, out, A, B, M, N, K, deviceId)."""
    a, b, c = W.dense_batched(3, range(3), 64, 48, 32, "uniform")
    out, ta, tb = dev(c), dev(a), dev(b)
    rc = L.lib().sb200_compat_dense_gemm(out.numel(), out.data_ptr(), ta.data_ptr(), tb.data_ptr(),
                                         64, 48, 32, 0)
    assert rc == L.OK
    assert rel_fro(out.cpu().numpy(), oracle.gemm(c, a, b)) <= 2e-3


@pytest.mark.parametrize("bcA,bcB", [(True, False), (False, True)])
def test_compat_gemm_matrixwise_broadcast_signature(ctx, oracle, bcA, bcB):
    """Sapphire::Compute::Dense::Cuda::GemmMatrixWiseBroadcast(out, A, B, M, N, K,
    batchSize, broadcastA, broadcastB, deviceId): out += A.B with one operand shared."""
    M, N, K, batch = 96, 80, 64, 5
    rng = np.random.default_rng(21)
    a = rng.standard_normal((1 if bcA else batch, M, K)).astype(np.float32)
    b = rng.standard_normal((1 if bcB else batch, K, N)).astype(np.float32)
    c = rng.uniform(-1, 1, (batch, M, N)).astype(np.float32)
    out, ta, tb = dev(c), dev(a), dev(b)
    L.lib().sb200_compat_set_mode(L.MODE_TF32X3)
    rc = L.lib().sb200_compat_dense_gemm_broadcast(out.data_ptr(), ta.data_ptr(), tb.data_ptr(),
                                                   M, N, K, batch, int(bcA), int(bcB), 0)
    L.lib().sb200_compat_set_mode(L.MODE_TF32)
    assert rc == L.OK
    want = oracle.gemm(c, np.broadcast_to(a, (batch, M, K)).copy(), np.broadcast_to(b, (batch, K, N)).copy())
    assert rel_fro(out.cpu().numpy(), want) <= 1e-5


@pytest.mark.parametrize("mode", [L.MODE_TF32, L.MODE_TF32X3])
def test_matmul_backward_accumulates_with_transposed_operand(ctx, oracle, mode):
    """MulBackProp (Sources/Sapphire/operations/Backward/MathBackward.cpp:46-50):
    da <- da + dy.b^T and db <- db + a^T.dy, each ONE call that both accumulates in
    place (C aliases D) and reads a transposed operand, batched."""
    batch, M, K, N = 3, 160, 96, 200
    rng = np.random.default_rng(22)
    a = rng.standard_normal((batch, M, K)).astype(np.float32)
    b = rng.standard_normal((batch, K, N)).astype(np.float32)
    dy = rng.standard_normal((batch, M, N)).astype(np.float32)
    da0 = rng.standard_normal((batch, M, K)).astype(np.float32)
    db0 = rng.standard_normal((batch, K, N)).astype(np.float32)
    # the CPU unit, itself pinned against the reference's MulBackProp (tests/test_oracle.py)
    want_da, want_db = oracle.matmul_backward(da0, db0, dy, a, b)
    da, db = dev(da0), dev(db0)
    ops.gemm(ctx, dev(dy), dev(b), da, da, trans_b=True, mode=mode)
    ops.gemm(ctx, dev(a), dev(dy), db, db, trans_a=True, mode=mode)
    ctx.check_device_status()
    assert ctx.last_path() == L.PATH_TCGEN05
    assert rel_fro(da.cpu().numpy(), want_da) <= TOL[mode]
    assert rel_fro(db.cpu().numpy(), want_db) <= TOL[mode]


@pytest.mark.parametrize("idx", [8, 9, 10])
def test_compat_compute_gemm_broadcast_families(ctx, idx):
    """The reference's BroadcastTest families (BroadcastTest.cpp:20-202) through the
    Compute::Gemm shim on the device, against fixtures written by the reference's own
    host path (tests/golden/compute_units_golden.npz) -- including the family whose pairing
    of y and a blocks is the reference's, not numpy's."""
    import ctypes as C
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    ys, as_, bs = mod.BROADCAST_CASES[idx]
    y0, a, b = mod.broadcast_case(idx)
    want = np.load(os.path.join(os.path.dirname(__file__), "golden", "compute_units_golden.npz"))[f"case{idx}"]
    ty, ta, tb = dev(y0), dev(a), dev(b)
    arr = lambda s: (C.c_int * len(s))(*s)
    L.lib().sb200_compat_set_mode(L.MODE_TF32X3)
    rc = L.lib().sb200_compat_compute_gemm(arr(ys), len(ys), ty.data_ptr(), arr(as_), len(as_),
                                           ta.data_ptr(), arr(bs), len(bs), tb.data_ptr(), 0)
    L.lib().sb200_compat_set_mode(L.MODE_TF32)
    assert rc == L.OK
    assert rel_fro(ty.cpu().numpy(), want) <= 1e-5


@pytest.mark.parametrize("mode", [L.MODE_TF32, L.MODE_TF32X3])
@pytest.mark.parametrize("B,n_in,n_out,path", [(64, 784, 512, L.PATH_AUTO), (64, 256, 12, L.PATH_AUTO),
                                               (16, 40, 24, L.PATH_AUTO), (7, 13, 5, L.PATH_SIMT),
                                               (512, 1024, 768, L.PATH_AUTO)])
def test_in_place_sgd_update_of_a_linear_layer(ctx, oracle, mode, B, n_in, n_out, path):
    """sgd_lr: W -= lr * x^T.dy and b -= lr * (1/B) colsum(dy) in one launch -- the weight
    and bias half of the reference's LinearBackProp with its SGD optimizer inside.
    Bit-identical to storing the gradients and running the SGD kernel on them (the
    same two roundings per element), and within the mode's tolerance of the CPU oracle's
    unit, which is itself pinned against the reference's."""
    rng = np.random.default_rng(B + n_in + n_out)
    x = rng.uniform(0, 1, (B, n_in)).astype(np.float32)
    dy = rng.standard_normal((B, n_out)).astype(np.float32)
    w = rng.standard_normal((n_in, n_out)).astype(np.float32)
    b = rng.standard_normal(n_out).astype(np.float32)
    lr = 0.01
    tx, tdy = dev(x), dev(dy)
    # gradients stored, then the SGD kernel
    dw, db = torch.empty(n_in, n_out, device=DEV), torch.empty(n_out, device=DEV)
    ops.gemm(ctx, tx, tdy, None, dw, trans_a=True, colsum_out=db, colsum_scale=1.0 / B, mode=mode, path=path)
    w_two, b_two = dev(w), dev(b)
    ops.sgd_update(ctx, w_two, dw, lr)
    ops.sgd_update(ctx, b_two, db, lr)
    # the same in one launch, in place
    w_one, b_one = dev(w), dev(b)
    ops.gemm(ctx, tx, tdy, w_one, w_one, trans_a=True, colsum_out=b_one, colsum_scale=1.0 / B, mode=mode,
             path=path, sgd_lr=lr)
    ctx.check_device_status()
    assert torch.equal(w_one, w_two) and torch.equal(b_one, b_two)
    net = oracle.MlpOracle([w], [b], lr)
    net.linear_backward(0, x, dy)
    # the update is lr * gradient on top of an O(1) weight: compare the steps taken
    step_w, step_b = w - net.W[0], b - net.b[0]
    tol = 1e-5 if (mode == L.MODE_TF32X3 or path == L.PATH_SIMT) else 2e-3
    assert rel_fro(w - w_one.cpu().numpy(), step_w) <= tol + 1e-4     # (+ the rounding of w - lr g itself)
    assert rel_fro(b - b_one.cpu().numpy(), step_b) <= tol + 1e-4
    # argument rules: needs C, no bias / relu / gate next to it
    with pytest.raises(L.Sb200Error):
        ops.gemm(ctx, tx, tdy, None, w_one, trans_a=True, sgd_lr=lr)
    with pytest.raises(L.Sb200Error):
        ops.gemm(ctx, tx, tdy, w_one, w_one, trans_a=True, sgd_lr=lr, relu=True)


def test_invalid_arguments(ctx):
    a = torch.zeros(4, 8, device=DEV)
    b = torch.zeros(8, 4, device=DEV)
    out = torch.zeros(4, 4, device=DEV)
    lib = L.lib()
    st = torch.cuda.current_stream().cuda_stream
    def call(**kw):
        args = dict(mode=0, path=0, ta=0, tb=0, M=4, N=4, K=8, lda=8, ldb=4, ldd=4, batch=1)
        args.update(kw)
        return lib.sb200_gemm_batched(ctx.handle, args["mode"], args["path"], args["ta"], args["tb"],
                                      args["M"], args["N"], args["K"], a.data_ptr(), args["lda"], 0,
                                      b.data_ptr(), args["ldb"], 0, None, 4, 0, out.data_ptr(),
                                      args["ldd"], 0, None, None, 1.0, args["batch"], st)
    assert call() == L.OK
    assert call(lda=7) == L.ERR_INVALID_ARG
    assert call(ldb=3) == L.ERR_INVALID_ARG
    assert call(ldd=3) == L.ERR_INVALID_ARG
    assert call(mode=5) == L.ERR_INVALID_ARG
    assert call(M=-1) == L.ERR_INVALID_ARG
    assert call(batch=2) == L.ERR_INVALID_ARG          # output batches would overlap (stride 0)
    torch.cuda.synchronize()


@pytest.mark.parametrize("mode", [L.MODE_TF32, L.MODE_TF32X3])
@pytest.mark.parametrize("M,N,K,batch,path", [
    (64, 512, 784, 1, L.PATH_TCGEN05),      # Linear forward of the MLP: one-CTA tensor-core kernel
    (200, 328, 100, 3, L.PATH_TCGEN05),     # ragged tiles, batch stride of the gate
    (1024, 512, 256, 40, L.PATH_AUTO),      # large enough for the two-CTA kernel (TF32 mode)
    (64, 10, 256, 1, L.PATH_AUTO),          # rows of 10 floats: CUDA-core kernel
    (33, 17, 9, 2, L.PATH_SIMT),
])
def test_relu_and_gate_epilogues_equal_the_separate_kernels(ctx, mode, M, N, K, batch, path):
    """The fused epilogue steps are exact elementwise functions of the unfused
    GEMM result: relu(x) = x > 0 ? x : 0 (NaiveBasic.cpp:159-165) and the ReLU
    backward gate 0 + (g > 0 ? x : 0) (NaiveBasic.cpp:167-174), so the fused and
    the unfused calls must agree bit for bit."""
    rng = np.random.default_rng(M + N + K)
    a = dev(rng.standard_normal((batch, M, K)).astype(np.float32))
    b = dev(rng.standard_normal((batch, K, N)).astype(np.float32))
    c = dev(rng.uniform(-1, 1, (batch, M, N)).astype(np.float32))
    bias = dev(rng.uniform(-1, 1, N).astype(np.float32))
    gate_np = rng.standard_normal((batch, M, N)).astype(np.float32)
    gate_np[:, ::3, ::5] = 0.0                                  # exact zeros do not pass the gate
    gate = dev(gate_np)
    plain = ops.gemm(ctx, a, b, c, bias=bias, mode=mode, path=path)
    want_relu = torch.where(plain > 0, plain, torch.zeros_like(plain))
    got = ops.gemm(ctx, a, b, c, bias=bias, mode=mode, path=path, relu=True)
    assert torch.equal(got, want_relu)
    want_gate = torch.where(gate > 0, plain, torch.zeros_like(plain)) + 0.0
    got = ops.gemm(ctx, a, b, c, bias=bias, mode=mode, path=path, relu_gate=gate)
    assert np.array_equal(bits(got.cpu().numpy()), bits(want_gate.cpu().numpy()))
    both = ops.gemm(ctx, a, b, c, bias=bias, mode=mode, path=path, relu=True, relu_gate=gate)
    want_both = torch.where(gate > 0, want_relu, torch.zeros_like(plain)) + 0.0
    assert np.array_equal(bits(both.cpu().numpy()), bits(want_both.cpu().numpy()))
    ctx.check_device_status()


def test_gate_argument_validation(ctx):
    a = torch.zeros(8, 8, device=DEV)
    e = L.GemmEpilogue()
    e.relu_gate, e.ld_gate, e.stride_gate = a.data_ptr(), 4, 0          # ld_gate < N
    rc = L.lib().sb200_gemm_batched_ex(ctx.handle, L.MODE_TF32, L.PATH_AUTO, 0, 0, 8, 8, 8,
                                       a.data_ptr(), 8, 0, a.data_ptr(), 8, 0, None, 8, 0,
                                       a.data_ptr(), 8, 0, C.byref(e), 1, None)
    assert rc == L.ERR_INVALID_ARG
    rc = L.lib().sb200_gemm_batched_ex(ctx.handle, L.MODE_TF32, L.PATH_AUTO, 0, 0, 8, 8, 8,
                                       a.data_ptr(), 8, 0, a.data_ptr(), 8, 0, None, 8, 0,
                                       a.data_ptr(), 8, 0, None, 1, None)
    assert rc == L.ERR_INVALID_ARG


@pytest.mark.parametrize("mode,tol", [(L.MODE_TF32, 2e-3), (L.MODE_TF32X3, 1e-5)])
@pytest.mark.parametrize("M,N,K,owners,ta", [
    (1024, 512, 256, 4, 1),       # one-CTA kernel, transposed A like dW = x^T.dy
    (4096, 4096, 512, 8, 1),      # enough tiles for the two-CTA kernel (TF32 mode)
    (512, 520, 100, 2, 0),        # ragged N and K: scalar tail reductions
    (256, 64, 64, 1, 0),          # a single owner: plain accumulate
])
def test_reduce_scatter_epilogue_on_one_gpu(ctx, oracle, mode, tol, M, N, K, owners, ta):
    """The reduce-scatter epilogue with every owner's buffer on this GPU: row block o
    of the product is added into buffer o; a second call adds it again."""
    rng = np.random.default_rng(M + N + K + owners)
    a = rng.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    b = rng.standard_normal((K, N)).astype(np.float32)
    want = (a.T if ta else a).astype(np.float64) @ b.astype(np.float64)
    bufs = [torch.full((M // owners, N), float(o + 1), device=DEV) for o in range(owners)]
    colsum = torch.empty(N, device=DEV)
    for rounds in (1, 2):
        ops.gemm_reduce_scatter(ctx, dev(a), dev(b), [t.data_ptr() for t in bufs], N, mode=mode,
                                trans_a=bool(ta), colsum_out=colsum, colsum_scale=0.5)
        got = torch.cat([t - float(o + 1) for o, t in enumerate(bufs)]).cpu().numpy()
        assert rel_fro(got, rounds * want) <= tol
    assert np.abs(colsum.cpu().numpy() - 0.5 * b.astype(np.float64).sum(0)).max() <= 1e-3
    ctx.check_device_status()


def test_reduce_scatter_argument_validation(ctx):
    a = torch.zeros(256, 64, device=DEV)
    bufs = [torch.zeros(96, 64, device=DEV) for _ in range(2)]
    with pytest.raises(L.Sb200Error) as e:           # 192 rows over 2 owners: blocks of 96, not tile-aligned
        ops.gemm_reduce_scatter(ctx, torch.zeros(192, 64, device=DEV), a[:64], [t.data_ptr() for t in bufs], 64)
    assert e.value.status == L.ERR_UNSUPPORTED
    with pytest.raises(L.Sb200Error) as e:
        ops.gemm_reduce_scatter(ctx, a, a[:64], [bufs[0].data_ptr()] * 9, 64)
    assert e.value.status == L.ERR_INVALID_ARG


def test_peer_window_single_rank_linear_backward(ctx):
    """world == 1: the windows are this GPU's own buffers; over five steps (the
    three windows come round again) dW and dB of the fused route equal the plain
    GEMM with its fused column sum."""
    from sapphire_b200 import runner
    rng = np.random.default_rng(5)
    reducer = runner.FusedWeightGradient(ctx, 256, 192)
    assert reducer.ok
    dw = torch.empty(256, 192, device=DEV)
    db = torch.empty(192, device=DEV)
    for _ in range(5):
        x = dev(rng.standard_normal((384, 256)).astype(np.float32))
        dy = dev(rng.standard_normal((384, 192)).astype(np.float32))
        reducer.start(x, dy, dw, db, mode=L.MODE_TF32X3)
        reducer.wait()
        want_db = torch.empty(192, device=DEV)
        want = ops.gemm(ctx, x, dy, trans_a=True, mode=L.MODE_TF32X3, colsum_out=want_db,
                        colsum_scale=1.0 / 384)
        assert rel_fro(dw.cpu().numpy(), want.cpu().numpy()) <= 1e-6
        assert torch.equal(db, want_db)
    reducer.close()


def test_peer_barrier_single_rank_and_bounded_wait(ctx):
    """sb200_peer_barrier with one rank passes at once and counts; with a second "rank"
    whose flag words nobody ever writes the wait runs out after the context's limit, the
    status word says so, and the context carries on (no rank is needed to make a wait
    expire, and nothing hangs)."""
    import ctypes as C
    from sapphire_b200 import runner
    bar = runner.PeerBarrier(ctx, 0, 1)
    for _ in range(3):
        bar()
    ctx.check_device_status()
    torch.cuda.synchronize()
    assert int(bar.window.mine.view(torch.int32)[0, 28]) == 3
    silent = torch.zeros(L.DP_FLAG_WORDS, dtype=torch.int32, device=DEV)     # the rank that never arrives
    arr = (C.c_void_p * 2)(int(bar.window.pointers[0]), silent.data_ptr())
    ctx.set_option(L.OPT_WAIT_LIMIT_US, 2000)
    try:
        rc = L.lib().sb200_peer_barrier(ctx.handle, arr, 2, 0, torch.cuda.current_stream().cuda_stream)
        assert rc == L.OK
        with pytest.raises(L.Sb200Error) as e:
            ctx.check_device_status()
        assert e.value.status == L.ERR_DEVICE_TIMEOUT
    finally:
        ctx.set_option(L.OPT_WAIT_LIMIT_US, 2000000)
    assert int(silent[20]) == 4                           # ... which was told that rank 0 had arrived
    bar()                                                # the context and the words still work
    ctx.check_device_status()
    bar.close()


def test_epilogue_steps_with_k_zero(ctx):
    """K == 0: D = gate(relu(C + bias)), no product."""
    rng = np.random.default_rng(9)
    c = dev(rng.standard_normal((40, 24)).astype(np.float32))
    bias = dev(rng.standard_normal(24).astype(np.float32))
    gate = dev(rng.standard_normal((40, 24)).astype(np.float32))
    a = torch.zeros(40, 0, device=DEV)
    b = torch.zeros(0, 24, device=DEV)
    got = ops.gemm(ctx, a, b, c, bias=bias, relu=True, relu_gate=gate)
    base = c + bias
    want = torch.where(gate > 0, torch.where(base > 0, base, torch.zeros_like(base)), torch.zeros_like(base)) + 0.0
    assert torch.equal(got, want)


@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (0, 1)])
@pytest.mark.parametrize("cmode", ["none", "separate", "in_place"])
def test_long_k_few_tiles_split_k(ctx, ta, tb, cmode):
    """256 x 192 x 8192: four output tiles, so the k range is cut into concurrent
    slices that add into D.  Checked against the fp64 product at the TF32 bound."""
    rng = np.random.default_rng(31 + ta + 2 * tb)
    M, N, K = 256, 192, 8192
    a = rng.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    b = rng.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    c = rng.standard_normal((M, N)).astype(np.float32)
    want = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    if cmode != "none":
        want = want + c
    if cmode == "none":
        got = ops.gemm(ctx, dev(a), dev(b), trans_a=bool(ta), trans_b=bool(tb))
    elif cmode == "separate":
        got = ops.gemm(ctx, dev(a), dev(b), dev(c), trans_a=bool(ta), trans_b=bool(tb))
    else:
        y = dev(c)
        got = ops.gemm(ctx, dev(a), dev(b), y, y, trans_a=bool(ta), trans_b=bool(tb))
    assert ctx.last_path() == L.PATH_TCGEN05
    assert rel_fro(got.cpu().numpy(), want) <= 2e-3
    ctx.check_device_status()
