"""GPU parity tests of the CSR sparse GEMM through the C ABI.

ROW and COL must equal the CPU oracle's bit for bit; values within 1e-5
(relative to the largest magnitude of the row set, accumulation order on the
GPU is not fixed).  The oracle is a restatement: the reference ships no sparse
GEMM, so reference parity for this path is unpinned.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from sapphire_b200 import _lib as L
from sapphire_b200 import ops
from sapphire_b200 import workloads as W

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_case(ctx, oracle, M, K, N, seedA, seedB, dens, dist, cap=4096, fn=None):
    rA, cA, vA = W.csr_random(seedA, M, K, dens, dist, zipf_cap=cap)
    rB, cB, vB = W.csr_random(seedB, K, N, dens, dist, zipf_cap=cap)
    A = ops.CsrMatrix.from_numpy(rA, cA, vA, M, K, DEV)
    B = ops.CsrMatrix.from_numpy(rB, cB, vB, K, N, DEV)
    Cm = (fn or ops.spgemm)(ctx, A, B)
    torch.cuda.synchronize()
    rc, cc, vc = Cm.to_numpy()
    orc, occ, ovc, _ = oracle.spgemm(rA, cA, vA, rB, cB, vB, M, N)
    assert np.array_equal(rc, orc), "ROW differs"
    assert np.array_equal(cc, occ), "COL differs"
    if ovc.size:
        assert np.abs(vc - ovc).max() <= 1e-5 * max(np.abs(ovc).max(), 1.0)
    return Cm


@pytest.mark.parametrize("M,K,N,dens,dist,cap", [
    (64, 64, 64, 0.05, "poisson", 0),            # tiny rows only (<= 32 products)
    (300, 200, 500, 0.02, "poisson", 0),         # rectangular, ragged N (not a multiple of 32)
    (2048, 2048, 2048, 0.01, "poisson", 0),      # bitmap rows
    (4096, 4096, 4096, None, "zipf", 512),       # mixed bins
    (8192, 8192, 8192, None, "zipf", 4096),      # heavy rows: output wider than the shared buffer
    (1000, 1000, 70000, 0.0005, "poisson", 0),   # wide N: bitmap larger than 2048 words
    (300, 400, 400000, 0.01, "poisson", 0),      # very wide N, long rows of B: heavy bin, rank windows
    (64, 2048, 65536, 0.02, "poisson", 0),       # ~37 k entries per output row: two windows each, one
                                                 # work item per window until the window queue is full
    (64, 2048, 65536, 0.05, "poisson", 0),       # nearly dense output rows: three windows, a queue
                                                 # that fills mid-row (empty items), single-item rows
])
def test_spgemm_matches_oracle(ctx, oracle, M, K, N, dens, dist, cap):
    run_case(ctx, oracle, M, K, N, 0, 1, dens, dist, cap or 4096)


@pytest.mark.parametrize("M,K,N,a,b", [
    # A (density | Zipf cap), B likewise: the walk classes of the mid-row kernel
    (500, 300, 65536, 0.05, 0.005),      # rows of B of ~330 entries: walked by the whole CTA
    (500, 300, 65536, 0.2, 0.005),       # the same with ~20 k products per row: heavy bin
    (400, 2000, 65536, 0.05, 0.00003),   # rows of B of <= 4 entries: walked by single threads
    (300, 1500, 65535, 0.03, 0.001),     # one column short of the rank-table kernels' width
    (300, 1500, 65537, 0.03, 0.001),     # one column beyond it: general row kernel
    (1, 4096, 65536, 0.5, 0.001),        # a single row of A with 2048 nonzeros
    (1500, 1500, 40000, ("zipf", 1024), 0.002),   # power-law A on uniform B
    (1500, 1500, 40000, 0.01, ("zipf", 1024)),    # uniform A on power-law B
    (700, 700, 33, 0.05, 0.5),           # 33 columns: every product collides
])
def test_spgemm_mixed_operands(ctx, oracle, M, K, N, a, b):
    """A and B drawn from different distributions, so that each way the kernels walk a
    row of B (single threads, 16-lane groups, the whole CTA) and each bin meets rows
    of the other kinds."""
    def draw(seed, rows, cols, spec):
        if isinstance(spec, tuple):
            return W.csr_random(seed, rows, cols, None, spec[0], zipf_cap=spec[1])
        return W.csr_random(seed, rows, cols, spec, "poisson")
    rA, cA, vA = draw(10, M, K, a)
    rB, cB, vB = draw(11, K, N, b)
    A = ops.CsrMatrix.from_numpy(rA, cA, vA, M, K, DEV)
    B = ops.CsrMatrix.from_numpy(rB, cB, vB, K, N, DEV)
    Cm = ops.spgemm(ctx, A, B)
    torch.cuda.synchronize()
    ctx.check_device_status()
    rc, cc, vc = Cm.to_numpy()
    orc, occ, ovc, _ = oracle.spgemm(rA, cA, vA, rB, cB, vB, M, N)
    assert np.array_equal(rc, orc), "ROW differs"
    assert np.array_equal(cc, occ), "COL differs"
    if ovc.size:
        assert np.abs(vc - ovc).max() <= 1e-5 * max(np.abs(ovc).max(), 1.0)


@pytest.mark.parametrize("dist,cap", [("poisson", 0), ("zipf", 2048)])
def test_spgemm_general_row_kernel_below_65536_columns(ctx, oracle, dist, cap):
    """Products of at most 65536 columns run their mid-sized rows on specialised
    kernels by default; with that switched off the general row kernel takes them.
    Both must match the oracle, hence each other."""
    ctx.set_option(L.OPT_SPGEMM_FAST_MID, 0)
    try:
        slow = run_case(ctx, oracle, 3000, 3000, 6000, 4, 5, 0.01, dist, cap or 4096)
    finally:
        ctx.set_option(L.OPT_SPGEMM_FAST_MID, 1)
    fast = run_case(ctx, oracle, 3000, 3000, 6000, 4, 5, 0.01, dist, cap or 4096)
    assert torch.equal(slow.row, fast.row) and torch.equal(slow.col, fast.col)


def test_spgemm_callee_allocated_output(ctx, oracle):
    """The drop-in call: the library allocates C, the caller frees it."""
    run_case(ctx, oracle, 1500, 1500, 1500, 2, 3, 0.01, "poisson", fn=ops.spgemm_callee_alloc)


def test_spgemm_through_sapphire_signature(ctx, oracle):
    """Sparse::Cuda::Gemm(hostOutput, cudaOutput, cudaA, cudaB, m, n, numMatrices, ...)."""
    def via_shim(ctx_, A, B):
        a, b, c = A.as_struct(), B.as_struct(), L.Csr()
        assert L.lib().sb200_compat_sparse_gemm(C.byref(a), C.byref(b), C.byref(c), 0) == L.OK
        n = int(c.NNZ)
        row = torch.empty(A.M + 1, dtype=torch.int32, device=DEV)
        col = torch.empty(max(n, 1), dtype=torch.int32, device=DEV)
        val = torch.empty(max(n, 1), dtype=torch.float32, device=DEV)
        st = torch.cuda.current_stream().cuda_stream
        assert L.lib().sb200_csr_copy_out(C.byref(c), row.data_ptr(), col.data_ptr(),
                                          val.data_ptr(), 0, st) == L.OK
        L.lib().sb200_csr_free(C.byref(c))
        return ops.CsrMatrix(row, col[:n], val[:n], A.M, B.N)
    run_case(ctx, oracle, 700, 700, 700, 4, 5, 0.02, "poisson", fn=via_shim)


def test_spgemm_keeps_structural_zeros(ctx, oracle):
    """Products that cancel exactly stay in the pattern (two-pass symbolic /
    numeric semantics).  Seeded random inputs do hit this: the 4096-row Zipf
    case above contains one entry whose two products are +-0.15941112."""
    rowA = np.array([0, 2, 3], np.uint32)
    colA = np.array([0, 1, 1], np.uint32)
    valA = np.array([1.0, -1.0, 2.0], np.float32)
    rowB = np.array([0, 2, 4], np.uint32)
    colB = np.array([3, 5, 3, 5], np.uint32)
    valB = np.array([0.5, 0.25, 0.5, 0.75], np.float32)
    A = ops.CsrMatrix.from_numpy(rowA, colA, valA, 2, 2, DEV)
    B = ops.CsrMatrix.from_numpy(rowB, colB, valB, 2, 8, DEV)
    r, c, v = ops.spgemm(ctx, A, B).to_numpy()
    assert r.tolist() == [0, 2, 4] and c.tolist() == [3, 5, 3, 5]
    assert v.tolist() == [0.0, -0.5, 1.0, 1.5]
    orc, occ, ovc, _ = oracle.spgemm(rowA, colA, valA, rowB, colB, valB, 2, 8)
    assert np.array_equal(r, orc) and np.array_equal(c, occ) and np.array_equal(v, ovc)


def test_spgemm_empty_and_degenerate(ctx, oracle):
    # all-empty A
    M = N = 128
    rowA = np.zeros(M + 1, np.uint32)
    A = ops.CsrMatrix.from_numpy(rowA, np.zeros(0, np.uint32), np.zeros(0, np.float32), M, N, DEV)
    rB, cB, vB = W.csr_random(1, N, N, 0.05)
    B = ops.CsrMatrix.from_numpy(rB, cB, vB, N, N, DEV)
    Cm = ops.spgemm(ctx, A, B)
    assert Cm.nnz == 0 and int(Cm.row.abs().sum()) == 0
    # identity x B == B
    eye = ops.CsrMatrix.from_numpy(np.arange(N + 1, dtype=np.uint32), np.arange(N, dtype=np.uint32),
                                   np.ones(N, np.float32), N, N, DEV)
    Cm = ops.spgemm(ctx, eye, B)
    r, c, v = Cm.to_numpy()
    assert np.array_equal(r, rB) and np.array_equal(c, cB) and np.array_equal(v, vB)
    # shape mismatch is rejected
    bad = ops.CsrMatrix.from_numpy(np.zeros(65, np.uint32), np.zeros(0, np.uint32),
                                   np.zeros(0, np.float32), 64, 64, DEV)
    with pytest.raises(L.Sb200Error) as e:
        ops.spgemm(ctx, A, bad)
    assert e.value.status == L.ERR_INVALID_ARG


@pytest.mark.parametrize("dist", ["poisson", "zipf"])
def test_config5_full_size_properties(ctx, dist):
    """65536 x 65536, 0.1 % density (and the Zipf variant): ROW monotone and
    consistent with NNZ, COL strictly ascending inside rows, and the checksum
    C.1 == A.(B.1) in float64."""
    import scipy.sparse as sp
    M = N = 65536
    rA, cA, vA = W.csr_random(0, M, N, 0.001, dist)
    rB, cB, vB = W.csr_random(1, N, N, 0.001, dist)
    A = ops.CsrMatrix.from_numpy(rA, cA, vA, M, N, DEV)
    B = ops.CsrMatrix.from_numpy(rB, cB, vB, N, N, DEV)
    Cm = ops.spgemm(ctx, A, B)
    torch.cuda.synchronize()
    row = Cm.row.long()
    assert int(row[0]) == 0 and int(row[-1]) == Cm.nnz
    assert bool((row[1:] >= row[:-1]).all())
    col = Cm.col.long()
    asc = col[1:] > col[:-1]
    starts = torch.zeros(Cm.nnz, dtype=torch.bool, device=DEV)
    inner = row[1:-1]
    starts[inner[inner < Cm.nnz]] = True
    assert bool((asc | starts[1:]).all())
    assert int(col.max()) < N and int(col.min()) >= 0
    rowsum = torch.zeros(M, dtype=torch.float64, device=DEV)
    ridx = torch.repeat_interleave(torch.arange(M, device=DEV), row[1:] - row[:-1])
    rowsum.index_add_(0, ridx, Cm.val.double())
    As = sp.csr_matrix((vA.astype(np.float64), cA, rA), shape=(M, N))
    Bs = sp.csr_matrix((vB.astype(np.float64), cB, rB), shape=(N, N))
    want = As @ (Bs @ np.ones(N))
    assert np.abs(rowsum.cpu().numpy() - want).max() <= 1e-4
    # two row blocks of the real product against the CPU oracle (full B): the first
    # 2048 rows, and 2048 rows around the row of A with the most scalar products
    from oracle import oracle as O
    from sapphire_b200 import runner
    work = W.csr_products(rA, cA, rB)
    heavy = int(np.argmax(work))
    lo = min(max(heavy - 1024, 0), M - 2048)
    rowC = Cm.row.cpu().numpy().view(np.uint32).astype(np.int64)
    for block in (range(0, 2048), range(lo, lo + 2048)):
        rb, cb, vb = runner.csr_row_block(rA, cA, vA, block)
        orow, ocol, oval, _ = O.spgemm(rb, cb, vb, rB, cB, vB, len(block), N)
        p0, p1 = rowC[block.start], rowC[block.stop]
        assert np.array_equal(rowC[block.start:block.stop + 1] - p0, orow.astype(np.int64)), "ROW differs"
        assert np.array_equal(Cm.col[p0:p1].cpu().numpy().view(np.uint32), ocol), "COL differs"
        got = Cm.val[p0:p1].cpu().numpy()
        assert np.abs(got - oval).max() <= 1e-5 * max(np.abs(oval).max(), 1.0)


def test_sparse_naive_gemm_signature_and_deep_copy_family(ctx, oracle):
    """Sapphire::Compute::Sparse::Naive::Gemm(output, a, b, m, n, numMatrices) with host
    arrays in and out, for two matrix pairs, and a round trip host -> device ->
    device -> host through the deep allocate / copy / free family
    (Includes/Sapphire/compute/sparse/Sparse.hpp)."""
    lib = L.lib()
    M = K = N = 700
    mats = [(W.csr_random(10 + i, M, K, 0.01), W.csr_random(20 + i, K, N, 0.01)) for i in range(2)]
    keep = []

    def host_array(which):
        arr = (L.Csr * 2)()
        for i, pair in enumerate(mats):
            r, c, v = (np.ascontiguousarray(x) for x in pair[which])
            keep.extend([r, c, v])
            arr[i].ROW, arr[i].COL, arr[i].V = r.ctypes.data, c.ctypes.data, v.ctypes.data
            arr[i].NNZ, arr[i].M, arr[i].N = c.size, M, (K if which == 0 else N)
        return arr

    hA, hB = host_array(0), host_array(1)
    out = C.POINTER(L.Csr)()
    assert lib.sb200_compat_sparse_naive_gemm(C.byref(out), hA, hB, M, N, 2) == L.OK
    for i, ((rA, cA, vA), (rB, cB, vB)) in enumerate(mats):
        orow, ocol, oval, _ = oracle.spgemm(rA, cA, vA, rB, cB, vB, M, N)
        m = out[i]
        assert (m.M, m.N, m.NNZ) == (M, N, ocol.size)
        as_np = lambda ptr, n, t: np.ctypeslib.as_array(C.cast(ptr, C.POINTER(t)), (n,))
        assert np.array_equal(as_np(m.ROW, M + 1, C.c_uint32), orow)
        assert np.array_equal(as_np(m.COL, m.NNZ, C.c_uint32), ocol)
        assert np.abs(as_np(m.V, m.NNZ, C.c_float) - oval).max() <= 1e-5 * max(np.abs(oval).max(), 1.0)
    assert lib.sb200_compat_deep_free_sparse_host(out, 2) == L.OK

    # deep copy round trip of hA
    d1, d2 = C.c_void_p(), C.c_void_p()
    assert lib.sb200_compat_deep_allocate_sparse_cuda(C.byref(d1), hA, 2, 0) == L.OK
    assert lib.sb200_compat_deep_allocate_sparse_cuda(C.byref(d2), hA, 2, 0) == L.OK
    assert lib.sb200_compat_deep_copy_host_to_device(d1, hA, 2, 0) == L.OK
    assert lib.sb200_compat_deep_copy_device_to_device(d2, d1, 2, 0) == L.OK
    back = C.POINTER(L.Csr)()
    nnz = (C.c_uint * 2)(hA[0].NNZ, hA[1].NNZ)
    assert lib.sb200_compat_deep_allocate_sparse_host(C.byref(back), M, K, nnz, 2) == L.OK
    assert lib.sb200_compat_deep_copy_device_to_host(back, d2, 2, 0) == L.OK
    again = C.POINTER(L.Csr)()
    assert lib.sb200_compat_deep_allocate_sparse_host(C.byref(again), M, K, nnz, 2) == L.OK
    assert lib.sb200_compat_deep_copy_host_to_host(again, back, 2) == L.OK
    for i, pair in enumerate(mats):
        r, c, v = pair[0]
        as_np = lambda ptr, n, t: np.ctypeslib.as_array(C.cast(ptr, C.POINTER(t)), (n,))
        assert np.array_equal(as_np(again[i].ROW, M + 1, C.c_uint32), r)
        assert np.array_equal(as_np(again[i].COL, c.size, C.c_uint32), c)
        assert np.array_equal(as_np(again[i].V, v.size, C.c_float), v)
    # a destination too small for the source is refused, not overrun
    small = (C.c_uint * 2)(1, 1)
    tiny = C.POINTER(L.Csr)()
    assert lib.sb200_compat_deep_allocate_sparse_host(C.byref(tiny), M, K, small, 2) == L.OK
    assert lib.sb200_compat_deep_copy_host_to_host(tiny, back, 2) != L.OK
    for h in (back, again, tiny):
        assert lib.sb200_compat_deep_free_sparse_host(h, 2) == L.OK
    assert lib.sb200_compat_deep_free_sparse_cuda(d1, 2, 0) == L.OK
    assert lib.sb200_compat_deep_free_sparse_cuda(d2, 2, 0) == L.OK


def test_sparse_workspace_lives_on_the_context_device(oracle):
    """A context of GPU 1 used while GPU 0 is current: the sparse work arrays must be
    allocated on the context's device (needs two GPUs)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx1 = ops.Context(1)
    torch.cuda.set_device(0)
    M = N = 512
    rA, cA, vA = W.csr_random(0, M, N, 0.02)
    rB, cB, vB = W.csr_random(1, N, N, 0.02)
    A = ops.CsrMatrix.from_numpy(rA, cA, vA, M, N, "cuda:1")
    B = ops.CsrMatrix.from_numpy(rB, cB, vB, N, N, "cuda:1")
    with torch.cuda.device(1):
        free_before = torch.cuda.mem_get_info(1)[0]
    with torch.cuda.device(0):
        free0_before = torch.cuda.mem_get_info(0)[0]
        torch.cuda.set_device(0)
        a, b = A.as_struct(), B.as_struct()
        row_c = torch.empty(M + 1, dtype=torch.int32, device="cuda:1")
        nnz = C.c_int64(0)
        st = torch.cuda.current_stream(torch.device("cuda:1")).cuda_stream
        assert L.lib().sb200_spgemm_csr_symbolic(ctx1.handle, C.byref(a), C.byref(b), row_c.data_ptr(),
                                                 C.byref(nnz), st) == L.OK
        free0_after = torch.cuda.mem_get_info(0)[0]
    orow, _, _, _ = oracle.spgemm(rA, cA, vA, rB, cB, vB, M, N)
    assert np.array_equal(row_c.cpu().numpy().view(np.uint32), orow)
    assert free0_after == free0_before                   # nothing was allocated on GPU 0
    torch.cuda.set_device(0)


def test_dense_csr_round_trip_and_product(ctx, oracle):
    """dense -> CSR -> dense is the identity (also with a padded row pitch), the
    CSR arrays equal numpy's, and CSR(A).CSR(B) densified equals the dense GEMM."""
    rng = np.random.default_rng(12)
    M, K, N = 96, 130, 75
    a = rng.standard_normal((M, K)).astype(np.float32) * (rng.random((M, K)) < 0.1)
    b = rng.standard_normal((K, N)).astype(np.float32) * (rng.random((K, N)) < 0.2)
    a[5] = 0.0                                                     # an empty row
    pitch = torch.zeros(M, K + 6, device=DEV)
    pitch[:, :K] = torch.from_numpy(a).to(DEV)
    A = ops.dense_to_csr(ctx, pitch[:, :K])
    r, c, v = A.to_numpy()
    want_r = np.concatenate([[0], np.cumsum((a != 0).sum(1))]).astype(np.uint32)
    rows, cols = np.nonzero(a)
    assert np.array_equal(r, want_r) and np.array_equal(c, cols.astype(np.uint32))
    assert np.array_equal(v, a[rows, cols])
    back = torch.full((M, K + 2), 7.0, device=DEV)
    ops.csr_to_dense(ctx, A, back[:, :K])
    assert np.array_equal(back[:, :K].cpu().numpy(), a)
    assert float(back[:, K:].min()) == 7.0                         # pitch padding untouched
    B = ops.dense_to_csr(ctx, torch.from_numpy(b).to(DEV))
    Cm = ops.spgemm(ctx, A, B)
    dense_c = ops.csr_to_dense(ctx, Cm).cpu().numpy()
    want = oracle.gemm(np.zeros((1, M, N), np.float32), a[None], b[None])[0]
    assert np.abs(dense_c - want).max() <= 1e-5 * max(np.abs(want).max(), 1.0)
