"""CPU tests of the boundary: the library loads, exports every symbol the
public headers declare, reports errors as status codes, and the host-side
broadcast planner reproduces Compute::Gemm's batch rules."""
import ctypes as C
import glob
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for h in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names += re.findall(r"\b(sb200_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    from sapphire_b200 import _lib as L
    handle = C.CDLL(L.LIB_PATH)
    decl = declared_symbols()
    assert len(decl) >= 15
    for name in decl:
        assert hasattr(handle, name), f"{name} declared in include/ but not exported"
    # and the ctypes table binds exactly the declared set
    assert sorted(L.SIGNATURES) == decl


def test_python_constants_equal_the_header_enumerators():
    """Every SB200_* enumerator of the public header has a constant of the same value
    in the ctypes table (named without the prefix), so an option or status added to
    one side cannot drift from the other."""
    from sapphire_b200 import _lib as L
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "sapphire_b200.h")).read(),
                  flags=re.S)
    enums = dict(re.findall(r"\bSB200_([A-Z0-9_]+)\s*=\s*(-?\d+)", text))
    assert len(enums) >= 20
    for name, value in enums.items():
        assert hasattr(L, name), f"SB200_{name} has no Python constant"
        assert getattr(L, name) == int(value), name


def test_status_strings():
    from sapphire_b200 import _lib as L
    assert L.status_string(L.OK) == "ok"
    seen = {L.status_string(i) for i in range(7)}
    assert len(seen) == 7
    assert "unknown" in L.status_string(99)


def test_csr_struct_is_48_bytes():
    from sapphire_b200 import _lib as L
    assert C.sizeof(L.Csr) == 48          # Sapphire's SparseMatrix is padded to 48 bytes


def test_no_device_is_an_error_not_a_fallback():
    """Without a GPU the product refuses to run; nothing routes to the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from sapphire_b200 import _lib as L
    from sapphire_b200 import ops
    h = C.c_void_p()
    assert L.lib().sb200_ctx_create(0, C.byref(h)) != L.OK
    with pytest.raises(RuntimeError):
        ops.Context(0)


def test_null_arguments_rejected():
    from sapphire_b200 import _lib as L
    lib = L.lib()
    assert lib.sb200_ctx_create(0, None) == L.ERR_INVALID_ARG
    assert lib.sb200_ctx_destroy(None) == L.ERR_INVALID_ARG
    assert lib.sb200_gemm_batched(None, 0, 0, 0, 0, 1, 1, 1, None, 1, 0, None, 1, 0, None, 1, 0,
                                  None, 1, 0, None, None, 0.0, 1, None) == L.ERR_INVALID_ARG
    assert lib.sb200_csr_free(None) == L.ERR_INVALID_ARG
    # the multi-GPU entry points check their arguments before they touch a device
    for fn in (lib.sb200_gemm_reduce_scatter, lib.sb200_gemm_scatter):
        assert fn(None, 0, 0, 0, 128, 4, 4, None, 4, None, 4, None, 1, 4, None, 0.0, None) == L.ERR_INVALID_ARG
    assert lib.sb200_sum_blocks(None, None, 4, None, 1, 0, 1, 4, 4, None) == L.ERR_INVALID_ARG
    assert lib.sb200_peer_barrier(None, None, 1, 0, None) == L.ERR_INVALID_ARG


def plan(y, a, b):
    from sapphire_b200 import _lib as L
    arr = lambda s: (C.c_int * len(s))(*s)
    cap = 4096
    out = (C.c_longlong * (6 * cap))()
    n = L.lib().sb200_compat_plan_gemm(arr(y), len(y), arr(a), len(a), arr(b), len(b), out, cap)
    return [tuple(out[6 * i:6 * i + 6]) for i in range(min(n, cap))]


def _golden_module():
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(ROOT, "tests", "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _run_plan_with_cpu_gemm(idx):
    """The plan's leaf calls executed with the reference's CPU GEMM arithmetic."""
    from oracle import oracle as O
    mod = _golden_module()
    ys, as_, bs = mod.BROADCAST_CASES[idx]
    y0, a, b = mod.broadcast_case(idx)
    M, N, K = ys[-2], ys[-1], as_[-1]
    got = y0.reshape(-1).copy()
    af, bf = a.reshape(-1), b.reshape(-1)
    for (oy, oa, ob, batch, sa, sb) in plan(ys, as_, bs):
        for i in range(batch):
            A = af[oa + i * sa: oa + i * sa + M * K].reshape(1, M, K)
            B = bf[ob + i * sb: ob + i * sb + K * N].reshape(1, K, N)
            seg = slice(oy + i * M * N, oy + (i + 1) * M * N)
            got[seg] = O.gemm(got[seg].reshape(1, M, N), A, B).reshape(-1)
    return got.reshape(ys), (y0, a, b)


@pytest.mark.parametrize("idx", range(11))
def test_plan_equals_the_reference_broadcast(idx):
    """The planner of the Sapphire-signature shims against the reference's own
    Compute::Gemm host path (shape expansion, BroadcastWith2Inputs, CPU GEMM: fixtures
    written by the reference build, and that build itself where it is present): the
    plan's leaf calls give the reference's result bit for bit -- also for
    [3,4,M,N] = [3,1,M,K].[3,4,K,N], where the reference pairs y block c with a block
    c % 3 and numpy's broadcast would pair it with c / 4."""
    from oracle import oracle as O
    gold = np.load(os.path.join(ROOT, "tests", "golden", "compute_units_golden.npz"))
    got, (y0, a, b) = _run_plan_with_cpu_gemm(idx)
    assert np.array_equal(got.view(np.uint32), gold[f"case{idx}"].view(np.uint32))
    if O.have_ref_ops():
        assert np.array_equal(got.view(np.uint32), O.ref_compute_gemm(y0, a, b).view(np.uint32))
    if idx not in (1, 8):                                # every other family is numpy's broadcast too
        want = y0.astype(np.float64) + np.matmul(a.astype(np.float64), b.astype(np.float64))
        assert np.allclose(got, want, rtol=1e-4, atol=1e-4)


def test_plan_folds_equal_batches_into_one_call():
    calls = plan([4, 256, 256], [4, 256, 256], [4, 256, 256])
    assert calls == [(0, 0, 0, 4, 256 * 256, 256 * 256)]
    calls = plan([8, 16, 16], [16, 16], [8, 16, 16])          # shared A: stride 0, still one call
    assert calls == [(0, 0, 0, 8, 0, 256)]
