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


def plan(y, a, b):
    from sapphire_b200 import _lib as L
    arr = lambda s: (C.c_int * len(s))(*s)
    cap = 4096
    out = (C.c_longlong * (6 * cap))()
    n = L.lib().sb200_compat_plan_gemm(arr(y), len(y), arr(a), len(a), arr(b), len(b), out, cap)
    return [tuple(out[6 * i:6 * i + 6]) for i in range(min(n, cap))]


def apply_plan(calls, y, a, b, M, N, K):
    """Executes a plan with numpy on flat buffers (float64), y += a.b per call."""
    y = y.copy()
    for (oy, oa, ob, batch, sa, sb) in calls:
        for i in range(batch):
            A = a[oa + i * sa: oa + i * sa + M * K].reshape(M, K)
            B = b[ob + i * sb: ob + i * sb + K * N].reshape(K, N)
            y[oy + i * M * N: oy + (i + 1) * M * N] += (A @ B).reshape(-1)
    return y


# shape families of the reference's broadcast tests
# (Tests/UnitTests/Sources/FunctionTest/BroadcastTest.cpp:20-202) and GemmTest.cpp:20-84
@pytest.mark.parametrize("ys,as_,bs", [
    ([4, 6, 5], [4, 6, 3], [4, 3, 5]),                   # equal batch: one call
    ([3, 4, 4, 5], [3, 1, 4, 2], [3, 4, 2, 5]),          # [b,1,M,K].[b,M,K,N]
    ([4, 4, 5], [4, 2], [4, 2, 5]),                      # [M,K].[M,K,N]: missing dimension
    ([5, 4, 4, 5], [4, 2], [5, 4, 2, 5]),                # [M,K].[N,M,K,N]
    ([6, 5], [6, 3], [3, 5]),                            # plain 2-D
    ([2, 3, 6, 5], [2, 3, 6, 3], [1, 1, 3, 5]),          # shared B
])
def test_plan_matches_numpy_broadcast(ys, as_, bs):
    rng = np.random.default_rng(0)
    a = rng.standard_normal(as_)
    b = rng.standard_normal(bs)
    y0 = rng.standard_normal(ys)
    M, N, K = ys[-2], ys[-1], as_[-1]
    calls = plan(ys, as_, bs)
    got = apply_plan(calls, y0.reshape(-1), a.reshape(-1), b.reshape(-1), M, N, K).reshape(ys)
    want = y0 + np.matmul(a, b)
    assert np.allclose(got, want)


def test_plan_folds_equal_batches_into_one_call():
    calls = plan([4, 256, 256], [4, 256, 256], [4, 256, 256])
    assert calls == [(0, 0, 0, 4, 256 * 256, 256 * 256)]
    calls = plan([8, 16, 16], [16, 16], [8, 16, 16])          # shared A: stride 0, still one call
    assert calls == [(0, 0, 0, 8, 0, 256)]
