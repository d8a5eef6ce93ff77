"""ctypes binding of libsapphire_b200.so.

The library is the product: there is no Python or CPU fallback.  If it has not
been built (``python -m sapphire_b200.build``) loading fails with an error.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsapphire_b200.so")

OK = 0
ERR_INVALID_ARG, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE_TIMEOUT, ERR_ALLOC, ERR_TOO_LARGE = range(1, 7)
MODE_TF32, MODE_TF32X3 = 0, 1
PATH_AUTO, PATH_TCGEN05, PATH_SIMT = 0, 1, 2
OPT_SPLIT_EXPLICIT_HI = 1
OPT_MERGE_MN_BOXES = 2
OPT_CTA_PAIRS = 3
OPT_SPLIT_TAIL_WAVE = 4
OPT_WAIT_LIMIT_US = 5
OPT_TEST_STALL_KBLOCKS = 6
OPT_SPGEMM_FAST_MID = 7
OPT_K_SLICES = 8
OPT_SPLIT_A_TMEM = 9
COUNTER_LAUNCHES, COUNTER_TENSOR_MAP_HITS, COUNTER_TENSOR_MAP_MISSES = 0, 1, 2


class Csr(C.Structure):
    """Mirror of sb200_csr (48 bytes)."""
    _fields_ = [("V", C.c_void_p), ("COL", C.c_void_p), ("ROW", C.c_void_p),
                ("NNZ", C.c_uint32), ("M", C.c_uint32), ("N", C.c_uint32),
                ("Padding", C.c_uint32 * 3)]


class GemmEpilogue(C.Structure):
    """Mirror of sb200_gemm_epilogue."""
    _fields_ = [("bias", C.c_void_p), ("colsum_out", C.c_void_p), ("colsum_scale", C.c_float),
                ("relu", C.c_int), ("relu_gate", C.c_void_p), ("ld_gate", C.c_int64),
                ("stride_gate", C.c_int64), ("sgd_lr", C.c_float)]


class ConvGeometry(C.Structure):
    """Mirror of sb200_conv_geometry."""
    _fields_ = [(n, C.c_int) for n in ("N", "C", "H", "W", "kh", "kw", "strideR", "strideC",
                                       "padR", "padC", "dilR", "dilC")]


class DpGroup(C.Structure):
    """Mirror of sb200_dp_group."""
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("grads", C.c_void_p * 8),
                ("reduced", C.c_void_p * 8), ("flags", C.c_void_p * 8)]


DP_FLAG_WORDS = 32


class Sb200Error(RuntimeError):
    def __init__(self, where: str, status: int):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} (status {status})")


_lib = None

# name -> (restype, argtypes); every symbol the public headers declare
SIGNATURES = {
    "sb200_ctx_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "sb200_ctx_destroy": (C.c_int, [C.c_void_p]),
    "sb200_status_string": (C.c_char_p, [C.c_int]),
    "sb200_last_path": (C.c_int, [C.c_void_p]),
    "sb200_launch_count": (C.c_int64, [C.c_void_p]),
    "sb200_ctx_counter": (C.c_int64, [C.c_void_p, C.c_int]),
    "sb200_ctx_set_option": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "sb200_check_device_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "sb200_gemm_batched": (C.c_int, [
        C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
        C.c_int64, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int64, C.c_int64,
        C.c_void_p, C.c_void_p, C.c_float,
        C.c_int64, C.c_void_p]),
    "sb200_gemm_batched_ex": (C.c_int, [
        C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
        C.c_int64, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int64, C.c_int64,
        C.POINTER(GemmEpilogue),
        C.c_int64, C.c_void_p]),
    "sb200_gemm_reduce_scatter": (C.c_int, [
        C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
        C.POINTER(C.c_void_p), C.c_int, C.c_int64, C.c_void_p, C.c_float, C.c_void_p]),
    "sb200_gemm_scatter": (C.c_int, [
        C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
        C.POINTER(C.c_void_p), C.c_int, C.c_int64, C.c_void_p, C.c_float, C.c_void_p]),
    "sb200_sum_blocks": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int64,
                                   C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "sb200_peer_barrier": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p]),
    "sb200_dp_reduce": (C.c_int, [C.c_void_p, C.POINTER(DpGroup), C.c_int64, C.c_void_p]),
    "sb200_dp_update": (C.c_int, [C.c_void_p, C.POINTER(DpGroup), C.c_void_p, C.c_int64, C.c_int64,
                                  C.c_float, C.c_void_p]),
    "sb200_peer_alloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]),
    "sb200_peer_open": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]),
    "sb200_peer_close": (C.c_int, [C.c_void_p, C.c_void_p]),
    "sb200_peer_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "sb200_spgemm_csr": (C.c_int, [C.c_void_p, C.POINTER(Csr), C.POINTER(Csr), C.POINTER(Csr),
                                   C.c_void_p]),
    "sb200_spgemm_csr_symbolic": (C.c_int, [C.c_void_p, C.POINTER(Csr), C.POINTER(Csr), C.c_void_p,
                                            C.POINTER(C.c_int64), C.c_void_p]),
    "sb200_spgemm_csr_numeric": (C.c_int, [C.c_void_p, C.POINTER(Csr), C.POINTER(Csr), C.c_void_p,
                                           C.c_void_p, C.c_void_p, C.c_void_p]),
    "sb200_csr_free": (C.c_int, [C.POINTER(Csr)]),
    "sb200_csr_copy_out": (C.c_int, [C.POINTER(Csr), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                     C.c_void_p]),
    "sb200_dense_to_csr": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_int64,
                                     C.POINTER(Csr), C.c_void_p]),
    "sb200_csr_to_dense": (C.c_int, [C.c_void_p, C.POINTER(Csr), C.c_void_p, C.c_int64, C.c_void_p]),
    "sb200_colsum_noalloc": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64,
                                       C.c_void_p, C.c_float, C.c_void_p]),
    "sb200_relu": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "sb200_relu_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                      C.c_void_p]),
    "sb200_softmax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "sb200_softmax_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                         C.c_int, C.c_void_p]),
    "sb200_cross_entropy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                      C.c_int, C.c_void_p]),
    "sb200_cross_entropy_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                               C.c_int, C.c_int, C.c_void_p]),
    "sb200_im2col": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(ConvGeometry), C.c_float,
                               C.c_void_p]),
    "sb200_col2im": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(ConvGeometry),
                               C.c_void_p]),
    "sb200_softmax_cross_entropy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_int64, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                              C.c_void_p]),
    "sb200_sgd_update": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int64,
                                   C.c_void_p]),
    "sb200_scale": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int64, C.c_void_p]),
    # Sapphire-signature shims (include/sapphire_b200_compat.h)
    "sb200_compat_set_mode": (C.c_int, [C.c_int]),
    "sb200_compat_dense_gemm": (C.c_int, [C.c_uint, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_uint, C.c_uint, C.c_uint, C.c_int]),
    "sb200_compat_dense_gemm_broadcast": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint,
                                                    C.c_uint, C.c_uint, C.c_uint, C.c_int, C.c_int,
                                                    C.c_int]),
    "sb200_compat_compute_gemm": (C.c_int, [C.POINTER(C.c_int), C.c_int, C.c_void_p,
                                            C.POINTER(C.c_int), C.c_int, C.c_void_p,
                                            C.POINTER(C.c_int), C.c_int, C.c_void_p, C.c_int]),
    "sb200_compat_plan_gemm": (C.c_longlong, [C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int),
                                              C.c_int, C.POINTER(C.c_int), C.c_int,
                                              C.POINTER(C.c_longlong), C.c_longlong]),
    "sb200_compat_sparse_gemm": (C.c_int, [C.POINTER(Csr), C.POINTER(Csr), C.POINTER(Csr), C.c_int]),
    "sb200_compat_sparse_naive_gemm": (C.c_int, [C.POINTER(C.POINTER(Csr)), C.POINTER(Csr),
                                                 C.POINTER(Csr), C.c_uint, C.c_uint, C.c_size_t]),
    "sb200_compat_deep_allocate_sparse_host": (C.c_int, [C.POINTER(C.POINTER(Csr)), C.c_uint, C.c_uint,
                                                         C.POINTER(C.c_uint), C.c_uint]),
    "sb200_compat_deep_free_sparse_host": (C.c_int, [C.POINTER(Csr), C.c_uint]),
    "sb200_compat_deep_allocate_sparse_cuda": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(Csr),
                                                         C.c_uint, C.c_int]),
    "sb200_compat_deep_free_sparse_cuda": (C.c_int, [C.c_void_p, C.c_uint, C.c_int]),
    "sb200_compat_deep_copy_host_to_device": (C.c_int, [C.c_void_p, C.POINTER(Csr), C.c_uint, C.c_int]),
    "sb200_compat_deep_copy_device_to_host": (C.c_int, [C.POINTER(Csr), C.c_void_p, C.c_uint, C.c_int]),
    "sb200_compat_deep_copy_device_to_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint, C.c_int]),
    "sb200_compat_deep_copy_host_to_host": (C.c_int, [C.POINTER(Csr), C.POINTER(Csr), C.c_uint]),
}


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m sapphire_b200.build` "
                "(there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().sb200_status_string(status).decode()


def check(where: str, status: int) -> None:
    if status != OK:
        raise Sb200Error(where, status)
