/*
 * sapphire_b200_compat.h -- C hooks onto the Sapphire-signature C++ shims
 * (sapphire_b200/compat/sapphire_b200_compat.hpp), so that a harness without a
 * C++ compiler (ctypes) can call the exact functions a Sapphire build would
 * link.  Each hook forwards to the shim, synchronises the per-thread stream
 * and returns a status code instead of throwing.
 */
#ifndef SAPPHIRE_B200_COMPAT_H
#define SAPPHIRE_B200_COMPAT_H

#include "sapphire_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Arithmetic mode the shims pass down (SB200_MODE_TF32 by default: the
 * reference's cublasSetMathMode(CUBLAS_TF32_TENSOR_OP_MATH),
 * Sources/Sapphire/compute/dense/cuda/Gemm.cu:31). */
int sb200_compat_set_mode(int mode);

/* Sapphire::Compute::Dense::Cuda::Gemm
 * (Includes/Sapphire/compute/dense/cuda/Gemm.cuh:15-18): out += A.B for
 * totalSize / (M*N) dense row-major batches. */
int sb200_compat_dense_gemm(unsigned totalSize, float* out, const float* A, const float* B,
                            unsigned M, unsigned N, unsigned K, int deviceId);

/* Sapphire::Compute::Dense::Cuda::GemmMatrixWiseBroadcast (Gemm.cuh:20-25). */
int sb200_compat_dense_gemm_broadcast(float* out, const float* A, const float* B, unsigned M,
                                      unsigned N, unsigned K, unsigned batch, int broadcastA,
                                      int broadcastB, int deviceId);

/* The batch / broadcast rules of Sapphire::Compute::Gemm over raw shapes
 * (Sources/Sapphire/compute/BasicOps.cpp:183-248,
 *  Includes/Sapphire/compute/Broadcast.hpp:82-133): y <- y + a.b, device pointers. */
int sb200_compat_compute_gemm(const int* yShape, int yDim, float* y, const int* aShape, int aDim,
                              const float* a, const int* bShape, int bDim, const float* b,
                              int deviceId);

/* The planner behind sb200_compat_compute_gemm, host only: writes up to cap
 * leaf calls as 6 int64 each (offY, offA, offB, batch, strideA, strideB) and
 * returns how many the shapes need. */
long long sb200_compat_plan_gemm(const int* yShape, int yDim, const int* aShape, int aDim,
                                 const int* bShape, int bDim, long long* out, long long cap);

/* Sapphire::Compute::Sparse::Cuda::Gemm
 * (Includes/Sapphire/compute/sparse/cuda/SparseGemm.cuh:38-41) for one matrix
 * pair given as host structs holding device arrays. */
int sb200_compat_sparse_gemm(const sb200_csr* A, const sb200_csr* B, sb200_csr* C, int deviceId);

#ifdef __cplusplus
}
#endif
#endif /* SAPPHIRE_B200_COMPAT_H */
