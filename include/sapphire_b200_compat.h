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

/* Sapphire::Compute::Sparse::Naive::Gemm
 * (Includes/Sapphire/compute/sparse/naive/SparseGemm.hpp:15-16): a and b are host
 * arrays of numMatrices structs holding HOST arrays; *output is a host array
 * allocated by the call (free it with sb200_compat_deep_free_sparse_host).  The
 * product itself runs on the current CUDA device; there is no CPU path. */
int sb200_compat_sparse_naive_gemm(sb200_csr** output, sb200_csr* a, sb200_csr* b, unsigned m,
                                   unsigned n, size_t numMatrices);

/* The deep allocate / free / copy family for arrays of sparse matrices
 * (Includes/Sapphire/compute/sparse/Sparse.hpp:20-25, 36, 49-51, 69-71, 92-94,
 * 119-121, 135-137, 149-150; declared there, defined nowhere in the reference).
 * "host array": numMatrices structs in host memory with host member arrays;
 * "device array": numMatrices structs in device memory with device member arrays. */
int sb200_compat_deep_allocate_sparse_host(sb200_csr** array, unsigned m, unsigned n,
                                           const unsigned* nnz, unsigned numMatrices);
int sb200_compat_deep_free_sparse_host(sb200_csr* array, unsigned numMatrices);
int sb200_compat_deep_allocate_sparse_cuda(sb200_csr** deviceArray, const sb200_csr* hostArray,
                                           unsigned numMatrices, int deviceId);
int sb200_compat_deep_free_sparse_cuda(sb200_csr* deviceArray, unsigned numMatrices, int deviceId);
int sb200_compat_deep_copy_host_to_device(sb200_csr* deviceDst, const sb200_csr* hostSrc,
                                          unsigned numMatrices, int deviceId);
int sb200_compat_deep_copy_device_to_host(sb200_csr* hostDst, sb200_csr* deviceSrc,
                                          unsigned numMatrices, int deviceId);
int sb200_compat_deep_copy_device_to_device(sb200_csr* deviceDst, sb200_csr* deviceSrc,
                                            unsigned numMatrices, int deviceId);
int sb200_compat_deep_copy_host_to_host(sb200_csr* hostDst, sb200_csr* hostSrc,
                                        unsigned numMatrices);

#ifdef __cplusplus
}
#endif
#endif /* SAPPHIRE_B200_COMPAT_H */
