// Source-compatible shims: Sapphire's own leaf signatures, implemented on the
// sapphire_b200 C ABI.  A Sapphire build drops its cuBLAS wrapper
// (Sources/Sapphire/compute/dense/cuda/Gemm.cu) and links these definitions
// instead; everything above the leaf (Compute::Gemm, the Linear unit) is
// untouched.  Errors from the C ABI become std::runtime_error, like the
// reference's CHECK_CUBLAS (Includes/Sapphire/compute/cudaUtil/CudaParams.cuh:51-58).
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

#include "../../include/sapphire_b200.h"

// Sapphire's CSR struct (Includes/Sapphire/compute/sparse/SparseMatrix.hpp:28-38) has the
// same members in the same order as sb200_csr; when Sapphire's header is not
// in the include path the ABI struct stands in for it.
#ifndef Sapphire_SPARSEMATRIX_HPP
typedef sb200_csr SparseMatrix;
#endif

namespace Sapphire::Compute::Dense::Cuda
{
// Includes/Sapphire/compute/dense/cuda/Gemm.cuh:15-18 -- out += A.B for
// totalSize / (M*N) batches, dense row-major, on device `deviceId`.
void Gemm(unsigned int totalSize, float* out, const float* A, const float* B,
          unsigned int M, unsigned int N, unsigned int K, int deviceId);

// Includes/Sapphire/compute/dense/cuda/Gemm.cuh:20-25 -- the same with one
// operand shared by every batch.
void GemmMatrixWiseBroadcast(float* out, const float* A, const float* B,
                             unsigned int M, unsigned int N, unsigned int K,
                             unsigned int batchSize, bool broadcastA,
                             bool broadcastB, int deviceId);
}  // namespace Sapphire::Compute::Dense::Cuda

namespace Sapphire::Compute::Sparse::Cuda
{
// Includes/Sapphire/compute/sparse/cuda/SparseGemm.cuh:38-41 -- cudaA / cudaB
// are device arrays of numMatrices structs whose V/COL/ROW are device arrays;
// the outputs (a device array of structs, and a host deep copy when
// copyResultToHost) are allocated here and owned by the caller.
void Gemm(SparseMatrix** hostOutput, SparseMatrix** cudaOutput,
          SparseMatrix* cudaA, SparseMatrix* cudaB, uint32_t m, uint32_t n,
          size_t numMatrices, int deviceId, bool copyResultToHost);
}  // namespace Sapphire::Compute::Sparse::Cuda

namespace Sapphire::Compute::Sparse::Naive
{
// Includes/Sapphire/compute/sparse/naive/SparseGemm.hpp:15-16 -- a / b are HOST
// arrays of numMatrices structs whose V/COL/ROW are host arrays; *output is
// allocated here (DeepAllocateSparseHost layout, freed with DeepFreeSparseHost).
// The reference declares this entry point without defining it.  Here it is the
// device path behind the host signature: operands are deep-copied to the
// current device, multiplied by Sparse::Cuda::Gemm and the result is deep-copied
// back; there is no CPU implementation behind it.
void Gemm(SparseMatrix** output, SparseMatrix* a, SparseMatrix* b, uint32_t m,
          uint32_t n, size_t numMatrices);
}  // namespace Sapphire::Compute::Sparse::Naive

namespace Sapphire::Compute
{
// The deep allocate / free / copy family of
// Includes/Sapphire/compute/sparse/Sparse.hpp:20-152 for SparseMatrix arrays
// (declared there without definitions; the LoadDistMatrix overloads belong to
// the reference's unfinished load-balancing scheme and are not provided).
// A "host array" is numMatrices structs in host memory whose V / COL / ROW are
// host arrays of NNZ / NNZ / M + 1 entries; a "device array" is numMatrices
// structs in device memory whose members are device arrays.
void DeepAllocateSparseHost(SparseMatrix** sparseMatrixArray, uint32_t m, uint32_t n,
                            const uint32_t nnz[], uint32_t numMatrices);
void DeepFreeSparseHost(SparseMatrix* sparseMatrixArray, uint32_t numMatrices);
// Sized after hostSparseMatrixArray (M, N, NNZ of each matrix); values are not copied.
void DeepAllocateSparseCuda(SparseMatrix** deviceSparseArray,
                            const SparseMatrix* hostSparseMatrixArray, uint32_t numMatrices,
                            int deviceId);
void DeepFreeSparseCuda(SparseMatrix* deviceSparseArray, uint32_t numMatrices, int deviceId);
void DeepCopyDeviceToDevice(SparseMatrix* deviceDstArray, SparseMatrix* deviceSrcArray,
                            uint32_t numMatrices, int deviceId);
void DeepCopyHostToDevice(SparseMatrix* deviceDstArray, const SparseMatrix* hostSrcArray,
                          uint32_t numMatrices, int deviceId);
void DeepCopyDeviceToHost(SparseMatrix* hostDstArray, SparseMatrix* deviceSrcArray,
                          uint32_t numMatrices, int deviceId);
void DeepCopyHostToHost(SparseMatrix* hostDstArray, SparseMatrix* hostSrcArray,
                        uint32_t numMatrices);
}  // namespace Sapphire::Compute

namespace sb200::compat
{
// Arithmetic mode used by the shims (process-wide; default SB200_MODE_TF32,
// what the reference asks of cuBLAS).
void SetMode(int mode);
int GetMode();

// Per (device, host thread) context, created on first use.
sb200_ctx* ContextFor(int deviceId);

// One strided-batched leaf call of a broadcast plan; offsets in elements.
struct LeafCall {
    long long offY, offA, offB;
    long long batch, strideA, strideB;
};

// Host-side planner that reproduces the batch/broadcast rules of
// Compute::Gemm (Sources/Sapphire/compute/BasicOps.cpp:183-248 with
// Includes/Sapphire/compute/Broadcast.hpp:82-133) by walking the reference's
// recursion with offsets in place of pointers: shapes are right-aligned and
// left-padded with 1s, the last two dimensions are the matrix, leading
// dimensions equal in all three tensors are folded, and at the first one that
// differs block c of the loop addresses block (c % extent) of each tensor --
// the reference's rule, also where it is not numpy's broadcast.  Instead of one
// leaf call per index it emits one strided call per run of consecutive y
// blocks whose operand blocks advance by a constant step (0 for a shared one).
std::vector<LeafCall> PlanGemm(const std::vector<int>& yShape, const std::vector<int>& aShape,
                               const std::vector<int>& bShape);

// y <- y + a.b over the planned calls (device pointers).
void Gemm(const std::vector<int>& yShape, float* y, const std::vector<int>& aShape,
          const float* a, const std::vector<int>& bShape, const float* b, int deviceId);
}  // namespace sb200::compat
