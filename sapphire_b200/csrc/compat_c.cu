// Definitions of the Sapphire-signature shims declared in
// compat/sapphire_b200_compat.hpp, plus C hooks so the test harness can drive
// them through ctypes.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "sapphire_b200_compat.hpp"

namespace {

int g_mode = SB200_MODE_TF32;

[[noreturn]] void fail(const char* where, int status)
{
    throw std::runtime_error(std::string(where) + ": " + sb200_status_string(status));
}

void check(const char* where, int status)
{
    if (status != SB200_OK)
        fail(where, status);
}

}  // namespace

namespace sb200::compat {

void SetMode(int mode) { g_mode = mode; }
int GetMode() { return g_mode; }

sb200_ctx* ContextFor(int deviceId)
{
    // one context per (device, host thread), as the reference keeps one
    // cuBLAS handle per (device, thread) -- Sources/Sapphire/compute/dense/cuda/Gemm.cu:24-30
    thread_local std::map<int, sb200_ctx*> table;
    auto it = table.find(deviceId);
    if (it != table.end())
        return it->second;
    sb200_ctx* ctx = nullptr;
    check("sb200_ctx_create", sb200_ctx_create(deviceId, &ctx));
    table[deviceId] = ctx;
    return ctx;
}

namespace {

struct MatrixTriple {
    long long y, a, b;                                 // element offsets of one M x N product
};

// The reference's recursion (Includes/Sapphire/compute/Broadcast.hpp:82-133), offsets instead
// of pointers, unsigned arithmetic and all: runs of leading dimensions that are equal in
// y, a and b are folded into `chunk`; at the first dimension that differs, index c of
// max(chunkOut, chunkA, chunkB) addresses block (c % chunkX) of each tensor.  (After a
// folded run that modulo is not numpy's broadcast -- [3,4,M,N] = [3,1,M,K].[3,4,K,N] pairs
// y block c with a block c % 3, not c / 4 -- and the plan follows the reference, whose
// loop stays in Sapphire when only the leaf is replaced.)
void Walk(const std::vector<unsigned>& y, const std::vector<unsigned>& a, const std::vector<unsigned>& b,
          unsigned totalOut, unsigned totalA, unsigned totalB, long long oy, long long oa, long long ob,
          unsigned shapeIdx, unsigned matY, unsigned matA, unsigned matB, std::vector<MatrixTriple>& out)
{
    const unsigned dims = static_cast<unsigned>(y.size());
    auto leaf = [&]() {
        // Dense::Cuda::Gemm(totalSizeOut, ...): totalSizeOut / (M N) matrices, packed
        const unsigned n = matY ? totalOut / matY : 0;
        for (unsigned i = 0; i < n; ++i)
            out.push_back({oy + static_cast<long long>(i) * matY, oa + static_cast<long long>(i) * matA,
                           ob + static_cast<long long>(i) * matB});
    };
    if (shapeIdx >= dims - 2)
        return leaf();
    unsigned chunk = 1;
    while (shapeIdx < dims - 2 && y[shapeIdx] == a[shapeIdx] && y[shapeIdx] == b[shapeIdx]) {
        chunk *= y[shapeIdx];
        shapeIdx += 1;
    }
    if (shapeIdx >= dims - 2)
        return leaf();
    const unsigned chunkA = chunk * a[shapeIdx], chunkB = chunk * b[shapeIdx], chunkOut = chunk * y[shapeIdx];
    if (chunkA == 0 || chunkB == 0 || chunkOut == 0)
        return;
    const unsigned strideA = totalA / chunkA, strideB = totalB / chunkB, strideOut = totalOut / chunkOut;
    const unsigned maxChunk = std::max(chunkOut, std::max(chunkA, chunkB));
    for (unsigned c = 0; c < maxChunk; ++c)
        Walk(y, a, b, strideOut, strideA, strideB, oy + static_cast<long long>(c % chunkOut) * strideOut,
             oa + static_cast<long long>(c % chunkA) * strideA, ob + static_cast<long long>(c % chunkB) * strideB,
             shapeIdx + 1, matY, matA, matB, out);
}

}  // namespace

std::vector<LeafCall> PlanGemm(const std::vector<int>& yShape, const std::vector<int>& aShape,
                               const std::vector<int>& bShape)
{
    // Shape::Expand: right-aligned, left-padded with 1s (Sources/Sapphire/util/shape.cpp:138-158)
    auto expanded = [](const std::vector<int>& s, size_t dim) {
        std::vector<unsigned> out(dim, 1);
        for (size_t i = 0; i < s.size(); ++i)
            out[dim - s.size() + i] = static_cast<unsigned>(s[i]);
        return out;
    };
    const size_t dim = std::max(std::max(yShape.size(), aShape.size()), std::max(bShape.size(), static_cast<size_t>(2)));
    const auto y = expanded(yShape, dim), a = expanded(aShape, dim), b = expanded(bShape, dim);
    const unsigned M = y[dim - 2], N = y[dim - 1], K = a[dim - 1];
    auto size = [](const std::vector<unsigned>& s) {
        unsigned n = 1;
        for (unsigned v : s) n *= v;
        return n;
    };
    std::vector<MatrixTriple> seq;
    Walk(y, a, b, size(y), size(a), size(b), 0, 0, 0, 0, M * N, M * K, K * N, seq);

    // The reference makes one leaf call per index of the loop above.  Here every maximal
    // run of products whose y blocks are consecutive and whose a and b blocks advance by
    // a constant, non-negative step (0 = shared operand) becomes one strided-batched call;
    // the runs keep the reference's order, so a y block that is addressed twice
    // accumulates as it does there.
    std::vector<LeafCall> plan;
    const long long matY = static_cast<long long>(M) * N;
    size_t i = 0;
    while (i < seq.size()) {
        LeafCall c{seq[i].y, seq[i].a, seq[i].b, 1, 0, 0};
        if (i + 1 < seq.size() && seq[i + 1].y == seq[i].y + matY && seq[i + 1].a >= seq[i].a &&
            seq[i + 1].b >= seq[i].b) {
            c.strideA = seq[i + 1].a - seq[i].a;
            c.strideB = seq[i + 1].b - seq[i].b;
            size_t j = i + 1;
            while (j < seq.size() && seq[j].y == seq[j - 1].y + matY && seq[j].a == seq[j - 1].a + c.strideA &&
                   seq[j].b == seq[j - 1].b + c.strideB)
                ++j;
            c.batch = static_cast<long long>(j - i);
        }
        plan.push_back(c);
        i += static_cast<size_t>(c.batch);
    }
    return plan;
}

void Gemm(const std::vector<int>& yShape, float* y, const std::vector<int>& aShape,
          const float* a, const std::vector<int>& bShape, const float* b, int deviceId)
{
    auto dimAt = [](const std::vector<int>& s, int fromEnd) {
        return static_cast<int>(s.size()) >= fromEnd ? s[s.size() - fromEnd] : 1;
    };
    const long long M = dimAt(yShape, 2), N = dimAt(yShape, 1), K = dimAt(aShape, 1);
    sb200_ctx* ctx = ContextFor(deviceId);
    for (const LeafCall& c : PlanGemm(yShape, aShape, bShape)) {
        check("sb200_gemm_batched",
              sb200_gemm_batched(ctx, g_mode, SB200_PATH_AUTO, 0, 0, M, N, K, a + c.offA, K,
                                 c.strideA, b + c.offB, N, c.strideB, y + c.offY, N, M * N,
                                 y + c.offY, N, M * N, nullptr, nullptr, 0.0f, c.batch,
                                 cudaStreamPerThread));
    }
}

}  // namespace sb200::compat

namespace Sapphire::Compute::Dense::Cuda {

void Gemm(unsigned int totalSize, float* out, const float* A, const float* B, unsigned int M,
          unsigned int N, unsigned int K, int deviceId)
{
    const unsigned long long per = static_cast<unsigned long long>(M) * N;
    const long long batch = per ? totalSize / per : 0;
    sb200_ctx* ctx = sb200::compat::ContextFor(deviceId);
    check("Dense::Cuda::Gemm",
          sb200_gemm_batched(ctx, g_mode, SB200_PATH_AUTO, 0, 0, M, N, K, A, K,
                             static_cast<long long>(M) * K, B, N, static_cast<long long>(K) * N,
                             out, N, per, out, N, per, nullptr, nullptr, 0.0f, batch,
                             cudaStreamPerThread));
}

void GemmMatrixWiseBroadcast(float* out, const float* A, const float* B, unsigned int M,
                             unsigned int N, unsigned int K, unsigned int batchSize,
                             bool broadcastA, bool broadcastB, int deviceId)
{
    const long long per = static_cast<long long>(M) * N;
    sb200_ctx* ctx = sb200::compat::ContextFor(deviceId);
    check("Dense::Cuda::GemmMatrixWiseBroadcast",
          sb200_gemm_batched(ctx, g_mode, SB200_PATH_AUTO, 0, 0, M, N, K, A, K,
                             broadcastA ? 0 : static_cast<long long>(M) * K, B, N,
                             broadcastB ? 0 : static_cast<long long>(K) * N, out, N, per, out, N,
                             per, nullptr, nullptr, 0.0f, batchSize, cudaStreamPerThread));
}

}  // namespace Sapphire::Compute::Dense::Cuda

namespace Sapphire::Compute::Sparse::Cuda {

void Gemm(SparseMatrix** hostOutput, SparseMatrix** cudaOutput, SparseMatrix* cudaA,
          SparseMatrix* cudaB, uint32_t m, uint32_t n, size_t numMatrices, int deviceId,
          bool copyResultToHost)
{
    (void)m;
    (void)n;
    sb200_ctx* ctx = sb200::compat::ContextFor(deviceId);
    std::vector<sb200_csr> hA(numMatrices), hB(numMatrices), hC(numMatrices);
    auto cu = [](cudaError_t e, const char* what) {
        if (e != cudaSuccess)
            throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    };
    cu(cudaMemcpy(hA.data(), cudaA, numMatrices * sizeof(sb200_csr), cudaMemcpyDeviceToHost),
       "copy A descriptors");
    cu(cudaMemcpy(hB.data(), cudaB, numMatrices * sizeof(sb200_csr), cudaMemcpyDeviceToHost),
       "copy B descriptors");
    for (size_t i = 0; i < numMatrices; ++i)
        check("sb200_spgemm_csr", sb200_spgemm_csr(ctx, &hA[i], &hB[i], &hC[i], cudaStreamPerThread));
    cu(cudaStreamSynchronize(cudaStreamPerThread), "sync");
    if (cudaOutput) {
        void* d = nullptr;
        cu(cudaMalloc(&d, numMatrices * sizeof(sb200_csr)), "alloc C descriptors");
        cu(cudaMemcpy(d, hC.data(), numMatrices * sizeof(sb200_csr), cudaMemcpyHostToDevice),
           "copy C descriptors");
        *cudaOutput = static_cast<SparseMatrix*>(d);
    }
    if (copyResultToHost && hostOutput) {
        SparseMatrix* h = static_cast<SparseMatrix*>(malloc(numMatrices * sizeof(SparseMatrix)));
        for (size_t i = 0; i < numMatrices; ++i) {
            h[i] = hC[i];
            const size_t nnz = hC[i].NNZ;
            h[i].V = static_cast<float*>(malloc((nnz ? nnz : 1) * 4));
            h[i].COL = static_cast<uint32_t*>(malloc((nnz ? nnz : 1) * 4));
            h[i].ROW = static_cast<uint32_t*>(malloc((static_cast<size_t>(hC[i].M) + 1) * 4));
            cu(cudaMemcpy(h[i].V, hC[i].V, nnz * 4, cudaMemcpyDeviceToHost), "copy V");
            cu(cudaMemcpy(h[i].COL, hC[i].COL, nnz * 4, cudaMemcpyDeviceToHost), "copy COL");
            cu(cudaMemcpy(h[i].ROW, hC[i].ROW, (static_cast<size_t>(hC[i].M) + 1) * 4,
                          cudaMemcpyDeviceToHost), "copy ROW");
        }
        *hostOutput = h;
    }
}

}  // namespace Sapphire::Compute::Sparse::Cuda

// ------------------------------------------- deep allocate / free / copy family
namespace Sapphire::Compute {

namespace {

void cuda_check(cudaError_t e, const char* what)
{
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    }
}

// The structs of a device array, read back so that their member pointers can be used.
std::vector<SparseMatrix> fetch_descriptors(const SparseMatrix* deviceArray, uint32_t numMatrices)
{
    std::vector<SparseMatrix> h(numMatrices);
    if (numMatrices)
        cuda_check(cudaMemcpy(h.data(), deviceArray, numMatrices * sizeof(SparseMatrix),
                              cudaMemcpyDeviceToHost), "read sparse descriptors");
    return h;
}

void copy_members(SparseMatrix& dst, const SparseMatrix& src, cudaMemcpyKind kind)
{
    if (dst.M != src.M || dst.NNZ < src.NNZ)
        throw std::runtime_error("DeepCopy: destination matrix is smaller than the source");
    cuda_check(cudaMemcpy(dst.ROW, src.ROW, (static_cast<size_t>(src.M) + 1) * 4, kind), "copy ROW");
    if (src.NNZ) {
        cuda_check(cudaMemcpy(dst.COL, src.COL, static_cast<size_t>(src.NNZ) * 4, kind), "copy COL");
        cuda_check(cudaMemcpy(dst.V, src.V, static_cast<size_t>(src.NNZ) * 4, kind), "copy V");
    }
}

}  // namespace

void DeepAllocateSparseHost(SparseMatrix** sparseMatrixArray, uint32_t m, uint32_t n,
                            const uint32_t nnz[], uint32_t numMatrices)
{
    SparseMatrix* h = static_cast<SparseMatrix*>(calloc(numMatrices ? numMatrices : 1, sizeof(SparseMatrix)));
    if (!h)
        throw std::bad_alloc();
    for (uint32_t i = 0; i < numMatrices; ++i) {
        const size_t k = nnz[i] ? nnz[i] : 1;
        h[i].M = m;
        h[i].N = n;
        h[i].NNZ = nnz[i];
        h[i].V = static_cast<float*>(calloc(k, 4));
        h[i].COL = static_cast<uint32_t*>(calloc(k, 4));
        h[i].ROW = static_cast<uint32_t*>(calloc(static_cast<size_t>(m) + 1, 4));
        if (!h[i].V || !h[i].COL || !h[i].ROW) {
            DeepFreeSparseHost(h, i + 1);
            throw std::bad_alloc();
        }
    }
    *sparseMatrixArray = h;
}

void DeepFreeSparseHost(SparseMatrix* sparseMatrixArray, uint32_t numMatrices)
{
    if (!sparseMatrixArray)
        return;
    for (uint32_t i = 0; i < numMatrices; ++i) {
        free(sparseMatrixArray[i].V);
        free(sparseMatrixArray[i].COL);
        free(sparseMatrixArray[i].ROW);
    }
    free(sparseMatrixArray);
}

void DeepAllocateSparseCuda(SparseMatrix** deviceSparseArray, const SparseMatrix* hostSparseMatrixArray,
                            uint32_t numMatrices, int deviceId)
{
    cuda_check(cudaSetDevice(deviceId), "cudaSetDevice");
    std::vector<SparseMatrix> d(numMatrices);
    try {
        for (uint32_t i = 0; i < numMatrices; ++i) {
            d[i] = hostSparseMatrixArray[i];
            d[i].V = nullptr; d[i].COL = nullptr; d[i].ROW = nullptr;
            const size_t k = d[i].NNZ ? d[i].NNZ : 1;
            cuda_check(cudaMalloc(&d[i].V, k * 4), "alloc V");
            cuda_check(cudaMalloc(&d[i].COL, k * 4), "alloc COL");
            cuda_check(cudaMalloc(&d[i].ROW, (static_cast<size_t>(d[i].M) + 1) * 4), "alloc ROW");
        }
        void* arr = nullptr;
        cuda_check(cudaMalloc(&arr, (numMatrices ? numMatrices : 1) * sizeof(SparseMatrix)),
                   "alloc sparse descriptors");
        if (numMatrices)
            cuda_check(cudaMemcpy(arr, d.data(), numMatrices * sizeof(SparseMatrix), cudaMemcpyHostToDevice),
                       "write sparse descriptors");
        *deviceSparseArray = static_cast<SparseMatrix*>(arr);
    } catch (...) {
        for (auto& x : d)
            sb200_csr_free(&x);
        throw;
    }
}

void DeepFreeSparseCuda(SparseMatrix* deviceSparseArray, uint32_t numMatrices, int deviceId)
{
    if (!deviceSparseArray)
        return;
    cuda_check(cudaSetDevice(deviceId), "cudaSetDevice");
    auto d = fetch_descriptors(deviceSparseArray, numMatrices);
    for (auto& x : d)
        sb200_csr_free(&x);
    cudaFree(deviceSparseArray);
}

void DeepCopyDeviceToDevice(SparseMatrix* deviceDstArray, SparseMatrix* deviceSrcArray,
                            uint32_t numMatrices, int deviceId)
{
    cuda_check(cudaSetDevice(deviceId), "cudaSetDevice");
    auto dst = fetch_descriptors(deviceDstArray, numMatrices);
    const auto src = fetch_descriptors(deviceSrcArray, numMatrices);
    for (uint32_t i = 0; i < numMatrices; ++i) {
        copy_members(dst[i], src[i], cudaMemcpyDeviceToDevice);
        dst[i].NNZ = src[i].NNZ;
        dst[i].N = src[i].N;
    }
    if (numMatrices)
        cuda_check(cudaMemcpy(deviceDstArray, dst.data(), numMatrices * sizeof(SparseMatrix),
                              cudaMemcpyHostToDevice), "write sparse descriptors");
}

void DeepCopyHostToDevice(SparseMatrix* deviceDstArray, const SparseMatrix* hostSrcArray,
                          uint32_t numMatrices, int deviceId)
{
    cuda_check(cudaSetDevice(deviceId), "cudaSetDevice");
    auto dst = fetch_descriptors(deviceDstArray, numMatrices);
    for (uint32_t i = 0; i < numMatrices; ++i) {
        copy_members(dst[i], hostSrcArray[i], cudaMemcpyHostToDevice);
        dst[i].NNZ = hostSrcArray[i].NNZ;
        dst[i].N = hostSrcArray[i].N;
    }
    if (numMatrices)
        cuda_check(cudaMemcpy(deviceDstArray, dst.data(), numMatrices * sizeof(SparseMatrix),
                              cudaMemcpyHostToDevice), "write sparse descriptors");
}

void DeepCopyDeviceToHost(SparseMatrix* hostDstArray, SparseMatrix* deviceSrcArray,
                          uint32_t numMatrices, int deviceId)
{
    cuda_check(cudaSetDevice(deviceId), "cudaSetDevice");
    const auto src = fetch_descriptors(deviceSrcArray, numMatrices);
    for (uint32_t i = 0; i < numMatrices; ++i) {
        copy_members(hostDstArray[i], src[i], cudaMemcpyDeviceToHost);
        hostDstArray[i].NNZ = src[i].NNZ;
        hostDstArray[i].N = src[i].N;
    }
}

void DeepCopyHostToHost(SparseMatrix* hostDstArray, SparseMatrix* hostSrcArray, uint32_t numMatrices)
{
    for (uint32_t i = 0; i < numMatrices; ++i) {
        SparseMatrix& d = hostDstArray[i];
        const SparseMatrix& s = hostSrcArray[i];
        if (d.M != s.M || d.NNZ < s.NNZ)
            throw std::runtime_error("DeepCopyHostToHost: destination matrix is smaller than the source");
        std::copy(s.ROW, s.ROW + s.M + 1, d.ROW);
        std::copy(s.COL, s.COL + s.NNZ, d.COL);
        std::copy(s.V, s.V + s.NNZ, d.V);
        d.NNZ = s.NNZ;
        d.N = s.N;
    }
}

}  // namespace Sapphire::Compute

namespace Sapphire::Compute::Sparse::Naive {

void Gemm(SparseMatrix** output, SparseMatrix* a, SparseMatrix* b, uint32_t m, uint32_t n,
          size_t numMatrices)
{
    int deviceId = 0;
    if (cudaGetDevice(&deviceId) != cudaSuccess)
        throw std::runtime_error("Sparse::Naive::Gemm: no CUDA device (this build has no CPU path)");
    const uint32_t count = static_cast<uint32_t>(numMatrices);
    SparseMatrix *dA = nullptr, *dB = nullptr, *dC = nullptr;
    try {
        DeepAllocateSparseCuda(&dA, a, count, deviceId);
        DeepAllocateSparseCuda(&dB, b, count, deviceId);
        DeepCopyHostToDevice(dA, a, count, deviceId);
        DeepCopyHostToDevice(dB, b, count, deviceId);
        Cuda::Gemm(output, &dC, dA, dB, m, n, numMatrices, deviceId, true);
    } catch (...) {
        DeepFreeSparseCuda(dA, count, deviceId);
        DeepFreeSparseCuda(dB, count, deviceId);
        DeepFreeSparseCuda(dC, count, deviceId);
        throw;
    }
    DeepFreeSparseCuda(dA, count, deviceId);
    DeepFreeSparseCuda(dB, count, deviceId);
    DeepFreeSparseCuda(dC, count, deviceId);
}

}  // namespace Sapphire::Compute::Sparse::Naive

// ------------------------------------------------------------- C test hooks
// These forward to the C++ shims and turn exceptions back into status codes so
// that a ctypes caller can exercise the Sapphire-signature layer.
extern "C" {

int sb200_compat_set_mode(int mode)
{
    if (mode != SB200_MODE_TF32 && mode != SB200_MODE_TF32X3)
        return SB200_ERR_INVALID_ARG;
    sb200::compat::SetMode(mode);
    return SB200_OK;
}

// Sapphire::Compute::Dense::Cuda::Gemm
int sb200_compat_dense_gemm(unsigned totalSize, float* out, const float* A, const float* B,
                            unsigned M, unsigned N, unsigned K, int deviceId)
{
    try {
        Sapphire::Compute::Dense::Cuda::Gemm(totalSize, out, A, B, M, N, K, deviceId);
        return cudaStreamSynchronize(cudaStreamPerThread) == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
    } catch (const std::exception&) {
        return SB200_ERR_CUDA;
    }
}

// Sapphire::Compute::Dense::Cuda::GemmMatrixWiseBroadcast
int sb200_compat_dense_gemm_broadcast(float* out, const float* A, const float* B, unsigned M,
                                      unsigned N, unsigned K, unsigned batch, int bcA, int bcB,
                                      int deviceId)
{
    try {
        Sapphire::Compute::Dense::Cuda::GemmMatrixWiseBroadcast(out, A, B, M, N, K, batch,
                                                                bcA != 0, bcB != 0, deviceId);
        return cudaStreamSynchronize(cudaStreamPerThread) == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
    } catch (const std::exception&) {
        return SB200_ERR_CUDA;
    }
}

// The Compute::Gemm broadcast rules over raw shapes; runs on the device.
int sb200_compat_compute_gemm(const int* yShape, int yDim, float* y, const int* aShape, int aDim,
                              const float* a, const int* bShape, int bDim, const float* b,
                              int deviceId)
{
    try {
        sb200::compat::Gemm(std::vector<int>(yShape, yShape + yDim), y,
                            std::vector<int>(aShape, aShape + aDim), a,
                            std::vector<int>(bShape, bShape + bDim), b, deviceId);
        return cudaStreamSynchronize(cudaStreamPerThread) == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
    } catch (const std::exception&) {
        return SB200_ERR_CUDA;
    }
}

// The planner alone (no GPU needed): writes up to `cap` calls as 6 int64 each
// (offY, offA, offB, batch, strideA, strideB) and returns the number planned.
long long sb200_compat_plan_gemm(const int* yShape, int yDim, const int* aShape, int aDim,
                                 const int* bShape, int bDim, long long* out, long long cap)
{
    const auto plan = sb200::compat::PlanGemm(std::vector<int>(yShape, yShape + yDim),
                                              std::vector<int>(aShape, aShape + aDim),
                                              std::vector<int>(bShape, bShape + bDim));
    long long n = 0;
    for (const auto& c : plan) {
        if (n < cap) {
            long long* o = out + 6 * n;
            o[0] = c.offY; o[1] = c.offA; o[2] = c.offB;
            o[3] = c.batch; o[4] = c.strideA; o[5] = c.strideB;
        }
        ++n;
    }
    return n;
}

// Sapphire::Compute::Sparse::Cuda::Gemm for one matrix pair given as host
// structs with device arrays; returns the output the same way.
int sb200_compat_sparse_gemm(const sb200_csr* A, const sb200_csr* B, sb200_csr* C, int deviceId)
{
    try {
        void *dA = nullptr, *dB = nullptr;
        if (cudaSetDevice(deviceId) != cudaSuccess ||
            cudaMalloc(&dA, sizeof(sb200_csr)) != cudaSuccess ||
            cudaMalloc(&dB, sizeof(sb200_csr)) != cudaSuccess)
            return SB200_ERR_ALLOC;
        cudaMemcpy(dA, A, sizeof(sb200_csr), cudaMemcpyHostToDevice);
        cudaMemcpy(dB, B, sizeof(sb200_csr), cudaMemcpyHostToDevice);
        SparseMatrix* dC = nullptr;
        Sapphire::Compute::Sparse::Cuda::Gemm(nullptr, &dC, static_cast<SparseMatrix*>(dA),
                                              static_cast<SparseMatrix*>(dB), A->M, B->N, 1,
                                              deviceId, false);
        cudaMemcpy(C, dC, sizeof(sb200_csr), cudaMemcpyDeviceToHost);
        cudaFree(dA);
        cudaFree(dB);
        cudaFree(dC);
        return SB200_OK;
    } catch (const std::exception&) {
        return SB200_ERR_CUDA;
    }
}

// Sapphire::Compute::Sparse::Naive::Gemm: host arrays in, host array out
// (free the output with sb200_compat_deep_free_sparse_host).
int sb200_compat_sparse_naive_gemm(sb200_csr** output, sb200_csr* a, sb200_csr* b, unsigned m,
                                   unsigned n, size_t numMatrices)
{
    try {
        Sapphire::Compute::Sparse::Naive::Gemm(output, a, b, m, n, numMatrices);
        return SB200_OK;
    } catch (const std::exception&) {
        return SB200_ERR_CUDA;
    }
}

// The deep allocate / free / copy family, one hook per function.
#define SB200_COMPAT_GUARD(call)                 \
    try {                                        \
        call;                                    \
        return SB200_OK;                         \
    } catch (const std::bad_alloc&) {            \
        return SB200_ERR_ALLOC;                  \
    } catch (const std::exception&) {            \
        return SB200_ERR_CUDA;                   \
    }

int sb200_compat_deep_allocate_sparse_host(sb200_csr** array, unsigned m, unsigned n,
                                           const unsigned* nnz, unsigned numMatrices)
{
    SB200_COMPAT_GUARD(Sapphire::Compute::DeepAllocateSparseHost(array, m, n, nnz, numMatrices))
}

int sb200_compat_deep_free_sparse_host(sb200_csr* array, unsigned numMatrices)
{
    SB200_COMPAT_GUARD(Sapphire::Compute::DeepFreeSparseHost(array, numMatrices))
}

int sb200_compat_deep_allocate_sparse_cuda(sb200_csr** deviceArray, const sb200_csr* hostArray,
                                           unsigned numMatrices, int deviceId)
{
    SB200_COMPAT_GUARD(Sapphire::Compute::DeepAllocateSparseCuda(deviceArray, hostArray, numMatrices, deviceId))
}

int sb200_compat_deep_free_sparse_cuda(sb200_csr* deviceArray, unsigned numMatrices, int deviceId)
{
    SB200_COMPAT_GUARD(Sapphire::Compute::DeepFreeSparseCuda(deviceArray, numMatrices, deviceId))
}

int sb200_compat_deep_copy_host_to_device(sb200_csr* deviceDst, const sb200_csr* hostSrc,
                                          unsigned numMatrices, int deviceId)
{
    SB200_COMPAT_GUARD(Sapphire::Compute::DeepCopyHostToDevice(deviceDst, hostSrc, numMatrices, deviceId))
}

int sb200_compat_deep_copy_device_to_host(sb200_csr* hostDst, sb200_csr* deviceSrc,
                                          unsigned numMatrices, int deviceId)
{
    SB200_COMPAT_GUARD(Sapphire::Compute::DeepCopyDeviceToHost(hostDst, deviceSrc, numMatrices, deviceId))
}

int sb200_compat_deep_copy_device_to_device(sb200_csr* deviceDst, sb200_csr* deviceSrc,
                                            unsigned numMatrices, int deviceId)
{
    SB200_COMPAT_GUARD(Sapphire::Compute::DeepCopyDeviceToDevice(deviceDst, deviceSrc, numMatrices, deviceId))
}

int sb200_compat_deep_copy_host_to_host(sb200_csr* hostDst, sb200_csr* hostSrc, unsigned numMatrices)
{
    SB200_COMPAT_GUARD(Sapphire::Compute::DeepCopyHostToHost(hostDst, hostSrc, numMatrices))
}

}  // extern "C"
