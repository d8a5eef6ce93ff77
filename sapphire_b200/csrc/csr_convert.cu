// Dense <-> CSR conversion on the device: the on-ramp for using the sparse
// GEMM from dense tensors.  The reference declares these conversions
// (Includes/Sapphire/compute/sparse/Sparse.hpp:154-162,
// CreateSparseMatrixWithDenseMatrix / ConvertSparseMatrixToDenseMatrix, with a
// padded row pitch `paddedN`) and ships no definition; an entry is "nonzero"
// when its value is not exactly 0.0f, columns come out ascending.
#include "common.cuh"

namespace sb200 {
namespace {

// one warp per row: count entries != 0
__global__ void __launch_bounds__(256)
dense_count_kernel(const float* __restrict__ dense, uint32_t M, uint32_t N, int64_t ld,
                   uint32_t* __restrict__ cnt)
{
    const int lane = threadIdx.x & 31;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t i = warp; i < M; i += nwarps) {
        const float* row = dense + static_cast<int64_t>(i) * ld;
        uint32_t c = 0;
        for (uint32_t j = lane; j < N; j += 32) c += row[j] != 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        if (lane == 0) cnt[i] = c;
    }
}

// rowptr[0] = 0, rowptr[i+1] = sum cnt[0..i]; one CTA
__global__ void __launch_bounds__(1024)
count_scan_kernel(const uint32_t* __restrict__ cnt, uint32_t M, uint32_t* __restrict__ rowptr,
                  unsigned long long* __restrict__ total_out)
{
    __shared__ unsigned long long s_warp[32];
    __shared__ unsigned long long s_carry;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        s_carry = 0;
        rowptr[0] = 0;
    }
    __syncthreads();
    for (uint32_t base = 0; base < M; base += 1024) {
        const uint32_t i = base + threadIdx.x;
        unsigned long long v = i < M ? cnt[i] : 0, incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        unsigned long long off = s_carry;
        for (int x = 0; x < warp; ++x) off += s_warp[x];
        if (i < M) rowptr[i + 1] = static_cast<uint32_t>(off + incl);
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = off + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) *total_out = s_carry;
}

// one warp per row: ballot compaction keeps the columns ascending
__global__ void __launch_bounds__(256)
dense_fill_kernel(const float* __restrict__ dense, uint32_t M, uint32_t N, int64_t ld,
                  const uint32_t* __restrict__ rowptr, uint32_t* __restrict__ col,
                  float* __restrict__ val)
{
    const int lane = threadIdx.x & 31;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t i = warp; i < M; i += nwarps) {
        const float* row = dense + static_cast<int64_t>(i) * ld;
        uint32_t out = rowptr[i];
        for (uint32_t j0 = 0; j0 < N; j0 += 32) {
            const uint32_t j = j0 + lane;
            const float v = j < N ? row[j] : 0.0f;
            const uint32_t mask = __ballot_sync(0xffffffffu, v != 0.0f);
            if (v != 0.0f) {
                const uint32_t pos = out + __popc(mask & ((1u << lane) - 1u));
                col[pos] = j;
                val[pos] = v;
            }
            out += __popc(mask);
        }
    }
}

__global__ void __launch_bounds__(256)
csr_scatter_kernel(const uint32_t* __restrict__ rowptr, const uint32_t* __restrict__ col,
                   const float* __restrict__ val, uint32_t M, float* __restrict__ dense, int64_t ld)
{
    const int lane = threadIdx.x & 31;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t i = warp; i < M; i += nwarps) {
        float* row = dense + static_cast<int64_t>(i) * ld;
        for (uint32_t p = rowptr[i] + lane; p < rowptr[i + 1]; p += 32) row[col[p]] = val[p];
    }
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" int sb200_dense_to_csr(sb200_ctx* ctx, const float* dense, uint32_t M, uint32_t N,
                                  int64_t ld, sb200_csr* out, sb200_stream stream_)
{
    if (!ctx || !out || (M && N && !dense) || ld < static_cast<int64_t>(N))
        return SB200_ERR_INVALID_ARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    out->V = nullptr; out->COL = nullptr; out->ROW = nullptr;
    out->NNZ = 0; out->M = M; out->N = N;
    out->Padding[0] = out->Padding[1] = out->Padding[2] = 0;
    int rc = ensure_workspace(ctx, (static_cast<size_t>(M) + 4) * 4 + 16);
    if (rc)
        return rc;
    uint32_t* cnt = reinterpret_cast<uint32_t*>(ctx->d_workspace);
    unsigned long long* d_total = reinterpret_cast<unsigned long long*>(
        (reinterpret_cast<uintptr_t>(cnt + M) + 7) & ~static_cast<uintptr_t>(7));
    if (cudaMalloc(&out->ROW, (static_cast<size_t>(M) + 1) * 4) != cudaSuccess)
        return SB200_ERR_ALLOC;
    const unsigned blocks = static_cast<unsigned>(ctx->sm_count) * 8;
    if (M) dense_count_kernel<<<blocks, 256, 0, stream>>>(dense, M, N, ld, cnt);
    count_scan_kernel<<<1, 1024, 0, stream>>>(cnt, M, out->ROW, d_total);
    ctx->launches += M ? 2 : 1;
    unsigned long long total = 0;
    if (cudaMemcpyAsync(&total, d_total, 8, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess) {
        sb200_csr_free(out);
        return SB200_ERR_CUDA;
    }
    if (total > 0xffffffffull) {
        sb200_csr_free(out);
        return SB200_ERR_TOO_LARGE;
    }
    out->NNZ = static_cast<uint32_t>(total);
    const size_t n = total ? total : 1;
    if (cudaMalloc(&out->COL, n * 4) != cudaSuccess || cudaMalloc(&out->V, n * 4) != cudaSuccess) {
        sb200_csr_free(out);
        return SB200_ERR_ALLOC;
    }
    if (M && total) {
        dense_fill_kernel<<<blocks, 256, 0, stream>>>(dense, M, N, ld, out->ROW, out->COL, out->V);
        ctx->launches += 1;
    }
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

extern "C" int sb200_csr_to_dense(sb200_ctx* ctx, const sb200_csr* src, float* dense, int64_t ld,
                                  sb200_stream stream_)
{
    if (!ctx || !src || !src->ROW || (src->M && src->N && !dense) ||
        ld < static_cast<int64_t>(src->N) || (src->NNZ && (!src->COL || !src->V)))
        return SB200_ERR_INVALID_ARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    if (src->M == 0 || src->N == 0)
        return SB200_OK;
    // zero only the M x N window of the (possibly padded) destination
    if (cudaMemset2DAsync(dense, static_cast<size_t>(ld) * 4, 0, static_cast<size_t>(src->N) * 4,
                          src->M, stream) != cudaSuccess)
        return SB200_ERR_CUDA;
    if (src->NNZ) {
        csr_scatter_kernel<<<static_cast<unsigned>(ctx->sm_count) * 8, 256, 0, stream>>>(
            src->ROW, src->COL, src->V, src->M, dense, ld);
        ctx->launches += 1;
    }
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}
