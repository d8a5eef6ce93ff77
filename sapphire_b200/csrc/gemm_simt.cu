// CUDA-core kernels of the dense path:
//
//  * gemm_simt_kernel   the general GEMM for requests the TMA-fed tensor-core
//                       kernel cannot take (leading dimensions or pointers
//                       that break TMA's 16-byte rules, e.g. Sapphire's
//                       [256,10] weight with a 40-byte row pitch) and for
//                       K == 0.  Products are rounded multiplies followed by
//                       rounded adds in ascending k from an fp32 zero, i.e. the
//                       operation order of the reference's CPU loop
//                       (Sources/Sapphire/compute/dense/naive/NaiveGemm.cpp:32-36),
//                       so its results are bit-identical to that loop.
//  * colsum kernels     column sums of op(B) (the bias gradient of a Linear
//                       layer) in two steps through a scratch buffer of
//                       per-slice partial sums.
#include "common.cuh"

namespace sb200 {
namespace {

constexpr int TS = 64;   // output tile edge
constexpr int TK = 16;   // k per shared-memory step

struct SimtParams {
    int transA, transB;
    long long M, N, K;
    const float* A; long long lda, strideA;
    const float* B; long long ldb, strideB;
    const float* C; long long ldc, strideC;
    float* D; long long ldd, strideD;
    const float* bias;
    int relu;                                    // D = D > 0 ? D : 0
    const float* mask; long long ldm, strideM;   // gate matrix or null: D = mask > 0 ? D : 0
};

__global__ void __launch_bounds__(256)
gemm_simt_kernel(const SimtParams p)
{
    __shared__ float As[TK][TS + 1];
    __shared__ float Bs[TK][TS + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long long m0 = static_cast<long long>(blockIdx.y) * TS;
    const long long n0 = static_cast<long long>(blockIdx.x) * TS;
    const long long b = blockIdx.z;
    const float* A = p.A + b * p.strideA;
    const float* B = p.B + b * p.strideB;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
            acc[i][j] = 0.0f;

    // Tiles go global -> registers -> shared memory; the loads of the next k-step
    // are issued before the current one is multiplied, so their latency hides
    // behind the arithmetic (small problems are a handful of CTAs walking K one
    // step at a time: latency is all there is).
    constexpr int PER = TK * TS / 256;
    float ra[PER], rb[PER];
    auto fetch = [&](long long k0) {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int i = threadIdx.x + e * 256;
            int kk, mm;
            if (p.transA) { mm = i % TS; kk = i / TS; }     // stored [K, M]: m contiguous
            else          { kk = i % TK; mm = i / TK; }     // stored [M, K]: k contiguous
            const long long m = m0 + mm, k = k0 + kk;
            ra[e] = 0.0f;
            if (m < p.M && k < p.K)
                ra[e] = p.transA ? A[k * p.lda + m] : A[m * p.lda + k];
            int kb, nn;
            if (p.transB) { kb = i % TK; nn = i / TK; }     // stored [N, K]: k contiguous
            else          { nn = i % TS; kb = i / TS; }     // stored [K, N]: n contiguous
            const long long n = n0 + nn, k2 = k0 + kb;
            rb[e] = 0.0f;
            if (n < p.N && k2 < p.K)
                rb[e] = p.transB ? B[n * p.ldb + k2] : B[k2 * p.ldb + n];
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int i = threadIdx.x + e * 256;
            if (p.transA) As[i / TS][i % TS] = ra[e]; else As[i % TK][i / TK] = ra[e];
            if (p.transB) Bs[i % TK][i / TK] = rb[e]; else Bs[i / TS][i % TS] = rb[e];
        }
    };
    if (p.K > 0) fetch(0);
    for (long long k0 = 0; k0 < p.K; k0 += TK) {
        stash();
        __syncthreads();
        if (k0 + TK < p.K) fetch(k0 + TK);
        const int klim = (p.K - k0) < TK ? static_cast<int>(p.K - k0) : TK;
        for (int kk = 0; kk < klim; ++kk) {
            float a[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], bv[j]));
        }
        __syncthreads();
    }

    const float* C = p.C ? p.C + b * p.strideC : nullptr;
    float* D = p.D + b * p.strideD;
    const float* G = p.mask ? p.mask + b * p.strideM : nullptr;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long m = m0 + ty + 16 * i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const long long n = n0 + tx + 16 * j;
            if (n >= p.N) continue;
            float base = C ? C[m * p.ldc + n] : 0.0f;
            if (p.bias) base = __fadd_rn(base, p.bias[n]);
            float o = __fadd_rn(base, acc[i][j]);
            if (p.relu) o = o > 0.0f ? o : 0.0f;
            if (G) o = __fadd_rn(0.0f, G[m * p.ldm + n] > 0.0f ? o : 0.0f);
            D[m * p.ldd + n] = o;
        }
    }
}

// partial[slice][n] = sum over the slice's k range of op(B)[k, n], ascending k
__global__ void __launch_bounds__(128)
colsum_partial_kernel(const float* __restrict__ B, int transB, long long K, long long N,
                      long long ldb, long long rows_per_slice, float* __restrict__ partial)
{
    const long long n = static_cast<long long>(blockIdx.x) * 128 + threadIdx.x;
    const long long k_lo = static_cast<long long>(blockIdx.y) * rows_per_slice;
    long long k_hi = k_lo + rows_per_slice;
    if (k_hi > K) k_hi = K;
    if (n >= N) return;
    float s = 0.0f;
    if (transB) {
        for (long long k = k_lo; k < k_hi; ++k) s = __fadd_rn(s, B[n * ldb + k]);
    } else {
        for (long long k = k_lo; k < k_hi; ++k) s = __fadd_rn(s, B[k * ldb + n]);
    }
    partial[static_cast<long long>(blockIdx.y) * N + n] = s;
}

__global__ void __launch_bounds__(128)
colsum_final_kernel(const float* __restrict__ partial, int slices, long long N, float scale,
                    float* __restrict__ out)
{
    const long long n = static_cast<long long>(blockIdx.x) * 128 + threadIdx.x;
    if (n >= N) return;
    float s = 0.0f;
    for (int i = 0; i < slices; ++i) s = __fadd_rn(s, partial[static_cast<long long>(i) * N + n]);
    out[n] = __fmul_rn(s, scale);
}

}  // namespace

int launch_gemm_simt(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream)
{
    if (g.M <= 0 || g.N <= 0 || g.batch <= 0)
        return SB200_OK;
    const long long gx = (g.N + TS - 1) / TS, gy = (g.M + TS - 1) / TS;
    if (gy > 65535 || g.batch > 65535)
        return SB200_ERR_TOO_LARGE;
    SimtParams p;
    p.transA = g.transA; p.transB = g.transB;
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.A = g.A; p.lda = g.lda; p.strideA = g.strideA;
    p.B = g.B; p.ldb = g.ldb; p.strideB = g.strideB;
    p.C = g.C; p.ldc = g.ldc; p.strideC = g.strideC;
    p.D = g.D; p.ldd = g.ldd; p.strideD = g.strideD;
    p.bias = g.bias;
    p.relu = g.relu;
    p.mask = g.mask; p.ldm = g.ldmask; p.strideM = g.strideMask;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(g.batch));
    gemm_simt_kernel<<<grid, 256, 0, stream>>>(p);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

// Slices the k range so that about two blocks per SM are in flight; one slice
// keeps the strict ascending-k order of the reference.
int colsum_slices(int sm_count, int64_t K, int64_t N)
{
    const int64_t col_blocks = (N + 127) / 128;
    int64_t want = (2 * static_cast<int64_t>(sm_count) + col_blocks - 1) / col_blocks;
    const int64_t max_by_rows = K / 64 > 0 ? K / 64 : 1;
    if (want > max_by_rows) want = max_by_rows;
    if (want < 1) want = 1;
    if (want > 1024) want = 1024;
    return static_cast<int>(want);
}

int launch_colsum_with_scratch(sb200_ctx* ctx, const float* B, int transB, int64_t K, int64_t N,
                               int64_t ldb, float* out, float scale, float* scratch, int slices,
                               cudaStream_t stream)
{
    const int64_t rows_per_slice = (K + slices - 1) / slices;
    dim3 grid(static_cast<unsigned>((N + 127) / 128), static_cast<unsigned>(slices));
    colsum_partial_kernel<<<grid, 128, 0, stream>>>(B, transB, K, N, ldb, rows_per_slice, scratch);
    colsum_final_kernel<<<static_cast<unsigned>((N + 127) / 128), 128, 0, stream>>>(
        scratch, slices, N, scale, out);
    if (ctx) ctx->launches += 2;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

int launch_colsum(sb200_ctx* ctx, const float* B, int transB, int64_t K, int64_t N, int64_t ldb,
                  float* out, float scale, cudaStream_t stream)
{
    if (N <= 0)
        return SB200_OK;
    const int slices = colsum_slices(ctx->sm_count, K, N);
    const int rc = ensure_workspace(ctx, static_cast<size_t>(slices) * N * sizeof(float));
    if (rc)
        return rc;
    return launch_colsum_with_scratch(ctx, B, transB, K, N, ldb, out, scale, ctx->d_workspace,
                                      slices, stream);
}

}  // namespace sb200
