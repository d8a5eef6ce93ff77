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

constexpr int TS = 64;   // edge of the standard output tile
// Rows and columns of an output tile (TM, TN: 64, or 16 -- columns for narrow outputs
// such as a 10-class layer, where a 64-wide tile would spend 5/6 of its arithmetic on
// masked columns; rows and columns when the launch would otherwise be a few CTAs: the
// ascending-k order forbids splitting k, so more and smaller tiles are the only way to
// put more SMs on a small product) and k per shared-memory step (TK: 16, or 64 when the launch is a handful of CTAs
// walking K, so that four times as many loads are in flight per step) are template
// parameters.  Neither changes the order of the additions.

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
    float acc_scale;                             // product times this before C is added (1 = off)
};

template <int TM, int TN, int TK>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const SimtParams p)
{
    constexpr int NI = TM / 16;                  // rows per thread
    constexpr int NJ = TN / 16;                  // columns per thread
    __shared__ float As[TK][TM + 1];
    __shared__ float Bs[TK][TN + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const long long m0 = static_cast<long long>(blockIdx.y) * TM;
    const long long n0 = static_cast<long long>(blockIdx.x) * TN;
    const long long b = blockIdx.z;
    const float* A = p.A + b * p.strideA;
    const float* B = p.B + b * p.strideB;

    float acc[NI][NJ];
#pragma unroll
    for (int i = 0; i < NI; ++i)
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            acc[i][j] = 0.0f;

    // Tiles go global -> registers -> shared memory; the loads of the next k-step
    // are issued before the current one is multiplied, so their latency hides
    // behind the arithmetic (small problems are a handful of CTAs walking K one
    // step at a time: latency is all there is).
    constexpr int PER_A = TK * TM / 256, PER_B = TK * TN / 256;
    static_assert(PER_A >= 1 && PER_B >= 1, "a tile step is at least one element per thread");
    float ra[PER_A], rb[PER_B];
    auto fetch = [&](long long k0) {
#pragma unroll
        for (int e = 0; e < PER_A; ++e) {
            const int i = threadIdx.x + e * 256;
            int kk, mm;
            if (p.transA) { mm = i % TM; kk = i / TM; }     // stored [K, M]: m contiguous
            else          { kk = i % TK; mm = i / TK; }     // stored [M, K]: k contiguous
            const long long m = m0 + mm, k = k0 + kk;
            ra[e] = 0.0f;
            if (m < p.M && k < p.K)
                ra[e] = p.transA ? A[k * p.lda + m] : A[m * p.lda + k];
        }
#pragma unroll
        for (int e = 0; e < PER_B; ++e) {
            const int i = threadIdx.x + e * 256;
            int kb, nn;
            if (p.transB) { kb = i % TK; nn = i / TK; }     // stored [N, K]: k contiguous
            else          { nn = i % TN; kb = i / TN; }     // stored [K, N]: n contiguous
            const long long n = n0 + nn, k2 = k0 + kb;
            rb[e] = 0.0f;
            if (n < p.N && k2 < p.K)
                rb[e] = p.transB ? B[n * p.ldb + k2] : B[k2 * p.ldb + n];
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int e = 0; e < PER_A; ++e) {
            const int i = threadIdx.x + e * 256;
            if (p.transA) As[i / TM][i % TM] = ra[e]; else As[i % TK][i / TK] = ra[e];
        }
#pragma unroll
        for (int e = 0; e < PER_B; ++e) {
            const int i = threadIdx.x + e * 256;
            if (p.transB) Bs[i % TK][i / TK] = rb[e]; else Bs[i / TN][i % TN] = rb[e];
        }
    };
    if (p.K > 0) fetch(0);
    for (long long k0 = 0; k0 < p.K; k0 += TK) {
        stash();
        __syncthreads();
        if (k0 + TK < p.K) fetch(k0 + TK);
        const int klim = (p.K - k0) < TK ? static_cast<int>(p.K - k0) : TK;
        auto k_step = [&](int kk) {
            float a[NI], bv[NJ];
#pragma unroll
            for (int i = 0; i < NI; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < NJ; ++j) bv[j] = Bs[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < NI; ++i)
#pragma unroll
                for (int j = 0; j < NJ; ++j)
                    acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], bv[j]));
        };
        if (NJ == 1 && klim == TK) {
            // narrow tiles, a whole step: unrolled, so that the shared-memory loads of
            // several k run ahead of the (strictly ordered) additions; a thread of a
            // 64-column tile has 16 independent sums to interleave and gains nothing
#pragma unroll 16
            for (int kk = 0; kk < TK; ++kk)
                k_step(kk);
        } else {
            for (int kk = 0; kk < klim; ++kk)
                k_step(kk);
        }
        __syncthreads();
    }

    const float* C = p.C ? p.C + b * p.strideC : nullptr;
    float* D = p.D + b * p.strideD;
    const float* G = p.mask ? p.mask + b * p.strideM : nullptr;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const long long m = m0 + ty + 16 * i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const long long n = n0 + tx + 16 * j;
            if (n >= p.N) continue;
            float base = C ? C[m * p.ldc + n] : 0.0f;
            if (p.bias) base = __fadd_rn(base, p.bias[n]);
            float o = __fadd_rn(base, p.acc_scale != 1.0f ? __fmul_rn(acc[i][j], p.acc_scale) : acc[i][j]);
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
                    float* __restrict__ out, float lr)
{
    const long long n = static_cast<long long>(blockIdx.x) * 128 + threadIdx.x;
    if (n >= N) return;
    float s = 0.0f;
    for (int i = 0; i < slices; ++i) s = __fadd_rn(s, partial[static_cast<long long>(i) * N + n]);
    const float g = __fmul_rn(s, scale);
    out[n] = lr != 0.0f ? __fsub_rn(out[n], __fmul_rn(g, lr)) : g;     // lr: in-place SGD update of a bias
}

}  // namespace

int launch_gemm_simt(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream)
{
    if (g.M <= 0 || g.N <= 0 || g.batch <= 0)
        return SB200_OK;
    // 16-column tiles for narrow outputs, and whenever 64-column tiles would leave
    // three quarters of the SMs without a CTA (four times as many CTAs share the walk);
    // 16-row tiles too when that still leaves three quarters idle
    const long long gy64 = (g.M + TS - 1) / TS;
    const bool narrow = g.N <= 32 || ((g.N + TS - 1) / TS) * gy64 * g.batch * 4 <= ctx->sm_count;
    const int tn = narrow ? 16 : TS;
    const long long gx = (g.N + tn - 1) / tn;
    const bool small = narrow && gx * gy64 * g.batch * 4 <= ctx->sm_count;
    const int tm = small ? 16 : TS;
    const long long gy = (g.M + tm - 1) / tm;
    if (gy > 65535 || g.batch > 65535)
        return SB200_ERR_TOO_LARGE;
    // a handful of CTAs walking K: longer steps, more loads in flight
    const bool few = gx * gy * g.batch <= 2ll * ctx->sm_count;
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
    p.acc_scale = g.acc_scale;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(g.batch));
    if (small)
        gemm_simt_kernel<16, 16, 64><<<grid, 256, 0, stream>>>(p);      // always a few CTAs
    else if (narrow)
        few ? gemm_simt_kernel<TS, 16, 64><<<grid, 256, 0, stream>>>(p)
            : gemm_simt_kernel<TS, 16, 16><<<grid, 256, 0, stream>>>(p);
    else
        few ? gemm_simt_kernel<TS, TS, 64><<<grid, 256, 0, stream>>>(p)
            : gemm_simt_kernel<TS, TS, 16><<<grid, 256, 0, stream>>>(p);
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

namespace {
int launch_colsum_kernels(sb200_ctx* ctx, const float* B, int transB, int64_t K, int64_t N,
                          int64_t ldb, float* out, float scale, float* scratch, int slices,
                          cudaStream_t stream, float lr)
{
    const int64_t rows_per_slice = (K + slices - 1) / slices;
    dim3 grid(static_cast<unsigned>((N + 127) / 128), static_cast<unsigned>(slices));
    colsum_partial_kernel<<<grid, 128, 0, stream>>>(B, transB, K, N, ldb, rows_per_slice, scratch);
    colsum_final_kernel<<<static_cast<unsigned>((N + 127) / 128), 128, 0, stream>>>(
        scratch, slices, N, scale, out, lr);
    if (ctx) ctx->launches += 2;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}
}  // namespace

int launch_colsum_with_scratch(sb200_ctx* ctx, const float* B, int transB, int64_t K, int64_t N,
                               int64_t ldb, float* out, float scale, float* scratch, int slices,
                               cudaStream_t stream)
{
    return launch_colsum_kernels(ctx, B, transB, K, N, ldb, out, scale, scratch, slices, stream, 0.0f);
}

int launch_colsum(sb200_ctx* ctx, const float* B, int transB, int64_t K, int64_t N, int64_t ldb,
                  float* out, float scale, cudaStream_t stream, float lr)
{
    if (N <= 0)
        return SB200_OK;
    const int slices = colsum_slices(ctx->sm_count, K, N);
    const int rc = ensure_workspace(ctx, static_cast<size_t>(slices) * N * sizeof(float));
    if (rc)
        return rc;
    return launch_colsum_kernels(ctx, B, transB, K, N, ldb, out, scale, ctx->d_workspace, slices, stream, lr);
}

}  // namespace sb200
