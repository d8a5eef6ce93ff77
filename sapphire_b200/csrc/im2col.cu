// The lowering that lets a convolution run on the batched GEMM: im2col builds,
// per image, the [C*kh*kw, outR*outC] matrix whose product with the
// [Cout, C*kh*kw] filter matrix is the convolution, and col2im is its adjoint
// (the input gradient).  Index conventions are those of Sapphire's host path
// (Sources/Sapphire/compute/dense/naive/Convolution.cpp:15-211): the taps of a channel are stored
// in reverse order, so the GEMM is a true (flipped-kernel) convolution, and
// pixels outside the image read a pad value.  Both kernels are pure data
// movement, bound by HBM: lanes walk the contiguous output-pixel dimension.
#include "common.cuh"

namespace sb200 {
namespace {

struct ConvGeom {
    int N, C, H, W, kh, kw, strideR, strideC, padR, padC, dilR, dilC;
    int outR, outC;
};

inline bool make_geom(const sb200_conv_geometry* g, ConvGeom* o)
{
    if (!g || g->N < 0 || g->C <= 0 || g->H <= 0 || g->W <= 0 || g->kh <= 0 || g->kw <= 0 ||
        g->strideR <= 0 || g->strideC <= 0 || g->padR < 0 || g->padC < 0 || g->dilR <= 0 || g->dilC <= 0)
        return false;
    const long long spanR = static_cast<long long>(g->H) + 2LL * g->padR - static_cast<long long>(g->dilR) * (g->kh - 1) - 1;
    const long long spanC = static_cast<long long>(g->W) + 2LL * g->padC - static_cast<long long>(g->dilC) * (g->kw - 1) - 1;
    if (spanR < 0 || spanC < 0)
        return false;                          // the filter does not fit the padded image
    *o = ConvGeom{g->N, g->C, g->H, g->W, g->kh, g->kw, g->strideR, g->strideC, g->padR, g->padC,
                  g->dilR, g->dilC, static_cast<int>(spanR / g->strideR + 1),
                  static_cast<int>(spanC / g->strideC + 1)};
    return true;
}

// One block per (image, channel) plane: a thread takes four consecutive output
// pixels, works out their input coordinates once and then writes them into each
// of the channel's kh*kw matrix rows (one 16-byte store per row when the row
// length allows), so the integer divisions are paid once per 4*kh*kw entries
// and the plane's re-reads (every pixel is wanted by kh*kw rows) hit L1.
__global__ void __launch_bounds__(256)
im2col_kernel(float* __restrict__ cols, const float* __restrict__ x, ConvGeom g, float pad, int vec_ok)
{
    const int taps = g.kh * g.kw;
    const long long P = static_cast<long long>(g.outR) * g.outC;
    const long long nc = blockIdx.x;                           // image * C + channel
    const float* xc = x + nc * static_cast<long long>(g.H) * g.W;
    float* out = cols + nc * taps * P;                         // this channel's first matrix row
    for (long long p0 = 4LL * threadIdx.x; p0 < P; p0 += 4LL * blockDim.x) {
        int orow = static_cast<int>(p0 / g.outC), ocol = static_cast<int>(p0 % g.outC);
        int r0[4], q0[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            r0[e] = p0 + e < P ? orow * g.strideR - g.padR : -(1 << 29);   // beyond the row: reads pad
            q0[e] = ocol * g.strideC - g.padC;
            if (++ocol == g.outC) {
                ocol = 0;
                ++orow;
            }
        }
        for (int fr = 0; fr < g.kh; ++fr)
            for (int fc = 0; fc < g.kw; ++fc) {
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = r0[e] + fr * g.dilR, q = q0[e] + fc * g.dilC;
                    const bool inside = r >= 0 && r < g.H && q >= 0 && q < g.W;
                    v[e] = inside ? __ldg(xc + static_cast<long long>(r) * g.W + q) : pad;
                }
                float* dst = out + (taps - 1 - (fr * g.kw + fc)) * P + p0;   // taps stored in reverse
                if (vec_ok) {                                  // P % 4 == 0 and cols 16-byte aligned
                    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (p0 + e < P) dst[e] = v[e];
                }
            }
    }
}

// One thread per input pixel gathers the matrix entries im2col read from it and
// adds them to the pixel in ascending (orow, ocol) order -- the order in which
// the reference's scatter loop reaches that pixel, so the sum is bit-identical.
__global__ void __launch_bounds__(256)
col2im_kernel(float* __restrict__ x, const float* __restrict__ cols, ConvGeom g)
{
    const int taps = g.kh * g.kw;
    const long long P = static_cast<long long>(g.outR) * g.outC;
    const long long plane = static_cast<long long>(g.H) * g.W;
    const long long total = static_cast<long long>(g.N) * g.C * plane;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long nc = idx / plane;
        const int r = static_cast<int>((idx % plane) / g.W), q = static_cast<int>(idx % g.W);
        const float* m = cols + nc * taps * P;                 // this image's rows of channel c
        float acc = x[idx];
        for (int fr = g.kh - 1; fr >= 0; --fr) {               // fr descending = orow ascending
            const int tr = r + g.padR - fr * g.dilR;
            if (tr < 0 || tr % g.strideR) continue;
            const int orow = tr / g.strideR;
            if (orow >= g.outR) continue;
            for (int fc = g.kw - 1; fc >= 0; --fc) {           // fc descending = ocol ascending
                const int tq = q + g.padC - fc * g.dilC;
                if (tq < 0 || tq % g.strideC) continue;
                const int ocol = tq / g.strideC;
                if (ocol >= g.outC) continue;
                const int row = taps - 1 - (fr * g.kw + fc);
                acc = __fadd_rn(acc, __ldg(m + row * P + static_cast<long long>(orow) * g.outC + ocol));
            }
        }
        x[idx] = acc;
    }
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" int sb200_im2col(sb200_ctx* ctx, float* cols, const float* x,
                            const sb200_conv_geometry* geometry, float pad_value, sb200_stream stream_)
{
    ConvGeom g;
    if (!ctx || !make_geom(geometry, &g))
        return SB200_ERR_INVALID_ARG;
    if (g.N == 0)
        return SB200_OK;
    if (!cols || !x)
        return SB200_ERR_INVALID_ARG;
    const long long rows = static_cast<long long>(g.C) * g.kh * g.kw;
    const long long P = static_cast<long long>(g.outR) * g.outC;
    if (rows * g.N > 0x7fffffffLL)
        return SB200_ERR_TOO_LARGE;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int vec_ok = (P % 4 == 0) && (reinterpret_cast<uintptr_t>(cols) % 16 == 0);
    const long long quads = (P + 3) / 4;
    const unsigned threads = quads >= 256 ? 256u : quads >= 128 ? 128u : quads >= 64 ? 64u : 32u;
    im2col_kernel<<<static_cast<unsigned>(static_cast<long long>(g.N) * g.C), threads, 0, stream>>>(
        cols, x, g, pad_value, vec_ok);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

extern "C" int sb200_col2im(sb200_ctx* ctx, float* x, const float* cols,
                            const sb200_conv_geometry* geometry, sb200_stream stream_)
{
    ConvGeom g;
    if (!ctx || !make_geom(geometry, &g))
        return SB200_ERR_INVALID_ARG;
    if (g.N == 0)
        return SB200_OK;
    if (!cols || !x)
        return SB200_ERR_INVALID_ARG;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const long long total = static_cast<long long>(g.N) * g.C * g.H * g.W;
    const long long want = (total + 255) / 256;
    const long long cap = static_cast<long long>(ctx->sm_count) * 32;
    col2im_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, stream>>>(x, cols, g);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}
