// The elementwise steps either side of the GEMMs in a Linear training step:
// ReLU, softmax, cross-entropy, their backward passes and the SGD update.
// Each restates the arithmetic of Sapphire's CPU leaf (operation order, where
// accumulation happens, the x == 0 floor of the cross-entropy), one thread per
// element or per row; softmax computes each row's maximum and sum once instead
// of once per element as the reference's device kernel does
// (Sources/Sapphire/compute/dense/cuda/kernels/ActivationKernel.cu:38-65).
#include "common.cuh"

namespace sb200 {
namespace {

constexpr float CE_FLOOR = 1.17549e-30f;

__global__ void relu_kernel(float* __restrict__ out, const float* __restrict__ in, int64_t n)
{
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[i] > 0.0f ? in[i] : 0.0f;
}

__global__ void relu_backward_kernel(float* __restrict__ dx, const float* __restrict__ dy,
                                     const float* __restrict__ x, int64_t n)
{
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) dx[i] = __fadd_rn(dx[i], x[i] > 0.0f ? dy[i] : 0.0f);
}

// one warp per row
__global__ void softmax_kernel(float* __restrict__ out, const float* __restrict__ in,
                               int64_t rows, int unit)
{
    const int lane = threadIdx.x & 31;
    const int64_t r = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (r >= rows) return;
    const float* x = in + r * unit;
    float* y = out + r * unit;
    float hi = -3.402823466e+38f;
    for (int i = lane; i < unit; i += 32) hi = fmaxf(hi, x[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    // the reference adds exp(x - max) in ascending element order: lane 0 does that
    // for short rows; long rows use a lane-strided sum
    float denom = 0.0f;
    if (unit <= 64) {
        for (int i = 0; i < unit; ++i) denom = __fadd_rn(denom, expf(x[i] - hi));
    } else {
        for (int i = lane; i < unit; i += 32) denom += expf(x[i] - hi);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
    }
    for (int i = lane; i < unit; i += 32) y[i] = __fdiv_rn(expf(x[i] - hi), denom);
}

// full-Jacobian form, dx accumulates; one thread per element
__global__ void softmax_backward_kernel(float* __restrict__ dx, const float* __restrict__ dy,
                                        const float* __restrict__ y, int64_t total, int unit)
{
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t o = (idx / unit) * unit;
    const int i = static_cast<int>(idx - o);
    const float yi = y[o + i];
    float s = 0.0f;
    for (int j = 0; j < unit; ++j) {
        const float yj = y[o + j];
        const float t = (i == j) ? __fmul_rn(dy[o + j], __fmul_rn(yj, __fsub_rn(1.0f, yj)))
                                 : __fmul_rn(dy[o + j], __fmul_rn(-yi, yj));
        s = __fadd_rn(s, t);
    }
    dx[idx] = __fadd_rn(dx[idx], s);
}

// loss[i] = -sum_j label*log(x), ascending j; one thread per sample
__global__ void cross_entropy_kernel(float* __restrict__ loss, const float* __restrict__ x,
                                     const float* __restrict__ label, int batch, int unit)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= batch) return;
    float s = 0.0f;
    for (int j = 0; j < unit; ++j) {
        const int64_t idx = static_cast<int64_t>(i) * unit + j;
        const float v = x[idx] == 0.0f ? CE_FLOOR : x[idx];
        s = __fsub_rn(s, __fmul_rn(label[idx], logf(v)));
    }
    loss[i] = s;
}

__global__ void cross_entropy_backward_kernel(float* __restrict__ dx, const float* __restrict__ x,
                                              const float* __restrict__ label, int64_t n)
{
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i] == 0.0f ? CE_FLOOR : x[i];
    dx[i] = __fsub_rn(dx[i], __fdiv_rn(label[i], v));
}

// softmax -> cross-entropy -> its backward -> softmax backward for one sample
// per warp, each stage with the arithmetic of the separate kernels above run on
// zero-initialised gradients; the probabilities and the cross-entropy gradient
// stay in shared memory between the stages.  WARPS rows per block; dynamic
// shared memory = WARPS * 2 * unit floats.
constexpr int FUSED_WARPS = 4;
constexpr int FUSED_MAX_UNIT = 1024;

__global__ void __launch_bounds__(FUSED_WARPS * 32)
softmax_ce_kernel(float* __restrict__ prob, float* __restrict__ loss, float* __restrict__ dlogits,
                  int64_t ld_dlogits, const float* __restrict__ logits,
                  const float* __restrict__ label, int batch, int unit)
{
    extern __shared__ float sh[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x * FUSED_WARPS + warp;
    if (r >= batch) return;                       // whole warps leave; only warp-level syncs below
    float* y = sh + static_cast<size_t>(warp) * 2 * unit;
    float* dp = y + unit;
    const float* x = logits + static_cast<int64_t>(r) * unit;
    const float* lab = label + static_cast<int64_t>(r) * unit;

    float hi = -3.402823466e+38f;
    for (int i = lane; i < unit; i += 32) hi = fmaxf(hi, x[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    float denom = 0.0f;
    if (unit <= 64) {
        for (int i = 0; i < unit; ++i) denom = __fadd_rn(denom, expf(x[i] - hi));
    } else {
        for (int i = lane; i < unit; i += 32) denom += expf(x[i] - hi);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
    }
    for (int i = lane; i < unit; i += 32) {
        const float p = __fdiv_rn(expf(x[i] - hi), denom);
        y[i] = p;
        if (prob) prob[static_cast<int64_t>(r) * unit + i] = p;
        const float v = p == 0.0f ? CE_FLOOR : p;
        dp[i] = __fsub_rn(0.0f, __fdiv_rn(lab[i], v));
    }
    __syncwarp();
    if (loss && lane == 0) {
        float s = 0.0f;
        for (int j = 0; j < unit; ++j) {
            const float v = y[j] == 0.0f ? CE_FLOOR : y[j];
            s = __fsub_rn(s, __fmul_rn(lab[j], logf(v)));
        }
        loss[r] = s;
    }
    for (int i = lane; i < unit; i += 32) {
        const float yi = y[i];
        float s = 0.0f;
        for (int j = 0; j < unit; ++j) {
            const float yj = y[j];
            const float t = (i == j) ? __fmul_rn(dp[j], __fmul_rn(yj, __fsub_rn(1.0f, yj)))
                                     : __fmul_rn(dp[j], __fmul_rn(-yi, yj));
            s = __fadd_rn(s, t);
        }
        dlogits[static_cast<int64_t>(r) * ld_dlogits + i] = __fadd_rn(0.0f, s);
    }
}

// z <- z - (lr * dz), two rounded operations like Scale then Sub
__global__ void sgd_kernel(float* __restrict__ z, const float* __restrict__ dz, float lr, int64_t n)
{
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) z[i] = __fsub_rn(z[i], __fmul_rn(dz[i], lr));
}

__global__ void scale_kernel(float* __restrict__ out, const float* __restrict__ in, float f,
                             int64_t n)
{
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fmul_rn(in[i], f);
}

inline unsigned blocks_for(int64_t n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

int finish(sb200_ctx* ctx)
{
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

}  // namespace
}  // namespace sb200

using namespace sb200;

#define SB200_PROLOGUE(cond)                                                   \
    if (!ctx || !(cond)) return SB200_ERR_INVALID_ARG;                         \
    if (cudaSetDevice(ctx->device) != cudaSuccess) return SB200_ERR_CUDA;      \
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

extern "C" int sb200_relu(sb200_ctx* ctx, float* out, const float* in, int64_t n,
                          sb200_stream stream_)
{
    SB200_PROLOGUE(n >= 0 && (n == 0 || (out && in)))
    if (n == 0) return SB200_OK;
    relu_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(out, in, n);
    return finish(ctx);
}

extern "C" int sb200_relu_backward(sb200_ctx* ctx, float* dx, const float* dy, const float* x,
                                   int64_t n, sb200_stream stream_)
{
    SB200_PROLOGUE(n >= 0 && (n == 0 || (dx && dy && x)))
    if (n == 0) return SB200_OK;
    relu_backward_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(dx, dy, x, n);
    return finish(ctx);
}

extern "C" int sb200_softmax(sb200_ctx* ctx, float* out, const float* in, int64_t total, int unit,
                             sb200_stream stream_)
{
    SB200_PROLOGUE(total >= 0 && unit > 0 && total % unit == 0 && (total == 0 || (out && in)))
    if (total == 0) return SB200_OK;
    const int64_t rows = total / unit;
    softmax_kernel<<<blocks_for(rows * 32, 256), 256, 0, stream>>>(out, in, rows, unit);
    return finish(ctx);
}

extern "C" int sb200_softmax_backward(sb200_ctx* ctx, float* dx, const float* dy, const float* y,
                                      int64_t total, int unit, sb200_stream stream_)
{
    SB200_PROLOGUE(total >= 0 && unit > 0 && total % unit == 0 && (total == 0 || (dx && dy && y)))
    if (total == 0) return SB200_OK;
    softmax_backward_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(dx, dy, y, total, unit);
    return finish(ctx);
}

extern "C" int sb200_cross_entropy(sb200_ctx* ctx, float* loss, const float* x, const float* label,
                                   int batch, int unit, sb200_stream stream_)
{
    SB200_PROLOGUE(batch >= 0 && unit > 0 && (batch == 0 || (loss && x && label)))
    if (batch == 0) return SB200_OK;
    cross_entropy_kernel<<<blocks_for(batch, 64), 64, 0, stream>>>(loss, x, label, batch, unit);
    return finish(ctx);
}

extern "C" int sb200_cross_entropy_backward(sb200_ctx* ctx, float* dx, const float* x,
                                            const float* label, int batch, int unit,
                                            sb200_stream stream_)
{
    SB200_PROLOGUE(batch >= 0 && unit > 0 && (batch == 0 || (dx && x && label)))
    if (batch == 0) return SB200_OK;
    const int64_t n = static_cast<int64_t>(batch) * unit;
    cross_entropy_backward_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(dx, x, label, n);
    return finish(ctx);
}

extern "C" int sb200_softmax_cross_entropy(sb200_ctx* ctx, float* prob, float* loss, float* dlogits,
                                           int64_t ld_dlogits, const float* logits,
                                           const float* label, int batch, int unit,
                                           sb200_stream stream_)
{
    SB200_PROLOGUE(batch >= 0 && unit > 0 && ld_dlogits >= unit &&
                   (batch == 0 || (dlogits && logits && label)))
    if (unit > FUSED_MAX_UNIT) return SB200_ERR_TOO_LARGE;
    if (batch == 0) return SB200_OK;
    const size_t smem = static_cast<size_t>(FUSED_WARPS) * 2 * unit * sizeof(float);
    softmax_ce_kernel<<<blocks_for(batch, FUSED_WARPS), FUSED_WARPS * 32, smem, stream>>>(
        prob, loss, dlogits, ld_dlogits, logits, label, batch, unit);
    return finish(ctx);
}

extern "C" int sb200_sgd_update(sb200_ctx* ctx, float* z, const float* dz, float lr, int64_t n,
                                sb200_stream stream_)
{
    SB200_PROLOGUE(n >= 0 && (n == 0 || (z && dz)))
    if (n == 0) return SB200_OK;
    sgd_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(z, dz, lr, n);
    return finish(ctx);
}

extern "C" int sb200_scale(sb200_ctx* ctx, float* out, const float* in, float factor, int64_t n,
                           sb200_stream stream_)
{
    SB200_PROLOGUE(n >= 0 && (n == 0 || (out && in)))
    if (n == 0) return SB200_OK;
    scale_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(out, in, factor, n);
    return finish(ctx);
}
