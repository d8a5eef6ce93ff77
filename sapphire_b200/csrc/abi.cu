// C ABI of libsapphire_b200: context life cycle, argument validation and the
// choice between the tensor-core kernel and the CUDA-core kernel.
#include <cstring>
#include <new>

#include "common.cuh"

using namespace sb200;

namespace sb200 {

int ensure_workspace(sb200_ctx* ctx, size_t bytes)
{
    ctx->sp_work_valid = 0;                // whoever asks is about to overwrite the buffer
    if (bytes <= ctx->workspace_bytes)
        return SB200_OK;
    // cudaFree waits for work that may still use the old buffer
    if (ctx->d_workspace)
        cudaFree(ctx->d_workspace);
    ctx->d_workspace = nullptr;
    ctx->workspace_bytes = 0;
    size_t want = bytes < (1u << 20) ? (1u << 20) : bytes + bytes / 4;
    void* p = nullptr;
    if (cudaMalloc(&p, want) != cudaSuccess)
        return SB200_ERR_ALLOC;
    ctx->d_workspace = static_cast<float*>(p);
    ctx->workspace_bytes = want;
    return SB200_OK;
}

}  // namespace sb200

extern "C" int sb200_ctx_create(int device, sb200_ctx** out)
{
    if (!out)
        return SB200_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count)
        return SB200_ERR_CUDA;
    if (cudaSetDevice(device) != cudaSuccess)
        return SB200_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess)
        return SB200_ERR_CUDA;
    if (prop.major != 10)
        return SB200_ERR_UNSUPPORTED;      // the kernels are sm_100a only
    sb200_ctx* ctx = new (std::nothrow) sb200_ctx();
    if (!ctx)
        return SB200_ERR_ALLOC;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->last_path = 0;
    ctx->launches = 0;
    ctx->d_workspace = nullptr;
    ctx->workspace_bytes = 0;
    ctx->split_explicit_hi = 0;
    ctx->split_a_tmem = 1;
    ctx->merge_mn_boxes = 1;
    ctx->use_cta_pairs = 1;
    ctx->split_tail_wave = 0;
    ctx->k_slices = 1;
    ctx->encode_tiled = nullptr;
    ctx->tmaps = nullptr;
    ctx->tmap_clock = 0;
    ctx->tmap_hits = 0;
    ctx->tmap_misses = 0;
    ctx->wait_limit_ns = 2000000000ull;
    ctx->test_stall_kb = -1;
    ctx->d_sp_pattern = nullptr;
    ctx->sp_pattern_bytes = 0;
    ctx->sp_valid = 0;
    ctx->sp_work_valid = 0;
    ctx->sp_fast_mid = 1;
    ctx->d_status = nullptr;
    if (cudaMalloc(&ctx->d_status, sb200::STATUS_WORDS * sizeof(unsigned)) != cudaSuccess ||
        cudaMemset(ctx->d_status, 0, sb200::STATUS_WORDS * sizeof(unsigned)) != cudaSuccess) {
        delete ctx;
        return SB200_ERR_ALLOC;
    }
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) !=
            cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
        cudaFree(ctx->d_status);
        delete ctx;
        return SB200_ERR_CUDA;
    }
    ctx->encode_tiled = fn;
    ctx->tmaps = new (std::nothrow) TensorMapSlot[TENSOR_MAP_SLOTS]();
    if (!ctx->tmaps) {
        cudaFree(ctx->d_status);
        delete ctx;
        return SB200_ERR_ALLOC;
    }
    *out = ctx;
    return SB200_OK;
}

extern "C" int sb200_ctx_destroy(sb200_ctx* ctx)
{
    if (!ctx)
        return SB200_ERR_INVALID_ARG;
    cudaSetDevice(ctx->device);
    if (ctx->d_workspace) cudaFree(ctx->d_workspace);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->d_sp_pattern) cudaFree(ctx->d_sp_pattern);
    delete[] ctx->tmaps;
    delete ctx;
    return SB200_OK;
}

extern "C" const char* sb200_status_string(int status)
{
    switch (status) {
        case SB200_OK: return "ok";
        case SB200_ERR_INVALID_ARG: return "invalid argument";
        case SB200_ERR_CUDA: return "CUDA call failed";
        case SB200_ERR_UNSUPPORTED: return "request not supported by this build or path";
        case SB200_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel expired";
        case SB200_ERR_ALLOC: return "allocation failed";
        case SB200_ERR_TOO_LARGE: return "size beyond a documented limit";
        default: return "unknown status";
    }
}

extern "C" int sb200_last_path(const sb200_ctx* ctx) { return ctx ? ctx->last_path : 0; }

extern "C" int64_t sb200_launch_count(const sb200_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int64_t sb200_ctx_counter(const sb200_ctx* ctx, int which)
{
    if (!ctx)
        return -1;
    switch (which) {
        case SB200_COUNTER_LAUNCHES: return ctx->launches;
        case SB200_COUNTER_TENSOR_MAP_HITS: return ctx->tmap_hits;
        case SB200_COUNTER_TENSOR_MAP_MISSES: return ctx->tmap_misses;
        default: return -1;
    }
}

extern "C" int sb200_ctx_set_option(sb200_ctx* ctx, int option, int value)
{
    if (!ctx)
        return SB200_ERR_INVALID_ARG;
    switch (option) {
        case SB200_OPT_SPLIT_EXPLICIT_HI:
            ctx->split_explicit_hi = value != 0;
            return SB200_OK;
        case SB200_OPT_MERGE_MN_BOXES:
            ctx->merge_mn_boxes = value != 0;
            return SB200_OK;
        case SB200_OPT_CTA_PAIRS:
            ctx->use_cta_pairs = value != 0;
            return SB200_OK;
        case SB200_OPT_SPLIT_TAIL_WAVE:
            ctx->split_tail_wave = value != 0;
            return SB200_OK;
        case SB200_OPT_K_SLICES:
            if (value < 0 || value > 16)
                return SB200_ERR_INVALID_ARG;
            ctx->k_slices = value;
            return SB200_OK;
        case SB200_OPT_SPLIT_A_TMEM:
            ctx->split_a_tmem = value != 0;
            return SB200_OK;
        case SB200_OPT_WAIT_LIMIT_US:
            if (value < 100)
                return SB200_ERR_INVALID_ARG;
            ctx->wait_limit_ns = static_cast<uint64_t>(value) * 1000ull;
            return SB200_OK;
        case SB200_OPT_SPGEMM_FAST_MID:
            ctx->sp_fast_mid = value != 0;
            return SB200_OK;
        case SB200_OPT_TEST_STALL_KBLOCKS:
            ctx->test_stall_kb = value < 0 ? -1 : value;
            return SB200_OK;
        default:
            return SB200_ERR_INVALID_ARG;
    }
}

extern "C" int sb200_check_device_status(sb200_ctx* ctx, sb200_stream stream_)
{
    if (!ctx)
        return SB200_ERR_INVALID_ARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    unsigned word = 0;
    if (cudaMemcpyAsync(&word, ctx->d_status, sizeof(word), cudaMemcpyDeviceToHost, stream) !=
            cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
        return SB200_ERR_CUDA;
    if (word == 0)
        return SB200_OK;
    cudaMemsetAsync(ctx->d_status, 0, sizeof(unsigned), stream);
    cudaStreamSynchronize(stream);
    return SB200_ERR_DEVICE_TIMEOUT;
}

namespace {

// Long-k products with few output tiles (say 256 x 256 x 8192: four tiles, each a
// serial walk over 256 k-blocks while most SMs idle): the k range is cut into
// slices that run as the batches of one launch and add their partial products
// into D through the reduction epilogue.  Returns the number of slices, 1 for
// "do not split".  fp32 adds in arrival order: the last bits of such a product
// can differ between runs.
int split_k_slices(const sb200_ctx* ctx, const GemmArgs& g, bool has_colsum)
{
    if (g.mode != SB200_MODE_TF32 || g.batch != 1 || g.relu || g.mask || g.bias || has_colsum ||
        g.acc_scale != 1.0f)
        return 1;
    if (g.K % 32)
        return 1;
    const long long kb = g.K / 32;
    const long long tiles = ((g.M + 127) / 128) * ((g.N + 127) / 128);
    if (kb < 64 || tiles * 4 > ctx->sm_count)
        return 1;
    long long s = ctx->sm_count / tiles;
    if (s > kb / 16) s = kb / 16;
    if (s > 32) s = 32;
    while (s > 1 && kb % s) --s;                     // equal slices of whole k-blocks
    return static_cast<int>(s);
}

// D <- C (or 0) ahead of a split-k launch, which only adds.
int preset_output(const GemmArgs& g, cudaStream_t stream)
{
    const size_t row_bytes = static_cast<size_t>(g.N) * 4;
    cudaError_t e = cudaSuccess;
    if (g.C == g.D)
        return SB200_OK;
    if (g.C)
        e = cudaMemcpy2DAsync(g.D, static_cast<size_t>(g.ldd) * 4, g.C, static_cast<size_t>(g.ldc) * 4,
                              row_bytes, static_cast<size_t>(g.M), cudaMemcpyDeviceToDevice, stream);
    else
        e = cudaMemset2DAsync(g.D, static_cast<size_t>(g.ldd) * 4, 0, row_bytes, static_cast<size_t>(g.M),
                              stream);
    return e == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

}  // namespace

extern "C" int sb200_gemm_batched(sb200_ctx* ctx, int mode, int path, int transA, int transB,
                                  int64_t M, int64_t N, int64_t K,
                                  const float* A, int64_t lda, int64_t strideA,
                                  const float* B, int64_t ldb, int64_t strideB,
                                  const float* C, int64_t ldc, int64_t strideC,
                                  float* D, int64_t ldd, int64_t strideD,
                                  const float* bias, float* colsum_out, float colsum_scale,
                                  int64_t batch, sb200_stream stream_)
{
    sb200_gemm_epilogue e;
    e.bias = bias;
    e.colsum_out = colsum_out;
    e.colsum_scale = colsum_scale;
    e.relu = 0;
    e.relu_gate = nullptr;
    e.ld_gate = 0;
    e.stride_gate = 0;
    e.sgd_lr = 0.0f;
    return sb200_gemm_batched_ex(ctx, mode, path, transA, transB, M, N, K, A, lda, strideA, B, ldb, strideB,
                                 C, ldc, strideC, D, ldd, strideD, &e, batch, stream_);
}

extern "C" int sb200_gemm_batched_ex(sb200_ctx* ctx, int mode, int path, int transA, int transB,
                                     int64_t M, int64_t N, int64_t K,
                                     const float* A, int64_t lda, int64_t strideA,
                                     const float* B, int64_t ldb, int64_t strideB,
                                     const float* C, int64_t ldc, int64_t strideC,
                                     float* D, int64_t ldd, int64_t strideD,
                                     const sb200_gemm_epilogue* epilogue,
                                     int64_t batch, sb200_stream stream_)
{
    TraceRange trace("sb200_gemm_batched");
    if (!ctx || !epilogue)
        return SB200_ERR_INVALID_ARG;
    const float* bias = epilogue->bias;
    float* colsum_out = epilogue->colsum_out;
    const float colsum_scale = epilogue->colsum_scale;
    const float* gate = epilogue->relu_gate;
    if (gate && (epilogue->ld_gate < N || epilogue->stride_gate < 0))
        return SB200_ERR_INVALID_ARG;
    if (mode != SB200_MODE_TF32 && mode != SB200_MODE_TF32X3)
        return SB200_ERR_INVALID_ARG;
    if (path != SB200_PATH_AUTO && path != SB200_PATH_TCGEN05 && path != SB200_PATH_SIMT)
        return SB200_ERR_INVALID_ARG;
    if (M < 0 || N < 0 || K < 0 || batch < 0)
        return SB200_ERR_INVALID_ARG;
    if (M == 0 || N == 0 || batch == 0)
        return SB200_OK;
    if (!D || (K > 0 && (!A || !B)))
        return SB200_ERR_INVALID_ARG;
    if (K > 0) {
        if (lda < (transA ? M : K) || ldb < (transB ? K : N))
            return SB200_ERR_INVALID_ARG;
        if (strideA < 0 || strideB < 0)
            return SB200_ERR_INVALID_ARG;
    }
    if (ldd < N || (C && ldc < N) || strideD < 0 || strideC < 0)
        return SB200_ERR_INVALID_ARG;
    if (batch > 1 && strideD < (M - 1) * ldd + N)
        return SB200_ERR_INVALID_ARG;      // output batches would overlap
    if (C == D && C && (ldc != ldd || strideC != strideD))
        return SB200_ERR_INVALID_ARG;      // aliasing is exact or not at all
    if (colsum_out && batch != 1)
        return SB200_ERR_INVALID_ARG;
    const float sgd_lr = epilogue->sgd_lr;
    if (sgd_lr != 0.0f && (!C || bias || epilogue->relu || gate))
        return SB200_ERR_INVALID_ARG;

    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;

    GemmArgs g;
    g.mode = mode; g.transA = transA != 0; g.transB = transB != 0;
    g.M = M; g.N = N; g.K = K; g.batch = batch;
    g.A = A; g.lda = lda; g.strideA = strideA;
    g.B = B; g.ldb = ldb; g.strideB = strideB;
    g.C = C; g.ldc = ldc; g.strideC = strideC;
    g.D = D; g.ldd = ldd; g.strideD = strideD;
    g.bias = bias;
    g.colsum_out = nullptr;
    g.colsum_scale = colsum_scale;
    g.relu = epilogue->relu != 0;
    g.mask = gate;
    g.ldmask = gate ? epilogue->ld_gate : 0;
    g.strideMask = gate ? epilogue->stride_gate : 0;
    for (int o = 0; o < MAX_OWNERS; ++o) g.owner[o] = nullptr;
    g.rows_per_owner = 0;
    if (sgd_lr != 0.0f) {
        g.acc_scale = -sgd_lr;
        g.colsum_lr = sgd_lr;
    }

    const bool tc_ok = tcgen05_eligible(g);
    int rc;
    if (path == SB200_PATH_TCGEN05 && !tc_ok)
        return SB200_ERR_UNSUPPORTED;
    bool fused_colsum = false;
    if ((path == SB200_PATH_AUTO && tc_ok) || path == SB200_PATH_TCGEN05) {
        // the TF32 tensor-core kernel takes the column sums along (extra warps read
        // the B tiles already in shared memory); other paths run them separately
        fused_colsum = colsum_out && mode == SB200_MODE_TF32 && K > 0;
        if (fused_colsum)
            g.colsum_out = colsum_out;
        const int slices = split_k_slices(ctx, g, colsum_out != nullptr);
        if (slices > 1) {
            if ((rc = preset_output(g, stream)))
                return rc;
            const int64_t ks = K / slices;
            g.batch = slices;
            g.K = ks;
            g.strideA = g.transA ? ks * lda : ks;          // slice s starts ks along k
            g.strideB = g.transB ? ks : ks * ldb;
            g.C = nullptr;
            g.owner[0] = D;                                // every tile adds into D itself
            g.rows_per_owner = int64_t(1) << 30;
        }
        rc = launch_gemm_tcgen05(ctx, g, stream);
        ctx->last_path = SB200_PATH_TCGEN05;
    } else {
        rc = launch_gemm_simt(ctx, g, stream);
        ctx->last_path = SB200_PATH_SIMT;
    }
    if (rc)
        return rc;
    if (colsum_out && !fused_colsum)
        rc = launch_colsum(ctx, B, g.transB, K, N, ldb, colsum_out, colsum_scale, stream, g.colsum_lr);
    return rc;
}

// ------------------------------------------------- GEMM -> reduce-scatter
namespace {
int gemm_to_owners(sb200_ctx* ctx, int mode, int transA, int transB, int64_t M, int64_t N, int64_t K,
                   const float* A, int64_t lda, const float* B, int64_t ldb, float* const* owners,
                   int n_owners, int64_t ld_out, float* colsum_out, float colsum_scale,
                   sb200_stream stream_, int store)
{
    TraceRange trace(store ? "sb200_gemm_scatter" : "sb200_gemm_reduce_scatter");
    if (!ctx || !owners || !A || !B)
        return SB200_ERR_INVALID_ARG;
    if (mode != SB200_MODE_TF32 && mode != SB200_MODE_TF32X3)
        return SB200_ERR_INVALID_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || n_owners < 1 || n_owners > MAX_OWNERS)
        return SB200_ERR_INVALID_ARG;
    if (lda < (transA ? M : K) || ldb < (transB ? K : N) || ld_out < N)
        return SB200_ERR_INVALID_ARG;
    // every 128-row tile of the product must lie inside one owner's row block,
    // and the adds are 16 bytes wide
    if (M % n_owners || (M / n_owners) % 128 || (ld_out & 3))
        return SB200_ERR_UNSUPPORTED;
    for (int o = 0; o < n_owners; ++o)
        if (!owners[o] || (reinterpret_cast<uintptr_t>(owners[o]) & 15))
            return SB200_ERR_INVALID_ARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;

    GemmArgs g;
    g.mode = mode; g.transA = transA != 0; g.transB = transB != 0;
    g.M = M; g.N = N; g.K = K; g.batch = 1;
    g.A = A; g.lda = lda; g.strideA = 0;
    g.B = B; g.ldb = ldb; g.strideB = 0;
    g.C = nullptr; g.ldc = N; g.strideC = 0;
    g.D = owners[0]; g.ldd = ld_out; g.strideD = 0;            // alignment checks only; tiles go to owner[]
    g.bias = nullptr;
    g.colsum_out = nullptr;
    g.colsum_scale = colsum_scale;
    g.relu = 0;
    g.mask = nullptr; g.ldmask = 0; g.strideMask = 0;
    for (int o = 0; o < MAX_OWNERS; ++o) g.owner[o] = o < n_owners ? owners[o] : nullptr;
    g.rows_per_owner = M / n_owners;
    g.owner_store = store;
    if (!tcgen05_eligible(g))
        return SB200_ERR_UNSUPPORTED;                           // the CUDA-core kernel has no such epilogue
    const bool fused_colsum = colsum_out && mode == SB200_MODE_TF32;
    if (fused_colsum)
        g.colsum_out = colsum_out;
    int rc = launch_gemm_tcgen05(ctx, g, stream);
    ctx->last_path = SB200_PATH_TCGEN05;
    if (rc)
        return rc;
    if (colsum_out && !fused_colsum)
        rc = launch_colsum(ctx, B, g.transB, K, N, ldb, colsum_out, colsum_scale, stream);
    return rc;
}

// out[r, c] = blocks[0][r, c] + blocks[1][r, c] + ... in that order
__global__ void __launch_bounds__(256)
sum_blocks_kernel(float* __restrict__ out, long long ld_out, const float* blocks, int n_blocks,
                  long long block_stride, long long rows, long long cols4, long long ld_block)
{
    const long long total = rows * cols4;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / cols4, c = (i % cols4) * 4;
        const float* src = blocks + r * ld_block + c;
        float4 s = *reinterpret_cast<const float4*>(src);
        for (int b = 1; b < n_blocks; ++b) {
            const float4 x = *reinterpret_cast<const float4*>(src + b * block_stride);
            s.x = __fadd_rn(s.x, x.x); s.y = __fadd_rn(s.y, x.y);
            s.z = __fadd_rn(s.z, x.z); s.w = __fadd_rn(s.w, x.w);
        }
        *reinterpret_cast<float4*>(out + r * ld_out + c) = s;      // (out may be blocks[0] itself)
    }
}
}  // namespace

extern "C" int sb200_gemm_reduce_scatter(sb200_ctx* ctx, int mode, int transA, int transB,
                                         int64_t M, int64_t N, int64_t K,
                                         const float* A, int64_t lda, const float* B, int64_t ldb,
                                         float* const* owners, int n_owners, int64_t ld_out,
                                         float* colsum_out, float colsum_scale, sb200_stream stream_)
{
    return gemm_to_owners(ctx, mode, transA, transB, M, N, K, A, lda, B, ldb, owners, n_owners, ld_out,
                          colsum_out, colsum_scale, stream_, 0);
}

extern "C" int sb200_gemm_scatter(sb200_ctx* ctx, int mode, int transA, int transB,
                                  int64_t M, int64_t N, int64_t K,
                                  const float* A, int64_t lda, const float* B, int64_t ldb,
                                  float* const* owners, int n_owners, int64_t ld_out,
                                  float* colsum_out, float colsum_scale, sb200_stream stream_)
{
    return gemm_to_owners(ctx, mode, transA, transB, M, N, K, A, lda, B, ldb, owners, n_owners, ld_out,
                          colsum_out, colsum_scale, stream_, 1);
}

extern "C" int sb200_sum_blocks(sb200_ctx* ctx, float* out, int64_t ld_out, const float* blocks, int n_blocks,
                                int64_t block_stride, int64_t rows, int64_t cols, int64_t ld_block,
                                sb200_stream stream_)
{
    if (!ctx || !out || !blocks || n_blocks < 1 || rows < 0 || cols < 0)
        return SB200_ERR_INVALID_ARG;
    if (ld_out < cols || ld_block < cols || block_stride < 0)
        return SB200_ERR_INVALID_ARG;
    if ((cols & 3) || (ld_out & 3) || (ld_block & 3) || (block_stride & 3) ||
        (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(blocks) & 15))
        return SB200_ERR_UNSUPPORTED;
    if (rows == 0 || cols == 0)
        return SB200_OK;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    const long long total = rows * (cols / 4);
    long long grid = (total + 255) / 256;
    if (grid > 8ll * ctx->sm_count)
        grid = 8ll * ctx->sm_count;
    sum_blocks_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
        out, ld_out, blocks, n_blocks, block_stride, rows, cols / 4, ld_block);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

// ------------------------------------------------- buffers other ranks map
extern "C" int sb200_peer_alloc(sb200_ctx* ctx, size_t bytes, void** ptr, unsigned char* handle64)
{
    if (!ctx || !ptr || !handle64 || bytes == 0)
        return SB200_ERR_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    *ptr = nullptr;
    if (cudaMalloc(ptr, bytes) != cudaSuccess) {
        cudaGetLastError();
        return SB200_ERR_ALLOC;
    }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, *ptr) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(*ptr);
        *ptr = nullptr;
        return SB200_ERR_CUDA;
    }
    memcpy(handle64, &h, sizeof(h));
    return SB200_OK;
}

extern "C" int sb200_peer_open(sb200_ctx* ctx, const unsigned char* handle64, void** ptr)
{
    if (!ctx || !ptr || !handle64)
        return SB200_ERR_INVALID_ARG;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    *ptr = nullptr;
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return SB200_ERR_CUDA;
    }
    return SB200_OK;
}

extern "C" int sb200_peer_close(sb200_ctx* ctx, void* ptr)
{
    if (!ctx || !ptr)
        return SB200_ERR_INVALID_ARG;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

extern "C" int sb200_peer_free(sb200_ctx* ctx, void* ptr)
{
    if (!ctx || !ptr)
        return SB200_ERR_INVALID_ARG;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    return cudaFree(ptr) == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}
