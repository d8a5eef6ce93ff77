// Gradient exchange of a data-parallel training step over peer memory, fused with
// the SGD update: two kernels per step, no collective library on the path.
//
// Every rank keeps three buffers that the other ranks of the node map (CUDA IPC):
// its gradient bucket, a buffer for the slice of the summed gradient it owns, and a
// few flag words.  Per step:
//
//   reduce   announces "my gradients are complete" in every peer's flag words,
//            waits until every peer has announced the same, then sums its own slice
//            (1 / world of the bucket) over all ranks' buckets -- peer loads over
//            NVLink, fixed rank order, so every run and every rank gets the same
//            bits -- into its slice buffer, and announces "my slice is reduced";
//   update   waits for every peer's "slice is reduced", then walks the whole
//            parameter vector: z <- z - lr * g with g read from the owning rank's
//            slice buffer (the all-gather happens inside the update), the elements
//            after `n_sum` scaled by 1 / world first (bias gradients are means).
//
// The announcements are release stores at system scope, the waits acquire loads
// with a time limit (the context's wait limit); a wait that runs out records
// SB200_ERR_DEVICE_TIMEOUT's status code and the kernel carries on, so nothing
// hangs when a rank is late or gone.  The step number lives in device memory and
// is advanced by the last CTA of `update`, so that a captured CUDA graph can replay
// the pair of kernels step after step.
//
// Buffer reuse is safe without further barriers: a rank's bucket is next written by
// its following backward pass, which starts after its `update`, which waited for
// every peer's "slice is reduced", which each peer announced after its last read of
// the bucket; a rank's slice buffer is next written in its following `reduce`, after
// every peer announced the next step's gradients, which each does after its
// `update` -- its last read of the slice buffer.
#include "common.cuh"

namespace sb200 {
namespace {

constexpr int DP_THREADS = 256;
// layout of a rank's flag words
constexpr int FLAG_READY = 0;                    // [0, 8): step number up to which rank r's gradients are complete
constexpr int FLAG_REDUCED = 8;                  // [8, 16): ... rank r's slice is reduced
constexpr int FLAG_STEP = 16;                    // steps completed by this rank
constexpr int FLAG_DONE_REDUCE = 17;             // CTAs of the running reduce kernel that have finished
constexpr int FLAG_DONE_UPDATE = 18;
constexpr int FLAG_BARRIER = 20;                 // [20, 28): barrier number rank r has reached
constexpr int FLAG_BARRIER_STEP = 28;            // barriers passed by this rank

struct DpGroup {
    int world, rank;
    const float* grads[8];
    float* reduced[8];
    uint32_t* flags[8];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// peer data: bypass L1, which is not coherent with another GPU's writes
__device__ __forceinline__ float4 ld_sys_v4(const float* p)
{
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ float ld_sys(const float* p)
{
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint64_t now_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Threads 0 .. world-1 each wait for one peer's flag to reach `step` (rank `skip` is
// not waited for); returns after a CTA-wide barrier.  A wait that runs out records
// `code` and gives up.
__device__ __forceinline__ void wait_flags(const uint32_t* mine, int world, int skip, int first, uint32_t step,
                                           unsigned long long limit_ns, unsigned* status, unsigned code)
{
    if (static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != skip) {
        const uint32_t* f = mine + first + threadIdx.x;
        uint64_t t0 = 0;                       // the timer is slow to read: started at the 16th try
        uint32_t spins = 0;
        while (static_cast<int32_t>(ld_acquire_sys(f) - step) < 0) {
            if ((++spins & 15u) == 0) {
                const uint64_t now = now_ns();
                if (t0 == 0) {
                    t0 = now;
                } else if (now - t0 > limit_ns) {
                    atomicCAS(status, 0u, code);
                    break;
                }
            }
        }
    }
    __syncthreads();
}

// Slice of rank r: [r * per, min((r + 1) * per, count)), per a multiple of 4.
__device__ __host__ __forceinline__ int64_t slice_len(int64_t count, int world)
{
    return ((count + world - 1) / world + 3) & ~static_cast<int64_t>(3);
}

__global__ void __launch_bounds__(DP_THREADS)
dp_reduce_kernel(DpGroup g, int64_t count, unsigned long long limit_ns, unsigned* status)
{
    uint32_t* mine = g.flags[g.rank];
    const uint32_t step = mine[FLAG_STEP] + 1;
    // every gradient kernel of this step has completed (stream order): tell the peers
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < g.world)
        st_release_sys(g.flags[threadIdx.x] + FLAG_READY + g.rank, step);
    // (this rank's own gradients are complete by stream order: no CTA waits for another CTA)
    wait_flags(mine, g.world, g.rank, FLAG_READY, step, limit_ns, status, FAULT_PEER_WAIT);

    const int64_t per = slice_len(count, g.world);
    const int64_t lo = g.rank * per, hi = min(lo + per, count);
    float* out = g.reduced[g.rank];
    const bool vec = (count & 3) == 0;
    for (int64_t i = lo + (static_cast<int64_t>(blockIdx.x) * DP_THREADS + threadIdx.x) * 4; i < hi;
         i += static_cast<int64_t>(gridDim.x) * DP_THREADS * 4) {
        if (vec || i + 4 <= hi) {
            float4 s = ld_sys_v4(g.grads[0] + i);
            for (int r = 1; r < g.world; ++r) {
                const float4 x = ld_sys_v4(g.grads[r] + i);
                s.x = __fadd_rn(s.x, x.x); s.y = __fadd_rn(s.y, x.y);
                s.z = __fadd_rn(s.z, x.z); s.w = __fadd_rn(s.w, x.w);
            }
            *reinterpret_cast<float4*>(out + i) = s;
        } else {
            for (int64_t j = i; j < hi; ++j) {
                float s = ld_sys(g.grads[0] + j);
                for (int r = 1; r < g.world; ++r) s = __fadd_rn(s, ld_sys(g.grads[r] + j));
                out[j] = s;
            }
        }
    }
    // last CTA out: the slice is complete, tell the peers
    __threadfence_system();
    __syncthreads();
    __shared__ uint32_t s_last;
    if (threadIdx.x == 0) s_last = atomicAdd(mine + FLAG_DONE_REDUCE, 1u) == gridDim.x - 1;
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        if (static_cast<int>(threadIdx.x) < g.world)
            st_release_sys(g.flags[threadIdx.x] + FLAG_REDUCED + g.rank, step);
        if (threadIdx.x == 0) mine[FLAG_DONE_REDUCE] = 0;
    }
}

__global__ void __launch_bounds__(DP_THREADS)
dp_update_kernel(DpGroup g, float* __restrict__ z, int64_t count, int64_t n_sum, float lr,
                 unsigned long long limit_ns, unsigned* status)
{
    uint32_t* mine = g.flags[g.rank];
    const uint32_t step = mine[FLAG_STEP] + 1;
    wait_flags(mine, g.world, g.rank, FLAG_REDUCED, step, limit_ns, status, FAULT_PEER_WAIT);

    const int64_t per = slice_len(count, g.world);
    const float inv = 1.0f / static_cast<float>(g.world);
    const bool vec = (count & 3) == 0 && (n_sum & 3) == 0;
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * DP_THREADS + threadIdx.x) * 4; i < count;
         i += static_cast<int64_t>(gridDim.x) * DP_THREADS * 4) {
        const float* src = g.reduced[i / per];                    // per is a multiple of 4: one owner per float4
        if (vec || i + 4 <= count) {
            float4 d = ld_sys_v4(src + i);
            const float e[4] = {d.x, d.y, d.z, d.w};
            float4 p = *reinterpret_cast<const float4*>(z + i);
            float o[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float gk = (i + k >= n_sum) ? __fmul_rn(e[k], inv) : e[k];
                o[k] = __fsub_rn(o[k], __fmul_rn(gk, lr));        // Scale then Sub, like the plain SGD kernel
            }
            *reinterpret_cast<float4*>(z + i) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
            for (int64_t j = i; j < count; ++j) {
                float gk = ld_sys(src + j);
                if (j >= n_sum) gk = __fmul_rn(gk, inv);
                z[j] = __fsub_rn(z[j], __fmul_rn(gk, lr));
            }
        }
    }
    // last CTA out: this rank has finished the step
    __syncthreads();
    __shared__ uint32_t s_last;
    if (threadIdx.x == 0) s_last = atomicAdd(mine + FLAG_DONE_UPDATE, 1u) == gridDim.x - 1;
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        mine[FLAG_DONE_UPDATE] = 0;
        mine[FLAG_STEP] = step;
    }
}

int check_group(const sb200_dp_group* g, DpGroup* out)
{
    if (!g || g->world < 1 || g->world > 8 || g->rank < 0 || g->rank >= g->world)
        return SB200_ERR_INVALID_ARG;
    out->world = g->world;
    out->rank = g->rank;
    for (int r = 0; r < 8; ++r) {
        const bool used = r < g->world;
        if (used && (!g->grads[r] || !g->reduced[r] || !g->flags[r]))
            return SB200_ERR_INVALID_ARG;
        if (used && ((reinterpret_cast<uintptr_t>(g->grads[r]) | reinterpret_cast<uintptr_t>(g->reduced[r])) & 15))
            return SB200_ERR_INVALID_ARG;
        out->grads[r] = used ? g->grads[r] : nullptr;
        out->reduced[r] = used ? g->reduced[r] : nullptr;
        out->flags[r] = used ? g->flags[r] : nullptr;
    }
    return SB200_OK;
}

// One warp: tell every peer that this rank's stream has reached barrier `step`, wait until
// every peer has said the same.  The count lives in the flag words: replays from a graph.
__global__ void __launch_bounds__(32)
peer_barrier_kernel(DpGroup g, unsigned long long limit_ns, unsigned* status)
{
    uint32_t* mine = g.flags[g.rank];
    const uint32_t step = mine[FLAG_BARRIER_STEP] + 1;
    __threadfence_system();
    if (static_cast<int>(threadIdx.x) < g.world)
        st_release_sys(g.flags[threadIdx.x] + FLAG_BARRIER + g.rank, step);
    wait_flags(mine, g.world, g.rank, FLAG_BARRIER, step, limit_ns, status, FAULT_PEER_WAIT);
    if (threadIdx.x == 0)
        mine[FLAG_BARRIER_STEP] = step;
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" int sb200_peer_barrier(sb200_ctx* ctx, uint32_t* const* flags, int world, int rank,
                                  sb200_stream stream_)
{
    TraceRange trace("sb200_peer_barrier");
    if (!ctx || !flags || world < 1 || world > 8 || rank < 0 || rank >= world)
        return SB200_ERR_INVALID_ARG;
    DpGroup g = {};
    g.world = world;
    g.rank = rank;
    for (int r = 0; r < world; ++r) {
        if (!flags[r] || (reinterpret_cast<uintptr_t>(flags[r]) & 3))
            return SB200_ERR_INVALID_ARG;
        g.flags[r] = flags[r];
    }
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(g, ctx->wait_limit_ns, ctx->d_status);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

extern "C" int sb200_dp_reduce(sb200_ctx* ctx, const sb200_dp_group* group, int64_t count,
                               sb200_stream stream_)
{
    TraceRange trace("sb200_dp_reduce");
    DpGroup g;
    if (!ctx || count < 0)
        return SB200_ERR_INVALID_ARG;
    if (const int rc = check_group(group, &g))
        return rc;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int64_t per = slice_len(count, g.world);
    int64_t blocks = (per / 4 + DP_THREADS - 1) / DP_THREADS;
    blocks = blocks < 1 ? 1 : (blocks > ctx->sm_count ? ctx->sm_count : blocks);
    dp_reduce_kernel<<<static_cast<unsigned>(blocks), DP_THREADS, 0, stream>>>(g, count, ctx->wait_limit_ns,
                                                                               ctx->d_status);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

extern "C" int sb200_dp_update(sb200_ctx* ctx, const sb200_dp_group* group, float* params, int64_t count,
                               int64_t n_sum, float lr, sb200_stream stream_)
{
    TraceRange trace("sb200_dp_update");
    DpGroup g;
    if (!ctx || count < 0 || n_sum < 0 || (count && !params) ||
        (reinterpret_cast<uintptr_t>(params) & 15))
        return SB200_ERR_INVALID_ARG;
    if (const int rc = check_group(group, &g))
        return rc;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int64_t blocks = (count / 4 + DP_THREADS) / DP_THREADS;
    blocks = blocks < 1 ? 1 : (blocks > 2 * ctx->sm_count ? 2 * ctx->sm_count : blocks);
    dp_update_kernel<<<static_cast<unsigned>(blocks), DP_THREADS, 0, stream>>>(g, params, count, n_sum, lr,
                                                                               ctx->wait_limit_ns, ctx->d_status);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}
