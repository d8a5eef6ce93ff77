// Batched fp32 GEMM on pairs of SMs (thread-block clusters of two CTAs,
// tcgen05 cta_group::2): one 256 x 256 output tile per pair.
//
// Each CTA of a pair holds 128 rows of op(A) and HALF of the tile's op(B) (128
// of its 256 columns) per stage; the pair's tensor cores read both halves.  Per
// k-block a CTA therefore receives 32 KB instead of the 48 KB a stand-alone
// 128 x 256 CTA needs, which is what limits the one-CTA kernel: its shared
// memory has to take in and feed back 96 KB per 128 x 256 x 32 MACs.
//
// Roles per CTA as in the one-CTA kernel (TMA producer, MMA issuer, four
// epilogue warps), with these differences:
//   * only the leader (cluster rank 0) issues tcgen05.mma, with M = 256;
//   * "stage filled" is one barrier in the leader: its producer announces the
//     bytes of both CTAs and both CTAs' TMA loads complete on it
//     (cp.async.bulk.tensor ... .cta_group::2, no multicast);
//   * "stage free" and "accumulator ready" are signalled to both CTAs by a
//     multicast tcgen05.commit; "accumulator drained" is one barrier in the
//     leader that the epilogue warps of both CTAs arrive on.
// TF32 mode only; the fp32-accurate split mode runs on the one-CTA kernel.
#include <cstdio>
#include <cstdlib>

#include "gemm_common.cuh"

namespace sb200 {

using namespace gemm;

namespace {

constexpr int PAIR_M = 256;             // rows per pair tile (128 per CTA)
constexpr int PAIR_N = 256;             // columns per pair tile (128 loaded per CTA)
constexpr int HALF_N = PAIR_N / 2;
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_PANEL = 8;           // row tiles (of 256 rows) per panel of the tile order
constexpr int B_HALF_BYTES = HALF_N * BLOCK_K * 4;              // 16 KB
constexpr int PAIR_STAGE_BYTES = A_TILE_BYTES + B_HALF_BYTES;   // 32 KB
constexpr int PAIR_TILES_BYTES = PAIR_STAGE_BYTES * PAIR_STAGES;
constexpr int PAIR_BAR_BYTES = ((2 * PAIR_STAGES + 4) * 8 + 16 + 15) & ~15;
constexpr int PAIR_SMEM = PAIR_TILES_BYTES + PAIR_BAR_BYTES + 4 * EPI_STAGE_BYTES_PER_WARP + 1024;

// waits of this kernel see arrivals from the peer CTA: cluster-scope acquire
__device__ __forceinline__ bool wait_bar_cluster(uint64_t* bar, uint32_t parity, const Abort& ab,
                                                 unsigned code)
{
    // The global timer is slow to read: the clock of a wait starts at its 64th failed
    // try, so the waits of the steady state (a few tries) never read it.
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (!ptx::mbar_try_wait_cluster(bar, parity)) {
        if ((++spins & 63u) == 0) {
            if (*ab.flag)
                return false;
            const uint64_t now = ptx::globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > ab.limit_ns) {
                *ab.flag = 1;
                atomicCAS(ab.status, 0u, code);
                return false;
            }
        }
    }
    return true;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap mapA,
                         const __grid_constant__ CUtensorMap mapB, const KernelParams p)
{
    constexpr uint32_t TMEM_COLS = 512;                          // two 256-column accumulators

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + PAIR_TILES_BYTES);
    uint64_t* empty_bar = full_bar + PAIR_STAGES;
    uint64_t* tmem_full = empty_bar + PAIR_STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* epi_stage = reinterpret_cast<float*>(smem + PAIR_TILES_BYTES + PAIR_BAR_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();                // 0 = leader
    const Abort ab{abort_flag, p.status, p.wait_limit_ns};

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);        // the leader's producer announces both CTAs' bytes
            ptx::mbar_init(&empty_bar[s], 1);       // one multicast commit
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&tmem_full[i], 1);       // one multicast commit
            ptx::mbar_init(&tmem_empty[i], 8);      // 4 epilogue warps x 2 CTAs (leader's copy used)
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&mapA);
        ptx::prefetch_tensormap(&mapB);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();                 // both CTAs' barriers and TMEM exist before any remote use
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const long long tiles_per_batch = static_cast<long long>(p.tiles_m) * p.tiles_n;
    const long long pair_id = blockIdx.x >> 1;
    const long long n_pairs = gridDim.x >> 1;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int issued = 0;
            for (long long t = pair_id; ok && t < p.total_tiles; t += n_pairs) {
                const int b = static_cast<int>(t / tiles_per_batch);
                const int r = static_cast<int>(t % tiles_per_batch);
                int tm, tn;
                tile_coords(r, p.tiles_m, p.tiles_n, PAIR_PANEL, tm, tn);
                const int m0 = tm * PAIR_M + static_cast<int>(rank) * BLOCK_M;
                const int n0 = tn * PAIR_N + static_cast<int>(rank) * HALF_N;
                const int ba = p.a_batched ? b : 0;
                const int bb = p.b_batched ? b : 0;
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (p.test_stall_kb >= 0 && issued++ >= p.test_stall_kb) {
                        ok = false;                        // test hook: the other roles' waits run out
                        break;
                    }
                    if (!(ok = wait_bar_cluster(&empty_bar[s], ph ^ 1u, ab, FAULT_PRODUCER_WAIT)))
                        break;
                    uint8_t* sa = smem + s * PAIR_STAGE_BYTES;
                    uint8_t* sb = sa + A_TILE_BYTES;
                    const int k0 = kb * BLOCK_K;
                    const uint32_t lead_full = ptx::map_to_cta(ptx::smem_u32(&full_bar[s]), 0);
                    // one arrival for the pair: a remote arrive per k-block from the peer's
                    // producer halves the throughput of the whole kernel
                    if (rank == 0)
                        ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * PAIR_STAGE_BYTES);
                    if (A_MN && p.a_merged) {
                        ptx::tma_load_4d_pair(sa, &mapA, lead_full, 0, k0, m0 / 32, ba);
                    } else if (A_MN) {
#pragma unroll
                        for (int c = 0; c < BLOCK_M / 32; ++c)
                            ptx::tma_load_3d_pair(sa + c * CHUNK_BYTES, &mapA, lead_full,
                                                  m0 + c * 32, k0, ba);
                    } else {
                        ptx::tma_load_3d_pair(sa, &mapA, lead_full, k0, m0, ba);
                    }
                    if (B_MN && p.b_merged) {
                        ptx::tma_load_4d_pair(sb, &mapB, lead_full, 0, k0, n0 / 32, bb);
                    } else if (B_MN) {
#pragma unroll
                        for (int c = 0; c < HALF_N / 32; ++c)
                            ptx::tma_load_3d_pair(sb + c * CHUNK_BYTES, &mapB, lead_full,
                                                  n0 + c * 32, k0, bb);
                    } else {
                        ptx::tma_load_3d_pair(sb, &mapB, lead_full, k0, n0, bb);
                    }
                    if (++s == PAIR_STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_tf32(PAIR_M, PAIR_N, A_MN, B_MN);
            constexpr uint32_t A_KSTEP = A_MN ? 1024u : UMMA_K * 4u;
            constexpr uint32_t B_KSTEP = B_MN ? 1024u : UMMA_K * 4u;
            constexpr uint32_t A_LBO = A_MN ? CHUNK_BYTES : 16u;
            constexpr uint32_t B_LBO = B_MN ? CHUNK_BYTES : 16u;
            constexpr uint32_t A_SBO = A_MN ? 512u : 1024u;
            constexpr uint32_t B_SBO = B_MN ? 512u : 1024u;
            constexpr uint32_t A_LAY = A_MN ? ptx::LAYOUT_SW128_BASE32 : ptx::LAYOUT_SW128;
            constexpr uint32_t B_LAY = B_MN ? ptx::LAYOUT_SW128_BASE32 : ptx::LAYOUT_SW128;
            int s = 0;
            uint32_t ph = 0;
            int acc = 0;
            uint32_t acc_ph = 0;
            bool ok = true;
            for (long long t = pair_id; ok && t < p.total_tiles; t += n_pairs) {
                if (!(ok = wait_bar_cluster(&tmem_empty[acc], acc_ph ^ 1u, ab, FAULT_MMA_WAIT_TMEM)))
                    break;
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * PAIR_N);
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (!(ok = wait_bar_cluster(&full_bar[s], ph, ab, FAULT_MMA_WAIT_FULL)))
                        break;
                    ptx::tc_fence_after_sync();
                    const uint32_t sa = ptx::smem_u32(smem + s * PAIR_STAGE_BYTES);
                    const uint32_t sb = sa + A_TILE_BYTES;
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t a_desc =
                            ptx::make_smem_desc(sa + k * A_KSTEP, A_LBO, A_SBO, A_LAY);
                        const uint64_t b_desc =
                            ptx::make_smem_desc(sb + k * B_KSTEP, B_LBO, B_SBO, B_LAY);
                        ptx::mma_tf32_pair(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    ptx::mma_commit_pair(&empty_bar[s], 3);     // stage free in both CTAs
                    if (++s == PAIR_STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (!ok)
                    break;
                ptx::mma_commit_pair(&tmem_full[acc], 3);       // accumulator ready in both CTAs
                acc ^= 1;
                if (acc == 0)
                    acc_ph ^= 1u;
            }
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int q = warp & 3;
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        const bool vec_ok = ((p.ldd & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) &&
                            ((p.strideD & 3) == 0) &&
                            (p.C == nullptr ||
                             (((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                              ((p.strideC & 3) == 0)));
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        for (long long t = pair_id; ok && t < p.total_tiles; t += n_pairs) {
            const int b = static_cast<int>(t / tiles_per_batch);
            const int r = static_cast<int>(t % tiles_per_batch);
            int tm, tn;
            tile_coords(r, p.tiles_m, p.tiles_n, PAIR_PANEL, tm, tn);
            const int m0 = tm * PAIR_M + static_cast<int>(rank) * BLOCK_M;
            const int n0 = tn * PAIR_N;
            const int row = m0 + q * 32 + lane;
            float* dmat = p.D + b * p.strideD;
            if (p.rows_per_owner) {
                // reduce-scatter: the tile lies inside one owner's row block; shift that
                // owner's buffer so that absolute row numbers index it
                // (a tile wholly beyond M maps past the last owner: clamp, its rows are masked)
                const int o = min(m0 / p.rows_per_owner, MAX_OWNERS - 1);
                dmat = p.owner[o] - static_cast<long long>(o) * p.rows_per_owner * p.ldd;
            }
            const float* cmat = p.C ? p.C + b * p.strideC : nullptr;
            float* drow = dmat + static_cast<long long>(row) * p.ldd;
            const float* crow = cmat ? cmat + static_cast<long long>(row) * p.ldc : nullptr;
            float* my_stage = epi_stage + q * (EPI_STAGE_BYTES_PER_WARP / 4);
            const Epilogue epi{p.bias, p.mask ? p.mask + b * p.strideM : nullptr, p.ldm, p.relu,
                               p.rows_per_owner != 0 && !p.owner_store};
            // the first chunk's C is requested before the wait for the accumulator: it
            // travels under the tile's main loop
            CChunk c_now, c_next;
            if (vec_ok)                                    // zeros when there is no C
                load_c_chunk(c_next, cmat, p.ldc, m0 + q * 32, n0, p.M, p.N);
            if (!(ok = wait_bar_cluster(&tmem_full[acc], acc_ph, ab, FAULT_EPI_WAIT)))
                break;
            ptx::tc_fence_after_sync();
#pragma unroll 1
            for (int c = 0; c < PAIR_N / 32; ++c) {
                const int col0 = n0 + c * 32;
                if (col0 >= p.N)
                    break;
                uint32_t v[32];
                ptx::tmem_ld_32x32(lane_base + static_cast<uint32_t>(acc * PAIR_N + c * 32), v);
                if (vec_ok && (cmat || c == 0)) {
                    c_now = c_next;
                    if (c + 1 < PAIR_N / 32 && col0 + 32 < p.N)          // next chunk's C, ahead of the stores
                        load_c_chunk(c_next, cmat, p.ldc, m0 + q * 32, col0 + 32, p.M, p.N);
                }
                ptx::tmem_ld_wait();
                if (vec_ok)
                    store_chunk_coalesced(v, my_stage, dmat, p.ldd, c_now, epi, m0 + q * 32,
                                          col0, p.M, p.N);
                else if (row < p.M)
                    store_row_chunk(v, drow, crow, epi,
                                    epi.mask ? epi.mask + static_cast<long long>(row) * p.ldm : nullptr,
                                    col0, p.N, false);
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&tmem_empty[acc]), 0));
            acc ^= 1;
            if (acc == 0)
                acc_ph ^= 1u;
        }
    }

    // common exit: no CTA may leave while its peer can still touch its barriers or TMEM
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

template <bool A_MN, bool B_MN>
int launch_pair_variant(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream)
{
    auto kern = gemm_tcgen05_pair_kernel<A_MN, B_MN>;
    static bool attr_done[16] = {};
    if (ctx->device >= 16 || !attr_done[ctx->device]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM) !=
            cudaSuccess)
            return SB200_ERR_CUDA;
        if (ctx->device < 16)
            attr_done[ctx->device] = true;
    }
    CUtensorMap mapA, mapB;
    int rc;
    const bool a_merged = A_MN && (g.M % 32 == 0) && ctx->merge_mn_boxes;
    const bool b_merged = B_MN && (g.N % 32 == 0) && ctx->merge_mn_boxes;
    if (a_merged)
        rc = make_map_merged(ctx, &mapA, g.A, g.M, g.K, g.lda, g.batch, g.strideA, BLOCK_M / 32);
    else if (A_MN)
        rc = make_map(ctx, &mapA, g.A, g.M, g.K, g.lda, g.batch, g.strideA, BLOCK_K, true);
    else
        rc = make_map(ctx, &mapA, g.A, g.K, g.M, g.lda, g.batch, g.strideA, BLOCK_M, false);
    if (rc)
        return rc;
    if (b_merged)
        rc = make_map_merged(ctx, &mapB, g.B, g.N, g.K, g.ldb, g.batch, g.strideB, HALF_N / 32);
    else if (B_MN)
        rc = make_map(ctx, &mapB, g.B, g.N, g.K, g.ldb, g.batch, g.strideB, BLOCK_K, true);
    else
        rc = make_map(ctx, &mapB, g.B, g.K, g.N, g.ldb, g.batch, g.strideB, HALF_N, false);
    if (rc)
        return rc;

    KernelParams p;
    p.M = static_cast<int>(g.M);
    p.N = static_cast<int>(g.N);
    p.K = static_cast<int>(g.K);
    p.batch = static_cast<int>(g.batch);
    p.tiles_m = static_cast<int>((g.M + PAIR_M - 1) / PAIR_M);
    p.tiles_n = static_cast<int>((g.N + PAIR_N - 1) / PAIR_N);
    p.num_kb = static_cast<int>((g.K + BLOCK_K - 1) / BLOCK_K);
    p.chunk_kb = p.num_kb > 0 ? p.num_kb : 1;
    p.total_tiles = static_cast<long long>(p.tiles_m) * p.tiles_n * g.batch;
    p.a_batched = g.strideA != 0;
    p.b_batched = g.strideB != 0;
    p.a_merged = a_merged;
    p.b_merged = b_merged;
    p.C = g.C; p.ldc = g.ldc; p.strideC = g.strideC;
    p.D = g.D; p.ldd = g.ldd; p.strideD = g.strideD;
    p.bias = g.bias;
    p.relu = g.relu;
    p.mask = g.mask; p.ldm = g.ldmask; p.strideM = g.strideMask;
    for (int o = 0; o < MAX_OWNERS; ++o) p.owner[o] = g.owner[o];
    p.rows_per_owner = static_cast<int>(g.rows_per_owner);
    p.owner_store = g.owner_store;
    p.status = ctx->d_status;
    p.wait_limit_ns = ctx->wait_limit_ns;
    p.test_stall_kb = ctx->test_stall_kb;
    p.explicit_hi = 0;
    p.colsum_out = nullptr;
    p.acc_scale = 1.0f;
    p.colsum_lr = 0.0f;
    p.colsum_scale = 0.0f;

    // a persistent grid must be fully co-resident: ask how many pairs fit at once
    static int cached_pairs[16] = {};
    int fit = ctx->device < 16 ? cached_pairs[ctx->device] : 0;
    if (fit == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(ctx->sm_count & ~1));
        cfg.blockDim = dim3(192);
        cfg.dynamicSmemBytes = PAIR_SMEM;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&fit, kern, &cfg) != cudaSuccess || fit < 1) {
            cudaGetLastError();
            fit = ctx->sm_count / 4;                 // conservative
        }
        if (fit > ctx->sm_count / 2)
            fit = ctx->sm_count / 2;
        if (ctx->device < 16)
            cached_pairs[ctx->device] = fit;
        if (getenv("SB200_VERBOSE"))
            fprintf(stderr, "sb200: %d CTA pairs co-resident on device %d\n", fit, ctx->device);
    }
    const long long max_pairs = fit;
    const long long pairs = p.total_tiles < max_pairs ? p.total_tiles : max_pairs;
    kern<<<static_cast<unsigned>(2 * pairs), 192, PAIR_SMEM, stream>>>(mapA, mapB, p);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

}  // namespace

// The pair kernel pays off when there are enough 256 x 256 tiles to fill the
// machine; smaller problems stay on the one-CTA kernel.
bool pair_kernel_preferred(const sb200_ctx* ctx, const GemmArgs& g)
{
    if (g.mode != SB200_MODE_TF32 || !ctx->use_cta_pairs)
        return false;
    // Fused column sums need a "stage filled" signal inside the CTA that holds the
    // B tile; in a pair that barrier lives in the leader only, so such requests
    // stay on the one-CTA kernel.
    if (g.colsum_out || g.acc_scale != 1.0f)           // (the in-place SGD epilogue likewise)
        return false;
    if (g.M < 2 * PAIR_M || g.N < PAIR_N)
        return false;
    const long long tiles = ((g.M + PAIR_M - 1) / PAIR_M) * ((g.N + PAIR_N - 1) / PAIR_N) * g.batch;
    return tiles >= ctx->sm_count / 2;
}

int launch_gemm_tcgen05_pair(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream)
{
    const bool a_mn = g.transA != 0;
    const bool b_mn = g.transB == 0;
    if (a_mn)
        return b_mn ? launch_pair_variant<true, true>(ctx, g, stream)
                    : launch_pair_variant<true, false>(ctx, g, stream);
    return b_mn ? launch_pair_variant<false, true>(ctx, g, stream)
                : launch_pair_variant<false, false>(ctx, g, stream);
}

}  // namespace sb200
