// Small TF32 GEMMs with a long inner dimension: split k inside a thread-block
// cluster.
//
// A product like 64 x 512 x 2048 (a wide Linear layer's forward pass at batch 64)
// has eight 128 x 64 output tiles and 64 k-blocks each.  One CTA per tile streams
// its 64 k-blocks through one SM, and one SM takes in about 100 GB/s however many
// stages are in flight: 0.27 us per k-block, 17 us of a serial walk while 140 SMs
// idle.  Here a cluster of S (2 or 4) CTAs shares one tile: CTA r multiplies
// k-blocks [r * kb_per, (r + 1) * kb_per) into its own TMEM accumulator, the
// CTAs r > 0 then write their partial accumulators into the leader's shared memory
// (distributed shared memory stores, one remote mbarrier arrive per warp and
// TILE, not per k-block), and the leader adds them to its own in fixed order
// (own + 1 + 2 + 3: bit-reproducible) and runs the ordinary epilogue -- C, bias,
// ReLU, gate -- so every epilogue the one-CTA kernel has survives the split.
//
// Roles per CTA as in the one-CTA kernel: warp 0 TMA producer, warp 1 MMA issuer,
// warps 2-5 epilogue.  Tiles are 128 x 64; 4 stages of 24 KB; the leader's buffer
// for the partial accumulators takes 3 x 34 KB.  Every wait is bounded; on expiry
// the CTA records a code, raises its abort flag and all roles fall to the common
// exit, a cluster barrier (no CTA leaves while a peer can still write its shared
// memory or arrive on its barriers).
#include "gemm_common.cuh"

namespace sb200 {

using namespace gemm;

namespace {

constexpr int SK_BLOCK_N = 64;
constexpr int SK_STAGES = 4;
constexpr int SK_MAX_SPLIT = 4;
constexpr int SK_PANEL = 16;
constexpr int SK_B_TILE_BYTES = SK_BLOCK_N * BLOCK_K * 4;                 // 8 KB
constexpr int SK_STAGE_BYTES = A_TILE_BYTES + SK_B_TILE_BYTES;            // 24 KB
constexpr int SK_TILES_BYTES = SK_STAGE_BYTES * SK_STAGES;
constexpr int SK_PART_LD = SK_BLOCK_N + 4;                                // floats per row of a partial tile (272 B:
                                                                          // 16-byte accesses of 32 rows hit 8 bank groups)
constexpr int SK_PART_BYTES = BLOCK_M * SK_PART_LD * 4;                   // one peer's partial accumulator
// barriers: full, empty per stage; tmem_full, tmem_empty x 2; partial_full, partial_free
constexpr int SK_BAR_BYTES = ((2 * SK_STAGES + 4 + 2) * 8 + 16 + 15) & ~15;
constexpr int SK_SMEM = SK_TILES_BYTES + SK_BAR_BYTES + (SK_MAX_SPLIT - 1) * SK_PART_BYTES +
                        4 * EPI_STAGE_BYTES_PER_WARP + 1024;
constexpr uint32_t SK_TMEM_COLS = 2 * SK_BLOCK_N;                         // two accumulators

__device__ __forceinline__ bool wait_cluster(uint64_t* bar, uint32_t parity, const Abort& ab, unsigned code)
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

__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, float4 v)
{
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(v.x), "f"(v.y),
                 "f"(v.z), "f"(v.w)
                 : "memory");
}

__device__ __forceinline__ void arrive_cluster_release(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ uint32_t cluster_size()
{
    uint32_t n;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
    return n;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_splitk_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                           const KernelParams p, const int kb_per_cta)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SK_TILES_BYTES);
    uint64_t* empty_bar = full_bar + SK_STAGES;
    uint64_t* tmem_full = empty_bar + SK_STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint64_t* partial_full = tmem_empty + 2;          // leader: every peer warp has written its part of the tile
    uint64_t* partial_free = partial_full + 1;        // peers: the leader has read the partial tiles
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(partial_free + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* partials = reinterpret_cast<float*>(smem + SK_TILES_BYTES + SK_BAR_BYTES);
    float* epi_stage = partials + (SK_MAX_SPLIT - 1) * (SK_PART_BYTES / 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();     // 0 = leader: owns the epilogue
    const uint32_t split = cluster_size();
    const Abort ab{abort_flag, p.status, p.wait_limit_ns};

    if (threadIdx.x == 0) {
        for (int s = 0; s < SK_STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&tmem_full[i], 1);
            ptx::mbar_init(&tmem_empty[i], 4);
        }
        ptx::mbar_init(partial_full, (split - 1) * 4);          // 4 epilogue warps of every peer
        ptx::mbar_init(partial_free, 4);                        // the leader's 4 epilogue warps
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&mapA);
        ptx::prefetch_tensormap(&mapB);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, SK_TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();                 // every CTA's barriers exist before any remote arrive or store
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // everything above touched only shared memory, TMEM and kernel parameters
    ptx::griddep_launch_dependents();
    ptx::griddep_wait();

    const long long tiles_per_batch = static_cast<long long>(p.tiles_m) * p.tiles_n;
    const long long cluster_id = blockIdx.x / split;
    const long long n_clusters = gridDim.x / split;
    const int kb_begin = static_cast<int>(rank) * kb_per_cta;
    const int kb_end = min(kb_begin + kb_per_cta, p.num_kb);    // the host guarantees kb_begin < num_kb

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int issued = 0;
            for (long long t = cluster_id; ok && t < p.total_tiles; t += n_clusters) {
                const int b = static_cast<int>(t / tiles_per_batch);
                const int r = static_cast<int>(t % tiles_per_batch);
                int tm, tn;
                tile_coords(r, p.tiles_m, p.tiles_n, SK_PANEL, tm, tn);
                const int m0 = tm * BLOCK_M;
                const int n0 = tn * SK_BLOCK_N;
                const int ba = p.a_batched ? b : 0;
                const int bb = p.b_batched ? b : 0;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (p.test_stall_kb >= 0 && issued++ >= p.test_stall_kb) {
                        ok = false;                        // test hook: the other roles' waits run out
                        break;
                    }
                    if (!(ok = wait_bar(&empty_bar[s], ph ^ 1u, ab, FAULT_PRODUCER_WAIT)))
                        break;
                    uint8_t* sa = smem + s * SK_STAGE_BYTES;
                    uint8_t* sb = sa + A_TILE_BYTES;
                    const int k0 = kb * BLOCK_K;
                    ptx::mbar_arrive_expect_tx(&full_bar[s], SK_STAGE_BYTES);
                    if (A_MN && p.a_merged) {
                        ptx::tma_load_4d(sa, &mapA, &full_bar[s], 0, k0, m0 / 32, ba);
                    } else if (A_MN) {
#pragma unroll
                        for (int c = 0; c < BLOCK_M / 32; ++c)
                            ptx::tma_load_3d(sa + c * CHUNK_BYTES, &mapA, &full_bar[s], m0 + c * 32, k0, ba);
                    } else {
                        ptx::tma_load_3d(sa, &mapA, &full_bar[s], k0, m0, ba);
                    }
                    if (B_MN && p.b_merged) {
                        ptx::tma_load_4d(sb, &mapB, &full_bar[s], 0, k0, n0 / 32, bb);
                    } else if (B_MN) {
#pragma unroll
                        for (int c = 0; c < SK_BLOCK_N / 32; ++c)
                            ptx::tma_load_3d(sb + c * CHUNK_BYTES, &mapB, &full_bar[s], n0 + c * 32, k0, bb);
                    } else {
                        ptx::tma_load_3d(sb, &mapB, &full_bar[s], k0, n0, bb);
                    }
                    if (++s == SK_STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_tf32(BLOCK_M, SK_BLOCK_N, A_MN, B_MN);
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
            for (long long t = cluster_id; ok && t < p.total_tiles; t += n_clusters) {
                if (!(ok = wait_bar(&tmem_empty[acc], acc_ph ^ 1u, ab, FAULT_MMA_WAIT_TMEM)))
                    break;
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * SK_BLOCK_N);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!(ok = wait_bar(&full_bar[s], ph, ab, FAULT_MMA_WAIT_FULL)))
                        break;
                    ptx::tc_fence_after_sync();
                    const uint32_t sa = ptx::smem_u32(smem + s * SK_STAGE_BYTES);
                    const uint32_t sb = sa + A_TILE_BYTES;
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t a_desc = ptx::make_smem_desc(sa + k * A_KSTEP, A_LBO, A_SBO, A_LAY);
                        const uint64_t b_desc = ptx::make_smem_desc(sb + k * B_KSTEP, B_LBO, B_SBO, B_LAY);
                        ptx::mma_tf32(d_tmem, a_desc, b_desc, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
                    }
                    ptx::mma_commit(&empty_bar[s]);
                    if (++s == SK_STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (!ok)
                    break;
                ptx::mma_commit(&tmem_full[acc]);
                acc ^= 1;
                if (acc == 0)
                    acc_ph ^= 1u;
            }
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int q = warp & 3;                           // TMEM lane quadrant of this warp
        int acc = 0;
        uint32_t acc_ph = 0, part_ph = 0;
        bool ok = true;
        const bool vec_ok = ((p.ldd & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) &&
                            ((p.strideD & 3) == 0) &&
                            (p.C == nullptr ||
                             (((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                              ((p.strideC & 3) == 0)));
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        // this lane's row inside a partial tile
        const uint32_t my_row_off = static_cast<uint32_t>((q * 32 + lane) * SK_PART_LD * 4);
        for (long long t = cluster_id; ok && t < p.total_tiles; t += n_clusters) {
            if (rank != 0) {
                // ---- a peer: hand the partial accumulator to the leader
                if (!(ok = wait_bar(&tmem_full[acc], acc_ph, ab, FAULT_EPI_WAIT)))
                    break;
                // the leader has read what this CTA wrote for the previous tile
                if (!(ok = wait_cluster(partial_free, part_ph ^ 1u, ab, FAULT_EPI_WAIT)))
                    break;
                ptx::tc_fence_after_sync();
                const uint32_t dst = ptx::map_to_cta(
                    ptx::smem_u32(partials) + (rank - 1) * SK_PART_BYTES + my_row_off, 0);
#pragma unroll
                for (int c = 0; c < SK_BLOCK_N / 32; ++c) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(lane_base + static_cast<uint32_t>(acc * SK_BLOCK_N + c * 32), v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        st_cluster_v4(dst + (c * 32 + j) * 4,
                                      make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                  __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])));
                }
                ptx::tc_fence_before_sync();
                asm volatile("fence.acq_rel.cluster;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    arrive_cluster_release(ptx::map_to_cta(ptx::smem_u32(partial_full), 0));
                    ptx::mbar_arrive(&tmem_empty[acc]);
                }
                part_ph ^= 1u;
            } else {
                // ---- the leader: own accumulator + the peers' partial tiles, then the epilogue proper
                const int b = static_cast<int>(t / tiles_per_batch);
                const int r = static_cast<int>(t % tiles_per_batch);
                int tm, tn;
                tile_coords(r, p.tiles_m, p.tiles_n, SK_PANEL, tm, tn);
                const int m0 = tm * BLOCK_M;
                const int n0 = tn * SK_BLOCK_N;
                const int row = m0 + q * 32 + lane;
                float* dmat = p.D + b * p.strideD;
                const float* cmat = p.C ? p.C + b * p.strideC : nullptr;
                float* drow = dmat + static_cast<long long>(row) * p.ldd;
                const float* crow = cmat ? cmat + static_cast<long long>(row) * p.ldc : nullptr;
                float* my_stage = epi_stage + q * (EPI_STAGE_BYTES_PER_WARP / 4);
                const Epilogue epi{p.bias, p.mask ? p.mask + b * p.strideM : nullptr, p.ldm, p.relu, false};
                const float* mrow = epi.mask ? epi.mask + static_cast<long long>(row) * p.ldm : nullptr;
                CChunk c_now, c_next;
                if (vec_ok)                                    // travels under the main loop
                    load_c_chunk(c_next, cmat, p.ldc, m0 + q * 32, n0, p.M, p.N);
                if (!(ok = wait_bar(&tmem_full[acc], acc_ph, ab, FAULT_EPI_WAIT)))
                    break;
                if (!(ok = wait_cluster(partial_full, part_ph, ab, FAULT_EPI_WAIT)))
                    break;
                ptx::tc_fence_after_sync();
                const float* my_part = reinterpret_cast<const float*>(
                    reinterpret_cast<const uint8_t*>(partials) + my_row_off);
#pragma unroll 1
                for (int c = 0; c < SK_BLOCK_N / 32; ++c) {
                    const int col0 = n0 + c * 32;
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(lane_base + static_cast<uint32_t>(acc * SK_BLOCK_N + c * 32), v);
                    if (vec_ok && (cmat || c == 0)) {
                        c_now = c_next;
                        if (c + 1 < SK_BLOCK_N / 32 && col0 + 32 < p.N)
                            load_c_chunk(c_next, cmat, p.ldc, m0 + q * 32, col0 + 32, p.M, p.N);
                    }
                    ptx::tmem_ld_wait();
                    for (uint32_t pr = 0; pr + 1 < split; ++pr) {          // fixed order: reproducible
                        const float4* src = reinterpret_cast<const float4*>(
                            my_part + pr * (SK_PART_BYTES / 4) + c * 32);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 x = src[j];
                            v[4 * j] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * j]), x.x));
                            v[4 * j + 1] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * j + 1]), x.y));
                            v[4 * j + 2] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * j + 2]), x.z));
                            v[4 * j + 3] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * j + 3]), x.w));
                        }
                    }
                    if (col0 >= p.N)
                        continue;                              // uniform across the warp
                    if (vec_ok)
                        store_chunk_coalesced(v, my_stage, dmat, p.ldd, c_now, epi, m0 + q * 32, col0, p.M, p.N);
                    else if (row < p.M)
                        store_row_chunk(v, drow, crow, epi, mrow, col0, p.N, false);
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    for (uint32_t pr = 1; pr < split; ++pr)
                        arrive_cluster_release(ptx::map_to_cta(ptx::smem_u32(partial_free), pr));
                    ptx::mbar_arrive(&tmem_empty[acc]);
                }
                part_ph ^= 1u;
            }
            acc ^= 1;
            if (acc == 0)
                acc_ph ^= 1u;
        }
    }

    // common exit: every thread arrives here, also after an abort; no CTA leaves while a
    // peer can still write its shared memory or arrive on its barriers
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, SK_TMEM_COLS);
    }
}

template <bool A_MN, bool B_MN>
int launch_splitk_variant(sb200_ctx* ctx, const GemmArgs& g, int split, cudaStream_t stream)
{
    auto kern = gemm_tcgen05_splitk_kernel<A_MN, B_MN>;
    static bool attr_done[16] = {};
    if (ctx->device >= 16 || !attr_done[ctx->device]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM) != cudaSuccess)
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
        rc = make_map_merged(ctx, &mapB, g.B, g.N, g.K, g.ldb, g.batch, g.strideB, SK_BLOCK_N / 32);
    else if (B_MN)
        rc = make_map(ctx, &mapB, g.B, g.N, g.K, g.ldb, g.batch, g.strideB, BLOCK_K, true);
    else
        rc = make_map(ctx, &mapB, g.B, g.K, g.N, g.ldb, g.batch, g.strideB, SK_BLOCK_N, false);
    if (rc)
        return rc;

    KernelParams p;
    p.M = static_cast<int>(g.M);
    p.N = static_cast<int>(g.N);
    p.K = static_cast<int>(g.K);
    p.batch = static_cast<int>(g.batch);
    p.tiles_m = static_cast<int>((g.M + BLOCK_M - 1) / BLOCK_M);
    p.tiles_n = static_cast<int>((g.N + SK_BLOCK_N - 1) / SK_BLOCK_N);
    p.num_kb = static_cast<int>((g.K + BLOCK_K - 1) / BLOCK_K);
    p.chunk_kb = p.num_kb;
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
    for (int o = 0; o < MAX_OWNERS; ++o) p.owner[o] = nullptr;
    p.rows_per_owner = 0;
    p.status = ctx->d_status;
    p.wait_limit_ns = ctx->wait_limit_ns;
    p.test_stall_kb = ctx->test_stall_kb;
    p.explicit_hi = 0;
    p.colsum_out = nullptr;
    p.colsum_scale = 0.0f;
    const int kb_per_cta = (p.num_kb + split - 1) / split;

    long long clusters = ctx->sm_count / split;
    if (clusters > p.total_tiles)
        clusters = p.total_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * split));
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = SK_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(split);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, mapA, mapB, p, kb_per_cta);
    ctx->launches += 1;
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? SB200_OK : SB200_ERR_CUDA;
}

}  // namespace

// How many CTAs should share each 128 x 64 tile of this request: 1 = the one-CTA
// kernel as before.  Only TF32 requests that the one-CTA kernel would run with
// 64-column tiles (few tiles) and whose inner dimension is long enough to pay for
// the cluster: measured against the one-CTA kernel (3.7 us + 0.27 us per k-block)
// a cluster of 2 costs 3.6 us more before it starts saving, a cluster of 4 5.7 us
// (cluster launch, two cluster barriers, the exchange of the partial tiles after
// the main loop), so both pay from about 32 k-blocks on: 64 x 512 x 784 is 11.3 us
// either way, 64 x 512 x 2048 14.0 against 21.6 us, 64 x 512 x 4096 18.5 against 39.2.
int cluster_split_k(const sb200_ctx* ctx, const GemmArgs& g)
{
    if (!ctx->cluster_split_k || g.mode != SB200_MODE_TF32 || g.colsum_out || g.rows_per_owner)
        return 1;
    const long long num_kb = (g.K + BLOCK_K - 1) / BLOCK_K;
    const long long tiles = ((g.M + BLOCK_M - 1) / BLOCK_M) * ((g.N + SK_BLOCK_N - 1) / SK_BLOCK_N) * g.batch;
    if (num_kb < 32)
        return 1;
    int split = tiles * 4 <= ctx->sm_count ? 4 : 2;
    if (tiles * split > ctx->sm_count)
        return 1;
    // every CTA of the cluster must own at least one k-block
    while (split > 1 && (split - 1) * ((num_kb + split - 1) / split) >= num_kb)
        split >>= 1;
    return split;
}

int launch_gemm_tcgen05_splitk(sb200_ctx* ctx, const GemmArgs& g, int split, cudaStream_t stream)
{
    const bool a_mn = g.transA != 0;
    const bool b_mn = g.transB == 0;
    if (a_mn)
        return b_mn ? launch_splitk_variant<true, true>(ctx, g, split, stream)
                    : launch_splitk_variant<true, false>(ctx, g, split, stream);
    return b_mn ? launch_splitk_variant<false, true>(ctx, g, split, stream)
                : launch_splitk_variant<false, false>(ctx, g, split, stream);
}

}  // namespace sb200
