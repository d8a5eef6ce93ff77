// Small TF32 GEMMs with few output tiles: slices of k on separate SMs, summed by
// whichever CTA of a tile finishes last.
//
// A product like 64 x 512 x 784 (a Linear layer's forward pass at batch 64) has
// eight 128 x 64 output tiles of 25 k-blocks each.  One CTA per tile streams its
// k-blocks through one SM at 0.27 us per k-block (the round trip commit -> producer
// -> TMA -> MMA over the eight stages one SM holds) while 140 SMs idle.  Here S CTAs
// share a tile: CTA r multiplies k-blocks [r * per, (r + 1) * per) into its TMEM
// accumulator, writes the partial tile to the context's workspace (L2) and takes a
// ticket from the tile's counter; the CTA that draws the last ticket adds the S
// partial tiles in slice order 0 .. S-1 -- its own from the workspace too, so the sum
// is the same whichever CTA does it: bit-reproducible -- and runs the ordinary
// epilogue (C, bias, ReLU, gate).  No CTA waits for another: no cluster, nothing to
// co-schedule, no spin.  The last CTA sets the counter back to zero for the next
// launch; a CTA whose waits ran out still takes its ticket, so the counters survive
// an abort.
//
// Roles per CTA as in the one-CTA kernel: warp 0 TMA producer, warp 1 MMA issuer,
// warps 2-5 epilogue.  Tiles are 128 x 64, 8 stages of 24 KB, one accumulator.
#include "gemm_common.cuh"

namespace sb200 {

using namespace gemm;

namespace {

constexpr int SL_BLOCK_N = 64;
constexpr int SL_STAGES = 8;
constexpr int SL_PANEL = 16;
constexpr int SL_B_TILE_BYTES = SL_BLOCK_N * BLOCK_K * 4;                 // 8 KB
constexpr int SL_STAGE_BYTES = A_TILE_BYTES + SL_B_TILE_BYTES;            // 24 KB
constexpr int SL_TILES_BYTES = SL_STAGE_BYTES * SL_STAGES;
constexpr int SL_BAR_BYTES = ((2 * SL_STAGES + 1) * 8 + 16 + 15) & ~15;   // full, empty per stage; tmem_full
constexpr int SL_SMEM = SL_TILES_BYTES + SL_BAR_BYTES + 4 * EPI_STAGE_BYTES_PER_WARP + 1024;
constexpr uint32_t SL_TMEM_COLS = SL_BLOCK_N;
constexpr int SL_PART_FLOATS = BLOCK_M * SL_BLOCK_N;                      // one partial tile: 32 KB

// epilogue warps only (threads 64 .. 191)
__device__ __forceinline__ void epilogue_barrier()
{
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_slices_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                           const KernelParams p, const int split, const int kb_per_cta, float* partials,
                           unsigned* tickets)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SL_TILES_BYTES);
    uint64_t* empty_bar = full_bar + SL_STAGES;
    uint64_t* tmem_full = empty_bar + SL_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* last_flag = abort_flag + 1;
    float* epi_stage = reinterpret_cast<float*>(smem + SL_TILES_BYTES + SL_BAR_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Abort ab{abort_flag, p.status, p.wait_limit_ns};

    if (threadIdx.x == 0) {
        for (int s = 0; s < SL_STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        ptx::mbar_init(tmem_full, 1);
        *abort_flag = 0;
        *last_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&mapA);
        ptx::prefetch_tensormap(&mapB);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, SL_TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // everything above touched only shared memory, TMEM and kernel parameters
    ptx::griddep_launch_dependents();
    ptx::griddep_wait();

    const long long tiles_per_batch = static_cast<long long>(p.tiles_m) * p.tiles_n;
    const long long tile = blockIdx.x / split;                  // one (tile, slice) per CTA
    const int slice = static_cast<int>(blockIdx.x % split);
    const int kb_begin = slice * kb_per_cta;
    const int kb_end = min(kb_begin + kb_per_cta, p.num_kb);    // the host guarantees kb_begin < num_kb
    const int b = static_cast<int>(tile / tiles_per_batch);
    int tm, tn;
    tile_coords(static_cast<int>(tile % tiles_per_batch), p.tiles_m, p.tiles_n, SL_PANEL, tm, tn);
    const int m0 = tm * BLOCK_M;
    const int n0 = tn * SL_BLOCK_N;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            int issued = 0;
            const int ba = p.a_batched ? b : 0;
            const int bb = p.b_batched ? b : 0;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (p.test_stall_kb >= 0 && issued++ >= p.test_stall_kb)
                    break;                                 // test hook: the other roles' waits run out
                if (!wait_bar(&empty_bar[s], ph ^ 1u, ab, FAULT_PRODUCER_WAIT))
                    break;
                uint8_t* sa = smem + s * SL_STAGE_BYTES;
                uint8_t* sb = sa + A_TILE_BYTES;
                const int k0 = kb * BLOCK_K;
                ptx::mbar_arrive_expect_tx(&full_bar[s], SL_STAGE_BYTES);
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
                    for (int c = 0; c < SL_BLOCK_N / 32; ++c)
                        ptx::tma_load_3d(sb + c * CHUNK_BYTES, &mapB, &full_bar[s], n0 + c * 32, k0, bb);
                } else {
                    ptx::tma_load_3d(sb, &mapB, &full_bar[s], k0, n0, bb);
                }
                if (++s == SL_STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_tf32(BLOCK_M, SL_BLOCK_N, A_MN, B_MN);
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
            bool ok = true;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (!(ok = wait_bar(&full_bar[s], ph, ab, FAULT_MMA_WAIT_FULL)))
                    break;
                ptx::tc_fence_after_sync();
                const uint32_t sa = ptx::smem_u32(smem + s * SL_STAGE_BYTES);
                const uint32_t sb = sa + A_TILE_BYTES;
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const uint64_t a_desc = ptx::make_smem_desc(sa + k * A_KSTEP, A_LBO, A_SBO, A_LAY);
                    const uint64_t b_desc = ptx::make_smem_desc(sb + k * B_KSTEP, B_LBO, B_SBO, B_LAY);
                    ptx::mma_tf32(tmem_base, a_desc, b_desc, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
                }
                ptx::mma_commit(&empty_bar[s]);
                if (++s == SL_STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
            if (ok)
                ptx::mma_commit(tmem_full);
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int q = warp & 3;                           // TMEM lane quadrant of this warp
        const int row_in_tile = q * 32 + lane;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        float* tile_parts = partials + tile * split * static_cast<long long>(SL_PART_FLOATS);
        const bool ok = wait_bar(tmem_full, 0, ab, FAULT_EPI_WAIT);
        if (ok) {
            // this CTA's partial tile as [column / 4][row][4]: lane = row, so every 16-byte
            // store of the warp lands in 512 contiguous bytes
            ptx::tc_fence_after_sync();
            float4* mine = reinterpret_cast<float4*>(tile_parts + slice * SL_PART_FLOATS) + row_in_tile;
#pragma unroll
            for (int c = 0; c < SL_BLOCK_N / 32; ++c) {
                uint32_t v[32];
                ptx::tmem_ld_32x32(lane_base + static_cast<uint32_t>(c * 32), v);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    mine[(c * 8 + j) * BLOCK_M] =
                        make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                    __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
            }
            __threadfence();
        }
        // the ticket is taken whatever happened above: the counter must come back to zero
        epilogue_barrier();
        if (warp == 2 && lane == 0) {
            const unsigned t = atomicAdd(&tickets[tile], 1u);
            if (t == static_cast<unsigned>(split - 1)) {
                tickets[tile] = 0;                        // every slice has drawn: ready for the next launch
                *last_flag = 1;
            }
        }
        epilogue_barrier();
        if (*last_flag && ok) {
            __threadfence();
            const bool vec_ok = ((p.ldd & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) &&
                                ((p.strideD & 3) == 0) &&
                                (p.C == nullptr ||
                                 (((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                                  ((p.strideC & 3) == 0)));
            const int row = m0 + row_in_tile;
            float* dmat = p.D + b * p.strideD;
            const float* cmat = p.C ? p.C + b * p.strideC : nullptr;
            float* drow = dmat + static_cast<long long>(row) * p.ldd;
            const float* crow = cmat ? cmat + static_cast<long long>(row) * p.ldc : nullptr;
            float* my_stage = epi_stage + q * (EPI_STAGE_BYTES_PER_WARP / 4);
            const Epilogue epi{p.bias, p.mask ? p.mask + b * p.strideM : nullptr, p.ldm, p.relu, false};
            const float* mrow = epi.mask ? epi.mask + static_cast<long long>(row) * p.ldm : nullptr;
            // the S partial tiles, in slice order (reproducible); a slice's 16 loads of 16
            // bytes are all in flight before the first add
            float acc[SL_BLOCK_N];
#pragma unroll
            for (int j = 0; j < SL_BLOCK_N; ++j)
                acc[j] = 0.0f;
#pragma unroll 1
            for (int r = 0; r < split; ++r) {
                const float4* src = reinterpret_cast<const float4*>(tile_parts + r * SL_PART_FLOATS) + row_in_tile;
                float4 x[SL_BLOCK_N / 4];
#pragma unroll
                for (int j = 0; j < SL_BLOCK_N / 4; ++j)
                    x[j] = __ldcg(src + j * BLOCK_M);      // written by other SMs: from L2, not through L1
#pragma unroll
                for (int j = 0; j < SL_BLOCK_N / 4; ++j) {
                    acc[4 * j] = __fadd_rn(acc[4 * j], x[j].x);
                    acc[4 * j + 1] = __fadd_rn(acc[4 * j + 1], x[j].y);
                    acc[4 * j + 2] = __fadd_rn(acc[4 * j + 2], x[j].z);
                    acc[4 * j + 3] = __fadd_rn(acc[4 * j + 3], x[j].w);
                }
            }
#pragma unroll
            for (int c = 0; c < SL_BLOCK_N / 32; ++c) {
                const int col0 = n0 + c * 32;
                if (col0 < p.N) {                          // uniform across the warp
                    CChunk cc;
                    if (vec_ok)                            // zeros when there is no C
                        load_c_chunk(cc, cmat, p.ldc, m0 + q * 32, col0, p.M, p.N);
                    uint32_t v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        v[j] = __float_as_uint(acc[c * 32 + j]);
                    if (vec_ok)
                        store_chunk_coalesced(v, my_stage, dmat, p.ldd, cc, epi, m0 + q * 32, col0, p.M, p.N);
                    else if (row < p.M)
                        store_row_chunk(v, drow, crow, epi, mrow, col0, p.N, false);
                }
            }
        }
    }

    // common exit: every thread arrives here, also after an abort
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, SL_TMEM_COLS);
    }
}

template <bool A_MN, bool B_MN>
int launch_slices_variant(sb200_ctx* ctx, const GemmArgs& g, int split, cudaStream_t stream)
{
    auto kern = gemm_tcgen05_slices_kernel<A_MN, B_MN>;
    static bool attr_done[16] = {};
    if (ctx->device >= 16 || !attr_done[ctx->device]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SL_SMEM) != cudaSuccess)
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
        rc = make_map_merged(ctx, &mapB, g.B, g.N, g.K, g.ldb, g.batch, g.strideB, SL_BLOCK_N / 32);
    else if (B_MN)
        rc = make_map(ctx, &mapB, g.B, g.N, g.K, g.ldb, g.batch, g.strideB, BLOCK_K, true);
    else
        rc = make_map(ctx, &mapB, g.B, g.K, g.N, g.ldb, g.batch, g.strideB, SL_BLOCK_N, false);
    if (rc)
        return rc;

    KernelParams p;
    p.M = static_cast<int>(g.M);
    p.N = static_cast<int>(g.N);
    p.K = static_cast<int>(g.K);
    p.batch = static_cast<int>(g.batch);
    p.tiles_m = static_cast<int>((g.M + BLOCK_M - 1) / BLOCK_M);
    p.tiles_n = static_cast<int>((g.N + SL_BLOCK_N - 1) / SL_BLOCK_N);
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
    p.owner_store = 0;
    p.status = ctx->d_status;
    p.wait_limit_ns = ctx->wait_limit_ns;
    p.test_stall_kb = ctx->test_stall_kb;
    p.explicit_hi = 0;
    p.colsum_out = nullptr;
    p.colsum_scale = 0.0f;
    p.acc_scale = 1.0f;
    p.colsum_lr = 0.0f;
    const int kb_per_cta = (p.num_kb + split - 1) / split;

    if (p.total_tiles > SLICE_TICKETS)
        return SB200_ERR_UNSUPPORTED;                       // the policy below never asks for this
    rc = ensure_workspace(ctx, static_cast<size_t>(p.total_tiles) * split * SL_PART_FLOATS * sizeof(float));
    if (rc)
        return rc;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(p.total_tiles * split));
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = SL_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, mapA, mapB, p, split, kb_per_cta, ctx->d_workspace,
                                               ctx->d_status + SLICE_TICKET_OFFSET);
    ctx->launches += 1;
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? SB200_OK : SB200_ERR_CUDA;
}

// Measured against the one-CTA kernel (64 x 512 x K, bias + ReLU, graph replay): the
// exchange (partial tile out, fence, ticket, the last CTA's reads) costs 2.3 us before
// the shorter walk starts to pay: 64 x 512 x 512 takes 9.4 us sliced and 8.7 us whole,
// 64 x 512 x 784 10.2 against 11.2, x 1024 10.5 against 13.1, x 2048 12.1 against 22.1.
constexpr int SL_MIN_KBLOCKS = 22;          // fewest k-blocks of a product worth slicing
constexpr int SL_MAX_SPLIT = 8;

}  // namespace

// How many CTAs should share each 128 x 64 tile of this request: 1 = the one-CTA
// kernel.  Only TF32 requests that the one-CTA kernel would run with 64-column tiles
// (few tiles), without column sums or row-block owners.
int k_slices(const sb200_ctx* ctx, const GemmArgs& g)
{
    if (!ctx->k_slices || g.mode != SB200_MODE_TF32 || g.colsum_out || g.rows_per_owner ||
        g.acc_scale != 1.0f)
        return 1;
    const long long num_kb = (g.K + BLOCK_K - 1) / BLOCK_K;
    const long long tiles = ((g.M + BLOCK_M - 1) / BLOCK_M) * ((g.N + SL_BLOCK_N - 1) / SL_BLOCK_N) * g.batch;
    if (tiles > SLICE_TICKETS || tiles * 2 > ctx->sm_count)
        return 1;
    long long split;
    if (ctx->k_slices > 1) {
        split = ctx->k_slices;                              // forced by the option (tests, tuning)
    } else {
        if (num_kb < SL_MIN_KBLOCKS)
            return 1;
        // after the fixed cost of the exchange: 0.28 us per k-block of the longest slice
        // and about 0.2 us more per slice for the CTA that adds them up
        long long max_split = ctx->sm_count / tiles;        // one wave
        if (max_split > SL_MAX_SPLIT)
            max_split = SL_MAX_SPLIT;
        split = 2;
        long long best = -1;
        for (long long s = 2; s <= max_split; ++s) {
            const long long cost = 28 * ((num_kb + s - 1) / s) + 20 * s;
            if (best < 0 || cost < best) {
                best = cost;
                split = s;
            }
        }
    }
    if (split > num_kb)
        split = num_kb;
    // every slice must own at least one k-block
    while (split > 1 && (split - 1) * ((num_kb + split - 1) / split) >= num_kb)
        --split;
    return static_cast<int>(split < 1 ? 1 : split);
}

int launch_gemm_tcgen05_slices(sb200_ctx* ctx, const GemmArgs& g, int split, cudaStream_t stream)
{
    const bool a_mn = g.transA != 0;
    const bool b_mn = g.transB == 0;
    if (a_mn)
        return b_mn ? launch_slices_variant<true, true>(ctx, g, split, stream)
                    : launch_slices_variant<true, false>(ctx, g, split, stream);
    return b_mn ? launch_slices_variant<false, true>(ctx, g, split, stream)
                : launch_slices_variant<false, false>(ctx, g, split, stream);
}

}  // namespace sb200
