// Batched fp32 GEMM  D = (C + bias) + op(A).op(B)  on the sm_100a tensor cores.
//
// One persistent CTA per SM walks over 128 x BLOCK_N output tiles.  Warp roles:
//   warp 0      TMA producer: fills a ring of shared-memory stages with one
//               128 x 32 tile of op(A) and one 32 x BLOCK_N tile of op(B) per
//               k-block (32 fp32 = one 128-byte swizzle row)
//   warp 1      MMA issuer: tcgen05.mma kind::tf32, accumulators in TMEM; two
//               accumulator buffers so the epilogue of one tile overlaps the
//               main loop of the next
//   warps 2-5   epilogue: tcgen05.ld the accumulator, add C and bias, store D
//   warps 6-9   (3xTF32 mode only) split every landed stage into a TF32 high
//               part and a TF32 low part; the issuer then runs lo.hi + hi.lo +
//               hi.hi per k-block into the same accumulator
//
// Transposed operands cost nothing extra: a tile whose contiguous dimension is
// M or N instead of K is loaded by TMA in its natural orientation ("MN-major",
// 32-element chunks along M/N, each 32 k-rows x 128 B) and the instruction
// descriptor's major bits tell the tensor core which way to read it.  Row-major
// B[K, N] -- the forward GEMM of a Linear layer -- is the MN-major case.
//
// Every wait on an mbarrier is bounded; when one expires the CTA records a code
// in the status word, raises a CTA-wide abort flag, and every role falls through
// to the common exit where TMEM is released.
#include "gemm_common.cuh"

namespace sb200 {

using namespace gemm;

namespace {

constexpr int TILE_PANEL = 16;          // row tiles (of 128 rows) per panel of the tile order

template <int BLOCK_N, int STAGES, bool SPLIT, bool A_TM = false>
struct SmemLayout {
    static constexpr int B_TILE_BYTES = BLOCK_N * BLOCK_K * 4;
    static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;   // one raw k-block (A + B)
    // 3xTF32: the low parts live in a ring of their own.  Only raw stages
    // have to cover the ~2 us from TMA issue to landed data; a low-part tile exists
    // just between the split warps and the MMAs that consume it (measured: 4 raw + 2 low
    // stages are slower than 3 + 3, the split warps need the slack).
    // A_TM: both parts of A go to TMEM instead (the tensor core reads them from
    // there), the ring holds the low part of B only.
    static constexpr int LO_STAGES = SPLIT ? (A_TM ? 4 : 3) : 0;
    static constexpr int LO_STAGE_BYTES = A_TM ? B_TILE_BYTES : STAGE_BYTES;
    static constexpr int TILES_BYTES = STAGE_BYTES * STAGES + LO_STAGE_BYTES * LO_STAGES;
    // accumulator buffers in TMEM (512 columns at most; A_TM: two accumulators and
    // LO_STAGES slots of 2 x 32 columns for the parts of A)
    static constexpr int NUM_ACC = SPLIT ? (A_TM ? 2 : 4) : 2;
    static constexpr int TMEM_COLS = A_TM ? 512 : NUM_ACC * BLOCK_N;
    static constexpr int A_TMEM_COL0 = NUM_ACC * BLOCK_N;
    static_assert(!A_TM || A_TMEM_COL0 + LO_STAGES * 2 * BLOCK_K <= 512, "TMEM columns");
    // barriers: full, empty per raw stage; lo_full, lo_empty per low-part stage; tmem_full,
    // tmem_empty per accumulator
    // (rounded to 16 bytes: the epilogue staging tiles that follow take float4 accesses)
    static constexpr int BAR_BYTES = ((2 * STAGES + 2 * LO_STAGES + 2 * NUM_ACC) * 8 + 16 + 15) & ~15;
    // + epilogue staging tiles (4 warps) + alignment slack
    static constexpr int TOTAL = TILES_BYTES + BAR_BYTES + 4 * EPI_STAGE_BYTES_PER_WARP +
                                 COLSUM_SCRATCH_BYTES + 1024;
    static_assert(TOTAL <= 227 * 1024, "shared memory per CTA");
};

// hi/lo split of one fp32 value for the 3xTF32 mode.  hi is exactly
// representable in TF32 (10 explicit mantissa bits), lo = x - hi is exact in
// fp32 and is itself cut to TF32 by the tensor core.
__device__ __forceinline__ void split_tf32(float x, bool rounded, float& hi, float& lo)
{
    uint32_t h;
    if (rounded)
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    else
        h = __float_as_uint(x) & 0xFFFFE000u;
    hi = __uint_as_float(h);
    lo = x - hi;
}

template <int BLOCK_N, int STAGES, bool A_MN, bool B_MN, bool SPLIT, bool COLSUM, bool A_TM>
__global__ void __launch_bounds__((SPLIT || COLSUM) ? 320 : 192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap mapA,
                    const __grid_constant__ CUtensorMap mapB, const KernelParams p)
{
    // A_TM (3xTF32 with A stored [M, K]): the split warps put both parts of A into TMEM
    static_assert(!A_TM || (SPLIT && !A_MN), "A in TMEM: 3xTF32 mode, A stored [M, K]");
    using L = SmemLayout<BLOCK_N, STAGES, SPLIT, A_TM>;
    constexpr int B_TILE_BYTES = L::B_TILE_BYTES;
    constexpr int HALF_STAGE = A_TILE_BYTES + B_TILE_BYTES;       // the hi (raw) tiles
    constexpr int LO_STAGES = L::LO_STAGES;
    constexpr int LO_STAGE_BYTES = L::LO_STAGE_BYTES;
    constexpr int NUM_ACC = L::NUM_ACC;
    constexpr uint32_t TMEM_COLS = L::TMEM_COLS;                   // 256 or 512: power of two
    static_assert(TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512,
                  "TMEM allocation must be a power of two");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::TILES_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* split_bar = empty_bar + STAGES;                     // "low parts written" per lo stage
    uint64_t* lo_empty = split_bar + LO_STAGES;                   // "low parts consumed" per lo stage
    uint64_t* tmem_full = lo_empty + LO_STAGES;
    uint8_t* lo_ring = smem + STAGES * L::STAGE_BYTES;            // LO_STAGES x (A + B) low-part tiles
    uint64_t* tmem_empty = tmem_full + NUM_ACC;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + NUM_ACC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* epi_stage = reinterpret_cast<float*>(smem + L::TILES_BYTES + L::BAR_BYTES);
    float* colsum_scratch = epi_stage + 4 * (EPI_STAGE_BYTES_PER_WARP / 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Abort ab{abort_flag, p.status, p.wait_limit_ns};

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], COLSUM ? 5 : 1);   // MMA commit (+ 4 column-sum warps)
        }
        for (int s = 0; s < LO_STAGES; ++s) {
            ptx::mbar_init(&split_bar[s], 4);
            ptx::mbar_init(&lo_empty[s], 1);
        }
        for (int i = 0; i < NUM_ACC; ++i) {
            ptx::mbar_init(&tmem_full[i], 1);
            ptx::mbar_init(&tmem_empty[i], 4);
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&mapA);
        ptx::prefetch_tensormap(&mapB);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched only shared memory, TMEM and kernel parameters: it may
    // overlap the tail of the previous kernel in the stream (small problems are a
    // chain of such prologues).  From here on global memory is read and written.
    ptx::griddep_launch_dependents();
    ptx::griddep_wait();

    const long long tiles_per_batch = static_cast<long long>(p.tiles_m) * p.tiles_n;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int issued = 0;
            for (long long t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                const int b = static_cast<int>(t / tiles_per_batch);
                const int r = static_cast<int>(t % tiles_per_batch);
                int tm, tn;
                tile_coords(r, p.tiles_m, p.tiles_n, TILE_PANEL, tm, tn);
                const int m0 = tm * BLOCK_M;
                const int n0 = tn * BLOCK_N;
                const int ba = p.a_batched ? b : 0;
                const int bb = p.b_batched ? b : 0;
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (p.test_stall_kb >= 0 && issued++ >= p.test_stall_kb) {
                        ok = false;                        // test hook: the other roles' waits run out
                        break;
                    }
                    if (!(ok = wait_bar(&empty_bar[s], ph ^ 1u, ab, FAULT_PRODUCER_WAIT)))
                        break;
                    uint8_t* sa = smem + s * L::STAGE_BYTES;
                    uint8_t* sb = sa + A_TILE_BYTES;
                    const int k0 = kb * BLOCK_K;
                    ptx::mbar_arrive_expect_tx(&full_bar[s], HALF_STAGE);
                    if (A_MN && p.a_merged) {
                        // stored [K, M], M % 32 == 0: all chunks in one 4-D box
                        ptx::tma_load_4d(sa, &mapA, &full_bar[s], 0, k0, m0 / 32, ba);
                    } else if (A_MN) {
                        // stored [K, M]: contiguous M, one 32(m) x 32(k) box per chunk
#pragma unroll
                        for (int c = 0; c < BLOCK_M / 32; ++c)
                            ptx::tma_load_3d(sa + c * CHUNK_BYTES, &mapA, &full_bar[s],
                                             m0 + c * 32, k0, ba);
                    } else {
                        // stored [M, K]: contiguous K, one 32(k) x 128(m) box
                        ptx::tma_load_3d(sa, &mapA, &full_bar[s], k0, m0, ba);
                    }
                    if (B_MN && p.b_merged) {
                        ptx::tma_load_4d(sb, &mapB, &full_bar[s], 0, k0, n0 / 32, bb);
                    } else if (B_MN) {
                        // stored [K, N]: contiguous N
#pragma unroll
                        for (int c = 0; c < BLOCK_N / 32; ++c)
                            ptx::tma_load_3d(sb + c * CHUNK_BYTES, &mapB, &full_bar[s],
                                             n0 + c * 32, k0, bb);
                    } else {
                        // stored [N, K]: contiguous K, one 32(k) x BLOCK_N(n) box
                        ptx::tma_load_3d(sb, &mapB, &full_bar[s], k0, n0, bb);
                    }
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_tf32(BLOCK_M, BLOCK_N, A_MN, B_MN);
            // byte step of the descriptor start address per UMMA_K
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
            int ls = 0;                                   // low-part stage (3xTF32)
            uint32_t lph = 0;
            int acc = 0;
            uint32_t acc_ph = 0;
            bool ok = true;
            for (long long t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                // One accumulator buffer per chunk of k-blocks.  In TF32 mode a
                // tile is a single chunk; in 3xTF32 mode the chain of tensor-core
                // accumulations is cut every SPLIT_CHUNK_KB k-blocks and the
                // partial sums are added up in fp32 registers by the epilogue.
                for (int kb0 = 0; ok && kb0 < p.num_kb; kb0 += p.chunk_kb) {
                    if (!(ok = wait_bar(&tmem_empty[acc], acc_ph ^ 1u, ab, FAULT_MMA_WAIT_TMEM)))
                        break;
                    ptx::tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
                    const int kb1 = min(kb0 + p.chunk_kb, p.num_kb);
                    for (int kb = kb0; kb < kb1; ++kb) {
                        // 3xTF32: the split warps signal once the low parts are written,
                        // which they do only after the raw stage has landed
                        if (!(ok = SPLIT ? wait_bar(&split_bar[ls], lph, ab, FAULT_MMA_WAIT_FULL)
                                         : wait_bar(&full_bar[s], ph, ab, FAULT_MMA_WAIT_FULL)))
                            break;
                        ptx::tc_fence_after_sync();
                        const uint32_t sa = ptx::smem_u32(smem + s * L::STAGE_BYTES);
                        const uint32_t sb = sa + A_TILE_BYTES;
#pragma unroll
                        for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                            const uint64_t a_hi =
                                ptx::make_smem_desc(sa + k * A_KSTEP, A_LBO, A_SBO, A_LAY);
                            const uint64_t b_hi =
                                ptx::make_smem_desc(sb + k * B_KSTEP, B_LBO, B_SBO, B_LAY);
                            const uint32_t first = (kb > kb0 || k > 0) ? 1u : 0u;
                            if (A_TM) {
                                const uint32_t a_hi_t =
                                    tmem_base + static_cast<uint32_t>(L::A_TMEM_COL0 +
                                                                      ls * 2 * BLOCK_K + k * UMMA_K);
                                const uint32_t a_lo_t = a_hi_t + BLOCK_K;
                                const uint64_t b_lo = ptx::make_smem_desc(
                                    ptx::smem_u32(lo_ring + ls * LO_STAGE_BYTES) + k * B_KSTEP, B_LBO,
                                    B_SBO, B_LAY);
                                // small terms first
                                ptx::mma_tf32_a_tmem(d_tmem, a_lo_t, b_hi, idesc, first);
                                ptx::mma_tf32_a_tmem(d_tmem, a_hi_t, b_lo, idesc, 1u);
                                ptx::mma_tf32_a_tmem(d_tmem, a_hi_t, b_hi, idesc, 1u);
                            } else if (SPLIT) {
                                const uint32_t la = ptx::smem_u32(lo_ring + ls * LO_STAGE_BYTES);
                                const uint64_t a_lo = ptx::make_smem_desc(
                                    la + k * A_KSTEP, A_LBO, A_SBO, A_LAY);
                                const uint64_t b_lo = ptx::make_smem_desc(
                                    la + A_TILE_BYTES + k * B_KSTEP, B_LBO, B_SBO, B_LAY);
                                // small terms first
                                ptx::mma_tf32(d_tmem, a_lo, b_hi, idesc, first);
                                ptx::mma_tf32(d_tmem, a_hi, b_lo, idesc, 1u);
                                ptx::mma_tf32(d_tmem, a_hi, b_hi, idesc, 1u);
                            } else {
                                ptx::mma_tf32(d_tmem, a_hi, b_hi, idesc, first);
                            }
                        }
                        ptx::mma_commit(&empty_bar[s]);   // stage free once these MMAs retire
                        if (++s == STAGES) {
                            s = 0;
                            ph ^= 1u;
                        }
                        if (SPLIT) {
                            ptx::mma_commit(&lo_empty[ls]);
                            if (++ls == LO_STAGES) {
                                ls = 0;
                                lph ^= 1u;
                            }
                        }
                    }
                    if (!ok)
                        break;
                    ptx::mma_commit(&tmem_full[acc]);     // this chunk's accumulator is complete
                    if (++acc == NUM_ACC) {
                        acc = 0;
                        acc_ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------- epilogue
        const int q = warp & 3;                           // TMEM lane quadrant of this warp
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        const bool vec_ok = ((p.ldd & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) &&
                            ((p.strideD & 3) == 0) &&
                            (p.C == nullptr ||
                             (((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                              ((p.strideC & 3) == 0)));
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        for (long long t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
            const int b = static_cast<int>(t / tiles_per_batch);
            const int r = static_cast<int>(t % tiles_per_batch);
            int tm, tn;
            tile_coords(r, p.tiles_m, p.tiles_n, TILE_PANEL, tm, tn);
            const int m0 = tm * BLOCK_M;
            const int n0 = tn * BLOCK_N;
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
            const float* mrow = epi.mask ? epi.mask + static_cast<long long>(row) * p.ldm : nullptr;
            if constexpr (!SPLIT) {
                // one chunk per tile: straight from TMEM to global memory.  The first
                // chunk's C is requested before the wait for the accumulator, so that it
                // travels under the tile's main loop (C may alias D, but this tile's
                // region of D is written by nobody else)
                CChunk c_now, c_next;
                if (vec_ok)                                    // zeros when there is no C
                    load_c_chunk(c_next, cmat, p.ldc, m0 + q * 32, n0, p.M, p.N);
                if (!(ok = wait_bar(&tmem_full[acc], acc_ph, ab, FAULT_EPI_WAIT)))
                    break;
                ptx::tc_fence_after_sync();
#pragma unroll 1
                for (int c = 0; c < BLOCK_N / 32; ++c) {
                    const int col0 = n0 + c * 32;
                    if (col0 >= p.N)
                        break;                             // uniform across the warp
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(lane_base + static_cast<uint32_t>(acc * BLOCK_N + c * 32), v);
                    if (vec_ok && (cmat || c == 0)) {
                        c_now = c_next;
                        if (c + 1 < BLOCK_N / 32 && col0 + 32 < p.N)     // next chunk's C, ahead of the stores
                            load_c_chunk(c_next, cmat, p.ldc, m0 + q * 32, col0 + 32, p.M, p.N);
                    }
                    ptx::tmem_ld_wait();
                    if (p.acc_scale != 1.0f) {             // in-place SGD: D = C + (-lr) * product
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            v[j] = __float_as_uint(__fmul_rn(__uint_as_float(v[j]), p.acc_scale));
                    }
                    if (vec_ok)
                        store_chunk_coalesced(v, my_stage, dmat, p.ldd, c_now, epi, m0 + q * 32,
                                              col0, p.M, p.N);
                    else if (row < p.M)
                        store_row_chunk(v, drow, crow, epi, mrow, col0, p.N, false);
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(&tmem_empty[acc]);
                if (++acc == NUM_ACC) {
                    acc = 0;
                    acc_ph ^= 1u;
                }
            } else {
                // 3xTF32: the tensor core cuts every fp32 accumulation short
                // (no round-to-nearest), which over thousands of k steps adds up
                // to ~1e-5 relative.  Each chunk of k-blocks therefore gets a
                // fresh TMEM accumulator and the chunks are summed here with
                // round-to-nearest adds.
                float sum[BLOCK_N];
#pragma unroll
                for (int j = 0; j < BLOCK_N; ++j)
                    sum[j] = 0.0f;
                for (int kb0 = 0; ok && kb0 < p.num_kb; kb0 += p.chunk_kb) {
                    if (!(ok = wait_bar(&tmem_full[acc], acc_ph, ab, FAULT_EPI_WAIT)))
                        break;
                    ptx::tc_fence_after_sync();
#pragma unroll
                    for (int c = 0; c < BLOCK_N / 32; ++c) {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32(lane_base + static_cast<uint32_t>(acc * BLOCK_N + c * 32),
                                           v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            sum[c * 32 + j] = __fadd_rn(sum[c * 32 + j], __uint_as_float(v[j]));
                    }
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0)
                        ptx::mbar_arrive(&tmem_empty[acc]);
                    if (++acc == NUM_ACC) {
                        acc = 0;
                        acc_ph ^= 1u;
                    }
                }
                if (!ok)
                    break;
#pragma unroll
                for (int c = 0; c < BLOCK_N / 32; ++c) {
                    const int col0 = n0 + c * 32;
                    if (col0 < p.N) {                      // uniform across the warp
                        uint32_t v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            v[j] = __float_as_uint(p.acc_scale != 1.0f ? __fmul_rn(sum[c * 32 + j], p.acc_scale)
                                                                       : sum[c * 32 + j]);
                        // one store per tile after many chunk drains: the plain row
                        // store keeps this path's register count down
                        if (row < p.M)
                            store_row_chunk(v, drow, crow, epi, mrow, col0, p.N, vec_ok);
                    }
                }
            }
        }
    } else if (SPLIT && warp < 10) {
        // --------------------------------------- hi/lo split (3xTF32 mode)
        // 128 threads; each float4 of the landed tiles is read once, its low
        // part is written to the twin tile at the same (swizzled) offset.
        const int tid = threadIdx.x - 6 * 32;
        int s = 0;
        uint32_t ph = 0;
        int ls = 0;
        uint32_t lph = 0;
        bool ok = true;
        const bool rounded = p.explicit_hi != 0;
        for (long long t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
            for (int kb = 0; kb < p.num_kb; ++kb) {
                if (!(ok = wait_bar(&full_bar[s], ph, ab, FAULT_SPLIT_WAIT)))
                    break;
                if (!(ok = wait_bar(&lo_empty[ls], lph ^ 1u, ab, FAULT_SPLIT_WAIT)))
                    break;
                if constexpr (A_TM) {
                    // A: this thread's row of the landed [128 rows x 32 k] tile (128 bytes,
                    // its 16-byte pieces permuted by the 128-byte swizzle) goes to TMEM
                    // lane = row, as the high part in 32 columns and the low part in the
                    // next 32.  Warp w of the CTA reaches TMEM lanes 32 (w % 4) .. + 31.
                    const int row = (warp & 3) * 32 + lane;
                    const float4* arow =
                        reinterpret_cast<const float4*>(smem + s * L::STAGE_BYTES + row * 128);
                    uint32_t h[32], l[32];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const float4 x = arow[c ^ (row & 7)];
                        float fh, fl;
                        split_tf32(x.x, rounded, fh, fl);
                        h[4 * c + 0] = __float_as_uint(fh); l[4 * c + 0] = __float_as_uint(fl);
                        split_tf32(x.y, rounded, fh, fl);
                        h[4 * c + 1] = __float_as_uint(fh); l[4 * c + 1] = __float_as_uint(fl);
                        split_tf32(x.z, rounded, fh, fl);
                        h[4 * c + 2] = __float_as_uint(fh); l[4 * c + 2] = __float_as_uint(fl);
                        split_tf32(x.w, rounded, fh, fl);
                        h[4 * c + 3] = __float_as_uint(fh); l[4 * c + 3] = __float_as_uint(fl);
                    }
                    const uint32_t slot = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) +
                                          static_cast<uint32_t>(L::A_TMEM_COL0 + ls * 2 * BLOCK_K);
                    ptx::tmem_st_32x32(slot, h);
                    ptx::tmem_st_32x32(slot + BLOCK_K, l);
                    // B: every float4 of the landed tile once, its low part to the twin tile
                    const float4* bhi =
                        reinterpret_cast<const float4*>(smem + s * L::STAGE_BYTES + A_TILE_BYTES);
                    float4* bhi_w = reinterpret_cast<float4*>(smem + s * L::STAGE_BYTES + A_TILE_BYTES);
                    float4* blo = reinterpret_cast<float4*>(lo_ring + ls * LO_STAGE_BYTES);
                    constexpr int PER_THREAD = B_TILE_BYTES / 16 / 128;
                    float4 x[PER_THREAD];
#pragma unroll
                    for (int j = 0; j < PER_THREAD; ++j)
                        x[j] = bhi[tid + j * 128];
#pragma unroll
                    for (int j = 0; j < PER_THREAD; ++j) {
                        float4 hh, ll;
                        split_tf32(x[j].x, rounded, hh.x, ll.x);
                        split_tf32(x[j].y, rounded, hh.y, ll.y);
                        split_tf32(x[j].z, rounded, hh.z, ll.z);
                        split_tf32(x[j].w, rounded, hh.w, ll.w);
                        blo[tid + j * 128] = ll;
                        if (rounded)
                            bhi_w[tid + j * 128] = hh;
                    }
                    ptx::tmem_st_wait();
                    ptx::tc_fence_before_sync();
                } else {
                float4* hi = reinterpret_cast<float4*>(smem + s * L::STAGE_BYTES);
                float4* lo = reinterpret_cast<float4*>(lo_ring + ls * LO_STAGE_BYTES);
                // all loads of a batch first, then the arithmetic, then the stores: the
                // split must finish well inside one k-block of tensor-core time
                constexpr int PER_THREAD = HALF_STAGE / 16 / 128;          // float4 per thread
                constexpr int BATCH = 8;
                static_assert(!SPLIT || PER_THREAD % BATCH == 0, "split batches");
#pragma unroll
                for (int b0 = 0; b0 < PER_THREAD; b0 += BATCH) {
                    float4 x[BATCH];
#pragma unroll
                    for (int j = 0; j < BATCH; ++j)
                        x[j] = hi[tid + (b0 + j) * 128];
#pragma unroll
                    for (int j = 0; j < BATCH; ++j) {
                        float4 h, l;
                        split_tf32(x[j].x, rounded, h.x, l.x);
                        split_tf32(x[j].y, rounded, h.y, l.y);
                        split_tf32(x[j].z, rounded, h.z, l.z);
                        split_tf32(x[j].w, rounded, h.w, l.w);
                        lo[tid + (b0 + j) * 128] = l;
                        if (rounded)
                            hi[tid + (b0 + j) * 128] = h;
                    }
                }
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(&split_bar[ls]);
                if (++s == STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
                if (++ls == LO_STAGES) {
                    ls = 0;
                    lph ^= 1u;
                }
            }
        }
    }

    if constexpr (COLSUM) {
        if (warp >= 6) {
            // ---------------------- column sums of op(B) (fused bias gradient)
            static_assert(!SPLIT, "column sums ride on the TF32 kernel");
            const int tid = threadIdx.x - 6 * 32;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (long long t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                const int r = static_cast<int>(t % tiles_per_batch);
                int tm, tn;
                tile_coords(r, p.tiles_m, p.tiles_n, TILE_PANEL, tm, tn);
                const bool mine = (t / tiles_per_batch == 0) && (tm == 0);
                const int n0 = tn * BLOCK_N;
                float4 acc4 = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    if (!(ok = wait_bar(&full_bar[s], ph, ab, FAULT_SPLIT_WAIT)))
                        break;
                    if (mine)
                        colsum_accumulate<B_MN, BLOCK_N>(smem + s * L::STAGE_BYTES + A_TILE_BYTES,
                                                         tid, acc4);
                    __syncwarp();
                    if (lane == 0)
                        ptx::mbar_arrive(&empty_bar[s]);
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (!ok)
                    break;
                if (mine)
                    colsum_finish<B_MN, BLOCK_N>(acc4, colsum_scratch, tid, p.colsum_out,
                                                 p.colsum_scale, n0, p.N, p.colsum_lr);
            }
        }
    }

    // common exit: every thread arrives here, also after an abort
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------- host

template <int BLOCK_N, int STAGES, bool A_MN, bool B_MN, bool SPLIT, bool COLSUM, bool A_TM = false>
int launch_variant(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream)
{
    using L = SmemLayout<BLOCK_N, STAGES, SPLIT, A_TM>;
    auto kern = gemm_tcgen05_kernel<BLOCK_N, STAGES, A_MN, B_MN, SPLIT, COLSUM, A_TM>;
    static bool attr_done[16] = {};
    if (ctx->device < 16 && !attr_done[ctx->device]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) !=
            cudaSuccess)
            return SB200_ERR_CUDA;
        attr_done[ctx->device] = true;
    } else if (ctx->device >= 16) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    }

    CUtensorMap mapA, mapB;
    int rc;
    const bool a_merged = A_MN && (g.M % 32 == 0) && ctx->merge_mn_boxes;
    const bool b_merged = B_MN && (g.N % 32 == 0) && ctx->merge_mn_boxes;
    if (a_merged)
        rc = make_map_merged(ctx, &mapA, g.A, g.M, g.K, g.lda, g.batch, g.strideA, BLOCK_M / 32);
    else if (A_MN)   // stored [K, M]
        rc = make_map(ctx, &mapA, g.A, g.M, g.K, g.lda, g.batch, g.strideA, BLOCK_K, true);
    else        // stored [M, K]
        rc = make_map(ctx, &mapA, g.A, g.K, g.M, g.lda, g.batch, g.strideA, BLOCK_M, false);
    if (rc)
        return rc;
    if (b_merged)
        rc = make_map_merged(ctx, &mapB, g.B, g.N, g.K, g.ldb, g.batch, g.strideB, BLOCK_N / 32);
    else if (B_MN)   // stored [K, N]
        rc = make_map(ctx, &mapB, g.B, g.N, g.K, g.ldb, g.batch, g.strideB, BLOCK_K, true);
    else        // stored [N, K]
        rc = make_map(ctx, &mapB, g.B, g.K, g.N, g.ldb, g.batch, g.strideB, BLOCK_N, false);
    if (rc)
        return rc;

    KernelParams p;
    p.M = static_cast<int>(g.M);
    p.N = static_cast<int>(g.N);
    p.K = static_cast<int>(g.K);
    p.batch = static_cast<int>(g.batch);
    p.tiles_m = static_cast<int>((g.M + BLOCK_M - 1) / BLOCK_M);
    p.tiles_n = static_cast<int>((g.N + BLOCK_N - 1) / BLOCK_N);
    p.num_kb = static_cast<int>((g.K + BLOCK_K - 1) / BLOCK_K);
    p.chunk_kb = SPLIT ? SPLIT_CHUNK_KB : (p.num_kb > 0 ? p.num_kb : 1);
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
    p.explicit_hi = ctx->split_explicit_hi;
    p.colsum_out = COLSUM ? g.colsum_out : nullptr;
    p.colsum_scale = g.colsum_scale;
    p.acc_scale = g.acc_scale;
    p.colsum_lr = COLSUM ? g.colsum_lr : 0.0f;

    const long long grid = p.total_tiles < ctx->sm_count ? p.total_tiles : ctx->sm_count;
    // programmatic stream serialization: the kernel's prologue may start while the
    // previous kernel of the stream is finishing (see griddep_wait in the kernel)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3((SPLIT || COLSUM) ? 320 : 192);
    cfg.dynamicSmemBytes = L::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, mapA, mapB, p);
    ctx->launches += 1;
    return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? SB200_OK : SB200_ERR_CUDA;
}

template <int BLOCK_N, int STAGES, bool SPLIT, bool COLSUM>
int launch_layout(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream)
{
    const bool a_mn = g.transA != 0;     // stored [K, M]
    const bool b_mn = g.transB == 0;     // stored [K, N]
    if constexpr (SPLIT) {
        // A stored [M, K]: its two parts live in TMEM, the shared memory that frees
        // holds a fourth raw stage and a fourth low-part tile of B
        if (!a_mn && ctx->split_a_tmem)
            return b_mn ? launch_variant<BLOCK_N, 4, false, true, SPLIT, COLSUM, true>(ctx, g, stream)
                        : launch_variant<BLOCK_N, 4, false, false, SPLIT, COLSUM, true>(ctx, g, stream);
    }
    if (a_mn)
        return b_mn ? launch_variant<BLOCK_N, STAGES, true, true, SPLIT, COLSUM>(ctx, g, stream)
                    : launch_variant<BLOCK_N, STAGES, true, false, SPLIT, COLSUM>(ctx, g, stream);
    return b_mn ? launch_variant<BLOCK_N, STAGES, false, true, SPLIT, COLSUM>(ctx, g, stream)
                : launch_variant<BLOCK_N, STAGES, false, false, SPLIT, COLSUM>(ctx, g, stream);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// TMA needs 16-byte aligned base addresses and 16-byte multiples for every
// stride; the tile coordinates the kernel uses are multiples of 32 elements.
bool tcgen05_eligible(const GemmArgs& g)
{
    if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.batch <= 0)
        return false;
    if (g.M > INT32_MAX || g.N > INT32_MAX || g.K > INT32_MAX || g.batch > INT32_MAX)
        return false;
    if (!aligned16(g.A) || !aligned16(g.B))
        return false;
    if ((g.lda & 3) || (g.ldb & 3))
        return false;
    // a batch stride is only ever added to the base when there is a second batch
    if (g.batch > 1 && ((g.strideA & 3) || (g.strideB & 3)))
        return false;
    if (g.strideA < 0 || g.strideB < 0)
        return false;
    return true;
}

namespace {

int launch_one_cta(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream)
{
    if (g.mode == SB200_MODE_TF32X3) {
        // 128-wide tiles: three raw stages plus a three-deep ring of low-part tiles
        return launch_layout<128, 3, true, false>(ctx, g, stream);
    }
    // Tile width: the widest of 256 / 128 / 64 columns that still gives every
    // second SM a tile.  Small problems are latency-bound; narrower tiles spread
    // them over more SMs and leave room for more stages (8 x 24 KB at width 64).
    const long long tiles_m = (g.M + BLOCK_M - 1) / BLOCK_M;
    auto tiles = [&](int bn) { return tiles_m * ((g.N + bn - 1) / bn) * g.batch; };
    const long long want = ctx->sm_count / 2;
    int bn = 256;
    if (g.N <= 64 || (tiles(128) < want && g.N > 64))
        bn = 64;
    else if (g.N <= 128 || tiles(256) < want)
        bn = 128;
    if (bn == 64) {
        // few tiles and a long inner dimension: a cluster of CTAs per tile, each a slice of k
        const int slices = k_slices(ctx, g);
        if (slices > 1)
            return launch_gemm_tcgen05_slices(ctx, g, slices, stream);
    }
    if (g.colsum_out) {
        if (bn == 256) return launch_layout<256, 4, false, true>(ctx, g, stream);
        if (bn == 128) return launch_layout<128, 6, false, true>(ctx, g, stream);
        return launch_layout<64, 8, false, true>(ctx, g, stream);
    }
    if (bn == 256) return launch_layout<256, 4, false, false>(ctx, g, stream);
    if (bn == 128) return launch_layout<128, 6, false, false>(ctx, g, stream);
    return launch_layout<64, 8, false, false>(ctx, g, stream);
}

// Wave quantisation of the pair kernel.  Its tiles all take the same time, so T
// tiles on P pairs cost ceil(T / P) waves: one 4096^3 product is 256 tiles on 74
// pairs, 3.46 waves of work in the time of 4.  When the last wave would be
// mostly empty the bottom rows of the product go to the one-CTA kernel instead
// (128 x 256 tiles, one per SM, about 0.56 of a pair wave each): rows [0, m1)
// stay on the pairs with m1 chosen so that they fill whole waves.  Returns m1
// (== M: do not split).  Costs are in pair waves.  A context option, off by
// default: on a power-capped part the SMs of a partly empty wave clock higher and
// the single launch measured faster (one 4096^3: 199 us whole, 212 us split).
int64_t pair_rows_before_tail(const sb200_ctx* ctx, const GemmArgs& g)
{
    if (g.rows_per_owner)                       // row numbers select the owner: keep one launch
        return g.M;
    const long long P = ctx->sm_count / 2, S = ctx->sm_count;
    const long long tiles_m = (g.M + 255) / 256, tiles_n = (g.N + 255) / 256;
    const long long T = tiles_m * tiles_n * g.batch;
    const double whole = static_cast<double>((T + P - 1) / P);
    if (whole > 8.0 || T % P == 0)
        return g.M;                             // long runs lose little to the last wave
    double best = whole * 0.93;                 // a second launch must buy a clear gain
    int64_t best_m1 = g.M;
    for (long long r = tiles_m - 1; r >= 1 && r >= tiles_m - 8; --r) {
        const long long t1 = r * tiles_n * g.batch;
        if (t1 < P)
            break;
        const long long rest_rows = g.M - r * 256;
        const long long t2 = ((rest_rows + 127) / 128) * tiles_n * g.batch;
        const double cost = static_cast<double>((t1 + P - 1) / P) +
                            0.56 * static_cast<double>((t2 + S - 1) / S) + 0.08;
        if (cost < best) {
            best = cost;
            best_m1 = r * 256;
        }
    }
    return best_m1;
}

}  // namespace

int launch_gemm_tcgen05(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream)
{
    if (!tcgen05_eligible(g))
        return SB200_ERR_UNSUPPORTED;
    if (pair_kernel_preferred(ctx, g)) {
        const int64_t m1 = ctx->split_tail_wave ? pair_rows_before_tail(ctx, g) : g.M;
        if (m1 >= g.M)
            return launch_gemm_tcgen05_pair(ctx, g, stream);
        GemmArgs top = g;
        top.M = m1;
        const int rc = launch_gemm_tcgen05_pair(ctx, top, stream);
        if (rc)
            return rc;
        GemmArgs rest = g;                      // rows [m1, M): same strides, shifted bases
        rest.M = g.M - m1;
        rest.A = g.transA ? g.A + m1 : g.A + m1 * g.lda;
        if (g.C) rest.C = g.C + m1 * g.ldc;
        rest.D = g.D + m1 * g.ldd;
        if (g.mask) rest.mask = g.mask + m1 * g.ldmask;
        return launch_one_cta(ctx, rest, stream);
    }
    return launch_one_cta(ctx, g, stream);
}

}  // namespace sb200
