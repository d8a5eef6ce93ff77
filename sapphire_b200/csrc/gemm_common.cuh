// Pieces shared by the one-CTA and the two-CTA tensor-core GEMM kernels:
// tile constants, kernel parameters, the bounded mbarrier wait, the epilogue
// store and the tensor-map builders.
#pragma once
#include <cstring>

#include "common.cuh"
#include "ptx.cuh"

namespace sb200 {
namespace gemm {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 32;                     // fp32 elements = 128 bytes
constexpr int UMMA_K = 8;                       // k per tcgen05.mma, kind::tf32
constexpr int A_TILE_BYTES = BLOCK_M * BLOCK_K * 4;
constexpr int CHUNK_BYTES = 32 * BLOCK_K * 4;   // one MN-major chunk: 32 k-rows x 128 B
constexpr uint64_t DEFAULT_WAIT_LIMIT_NS = 2000000000ull;   // a context option shortens it
constexpr int SPLIT_CHUNK_KB = 8;               // 3xTF32: 256 k per tensor-core accumulation chain

struct KernelParams {
    int M, N, K, batch;
    int tiles_m, tiles_n, num_kb;
    int chunk_kb;                               // k-blocks per TMEM accumulation chain
    long long total_tiles;
    int a_batched, b_batched;                   // 0: batch stride 0, always read matrix 0
    int a_merged, b_merged;                     // MN-major tile fetched by one 4-D TMA box
    const float* C; long long ldc, strideC;
    float* D; long long ldd, strideD;
    const float* bias;
    unsigned* status;
    int explicit_hi;
    float* colsum_out;                          // column sums of op(B) (fused bias gradient) or null
    float colsum_scale;
    int relu;                                   // ReLU of the result
    const float* mask; long long ldm, strideM;  // ReLU-backward gate matrix or null
    float* owner[MAX_OWNERS];                   // reduce-scatter epilogue: row-block owners' buffers
    int rows_per_owner;                         // 0: plain store to D
    int owner_store;                            // with owners: store the tile instead of adding it
    unsigned long long wait_limit_ns;           // bound of every mbarrier wait
    int test_stall_kb;                          // >= 0: the TMA producer stops after this many k-blocks
                                                // (test hook: every other role's wait then runs out)
    float acc_scale;                            // accumulator times this before C is added (1 = off;
                                                // -lr: D = C - lr * product, the in-place SGD update)
    float colsum_lr;                            // != 0: colsum_out[n] -= colsum_lr * (colsum_scale * sum)
};

// What the epilogue does with an accumulator: D = post((C + bias) + acc), where
// post is the optional ReLU followed by the optional gate "keep where mask > 0,
// else 0" (the backward pass of a ReLU whose output, or input, is `mask`).
struct Epilogue {
    const float* bias;      // [N] or null
    const float* mask;      // this batch's [M, N] gate matrix or null
    long long ldm;
    int relu;
    int reduce;             // add the result into D (system-scope reduction) instead of storing it
};

__device__ __forceinline__ float post_op(float o, int relu, const float* m)
{
    if (relu) o = o > 0.0f ? o : 0.0f;
    // 0 + x like the reference's accumulation into a zeroed gradient (turns -0 into +0)
    if (m) o = __fadd_rn(0.0f, __ldg(m) > 0.0f ? o : 0.0f);
    return o;
}

// The same with the gate value already in a register.
__device__ __forceinline__ float post_op_value(float o, int relu, bool gated, float gate)
{
    if (relu) o = o > 0.0f ? o : 0.0f;
    if (gated) o = __fadd_rn(0.0f, gate > 0.0f ? o : 0.0f);
    return o;
}

// Tile r of a batch -> (row tile, column tile).  Tiles are taken in panels of
// `panel` row tiles, column tiles fastest inside a panel: the ~150 tiles in
// flight at any time then cover a near-square patch of the output (panel x ~9
// tiles), which needs fewer distinct rows of A and columns of B per k-slice --
// fewer bytes from HBM per wave -- than a full-height stripe a few columns wide.
__device__ __forceinline__ void tile_coords(int r, int tiles_m, int tiles_n, int panel, int& tm, int& tn)
{
    const int per_panel = panel * tiles_n;
    const int first = (r / per_panel) * panel;                  // first row tile of this panel
    const int height = min(panel, tiles_m - first);
    const int within = r - (r / per_panel) * per_panel;
    tn = within / height;
    tm = first + within % height;
}

struct Abort {
    volatile int* flag;
    unsigned* status;
    unsigned long long limit_ns;
};

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, const Abort& ab,
                                         unsigned code)
{
    // The global timer is slow to read: the clock of a wait starts at its 64th failed
    // try, so the waits of the steady state (a few tries) never read it.
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
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

// One thread's 32 consecutive output columns of one row: D = post((C + bias) + acc);
// mrow is the row of the gate matrix or null.
__device__ __forceinline__ void store_row_chunk(const uint32_t (&v)[32], float* drow,
                                                const float* crow, const Epilogue& ep,
                                                const float* mrow, int col0, int N, bool vec_ok)
{
    const float* bias = ep.bias;
    const bool post = ep.relu || mrow;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const int col = col0 + j;
        if (vec_ok && col + 3 < N) {
            float4 base = make_float4(0.f, 0.f, 0.f, 0.f);
            if (crow)
                base = *reinterpret_cast<const float4*>(crow + col);
            if (bias) {
                base.x = base.x + __ldg(bias + col);
                base.y = base.y + __ldg(bias + col + 1);
                base.z = base.z + __ldg(bias + col + 2);
                base.w = base.w + __ldg(bias + col + 3);
            }
            float4 o;
            o.x = base.x + __uint_as_float(v[j]);
            o.y = base.y + __uint_as_float(v[j + 1]);
            o.z = base.z + __uint_as_float(v[j + 2]);
            o.w = base.w + __uint_as_float(v[j + 3]);
            if (post) {
                o.x = post_op(o.x, ep.relu, mrow ? mrow + col : nullptr);
                o.y = post_op(o.y, ep.relu, mrow ? mrow + col + 1 : nullptr);
                o.z = post_op(o.z, ep.relu, mrow ? mrow + col + 2 : nullptr);
                o.w = post_op(o.w, ep.relu, mrow ? mrow + col + 3 : nullptr);
            }
            if (ep.reduce)
                ptx::red_add_sys_v4(drow + col, o);
            else
                *reinterpret_cast<float4*>(drow + col) = o;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (col + e < N) {
                    float base = crow ? crow[col + e] : 0.f;
                    if (bias)
                        base = base + __ldg(bias + col + e);
                    float o = base + __uint_as_float(v[j + e]);
                    if (post) o = post_op(o, ep.relu, mrow ? mrow + col + e : nullptr);
                    if (ep.reduce)
                        ptx::red_add_sys(drow + col + e, o);
                    else
                        drow[col + e] = o;
                }
            }
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Coalesced epilogue store of one warp's 32 rows x 32 columns.  After
// tcgen05.ld lane l holds 32 columns of row l; going through a per-warp
// shared-memory tile (32 rows x 36 floats) the warp instead moves 4 rows x 128
// contiguous bytes per instruction: 8 lanes per row, one float4 each: lane l
// handles rows 4 i + l / 8 (i = 0..7), columns col0 + 4 (l % 8) .. + 3.
// `row0` is the global row of lane 0's TMEM lane; D / C point at the matrix
// origin of the batch.  Requires 16-byte aligned rows.
//
// C is read by load_c_chunk BEFORE the stores of the previous chunk are issued:
// C may alias D (in-place y <- y + a.b), so the compiler keeps every load of C
// behind every earlier store to D, and a load issued only when its value is
// needed costs a full memory round trip per float4.  Fetching the next chunk's
// C ahead keeps eight loads per lane in flight across the stores.
constexpr int EPI_STAGE_LD = 36;                                 // floats per staged row
constexpr int EPI_STAGE_BYTES_PER_WARP = 32 * EPI_STAGE_LD * 4;

struct CChunk {
    float4 v[8];
};

__device__ __forceinline__ void load_c_chunk(CChunk& cc, const float* C, long long ldc, int row0,
                                             int col0, int M, int N)
{
    const int lane = threadIdx.x & 31;
    const int sub = lane >> 3, col = col0 + (lane & 7) * 4;
    if (C && row0 + 32 <= M && col0 + 32 <= N) {                 // inside the matrix: no predicates
        const float* cptr = C + static_cast<long long>(row0 + sub) * ldc + col;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            cc.v[i] = *reinterpret_cast<const float4*>(cptr);
            cptr += 4 * ldc;
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int grow = row0 + i * 4 + sub;
        cc.v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (C && grow < M) {
            const float* crow = C + static_cast<long long>(grow) * ldc;
            if (col + 3 < N) {
                cc.v[i] = *reinterpret_cast<const float4*>(crow + col);
            } else {
                if (col < N) cc.v[i].x = crow[col];
                if (col + 1 < N) cc.v[i].y = crow[col + 1];
                if (col + 2 < N) cc.v[i].z = crow[col + 2];
            }
        }
    }
}

// A chunk that lies inside the matrix (the common case by far): no predicate and
// no address multiplication per element.  The general version below costs ~500
// instructions per chunk, and with one warp per 32 rows of a 256-column tile
// that, not memory, bounded short-k problems.  The gate matrix, when there is
// one, must have 16-byte aligned rows.  EXTRAS = false compiles the gate and the
// reduction variant out: the plain store is the hot case and even their
// never-taken branches cost it 15 % (registers, scheduling freedom).
template <bool EXTRAS>
__device__ __forceinline__ void store_chunk_interior(const uint32_t (&v)[32], float* stage, float* D, long long ldd,
                                                    const CChunk& cc, const Epilogue& e, int row0, int col0,
                                                    int M, int N)
{
    const int lane = threadIdx.x & 31;
    const float* bias = e.bias;
    const int sub = lane >> 3, cq = (lane & 7) * 4;
    const int col = col0 + cq;
    // gate values: four 16-byte loads in flight at a time, issued before the
    // shared-memory round trip
    float4 g4[4];
    const float* gptr = (EXTRAS && e.mask) ? e.mask + static_cast<long long>(row0 + sub) * e.ldm + col : nullptr;
    if (gptr) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
            g4[k] = __ldg(reinterpret_cast<const float4*>(gptr + static_cast<long long>(k) * 4 * e.ldm));
    }
#pragma unroll
    for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(stage + lane * EPI_STAGE_LD + j) =
            make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                        __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
    __syncwarp();
    float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias) bv = make_float4(__ldg(bias + col), __ldg(bias + col + 1), __ldg(bias + col + 2),
                               __ldg(bias + col + 3));
    float* dptr = D + static_cast<long long>(row0 + sub) * ldd + col;
    const float* sptr = stage + sub * EPI_STAGE_LD + cq;
    const bool relu = e.relu != 0;
    // all eight results first, the stores after them: the reduction variant is an
    // asm statement with a memory clobber, inside this loop it would order every
    // shared-memory read behind the previous store and serialise the chunk
    float4 o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (i == 4 && gptr) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                g4[k] = __ldg(reinterpret_cast<const float4*>(gptr + static_cast<long long>(4 + k) * 4 * e.ldm));
        }
        const float4 a = *reinterpret_cast<const float4*>(sptr + i * 4 * EPI_STAGE_LD);
        o[i] = make_float4((cc.v[i].x + bv.x) + a.x, (cc.v[i].y + bv.y) + a.y,
                           (cc.v[i].z + bv.z) + a.z, (cc.v[i].w + bv.w) + a.w);
        if (relu) {
            o[i].x = o[i].x > 0.0f ? o[i].x : 0.0f;
            o[i].y = o[i].y > 0.0f ? o[i].y : 0.0f;
            o[i].z = o[i].z > 0.0f ? o[i].z : 0.0f;
            o[i].w = o[i].w > 0.0f ? o[i].w : 0.0f;
        }
        if (gptr) {
            const float4 g = g4[i & 3];
            o[i].x = __fadd_rn(0.0f, g.x > 0.0f ? o[i].x : 0.0f);
            o[i].y = __fadd_rn(0.0f, g.y > 0.0f ? o[i].y : 0.0f);
            o[i].z = __fadd_rn(0.0f, g.z > 0.0f ? o[i].z : 0.0f);
            o[i].w = __fadd_rn(0.0f, g.w > 0.0f ? o[i].w : 0.0f);
        }
    }
    if (EXTRAS && e.reduce) {
#pragma unroll
        for (int i = 0; i < 8; ++i) ptx::red_add_sys_v4(dptr + static_cast<long long>(i) * 4 * ldd, o[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(dptr + static_cast<long long>(i) * 4 * ldd) = o[i];
    }
    __syncwarp();
}

// Any chunk: every row and column is checked against M and N.
__device__ __forceinline__ void store_chunk_edge(const uint32_t (&v)[32], float* stage, float* D, long long ldd,
                                                    const CChunk& cc, const Epilogue& e, int row0, int col0,
                                                    int M, int N)
{
    const int lane = threadIdx.x & 31;
    const float* bias = e.bias;
    const int sub = lane >> 3, cq = (lane & 7) * 4;
    const int col = col0 + cq;
    const bool post = e.relu || e.mask;
    // the gate values of this lane's float4s are fetched four rows at a time, the
    // four loads in flight together (fetched one by one where they are needed
    // they would cost a memory round trip each)
    float4 gate[4];
    const bool gate_vec = e.mask && ((e.ldm & 3) == 0) && ((reinterpret_cast<uintptr_t>(e.mask) & 15) == 0);
    auto load_gates = [&](int first) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int grow = row0 + (first + k) * 4 + sub;
            gate[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (grow < M && col < N) {
                const float* mp = e.mask + static_cast<long long>(grow) * e.ldm + col;
                if (gate_vec && col + 3 < N) {
                    gate[k] = __ldg(reinterpret_cast<const float4*>(mp));
                } else {
                    gate[k].x = __ldg(mp);
                    if (col + 1 < N) gate[k].y = __ldg(mp + 1);
                    if (col + 2 < N) gate[k].z = __ldg(mp + 2);
                    if (col + 3 < N) gate[k].w = __ldg(mp + 3);
                }
            }
        }
    };
    if (e.mask) load_gates(0);
#pragma unroll
    for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(stage + lane * EPI_STAGE_LD + j) =
            make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                        __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
    __syncwarp();
    float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias) {
        if (col < N) bv.x = __ldg(bias + col);
        if (col + 1 < N) bv.y = __ldg(bias + col + 1);
        if (col + 2 < N) bv.z = __ldg(bias + col + 2);
        if (col + 3 < N) bv.w = __ldg(bias + col + 3);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (i == 4 && e.mask) load_gates(4);
        const int r = i * 4 + sub;
        const int grow = row0 + r;
        const float4 a = *reinterpret_cast<const float4*>(stage + r * EPI_STAGE_LD + cq);
        if (grow < M && col < N) {
            float* drow = D + static_cast<long long>(grow) * ldd;
            float4 o;
            o.x = (cc.v[i].x + bv.x) + a.x;
            o.y = (cc.v[i].y + bv.y) + a.y;
            o.z = (cc.v[i].z + bv.z) + a.z;
            o.w = (cc.v[i].w + bv.w) + a.w;
            if (post) {
                const bool gated = e.mask != nullptr;
                o.x = post_op_value(o.x, e.relu, gated, gate[i & 3].x);
                o.y = post_op_value(o.y, e.relu, gated, gate[i & 3].y);
                o.z = post_op_value(o.z, e.relu, gated, gate[i & 3].z);
                o.w = post_op_value(o.w, e.relu, gated, gate[i & 3].w);
            }
            if (e.reduce) {
                if (col + 3 < N) {
                    ptx::red_add_sys_v4(drow + col, o);
                } else {
                    ptx::red_add_sys(drow + col, o.x);
                    if (col + 1 < N) ptx::red_add_sys(drow + col + 1, o.y);
                    if (col + 2 < N) ptx::red_add_sys(drow + col + 2, o.z);
                }
            } else if (col + 3 < N) {
                *reinterpret_cast<float4*>(drow + col) = o;
            } else {
                drow[col] = o.x;
                if (col + 1 < N) drow[col + 1] = o.y;
                if (col + 2 < N) drow[col + 2] = o.z;
            }
        }
    }
    __syncwarp();
}

__device__ __forceinline__ void store_chunk_coalesced(const uint32_t (&v)[32], float* stage, float* D, long long ldd,
                                                    const CChunk& cc, const Epilogue& e, int row0, int col0,
                                                    int M, int N)
{
    const bool gate_aligned =
        !e.mask || (((e.ldm & 3) == 0) && ((reinterpret_cast<uintptr_t>(e.mask) & 15) == 0));
    if (gate_aligned && row0 + 32 <= M && col0 + 32 <= N) {
        if (e.mask || e.reduce)
            store_chunk_interior<true>(v, stage, D, ldd, cc, e, row0, col0, M, N);
        else
            store_chunk_interior<false>(v, stage, D, ldd, cc, e, row0, col0, M, N);
    } else
        store_chunk_edge(v, stage, D, ldd, cc, e, row0, col0, M, N);
}

// ---------------------------------------------------------------- column sums
// Column sums of op(B) taken from the B tiles as they pass through shared
// memory (the bias gradient of a Linear layer: B = dy).  Four extra warps (128
// threads) consume every stage next to the tensor core; only the CTAs of the
// first row of tiles add anything up, so the sums cost no extra global traffic.
constexpr int COLSUM_THREADS = 128;
constexpr int COLSUM_SCRATCH_BYTES = 2048;

// Adds one k-block (32 k) of the staged B tile to this thread's partial sums.
//   MN-major tile ([chunk][32 k rows][128 B], 32-byte-atom swizzle): thread owns
//     one 16-byte unit (4 columns) and a share of the k rows -> acc4;
//   K-major tile ([column][128 B of k], 16-byte swizzle): thread owns whole
//     rows (= columns of op(B)), tid and tid + 128 -> acc4.x / acc4.y.
template <bool B_MN, int NCOLS>
__device__ __forceinline__ void colsum_accumulate(const uint8_t* sb, int tid, float4& acc4)
{
    if (B_MN) {
        constexpr int UNITS = NCOLS / 4;                  // 16-byte units across the tile
        constexpr int PARTS = COLSUM_THREADS / UNITS;     // k shares
        constexpr int ROWS = BLOCK_K / PARTS;
        const int u = tid % UNITS, part = tid / UNITS;
        const uint8_t* base = sb + (u >> 3) * CHUNK_BYTES;
        const int uu = u & 7;
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int k = part * ROWS + i;
            const int phys = uu ^ ((k & 3) << 1);
            const float4 x = *reinterpret_cast<const float4*>(base + k * 128 + phys * 16);
            acc4.x += x.x; acc4.y += x.y; acc4.z += x.z; acc4.w += x.w;
        }
    } else {
#pragma unroll
        for (int h = 0; h < (NCOLS + COLSUM_THREADS - 1) / COLSUM_THREADS; ++h) {
            const int row = tid + h * COLSUM_THREADS;
            if (row >= NCOLS)
                break;
            const uint8_t* r = sb + row * 128;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 x = *reinterpret_cast<const float4*>(r + (((i + row) & 7) << 4));
                s += (x.x + x.y) + (x.z + x.w);
            }
            if (h == 0) acc4.x += s; else acc4.y += s;
        }
    }
}

// What a finished column sum does to out[n]: store scale * sum, or, for the in-place SGD
// update of a bias, subtract lr times that (each product rounded on its own).
__device__ __forceinline__ void colsum_store(float* out, float sum, float scale, float lr)
{
    const float g = __fmul_rn(sum, scale);
    *out = lr != 0.0f ? __fsub_rn(*out, __fmul_rn(g, lr)) : g;
}

// Combines the threads' partial sums and writes scale * sum for columns
// [n0, n0 + NCOLS) below N.  `scratch`: COLSUM_SCRATCH_BYTES of shared memory.
// Uses named barrier 1 among the 128 column-sum threads.

template <bool B_MN, int NCOLS>
__device__ __forceinline__ void colsum_finish(float4 acc4, float* scratch, int tid, float* out,
                                              float scale, int n0, int N, float lr)
{
    if (B_MN) {
        constexpr int UNITS = NCOLS / 4;
        constexpr int PARTS = COLSUM_THREADS / UNITS;
        reinterpret_cast<float4*>(scratch)[tid] = acc4;   // [part][unit]
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tid < UNITS) {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int q = 0; q < PARTS; ++q) {
                const float4 x = reinterpret_cast<const float4*>(scratch)[q * UNITS + tid];
                s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
            }
            const int col = n0 + tid * 4;
            const float v[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (col + e < N) colsum_store(out + col + e, v[e], scale, lr);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
    } else {
        if (tid < NCOLS && n0 + tid < N) colsum_store(out + n0 + tid, acc4.x, scale, lr);
        if (NCOLS > COLSUM_THREADS && n0 + tid + COLSUM_THREADS < N)
            colsum_store(out + n0 + tid + COLSUM_THREADS, acc4.y, scale, lr);
    }
}

// Looks the descriptor up in the context's cache; on a miss encodes it into the
// least recently used slot.  `encode` fills a CUtensorMap and returns a CUresult.
template <typename Encode>
inline int cached_map(sb200_ctx* ctx, CUtensorMap* out, const TensorMapKey& key, Encode encode)
{
    TensorMapSlot* slots = ctx->tmaps;
    int victim = 0;
    uint64_t oldest = ~0ull;
    for (int i = 0; i < TENSOR_MAP_SLOTS; ++i) {
        if (slots[i].stamp && memcmp(&slots[i].key, &key, sizeof(key)) == 0) {
            slots[i].stamp = ++ctx->tmap_clock;
            ctx->tmap_hits += 1;
            memcpy(out, &slots[i].map, sizeof(CUtensorMap));
            return SB200_OK;
        }
        if (slots[i].stamp < oldest) {
            oldest = slots[i].stamp;
            victim = i;
        }
    }
    ctx->tmap_misses += 1;
    TensorMapSlot& v = slots[victim];
    v.stamp = 0;
    if (encode(&v.map) != CUDA_SUCCESS)
        return SB200_ERR_CUDA;
    v.key = key;
    v.stamp = ++ctx->tmap_clock;
    memcpy(out, &v.map, sizeof(CUtensorMap));
    return SB200_OK;
}

// Tensor map over a stack of row-major matrices: dim0 = contiguous extent,
// dim1 = rows, dim2 = batch; box = 32 contiguous elements x box_rows x 1,
// out-of-range elements read as zero.  K-major tiles use the plain 128-byte
// swizzle; MN-major tiles the 128-byte swizzle with a 32-byte atom, the only
// MN-major layout the tensor core reads for 32-bit operands.
inline int make_map(sb200_ctx* ctx, CUtensorMap* map, const float* base, int64_t contig, int64_t rows,
             int64_t ld, int64_t batch, int64_t batch_stride, int box_rows, bool mn_major)
{
    EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
    if (!enc)
        return SB200_ERR_UNSUPPORTED;
    const int64_t nb = (batch_stride == 0) ? 1 : batch;
    const int64_t bs = (batch_stride == 0 || nb == 1) ? rows * ld : batch_stride;
    const TensorMapKey key{reinterpret_cast<uint64_t>(base), contig, rows, ld, nb, bs, box_rows,
                           mn_major ? 1 : 0};
    return cached_map(ctx, map, key, [&](CUtensorMap* m) {
        cuuint64_t dims[3] = {static_cast<cuuint64_t>(contig), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(nb)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 4, static_cast<cuuint64_t>(bs) * 4};
        cuuint32_t box[3] = {32, static_cast<cuuint32_t>(box_rows), 1};
        cuuint32_t estr[3] = {1, 1, 1};
        return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    });
}

// MN-major operand whose contiguous extent is a multiple of 32: view it as
// [batch][chunk = contig / 32][row][32] so that one box of 32 x 32 rows x
// `chunks` chunks brings a whole tile (same shared-memory image as `chunks`
// separate 32 x 32 boxes: chunk-major, 32 rows of 128 B each).
inline int make_map_merged(sb200_ctx* ctx, CUtensorMap* map, const float* base, int64_t contig,
                    int64_t rows, int64_t ld, int64_t batch, int64_t batch_stride, int chunks)
{
    EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
    if (!enc)
        return SB200_ERR_UNSUPPORTED;
    const int64_t nb = (batch_stride == 0) ? 1 : batch;
    const int64_t bs = (batch_stride == 0 || nb == 1) ? rows * ld : batch_stride;
    const TensorMapKey key{reinterpret_cast<uint64_t>(base), contig, rows, ld, nb, bs, chunks, 2};
    return cached_map(ctx, map, key, [&](CUtensorMap* m) {
        cuuint64_t dims[4] = {32, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(contig / 32),
                              static_cast<cuuint64_t>(nb)};
        cuuint64_t strides[3] = {static_cast<cuuint64_t>(ld) * 4, 128, static_cast<cuuint64_t>(bs) * 4};
        cuuint32_t box[4] = {32, static_cast<cuuint32_t>(BLOCK_K), static_cast<cuuint32_t>(chunks), 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    });
}

}  // namespace gemm
}  // namespace sb200
