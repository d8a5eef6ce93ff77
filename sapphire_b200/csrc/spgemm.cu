// CSR x CSR sparse GEMM, C = A.B, two passes (symbolic: row sizes; numeric:
// columns and values), columns ascending inside every row.
//
// Rows of A are binned by their number of scalar products
//   P(i) = sum over nonzeros (i,k) of A of nnz(B row k):
//
//   P == 0          empty output row
//   P <= 32         "tiny": one warp per row; the products sit one per lane,
//                   are sorted by column with a shuffle bitonic network and
//                   equal columns are merged with a segmented warp reduction
//   otherwise       one CTA per row with a dense accumulator in shared memory:
//                   a bitmap of the N columns marks the row's pattern
//                   (atomicOr), a prefix sum of the bitmap's popcounts turns a
//                   column into its rank inside the sorted output row, and the
//                   values are accumulated with shared-memory atomicAdd at that
//                   rank.  Reading the bitmap back in word order yields the
//                   columns already sorted, so no sort is needed.  Rows whose
//                   output exceeds the shared value buffer accumulate straight
//                   into their slice of C.V in global memory.
//   rows with P above a threshold are queued first so that the longest CTAs
//   start early.
//
// The symbolic pass runs the pattern part only (tiny: count distinct sorted
// keys; CTA: popcount of the bitmap); an exclusive scan of the counts gives ROW.
//
// Accumulation order inside an output entry is not fixed (atomics), hence
// values agree with a sequential sum to rounding, while ROW and COL are exact.
#include "common.cuh"

namespace sb200 {
namespace {

constexpr int TINY_MAX = 32;
constexpr unsigned HEAVY_MIN = 16384;
constexpr int ROW_THREADS = 256;
constexpr int VAL_CAP = 6144;            // fp32 accumulators per CTA in shared memory
constexpr uint32_t MAX_COLS = 1u << 20;  // bitmap of N bits must fit in shared memory

struct Csr {
    const uint32_t* row;
    const uint32_t* col;
    const float* val;
    uint32_t M, N;
};

struct Work {
    uint32_t* prod;        // [M] scalar products per row, saturating
    uint32_t* cnt;         // [M] nnz of each output row
    uint32_t* list_tiny;   // [M]
    uint32_t* list_mid;    // [M]
    uint32_t* list_heavy;  // [M]
    uint32_t* counters;    // [4]: tiny, mid, heavy, unused
};

// ------------------------------------------------------------ row work
__global__ void __launch_bounds__(256)
row_products_kernel(Csr A, const uint32_t* __restrict__ rowB, Work w)
{
    const int lane = threadIdx.x & 31;
    const uint32_t warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t i = warp_global; i < A.M; i += nwarps) {
        unsigned long long s = 0;
        for (uint32_t p = A.row[i] + lane; p < A.row[i + 1]; p += 32) {
            const uint32_t k = A.col[p];
            s += rowB[k + 1] - rowB[k];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) {
            const uint32_t P = s > 0xffffffffull ? 0xffffffffu : static_cast<uint32_t>(s);
            w.prod[i] = P;
            if (P == 0) {
                w.cnt[i] = 0;
            } else if (P <= TINY_MAX) {
                w.list_tiny[atomicAdd(&w.counters[0], 1u)] = i;
            } else if (P < HEAVY_MIN) {
                w.list_mid[atomicAdd(&w.counters[1], 1u)] = i;
            } else {
                w.list_heavy[atomicAdd(&w.counters[2], 1u)] = i;
            }
        }
    }
}

// ------------------------------------------------------------ tiny rows
// One warp per row.  Gathers the (<= 32) products into lanes, sorts by column.
__device__ __forceinline__ void tiny_gather(const Csr& A, const Csr& B, uint32_t i, int lane,
                                            uint32_t* s_key, float* s_val, bool with_values,
                                            uint32_t& key, float& val)
{
    s_key[lane] = 0xffffffffu;
    s_val[lane] = 0.0f;
    __syncwarp();
    uint32_t base = 0;
    const uint32_t pa = A.row[i], pe = A.row[i + 1];
    for (uint32_t p0 = pa; p0 < pe; p0 += 32) {
        const uint32_t p = p0 + lane;
        uint32_t qs = 0, len = 0;
        float av = 0.0f;
        if (p < pe) {
            const uint32_t k = A.col[p];
            qs = B.row[k];
            len = B.row[k + 1] - qs;
            if (with_values) av = A.val[p];
        }
        uint32_t incl = len;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        const uint32_t off = base + incl - len;
        for (uint32_t t = 0; t < len; ++t) {
            const uint32_t slot = off + t;
            if (slot < TINY_MAX) {
                s_key[slot] = B.col[qs + t];
                if (with_values) s_val[slot] = __fmul_rn(av, B.val[qs + t]);
            }
        }
        base += __shfl_sync(0xffffffffu, incl, 31);
    }
    __syncwarp();
    key = s_key[lane];
    val = s_val[lane];
    // bitonic sort of 32 (key, val) pairs across the warp, ascending key
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            const uint32_t okey = __shfl_xor_sync(0xffffffffu, key, j);
            const float oval = __shfl_xor_sync(0xffffffffu, val, j);
            const bool up = ((lane & k) == 0);
            const bool lower = ((lane & j) == 0);
            const bool take = (lower == up) ? (okey < key) : (okey > key);
            if (take) {
                key = okey;
                val = oval;
            }
        }
    }
}

template <bool NUMERIC>
__global__ void __launch_bounds__(256)
tiny_rows_kernel(Csr A, Csr B, Work w, const uint32_t* __restrict__ rowC,
                 uint32_t* __restrict__ colC, float* __restrict__ valC)
{
    __shared__ uint32_t s_key[8][32];
    __shared__ float s_val[8][32];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const uint32_t warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t count = w.counters[0];
    for (uint32_t idx = warp_global; idx < count; idx += nwarps) {
        const uint32_t i = w.list_tiny[idx];
        uint32_t key;
        float val;
        tiny_gather(A, B, i, lane, s_key[wib], s_val[wib], NUMERIC, key, val);
        // ties between equal keys keep no fixed order; the sum below is over
        // lanes in ascending lane order of the sorted sequence
        const uint32_t prev = __shfl_up_sync(0xffffffffu, key, 1);
        const bool valid = key != 0xffffffffu;
        const bool head = valid && (lane == 0 || prev != key);
        const uint32_t heads = __ballot_sync(0xffffffffu, head);
        if (!NUMERIC) {
            if (lane == 0) w.cnt[i] = __popc(heads);
        } else {
            // segmented sum: every head adds the values of the lanes up to the next head
            const uint32_t after = heads & ~((2u << lane) - 1u);        // heads above this lane
            const uint32_t valid_mask = __ballot_sync(0xffffffffu, valid);
            const int seg_end = after ? (__ffs(after) - 1) : (32 - __clz(valid_mask));
            float s = val;
            for (int l = 1; l < 32; ++l) {              // uniform trip count: shuffles stay converged
                const float v = __shfl_sync(0xffffffffu, val, l);
                if (head && l > lane && l < seg_end) s = __fadd_rn(s, v);
            }
            if (head) {
                const uint32_t pos = rowC[i] + __popc(heads & ((1u << lane) - 1u));
                colC[pos] = key;
                valC[pos] = s;
            }
        }
        __syncwarp();
    }
}

// ------------------------------------------------------- CTA-per-row path
constexpr int A_CHUNK = 512;             // nonzeros of A's row staged in shared memory at a time
constexpr int WALK_UNROLL = 4;           // independent loads in flight per thread

// Per-chunk staging of A's row: for nonzero p of the chunk, where B's row
// starts (qs), the running count of products before it (pref) and A's value.
struct RowChunk {
    uint32_t* qs;      // [A_CHUNK]
    uint32_t* pref;    // [A_CHUNK + 1]
    float* aval;       // [A_CHUNK]   (numeric only)
};

__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* s_warp,
                                                         uint32_t& total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    __syncthreads();                      // s_warp may still be read from a previous call
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    uint32_t warp_off = 0, tot = 0;
#pragma unroll
    for (int i = 0; i < ROW_THREADS / 32; ++i) {
        const uint32_t x = s_warp[i];
        if (i < warp) warp_off += x;
        tot += x;
    }
    total = tot;
    return warp_off + incl - v;
}

// Stages nonzeros [p0, p0 + n) of A's row i and returns the chunk's product count.
template <bool NUMERIC>
__device__ __forceinline__ uint32_t load_chunk(const Csr& A, const Csr& B, uint32_t p0, uint32_t n,
                                               const RowChunk& ch, uint32_t* s_warp)
{
    // two nonzeros per thread (A_CHUNK == 2 * ROW_THREADS)
    uint32_t len[2], qs[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const uint32_t e = threadIdx.x * 2 + u;
        len[u] = 0;
        qs[u] = 0;
        if (e < n) {
            const uint32_t k = A.col[p0 + e];
            qs[u] = B.row[k];
            len[u] = B.row[k + 1] - qs[u];
            if (NUMERIC) ch.aval[e] = A.val[p0 + e];
        }
    }
    uint32_t total;
    const uint32_t off = block_exclusive_scan(len[0] + len[1], s_warp, total);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const uint32_t e = threadIdx.x * 2 + u;
        if (e < n) {
            ch.qs[e] = qs[u];
            ch.pref[e] = off + (u ? len[0] : 0);
        }
    }
    if (threadIdx.x == 0) ch.pref[n] = total;
    __syncthreads();
    return total;
}

// Calls f(column, a_value * b_value) for every product of the staged chunk.
//
// Two schedules, chosen per chunk by the mean length of B's rows:
//  * rows of B of 16+ entries: one warp per nonzero of A, lanes stride B's row
//    with four loads in flight; no search, ~10 instructions per product;
//  * short rows: product t of the chunk belongs to the nonzero p with
//    pref[p] <= t < pref[p+1] (binary search); thread tid takes t = tid,
//    tid + 256, ... so that no lane idles on a one-entry row.
template <bool NUMERIC, typename F>
__device__ __forceinline__ void walk_chunk(const Csr& B, const RowChunk& ch, uint32_t n,
                                           uint32_t total, F f)
{
    if (total >= 16u * n) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        for (uint32_t p = warp; p < n; p += ROW_THREADS / 32) {
            const uint32_t qs = ch.qs[p];
            const uint32_t len = ch.pref[p + 1] - ch.pref[p];
            const float av = NUMERIC ? ch.aval[p] : 0.0f;
            for (uint32_t o = lane; o < len; o += 32 * WALK_UNROLL) {
                uint32_t col[WALK_UNROLL];
                float bv[WALK_UNROLL];
#pragma unroll
                for (int u = 0; u < WALK_UNROLL; ++u) {
                    if (o + 32 * u < len) {
                        col[u] = __ldg(B.col + qs + o + 32 * u);
                        if (NUMERIC) bv[u] = __ldg(B.val + qs + o + 32 * u);
                    }
                }
#pragma unroll
                for (int u = 0; u < WALK_UNROLL; ++u)
                    if (o + 32 * u < len) f(col[u], NUMERIC ? __fmul_rn(av, bv[u]) : 0.0f);
            }
        }
        return;
    }
    uint32_t p = 0;
    for (uint32_t base = threadIdx.x; base < total; base += ROW_THREADS * WALK_UNROLL) {
        uint32_t q[WALK_UNROLL], col[WALK_UNROLL];
        float av[WALK_UNROLL], bv[WALK_UNROLL];
#pragma unroll
        for (int u = 0; u < WALK_UNROLL; ++u) {
            const uint32_t t = base + u * ROW_THREADS;
            q[u] = 0xffffffffu;
            if (t < total) {
                uint32_t lo = p, hi = n;            // pref[lo] <= t < pref[hi]
                while (hi - lo > 1) {
                    const uint32_t mid = (lo + hi) >> 1;
                    if (ch.pref[mid] <= t) lo = mid; else hi = mid;
                }
                p = lo;
                q[u] = ch.qs[p] + (t - ch.pref[p]);
                if (NUMERIC) av[u] = ch.aval[p];
            }
        }
#pragma unroll
        for (int u = 0; u < WALK_UNROLL; ++u) {
            if (q[u] != 0xffffffffu) {
                col[u] = __ldg(B.col + q[u]);
                if (NUMERIC) bv[u] = __ldg(B.val + q[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < WALK_UNROLL; ++u)
            if (q[u] != 0xffffffffu) f(col[u], NUMERIC ? __fmul_rn(av[u], bv[u]) : 0.0f);
    }
}

// One CTA per row.
//   SYMBOLIC (NUMERIC == false): mark the row's columns in a shared-memory
//       bitmap, count them, and -- when `pattern` is given -- keep the bitmap in
//       global memory for the numeric pass (words * 4 bytes per row).
//   NUMERIC: rebuild the bitmap (FROM_PATTERN == false) or read it back,
//       prefix-sum its popcounts so that rank(j) = prefix[j / 32] +
//       popc(bits below j) is the position of column j in the sorted output row,
//       emit the columns in bitmap order, then accumulate every product at its rank.
template <bool NUMERIC, bool FROM_PATTERN>
__global__ void __launch_bounds__(ROW_THREADS, 4)
cta_rows_kernel(Csr A, Csr B, Work w, uint32_t words, uint32_t* __restrict__ pattern,
                const uint32_t* __restrict__ rowC, uint32_t* __restrict__ colC,
                float* __restrict__ valC)
{
    extern __shared__ uint32_t sm[];
    // symbolic: bitmap[words]; numeric: packed[words] = {bits, prefix}
    uint32_t* bitmap = sm;
    uint2* packed = reinterpret_cast<uint2*>(sm);
    uint32_t* after_map = sm + (NUMERIC ? 2 * words : words);
    RowChunk ch;
    ch.qs = after_map;                                           // [A_CHUNK]
    ch.pref = ch.qs + A_CHUNK;                                   // [A_CHUNK + 1] (+ pad)
    ch.aval = reinterpret_cast<float*>(ch.pref + A_CHUNK + 4);   // [A_CHUNK]   (numeric)
    float* vals = ch.aval + A_CHUNK;                             // [VAL_CAP]   (numeric)
    __shared__ uint32_t s_warp[ROW_THREADS / 32];

    const uint32_t n_heavy = w.counters[2];
    const uint32_t n_rows = n_heavy + w.counters[1];
    const uint32_t per_thread = (words + ROW_THREADS - 1) / ROW_THREADS;
    const uint32_t w_lo = threadIdx.x * per_thread;
    const uint32_t w_hi = min(w_lo + per_thread, words);

    for (uint32_t idx = blockIdx.x; idx < n_rows; idx += gridDim.x) {
        const uint32_t i = idx < n_heavy ? w.list_heavy[idx] : w.list_mid[idx - n_heavy];
        const uint32_t pa = A.row[i], pe = A.row[i + 1];
        const bool one_chunk = (pe - pa) <= A_CHUNK;
        uint32_t chunk_total = 0;
        uint32_t mine = 0;                                       // set bits in this thread's words

        if (!(NUMERIC && FROM_PATTERN)) {
            // ---- pattern: mark every product's column
            if (NUMERIC) {
                for (uint32_t x = threadIdx.x; x < words; x += ROW_THREADS)
                    packed[x] = make_uint2(0u, 0u);
            } else {
                for (uint32_t x = threadIdx.x; x < words; x += ROW_THREADS) bitmap[x] = 0;
            }
            __syncthreads();
            for (uint32_t p0 = pa; p0 < pe; p0 += A_CHUNK) {
                const uint32_t n = min(static_cast<uint32_t>(A_CHUNK), pe - p0);
                chunk_total = load_chunk<NUMERIC>(A, B, p0, n, ch, s_warp);
                walk_chunk<false>(B, ch, n, chunk_total, [&](uint32_t j, float) {
                    if (NUMERIC)
                        atomicOr(&packed[j >> 5].x, 1u << (j & 31));
                    else
                        atomicOr(&bitmap[j >> 5], 1u << (j & 31));
                });
                __syncthreads();
            }
            if (!NUMERIC && pattern) {
                // lane-contiguous copy: full 128-byte lines per warp
                uint32_t* dst = pattern + static_cast<size_t>(i) * words;
                for (uint32_t x = threadIdx.x; x < words; x += ROW_THREADS) dst[x] = bitmap[x];
            }
            for (uint32_t x = w_lo; x < w_hi; ++x)
                mine += __popc(NUMERIC ? packed[x].x : bitmap[x]);
        } else {
            // ---- pattern kept by the symbolic pass
            const uint32_t* src = pattern + static_cast<size_t>(i) * words;
            for (uint32_t x = threadIdx.x; x < words; x += ROW_THREADS) packed[x].x = src[x];
            __syncthreads();
            for (uint32_t x = w_lo; x < w_hi; ++x) mine += __popc(packed[x].x);
        }
        uint32_t total;
        uint32_t run = block_exclusive_scan(mine, s_warp, total);
        if (!NUMERIC) {
            if (threadIdx.x == 0) w.cnt[i] = total;
            __syncthreads();
            continue;
        }
        const uint32_t out0 = rowC[i];
        const bool in_smem = total <= VAL_CAP;
        // columns come out ascending: word order, then bit order.  They are
        // staged in the (not yet used) value buffer so that the global store is
        // lane-contiguous; rows wider than the buffer store them directly.
        uint32_t* stage = reinterpret_cast<uint32_t*>(vals);
        for (uint32_t x = w_lo; x < w_hi; ++x) {
            uint32_t bits = packed[x].x;
            packed[x].y = run;
            while (bits) {
                const int bpos = __ffs(bits) - 1;
                bits &= bits - 1;
                if (in_smem)
                    stage[run] = x * 32 + bpos;
                else
                    colC[out0 + run] = x * 32 + bpos;
                ++run;
            }
        }
        __syncthreads();
        if (in_smem) {
            for (uint32_t x = threadIdx.x; x < total; x += ROW_THREADS) {
                colC[out0 + x] = stage[x];
                vals[x] = 0.0f;                    // same word, same thread: no hazard
            }
        } else {
            for (uint32_t x = threadIdx.x; x < total; x += ROW_THREADS) valC[out0 + x] = 0.0f;
        }
        __syncthreads();
        // ---- values: accumulate every product at the rank of its column
        float* acc = in_smem ? vals : (valC + out0);
        for (uint32_t p0 = pa; p0 < pe; p0 += A_CHUNK) {
            const uint32_t n = min(static_cast<uint32_t>(A_CHUNK), pe - p0);
            if (FROM_PATTERN || !one_chunk)
                chunk_total = load_chunk<NUMERIC>(A, B, p0, n, ch, s_warp);
            walk_chunk<true>(B, ch, n, chunk_total, [&](uint32_t j, float prod) {
                const uint2 wp = packed[j >> 5];
                const uint32_t rank = wp.y + __popc(wp.x & ((1u << (j & 31)) - 1u));
                atomicAdd(&acc[rank], prod);
            });
            __syncthreads();
        }
        if (in_smem)
            for (uint32_t x = threadIdx.x; x < total; x += ROW_THREADS) valC[out0 + x] = vals[x];
        __syncthreads();
    }
}

// --------------------------------------------------------------- row scan
// rowC[0] = 0, rowC[i+1] = sum cnt[0..i]; one CTA, chunks of 1024 with carry.
__global__ void __launch_bounds__(1024)
row_scan_kernel(const uint32_t* __restrict__ cnt, uint32_t M, uint32_t* __restrict__ rowC,
                unsigned long long* __restrict__ total_out)
{
    __shared__ unsigned long long s_warp[32];
    __shared__ unsigned long long s_carry;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        s_carry = 0;
        rowC[0] = 0;
    }
    __syncthreads();
    for (uint32_t base = 0; base < M; base += 1024) {
        const uint32_t i = base + threadIdx.x;
        unsigned long long v = i < M ? cnt[i] : 0, incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        unsigned long long off = s_carry;
        for (int x = 0; x < warp; ++x) off += s_warp[x];
        if (i < M) rowC[i + 1] = static_cast<uint32_t>(off + incl);
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = off + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) *total_out = s_carry;
}

// ------------------------------------------------------------------- host
struct Plan {
    Csr A, B;
    Work w;
    uint32_t words;
    size_t smem_symbolic, smem_numeric;
    unsigned long long* d_total;
    uint32_t* pattern;          // [M][words] row bitmaps kept between the passes, or null
};

int make_plan(sb200_ctx* ctx, const sb200_csr* A, const sb200_csr* B, Plan* pl)
{
    if (!ctx || !A || !B)
        return SB200_ERR_INVALID_ARG;
    if (A->N != B->M)
        return SB200_ERR_INVALID_ARG;
    if (!A->ROW || !B->ROW || (A->NNZ && (!A->COL || !A->V)) || (B->NNZ && (!B->COL || !B->V)))
        return SB200_ERR_INVALID_ARG;
    if (B->N > MAX_COLS)
        return SB200_ERR_TOO_LARGE;
    pl->A = Csr{A->ROW, A->COL, A->V, A->M, A->N};
    pl->B = Csr{B->ROW, B->COL, B->V, B->M, B->N};
    const size_t M = A->M;
    const size_t words32 = 5 * M + 8;        // prod, cnt, 3 lists, counters
    const int rc = ensure_workspace(ctx, words32 * 4 + 16);
    if (rc)
        return rc;
    uint32_t* base = reinterpret_cast<uint32_t*>(ctx->d_workspace);
    pl->w.prod = base;
    pl->w.cnt = base + M;
    pl->w.list_tiny = base + 2 * M;
    pl->w.list_mid = base + 3 * M;
    pl->w.list_heavy = base + 4 * M;
    pl->w.counters = base + 5 * M;
    pl->d_total = reinterpret_cast<unsigned long long*>(base + 5 * M + 4);
    // keep the 64-bit total 8-byte aligned
    if (reinterpret_cast<uintptr_t>(pl->d_total) & 7)
        pl->d_total = reinterpret_cast<unsigned long long*>(base + 5 * M + 5);
    pl->words = (B->N + 31) / 32;
    if (pl->words == 0)
        pl->words = 1;
    const size_t chunk_bytes = (3 * A_CHUNK + 4) * 4;   // qs, pref (+pad), aval
    pl->pattern = nullptr;
    pl->smem_symbolic = static_cast<size_t>(pl->words) * 4 + chunk_bytes;
    pl->smem_numeric = static_cast<size_t>(pl->words) * 8 + chunk_bytes + VAL_CAP * 4;
    return SB200_OK;
}

int bin_rows(sb200_ctx* ctx, const Plan& pl, cudaStream_t stream)
{
    if (cudaMemsetAsync(pl.w.counters, 0, 16, stream) != cudaSuccess)
        return SB200_ERR_CUDA;
    if (pl.A.M == 0)
        return SB200_OK;
    const unsigned blocks = static_cast<unsigned>(ctx->sm_count) * 8;
    row_products_kernel<<<blocks, 256, 0, stream>>>(pl.A, pl.B.row, pl.w);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

// Identity of the operands a kept pattern belongs to.
bool same_operands(const sb200_ctx* ctx, const sb200_csr* A, const sb200_csr* B)
{
    const SpPatternKey& k = ctx->sp_key;
    return ctx->sp_valid && k.rowA == A->ROW && k.colA == A->COL && k.rowB == B->ROW &&
           k.colB == B->COL && k.M == A->M && k.K == A->N && k.N == B->N && k.nnzA == A->NNZ &&
           k.nnzB == B->NNZ;
}

// Row bitmaps are kept when they fit the budget (M * ceil(N / 32) * 4 bytes).
constexpr size_t PATTERN_BUDGET = static_cast<size_t>(2) << 30;

int prepare_pattern(sb200_ctx* ctx, Plan* pl, const sb200_csr* A, const sb200_csr* B)
{
    ctx->sp_valid = 0;
    const size_t need = static_cast<size_t>(A->M) * pl->words * 4;
    if (need == 0 || need > PATTERN_BUDGET)
        return SB200_OK;                       // numeric pass rebuilds the bitmaps
    if (need > ctx->sp_pattern_bytes) {
        if (ctx->d_sp_pattern) cudaFree(ctx->d_sp_pattern);
        ctx->d_sp_pattern = nullptr;
        ctx->sp_pattern_bytes = 0;
        void* p = nullptr;
        if (cudaMalloc(&p, need) != cudaSuccess) {
            cudaGetLastError();
            return SB200_OK;                   // no room: fall back to rebuilding
        }
        ctx->d_sp_pattern = static_cast<uint32_t*>(p);
        ctx->sp_pattern_bytes = need;
    }
    pl->pattern = ctx->d_sp_pattern;
    ctx->sp_key = SpPatternKey{A->ROW, A->COL, B->ROW, B->COL, A->M, A->N, B->N, A->NNZ, B->NNZ};
    return SB200_OK;
}

template <bool NUMERIC, bool FROM_PATTERN>
int run_rows(sb200_ctx* ctx, const Plan& pl, const uint32_t* rowC, uint32_t* colC, float* valC,
             cudaStream_t stream)
{
    if (pl.A.M == 0)
        return SB200_OK;
    const size_t smem = NUMERIC ? pl.smem_numeric : pl.smem_symbolic;
    auto kern = cta_rows_kernel<NUMERIC, FROM_PATTERN>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
        return SB200_ERR_CUDA;
    int per_sm = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, ROW_THREADS, smem) !=
            cudaSuccess || per_sm < 1)
        per_sm = 1;
    const unsigned grid = static_cast<unsigned>(ctx->sm_count) * per_sm;
    kern<<<grid, ROW_THREADS, smem, stream>>>(pl.A, pl.B, pl.w, pl.words, pl.pattern, rowC, colC,
                                              valC);
    tiny_rows_kernel<NUMERIC><<<static_cast<unsigned>(ctx->sm_count) * 8, 256, 0, stream>>>(
        pl.A, pl.B, pl.w, rowC, colC, valC);
    ctx->launches += 2;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" int sb200_spgemm_csr_symbolic(sb200_ctx* ctx, const sb200_csr* A, const sb200_csr* B,
                                         uint32_t* rowC, int64_t* nnzC, sb200_stream stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!rowC || !nnzC)
        return SB200_ERR_INVALID_ARG;
    Plan pl;
    int rc = make_plan(ctx, A, B, &pl);
    if (rc)
        return rc;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    if ((rc = prepare_pattern(ctx, &pl, A, B)) || (rc = bin_rows(ctx, pl, stream)))
        return rc;
    if ((rc = run_rows<false, false>(ctx, pl, nullptr, nullptr, nullptr, stream)))
        return rc;
    ctx->sp_valid = pl.pattern != nullptr;
    row_scan_kernel<<<1, 1024, 0, stream>>>(pl.w.cnt, pl.A.M, rowC, pl.d_total);
    ctx->launches += 1;
    unsigned long long total = 0;
    if (cudaMemcpyAsync(&total, pl.d_total, sizeof(total), cudaMemcpyDeviceToHost, stream) !=
            cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
        return SB200_ERR_CUDA;
    if (total > 0xffffffffull)
        return SB200_ERR_TOO_LARGE;       // NNZ and ROW are 32-bit in the CSR struct
    *nnzC = static_cast<int64_t>(total);
    return SB200_OK;
}

// The row bins are rebuilt here, so the call works on its own.  When the
// immediately preceding symbolic call on this context had the same operand
// arrays (same pointers and sizes; their contents must not have changed) the
// row patterns it kept are read back instead of being recomputed.
extern "C" int sb200_spgemm_csr_numeric(sb200_ctx* ctx, const sb200_csr* A, const sb200_csr* B,
                                        const uint32_t* rowC, uint32_t* colC, float* valC,
                                        sb200_stream stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!rowC)
        return SB200_ERR_INVALID_ARG;
    Plan pl;
    int rc = make_plan(ctx, A, B, &pl);
    if (rc)
        return rc;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    if ((rc = bin_rows(ctx, pl, stream)))
        return rc;
    if (same_operands(ctx, A, B)) {
        pl.pattern = ctx->d_sp_pattern;
        return run_rows<true, true>(ctx, pl, rowC, colC, valC, stream);
    }
    return run_rows<true, false>(ctx, pl, rowC, colC, valC, stream);
}

extern "C" int sb200_spgemm_csr(sb200_ctx* ctx, const sb200_csr* A, const sb200_csr* B,
                                sb200_csr* C, sb200_stream stream_)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!C)
        return SB200_ERR_INVALID_ARG;
    Plan pl;
    int rc = make_plan(ctx, A, B, &pl);
    if (rc)
        return rc;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    C->V = nullptr; C->COL = nullptr; C->ROW = nullptr;
    C->NNZ = 0; C->M = A->M; C->N = B->N;
    C->Padding[0] = C->Padding[1] = C->Padding[2] = 0;
    if (cudaMalloc(&C->ROW, (static_cast<size_t>(A->M) + 1) * 4) != cudaSuccess)
        return SB200_ERR_ALLOC;
    // symbolic: bins stay valid in the workspace for the numeric pass below
    if ((rc = prepare_pattern(ctx, &pl, A, B)) || (rc = bin_rows(ctx, pl, stream)) ||
        (rc = run_rows<false, false>(ctx, pl, nullptr, nullptr, nullptr, stream))) {
        sb200_csr_free(C);
        return rc;
    }
    row_scan_kernel<<<1, 1024, 0, stream>>>(pl.w.cnt, pl.A.M, C->ROW, pl.d_total);
    ctx->launches += 1;
    unsigned long long total = 0;
    if (cudaMemcpyAsync(&total, pl.d_total, sizeof(total), cudaMemcpyDeviceToHost, stream) !=
            cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess) {
        sb200_csr_free(C);
        return SB200_ERR_CUDA;
    }
    if (total > 0xffffffffull) {
        sb200_csr_free(C);
        return SB200_ERR_TOO_LARGE;
    }
    C->NNZ = static_cast<uint32_t>(total);
    const size_t n = total ? total : 1;
    if (cudaMalloc(&C->COL, n * 4) != cudaSuccess || cudaMalloc(&C->V, n * 4) != cudaSuccess) {
        sb200_csr_free(C);
        return SB200_ERR_ALLOC;
    }
    rc = pl.pattern ? run_rows<true, true>(ctx, pl, C->ROW, C->COL, C->V, stream)
                    : run_rows<true, false>(ctx, pl, C->ROW, C->COL, C->V, stream);
    ctx->sp_valid = 0;
    if (rc) {
        sb200_csr_free(C);
        return rc;
    }
    return SB200_OK;
}

extern "C" int sb200_csr_free(sb200_csr* C)
{
    if (!C)
        return SB200_ERR_INVALID_ARG;
    if (C->V) cudaFree(C->V);
    if (C->COL) cudaFree(C->COL);
    if (C->ROW) cudaFree(C->ROW);
    C->V = nullptr; C->COL = nullptr; C->ROW = nullptr;
    C->NNZ = 0;
    return SB200_OK;
}

extern "C" int sb200_csr_copy_out(const sb200_csr* src, uint32_t* row, uint32_t* col, float* val,
                                  int to_host, sb200_stream stream_)
{
    if (!src || !row || !src->ROW || (src->NNZ && (!col || !val || !src->COL || !src->V)))
        return SB200_ERR_INVALID_ARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const cudaMemcpyKind kind = to_host ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    const size_t n = src->NNZ;
    if (cudaMemcpyAsync(row, src->ROW, (static_cast<size_t>(src->M) + 1) * 4, kind, stream) !=
        cudaSuccess)
        return SB200_ERR_CUDA;
    if (n && (cudaMemcpyAsync(col, src->COL, n * 4, kind, stream) != cudaSuccess ||
              cudaMemcpyAsync(val, src->V, n * 4, kind, stream) != cudaSuccess))
        return SB200_ERR_CUDA;
    return cudaStreamSynchronize(stream) == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}
