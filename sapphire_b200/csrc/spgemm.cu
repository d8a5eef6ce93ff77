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
constexpr uint32_t MAX_COLS = 1u << 19;  // bitmap + prefix of N columns must fit in shared memory

struct Csr {
    const uint32_t* row;
    const uint32_t* col;
    const float* val;
    uint32_t M, N;
};

struct Work {
    uint32_t* cnt;         // [M] nnz of each output row
    uint32_t* bq;          // [nnzA] for every nonzero (i,k) of A: where B's row k starts
    uint32_t* blen;        // [nnzA] ... and its length
    uint4* rows_mid;       // [M] {row, first nonzero, end nonzero, products} per CTA-path row
    uint4* rows_heavy;     // [M] the same for rows with many products (queued first)
    uint32_t* list_tiny;   // [M]
    uint32_t* counters;    // [4]: tiny, mid, heavy, next row of the running row kernel
};

// ------------------------------------------------------------ row work
// One warp per row of A: records where each nonzero's row of B lies (so that
// the row kernels read it with one coalesced load instead of a dependent
// gather), counts the row's scalar products and queues the row in its bin.
// In the numeric pass (rowC given) a row whose output is wider than the small
// value buffer also goes to the heavy bin, whose kernel has a large one.
__global__ void __launch_bounds__(256)
row_products_kernel(Csr A, const uint32_t* __restrict__ rowB, Work w,
                    const uint32_t* __restrict__ rowC)
{
    const int lane = threadIdx.x & 31;
    const uint32_t warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t i = warp_global; i < A.M; i += nwarps) {
        unsigned long long s = 0;
        const uint32_t pa = A.row[i], pe = A.row[i + 1];
        for (uint32_t p = pa + lane; p < pe; p += 32) {
            const uint32_t k = A.col[p];
            const uint32_t q0 = rowB[k], q1 = rowB[k + 1];
            w.bq[p] = q0;
            w.blen[p] = q1 - q0;
            s += q1 - q0;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) {
            const uint32_t P = s > 0xffffffffull ? 0xffffffffu : static_cast<uint32_t>(s);
            if (P == 0) {
                w.cnt[i] = 0;
            } else if (P <= TINY_MAX) {
                w.list_tiny[atomicAdd(&w.counters[0], 1u)] = i;
            } else if (P < HEAVY_MIN && !(rowC && rowC[i + 1] - rowC[i] > VAL_CAP)) {
                w.rows_mid[atomicAdd(&w.counters[1], 1u)] = make_uint4(i, pa, pe, P);
            } else {
                w.rows_heavy[atomicAdd(&w.counters[2], 1u)] = make_uint4(i, pa, pe, P);
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

// Shared-memory staging of a chunk of A's row.
struct RowChunk {
    uint32_t* qs;      // [A_CHUNK]     start of B's row
    uint32_t* len;     // [A_CHUNK]     its length
    float* aval;       // [A_CHUNK]     A's value (numeric only)
    uint32_t* longs;   // [A_CHUNK]     nonzeros whose row of B the whole CTA walks
    uint32_t* n_long;  // [1]
};

template <int THREADS>
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* s_warp,
                                                         uint32_t& total)
{
    constexpr int NWARPS = THREADS / 32;
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
    for (int i = 0; i < NWARPS; ++i) {
        const uint32_t x = s_warp[i];
        if (i < warp) warp_off += x;
        tot += x;
    }
    total = tot;
    return warp_off + incl - v;
}

// Copies nonzeros [p0, p0 + n) of A's row into shared memory (coalesced reads
// of the arrays the row-work kernel prepared) and lists the ones whose row of B
// is long enough for the whole CTA.  *ch.n_long must be zero on entry (a barrier
// earlier); no barrier inside.
template <int THREADS, bool NUMERIC>
__device__ __forceinline__ void stage_chunk(const Csr& A, const Work& w, uint32_t p0, uint32_t n,
                                            const RowChunk& ch)
{
    for (uint32_t e = threadIdx.x; e < n; e += THREADS) {
        const uint32_t len = w.blen[p0 + e];
        ch.qs[e] = w.bq[p0 + e];
        ch.len[e] = len;
        if (NUMERIC) ch.aval[e] = A.val[p0 + e];
        if (len >= static_cast<uint32_t>(THREADS)) ch.longs[atomicAdd(ch.n_long, 1u)] = e;
    }
}

// Calls f(column, a_value * b_value) for every product of the staged chunk.
//  * rows of B of THREADS or more entries: the whole CTA strides the row (a
//    4096-entry row would otherwise keep one warp busy while 31 wait);
//  * rows with more than SHORT_ROW entries: one warp per nonzero of A, lanes
//    stride B's row with four loads in flight;
//  * shorter rows: one thread per nonzero, so that a warp is not spent on a
//    one-entry row (power-law matrices are mostly such rows).
constexpr uint32_t SHORT_ROW = 8;

template <int THREADS, bool NUMERIC, typename F>
__device__ __forceinline__ void walk_chunk(const Csr& B, const RowChunk& ch, uint32_t n, F f)
{
    constexpr int NWARPS = THREADS / 32;
    const uint32_t n_long = *ch.n_long;
    for (uint32_t l = 0; l < n_long; ++l) {
        const uint32_t e = ch.longs[l];
        const uint32_t qs = ch.qs[e], len = ch.len[e];
        const float av = NUMERIC ? ch.aval[e] : 0.0f;
        for (uint32_t o = threadIdx.x; o < len; o += THREADS * 2) {
            const bool second = o + THREADS < len;
            const uint32_t c0 = __ldg(B.col + qs + o);
            const uint32_t c1 = second ? __ldg(B.col + qs + o + THREADS) : 0u;
            float v0 = 0.0f, v1 = 0.0f;
            if (NUMERIC) {
                v0 = __ldg(B.val + qs + o);
                if (second) v1 = __ldg(B.val + qs + o + THREADS);
            }
            f(c0, NUMERIC ? __fmul_rn(av, v0) : 0.0f);
            if (second) f(c1, NUMERIC ? __fmul_rn(av, v1) : 0.0f);
        }
    }
    for (uint32_t e = threadIdx.x; e < n; e += THREADS) {
        const uint32_t len = ch.len[e];
        if (len <= SHORT_ROW) {
            const uint32_t qs = ch.qs[e];
            const float av = NUMERIC ? ch.aval[e] : 0.0f;
            for (uint32_t q = 0; q < len; ++q)
                f(__ldg(B.col + qs + q), NUMERIC ? __fmul_rn(av, __ldg(B.val + qs + q)) : 0.0f);
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t p = warp; p < n; p += NWARPS) {
        const uint32_t len = ch.len[p];
        if (len <= SHORT_ROW || len >= static_cast<uint32_t>(THREADS))
            continue;
        const uint32_t qs = ch.qs[p];
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
}

// One CTA per row.
//   SYMBOLIC (NUMERIC == false): mark the row's columns in a shared-memory
//       bitmap, count them, and -- when `pattern` is given -- keep the bitmap in
//       global memory for the numeric pass (words * 4 bytes per row).
//   NUMERIC: rebuild the bitmap (FROM_PATTERN == false) or read it back,
//       prefix-sum its popcounts so that rank(j) = prefix[j / 32] +
//       popc(bits below j) is the position of column j in the sorted output row,
//       emit the columns in bitmap order, then accumulate every product at its rank.
// The bitmap is split into one contiguous range of `wpw` words per warp; inside
// a range lane l owns words l, l + 32, ... so every shared-memory access of the
// scans is conflict-free and the prefix needs only warp shuffles.
template <int THREADS, int MIN_BLOCKS, bool NUMERIC, bool FROM_PATTERN>
__global__ void __launch_bounds__(THREADS, MIN_BLOCKS)
cta_rows_kernel(Csr A, Csr B, Work w, const uint4* __restrict__ rows,
                const uint32_t* __restrict__ n_rows_ptr, uint32_t* __restrict__ next_row,
                uint32_t words, uint32_t wpw,
                uint32_t val_cap, uint32_t* __restrict__ pattern,
                const uint32_t* __restrict__ rowC, uint32_t* __restrict__ colC,
                float* __restrict__ valC)
{
    constexpr int NWARPS = THREADS / 32;
    extern __shared__ uint32_t sm[];
    const uint32_t padded = wpw * NWARPS;                        // >= words
    // symbolic: bitmap[padded]; numeric: packed[padded] = {bits, prefix}
    uint32_t* bitmap = sm;
    uint2* packed = reinterpret_cast<uint2*>(sm);
    uint32_t* after_map = sm + (NUMERIC ? 2 * padded : padded);
    RowChunk ch;
    ch.qs = after_map;
    ch.len = ch.qs + A_CHUNK;
    ch.aval = reinterpret_cast<float*>(ch.len + A_CHUNK);
    ch.longs = reinterpret_cast<uint32_t*>(ch.aval + A_CHUNK);
    float* vals = reinterpret_cast<float*>(ch.longs + A_CHUNK);  // [val_cap]   (numeric)
    __shared__ uint32_t s_tot[NWARPS];
    __shared__ uint32_t s_n_long;
    __shared__ uint32_t s_next;
    ch.n_long = &s_n_long;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t n_rows = *n_rows_ptr;
    const uint32_t wbase = warp * wpw;                           // this warp's word range

    auto bits_at = [&](uint32_t x) -> uint32_t { return NUMERIC ? packed[x].x : bitmap[x]; };

    // Rows are handed out through a counter: their cost varies by an order of
    // magnitude in the heavy bin, a fixed stride would leave SMs idle.
    for (;;) {
        if (threadIdx.x == 0) {
            s_next = atomicAdd(next_row, 1u);
            s_n_long = 0;
        }
        __syncthreads();
        const uint32_t idx = s_next;
        if (idx >= n_rows)
            break;
        const uint4 d = rows[idx];
        const uint32_t i = d.x, pa = d.y, pe = d.z;
        const uint32_t nnzA = pe - pa;
        const bool one_chunk = nnzA <= A_CHUNK;
        const uint32_t out0 = NUMERIC ? rowC[i] : 0;

        const uint32_t n0 = min(static_cast<uint32_t>(A_CHUNK), nnzA);
        stage_chunk<THREADS, NUMERIC>(A, w, pa, n0, ch);
        if (NUMERIC && FROM_PATTERN) {
            const uint32_t* src = pattern + static_cast<size_t>(i) * words;
            for (uint32_t x = threadIdx.x; x < padded; x += THREADS)
                packed[x].x = x < words ? src[x] : 0u;
        } else if (NUMERIC) {
            for (uint32_t x = threadIdx.x; x < padded; x += THREADS)
                packed[x] = make_uint2(0u, 0u);
        } else {
            for (uint32_t x = threadIdx.x; x < padded; x += THREADS) bitmap[x] = 0;
        }
        __syncthreads();

        if (!(NUMERIC && FROM_PATTERN)) {
            // ---- pattern: mark every product's column
            for (uint32_t p0 = pa; p0 < pe; p0 += A_CHUNK) {
                const uint32_t n = min(static_cast<uint32_t>(A_CHUNK), pe - p0);
                if (p0 != pa) {
                    if (threadIdx.x == 0) s_n_long = 0;          // previous walk ended at a barrier
                    __syncthreads();
                    stage_chunk<THREADS, NUMERIC>(A, w, p0, n, ch);
                    __syncthreads();
                }
                walk_chunk<THREADS, false>(B, ch, n, [&](uint32_t j, float) {
                    if (NUMERIC)
                        atomicOr(&packed[j >> 5].x, 1u << (j & 31));
                    else
                        atomicOr(&bitmap[j >> 5], 1u << (j & 31));
                });
                __syncthreads();
            }
            if (!NUMERIC && pattern) {
                uint32_t* dst = pattern + static_cast<size_t>(i) * words;
                for (uint32_t x = threadIdx.x; x < words; x += THREADS) dst[x] = bitmap[x];
            }
        }

        // ---- popcounts: warp-local running prefix over this warp's word range
        uint32_t carry = 0;
        for (uint32_t m = 0; m < wpw; m += 32) {
            const uint32_t x = wbase + m + lane;
            const uint32_t c = __popc(bits_at(x));
            uint32_t incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            if (NUMERIC) packed[x].y = carry + incl - c;          // relative to the warp's range
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) s_tot[warp] = carry;
        __syncthreads();
        uint32_t woff = 0, total = 0;
#pragma unroll
        for (int v = 0; v < NWARPS; ++v) {
            const uint32_t t = s_tot[v];
            if (v < warp) woff += t;
            total += t;
        }
        if (!NUMERIC) {
            if (threadIdx.x == 0) w.cnt[i] = total;
            __syncthreads();                                      // s_tot, bitmap reused next row
            continue;
        }

        // ---- columns: ascending = word order, then bit order.  Staged in the (not
        // yet used) value buffer so that the global store is lane-contiguous; rows
        // wider than the buffer store them directly.
        const bool staged = total <= val_cap;
        uint32_t* stage = reinterpret_cast<uint32_t*>(vals);
        for (uint32_t m = 0; m < wpw; m += 32) {
            const uint32_t x = wbase + m + lane;
            uint2 wp = packed[x];
            wp.y += woff;
            packed[x].y = wp.y;
            uint32_t bits = wp.x, run = wp.y;
            while (bits) {
                const int bpos = __ffs(bits) - 1;
                bits &= bits - 1;
                if (staged)
                    stage[run] = x * 32 + bpos;
                else
                    colC[out0 + run] = x * 32 + bpos;
                ++run;
            }
        }
        __syncthreads();
        if (staged)
            for (uint32_t x = threadIdx.x; x < total; x += THREADS) colC[out0 + x] = stage[x];

        // ---- values: accumulate every product at the rank of its column.  Rows
        // with more output entries than the value buffer take one pass over the
        // products per buffer-sized window of ranks.
        for (uint32_t r0 = 0; r0 < total; r0 += val_cap) {
            const uint32_t span = min(val_cap, total - r0);
            __syncthreads();
            for (uint32_t x = threadIdx.x; x < span; x += THREADS) vals[x] = 0.0f;
            __syncthreads();
            for (uint32_t p0 = pa; p0 < pe; p0 += A_CHUNK) {
                const uint32_t n = min(static_cast<uint32_t>(A_CHUNK), pe - p0);
                if (!one_chunk) {
                    __syncthreads();
                    if (threadIdx.x == 0) s_n_long = 0;
                    __syncthreads();
                    stage_chunk<THREADS, NUMERIC>(A, w, p0, n, ch);
                    __syncthreads();
                }
                walk_chunk<THREADS, true>(B, ch, n, [&](uint32_t j, float prod) {
                    const uint2 wp = packed[j >> 5];
                    const uint32_t rank = wp.y + __popc(wp.x & ((1u << (j & 31)) - 1u)) - r0;
                    if (rank < span) atomicAdd(&vals[rank], prod);
                });
            }
            __syncthreads();
            for (uint32_t x = threadIdx.x; x < span; x += THREADS) valC[out0 + r0 + x] = vals[x];
        }
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
    uint32_t words;             // bitmap words per row
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
    const size_t M = A->M, nnzA = A->NNZ;
    // cnt[M] | bq[nnzA] | blen[nnzA] | list_tiny[M] | counters[4] | total (8 B) | pad |
    // rows_mid[M] (16 B each) | rows_heavy[M]
    const size_t head_words = (2 * M + 2 * nnzA + 4 + 2 + 3) & ~static_cast<size_t>(3);
    const size_t bytes = head_words * 4 + 2 * M * sizeof(uint4) + 64;
    const int rc = ensure_workspace(ctx, bytes);
    if (rc)
        return rc;
    uint32_t* base = reinterpret_cast<uint32_t*>(ctx->d_workspace);
    pl->w.cnt = base;
    pl->w.bq = base + M;
    pl->w.blen = base + M + nnzA;
    pl->w.list_tiny = base + M + 2 * nnzA;
    pl->w.counters = base + 2 * M + 2 * nnzA;
    uintptr_t tot = reinterpret_cast<uintptr_t>(pl->w.counters + 4);
    tot = (tot + 7) & ~static_cast<uintptr_t>(7);
    pl->d_total = reinterpret_cast<unsigned long long*>(tot);
    uintptr_t desc = (reinterpret_cast<uintptr_t>(base + head_words) + 15) & ~static_cast<uintptr_t>(15);
    pl->w.rows_mid = reinterpret_cast<uint4*>(desc);
    pl->w.rows_heavy = pl->w.rows_mid + M;
    pl->words = (B->N + 31) / 32;
    if (pl->words == 0)
        pl->words = 1;
    pl->pattern = nullptr;
    return SB200_OK;
}

int bin_rows(sb200_ctx* ctx, const Plan& pl, const uint32_t* rowC, cudaStream_t stream)
{
    if (cudaMemsetAsync(pl.w.counters, 0, 16, stream) != cudaSuccess)
        return SB200_ERR_CUDA;
    if (pl.A.M == 0)
        return SB200_OK;
    const unsigned blocks = static_cast<unsigned>(ctx->sm_count) * 8;
    row_products_kernel<<<blocks, 256, 0, stream>>>(pl.A, pl.B.row, pl.w, rowC);
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

// Row bitmaps are kept when they fit the limit (M * ceil(N / 32) * 4 bytes).
constexpr size_t PATTERN_LIMIT = static_cast<size_t>(2) << 30;

int prepare_pattern(sb200_ctx* ctx, Plan* pl, const sb200_csr* A, const sb200_csr* B)
{
    ctx->sp_valid = 0;
    const size_t need = static_cast<size_t>(A->M) * pl->words * 4;
    if (need == 0 || need > PATTERN_LIMIT)
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

constexpr int HEAVY_THREADS = 1024;
constexpr uint32_t HEAVY_VAL_CAP = 40960;     // 160 KB of fp32 accumulators, one CTA per SM

template <int THREADS, int MIN_BLOCKS, bool NUMERIC, bool FROM_PATTERN>
int launch_rows(sb200_ctx* ctx, const Plan& pl, const uint4* rows, const uint32_t* n_rows,
                uint32_t* next_row, uint32_t val_cap, const uint32_t* rowC, uint32_t* colC, float* valC,
                cudaStream_t stream)
{
    constexpr int NWARPS = THREADS / 32;
    const uint32_t wpw = ((pl.words + NWARPS - 1) / NWARPS + 31) & ~31u;
    const size_t padded = static_cast<size_t>(wpw) * NWARPS;
    const size_t chunk_bytes = 4 * A_CHUNK * 4;                // qs, len, aval, longs
    if (NUMERIC) {
        // the value buffer takes what the bitmap leaves of the 227 KB per CTA
        const size_t room = 226 * 1024, fixed = padded * 8 + chunk_bytes;
        if (fixed + 1024 * 4 > room)
            return SB200_ERR_TOO_LARGE;
        if (fixed + static_cast<size_t>(val_cap) * 4 > room)
            val_cap = static_cast<uint32_t>((room - fixed) / 4);
    }
    const size_t smem = NUMERIC ? padded * 8 + chunk_bytes + static_cast<size_t>(val_cap) * 4
                                : padded * 4 + chunk_bytes;
    auto kern = cta_rows_kernel<THREADS, MIN_BLOCKS, NUMERIC, FROM_PATTERN>;
    // attribute and occupancy of this instance, remembered per (device, smem size)
    static thread_local int cached_dev = -1, cached_per_sm = 1;
    static thread_local size_t cached_smem = 0;
    if (cached_dev != ctx->device || cached_smem != smem) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)) != cudaSuccess) {
            cudaGetLastError();
            return SB200_ERR_TOO_LARGE;                         // bitmap beyond shared memory
        }
        int n = 1;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, THREADS, smem) !=
                cudaSuccess || n < 1)
            n = 1;
        cached_dev = ctx->device;
        cached_smem = smem;
        cached_per_sm = n;
    }
    const int per_sm = cached_per_sm;
    const unsigned grid = static_cast<unsigned>(ctx->sm_count) * per_sm;
    if (cudaMemsetAsync(next_row, 0, 4, stream) != cudaSuccess)
        return SB200_ERR_CUDA;
    kern<<<grid, THREADS, smem, stream>>>(pl.A, pl.B, pl.w, rows, n_rows, next_row, pl.words, wpw, val_cap,
                                          pl.pattern, rowC, colC, valC);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

template <bool NUMERIC, bool FROM_PATTERN>
int run_rows(sb200_ctx* ctx, const Plan& pl, const uint32_t* rowC, uint32_t* colC, float* valC,
             cudaStream_t stream)
{
    if (pl.A.M == 0)
        return SB200_OK;
    // heavy rows first: 1024 threads and a large value buffer, one CTA per SM
    int rc = launch_rows<HEAVY_THREADS, 1, NUMERIC, FROM_PATTERN>(
        ctx, pl, pl.w.rows_heavy, pl.w.counters + 2, pl.w.counters + 3, HEAVY_VAL_CAP, rowC, colC, valC, stream);
    if (rc)
        return rc;
    rc = launch_rows<ROW_THREADS, 4, NUMERIC, FROM_PATTERN>(
        ctx, pl, pl.w.rows_mid, pl.w.counters + 1, pl.w.counters + 3, VAL_CAP, rowC, colC, valC, stream);
    if (rc)
        return rc;
    tiny_rows_kernel<NUMERIC><<<static_cast<unsigned>(ctx->sm_count) * 8, 256, 0, stream>>>(
        pl.A, pl.B, pl.w, rowC, colC, valC);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

}  // namespace
}  // namespace sb200

using namespace sb200;

extern "C" int sb200_spgemm_csr_symbolic(sb200_ctx* ctx, const sb200_csr* A, const sb200_csr* B,
                                         uint32_t* rowC, int64_t* nnzC, sb200_stream stream_)
{
    TraceRange trace("sb200_spgemm_csr_symbolic");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!rowC || !nnzC)
        return SB200_ERR_INVALID_ARG;
    Plan pl;
    int rc = make_plan(ctx, A, B, &pl);
    if (rc)
        return rc;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    if ((rc = prepare_pattern(ctx, &pl, A, B)) || (rc = bin_rows(ctx, pl, nullptr, stream)))
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
    TraceRange trace("sb200_spgemm_csr_numeric");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!rowC)
        return SB200_ERR_INVALID_ARG;
    Plan pl;
    int rc = make_plan(ctx, A, B, &pl);
    if (rc)
        return rc;
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    if ((rc = bin_rows(ctx, pl, rowC, stream)))
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
    TraceRange trace("sb200_spgemm_csr");
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
    if ((rc = prepare_pattern(ctx, &pl, A, B)) || (rc = bin_rows(ctx, pl, nullptr, stream)) ||
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
    // bin again, now that the output row sizes are known
    if ((rc = bin_rows(ctx, pl, C->ROW, stream))) {
        sb200_csr_free(C);
        return rc;
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
