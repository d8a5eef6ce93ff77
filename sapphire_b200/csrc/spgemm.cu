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
//                   column into its rank inside the sorted output row, and every
//                   product stores its column and adds its value at that rank in
//                   a shared-memory window, which is then copied to C with
//                   16-byte stores: the columns come out sorted without a sort.
//                   Rows with more output entries than the window take one walk
//                   over their products per window (no global atomics).
//   rows with many products, or with an output wider than the small window, go
//   to a second instance of the same kernel with 1024 threads, one CTA per SM
//   and a large window.
//
// The symbolic pass runs the pattern part only (tiny: count distinct sorted
// keys; CTA: popcount of the bitmap); an exclusive scan of the counts gives ROW.
//
// Accumulation order inside an output entry is not fixed (atomics), hence
// values agree with a sequential sum to rounding, while ROW and COL are exact.
#include "common.cuh"

// the symbolic instance of the row kernel folds the output offset to zero, which
// turns a bounds check of its (dead) numeric half into "unsigned >= 0"
#pragma nv_diag_suppress 186

namespace sb200 {
namespace {

constexpr int TINY_MAX = 32;
constexpr uint32_t ALL_WINDOWS = 0xffffffffu;   // work item covers the whole output row
constexpr unsigned HEAVY_MIN = 16384;
constexpr int ROW_THREADS = 256;
// Output entries a mid-bin CTA holds in shared memory (wider rows go to the heavy
// bin): with 16-bit staged columns four CTAs fit on an SM, with 32-bit ones three.
__host__ __device__ constexpr uint32_t mid_cap(uint32_t n_cols) { return n_cols <= 65536 ? 5376u : 6144u; }
constexpr uint32_t MAX_COLS = 1u << 19;  // bitmap + prefix of N columns must fit in shared memory

struct Csr {
    const uint32_t* row;
    const uint32_t* col;
    const float* val;
    uint32_t M, N;
};

struct Work {
    uint32_t* cnt;         // [M] nnz of each output row
    uint32_t* prod;        // [M] scalar products of each row (saturating)
    uint32_t* bq;          // [nnzA] for every nonzero (i,k) of A: where B's row k starts
    uint32_t* blen;        // [nnzA] ... and its length
    uint4* rows_mid;       // [M] {row, first nonzero, end nonzero, window} per CTA-path row
    uint4* rows_heavy;     // [2M] the same for rows with many products or a wide output;
                           //      numeric pass: one entry per window of the output row
    uint32_t* list_tiny;   // [M]
    uint32_t* counters;    // [8]: tiny, mid, heavy, next row of the running row kernel, heavy windows
};

// Queues a heavy row.  In the numeric pass (width = its output entries) a row
// wider than one window of `heavy_cap` entries is cut into one work item per
// window, so that it spreads over several SMs; these items go to the second
// half of the queue (rows_heavy[M .. 2M), counters[4]).  When that half is full
// the row stays a single item whose CTA walks the windows itself.
__device__ __forceinline__ void queue_heavy(const Work& w, uint32_t M, uint32_t i, uint32_t pa,
                                            uint32_t pe, uint32_t width, uint32_t heavy_cap)
{
    const uint32_t nw = heavy_cap ? (width + heavy_cap - 1) / heavy_cap : 1u;
    if (nw > 1) {
        const uint32_t at = atomicAdd(&w.counters[4], nw);
        if (at + nw <= M) {
            for (uint32_t k = 0; k < nw; ++k) w.rows_heavy[M + at + k] = make_uint4(i, pa, pe, k);
            return;
        }
        for (uint32_t k = 0; k < nw && at + k < M; ++k)           // taken but unused: empty items
            w.rows_heavy[M + at + k] = make_uint4(ALL_WINDOWS, 0u, 0u, 0u);
    }
    w.rows_heavy[atomicAdd(&w.counters[2], 1u)] = make_uint4(i, pa, pe, ALL_WINDOWS);
}

// ------------------------------------------------------------ row work
// One warp per row of A: records where each nonzero's row of B lies (so that
// the row kernels read it with one coalesced load instead of a dependent
// gather), counts the row's scalar products and queues the row in its bin.
// In the numeric pass (rowC given) a row whose output is wider than the small
// value buffer also goes to the heavy bin, whose kernel has a large one.
__global__ void __launch_bounds__(256)
row_products_kernel(Csr A, const uint32_t* __restrict__ rowB, Work w,
                    const uint32_t* __restrict__ rowC, uint32_t cap, uint32_t heavy_cap)
{
    const int lane = threadIdx.x & 31;
    const uint32_t warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t i = warp_global; i < A.M; i += nwarps) {
        unsigned long long s = 0;
        const uint32_t pa = A.row[i], pe = A.row[i + 1];
        // four nonzeros per lane and step: the gathers from B.ROW are dependent
        // loads, a row of A with thousands of nonzeros would otherwise crawl
        for (uint32_t p = pa + lane; p < pe; p += 128) {
            uint32_t k[4], q0[4], q1[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) k[u] = p + 32 * u < pe ? A.col[p + 32 * u] : 0u;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                q0[u] = rowB[k[u]];
                q1[u] = rowB[k[u] + 1];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (p + 32 * u < pe) {
                    w.bq[p + 32 * u] = q0[u];
                    w.blen[p + 32 * u] = q1[u] - q0[u];
                    s += q1[u] - q0[u];
                }
            }
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
            } else if (P < HEAVY_MIN && !(rowC && rowC[i + 1] - rowC[i] > cap)) {
                w.rows_mid[atomicAdd(&w.counters[1], 1u)] = make_uint4(i, pa, pe, ALL_WINDOWS);
            } else {
                queue_heavy(w, A.M, i, pa, pe, rowC ? rowC[i + 1] - rowC[i] : 0u, rowC ? heavy_cap : 0u);
            }
        }
    }
}

// The bins again, from the product counts a previous row_products_kernel left in
// the workspace, now that the output row sizes are known (one thread per row).
__global__ void __launch_bounds__(256)
rebin_kernel(Csr A, Work w, const uint32_t* __restrict__ rowC, uint32_t cap, uint32_t heavy_cap)
{
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < A.M; i += gridDim.x * blockDim.x) {
        const uint32_t P = w.prod[i];
        if (P == 0)
            continue;
        if (P <= TINY_MAX)
            w.list_tiny[atomicAdd(&w.counters[0], 1u)] = i;
        else if (P < HEAVY_MIN && rowC[i + 1] - rowC[i] <= cap)
            w.rows_mid[atomicAdd(&w.counters[1], 1u)] = make_uint4(i, A.row[i], A.row[i + 1], ALL_WINDOWS);
        else
            queue_heavy(w, A.M, i, A.row[i], A.row[i + 1], rowC[i + 1] - rowC[i], heavy_cap);
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
constexpr uint32_t SHORT_ROW = 8;        // rows of B up to this length are walked by one thread
constexpr uint32_t SUB = 16;             // lanes that share one descriptor (a piece of a row of B)
constexpr uint32_t TILE_WORDS = 2048;    // bitmap words covered by one block-wide prefix step
constexpr int PIECES_IN_FLIGHT = 4;      // descriptors a lane group loads before it accumulates

// Shared-memory work lists of the product walk.  A nonzero (i,k) of A whose
// row of B has SHORT_ROW < len < THREADS entries is cut into pieces of SUB
// entries; every piece gets a descriptor and SUB adjacent lanes take one piece
// at a time, so that a warp works on two pieces with most lanes busy whatever
// the row lengths are (16 and 8 lanes per piece time alike on uniform rows, 16
// is a few per cent ahead on power-law rows: half the descriptors).  Rows of THREADS or more entries are listed in
// the same arrays (used before the descriptors) and walked by the whole CTA.
template <int THREADS>
struct WalkLists {
    static constexpr uint32_t CAP = 3 * THREADS;                 // descriptors per round
    static constexpr size_t BYTES = CAP * 4 + CAP * 4 + CAP;     // off, aval, n
    uint32_t* off;     // [CAP]  first entry of the piece in B.col / B.val
                       //        (long rows: [0, THREADS) starts, [THREADS, 2 THREADS) lengths)
    float* aval;       // [CAP]  A's value
    uint8_t* n;        // [CAP]  entries in the piece (1..SUB)
};

__device__ __forceinline__ void prefetch_l2(const void* p)
{
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

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

// Calls f(column, a_value * b_value) for every scalar product of A's nonzeros
// [pa, pe).  The whole CTA must call it; *n_long must be zero on entry and is
// zero again on return; the lists must not be in use (a barrier earlier).  No
// barrier after the last call of f.
template <int THREADS, bool WITH_VALUES, typename F>
__device__ __forceinline__ void walk_products(const Csr& A, const Csr& B, const Work& w,
                                              uint32_t pa, uint32_t pe, const WalkLists<THREADS>& wl,
                                              uint32_t* n_long, uint32_t* s_warp, F f)
{
    constexpr uint32_t CAP = WalkLists<THREADS>::CAP;
    constexpr uint32_t NGROUPS = THREADS / SUB;
    const uint32_t sub = threadIdx.x & (SUB - 1), group = threadIdx.x / SUB;
    uint32_t* long_len = wl.off + THREADS;

    for (uint32_t p0 = pa; p0 < pe; p0 += THREADS) {
        const uint32_t e = p0 + threadIdx.x;
        uint32_t len = 0, qs = 0;
        float av = 0.0f;
        if (e < pe) {
            len = w.blen[e];
            qs = w.bq[e];
            if (WITH_VALUES) av = A.val[e];
        }
        const bool is_long = len >= static_cast<uint32_t>(THREADS);
        const bool is_mid = len > SHORT_ROW && !is_long;
        if (is_long) {
            const uint32_t s = atomicAdd(n_long, 1u);
            wl.off[s] = qs;
            long_len[s] = len;
            if (WITH_VALUES) wl.aval[s] = av;
        }
        const uint32_t pieces = is_mid ? (len + SUB - 1) / SUB : 0u;
        uint32_t total_pieces;
        const uint32_t first = block_exclusive_scan<THREADS>(pieces, s_warp, total_pieces);

        // ---- rows of B walked by the whole CTA
        const uint32_t nl = *n_long;
        if (nl) {
            for (uint32_t l = 0; l < nl; ++l) {
                const uint32_t lq = wl.off[l], ll = long_len[l];
                const float la = WITH_VALUES ? wl.aval[l] : 0.0f;
                for (uint32_t o = threadIdx.x; o < ll; o += THREADS * 2) {
                    const bool second = o + THREADS < ll;
                    const uint32_t c0 = __ldg(B.col + lq + o);
                    const uint32_t c1 = second ? __ldg(B.col + lq + o + THREADS) : 0u;
                    float v0 = 0.0f, v1 = 0.0f;
                    if (WITH_VALUES) {
                        v0 = __ldg(B.val + lq + o);
                        if (second) v1 = __ldg(B.val + lq + o + THREADS);
                    }
                    const uint32_t cc[2] = {c0, c1};
                    const float pp[2] = {WITH_VALUES ? __fmul_rn(la, v0) : 0.0f,
                                         WITH_VALUES ? __fmul_rn(la, v1) : 0.0f};
                    const bool aa[2] = {true, second};
                    f(cc, pp, aa);
                }
            }
            __syncthreads();                                      // the lists become descriptors
            if (threadIdx.x == 0) *n_long = 0;
        }

        // ---- short rows: one thread each, straight from registers
        if (len <= SHORT_ROW)
            for (uint32_t q = 0; q < len; ++q) {
                const uint32_t cc[1] = {__ldg(B.col + qs + q)};
                const float pp[1] = {WITH_VALUES ? __fmul_rn(av, __ldg(B.val + qs + q)) : 0.0f};
                const bool aa[1] = {true};
                f(cc, pp, aa);
            }

        // ---- everything between: pieces of SUB entries, SUB lanes per piece
        for (uint32_t base = 0; base < total_pieces; base += CAP) {
            if (base) __syncthreads();                            // previous round consumed
            if (pieces) {
                const uint32_t c_lo = base > first ? base - first : 0u;
                const uint32_t c_hi = min(pieces, base + CAP > first ? base + CAP - first : 0u);
                for (uint32_t c = c_lo; c < c_hi; ++c) {
                    const uint32_t slot = first + c - base;
                    wl.off[slot] = qs + c * SUB;
                    wl.n[slot] = static_cast<uint8_t>(min(SUB, len - c * SUB));
                    if (WITH_VALUES) wl.aval[slot] = av;
                }
            }
            __syncthreads();
            const uint32_t nd = min(CAP, total_pieces - base);
            for (uint32_t d = group; d < nd; d += PIECES_IN_FLIGHT * NGROUPS) {
                uint32_t o[PIECES_IN_FLIGHT], cc[PIECES_IN_FLIGHT];
                float pp[PIECES_IN_FLIGHT];
                bool aa[PIECES_IN_FLIGHT];
#pragma unroll
                for (int u = 0; u < PIECES_IN_FLIGHT; ++u) {
                    const uint32_t du = d + u * NGROUPS;
                    aa[u] = du < nd && sub < wl.n[du];
                    o[u] = aa[u] ? wl.off[du] + sub : 0u;
                }
#pragma unroll
                for (int u = 0; u < PIECES_IN_FLIGHT; ++u) {
                    cc[u] = aa[u] ? __ldg(B.col + o[u]) : 0u;
                    pp[u] = (WITH_VALUES && aa[u]) ? __ldg(B.val + o[u]) : 0.0f;
                }
                if (WITH_VALUES) {
#pragma unroll
                    for (int u = 0; u < PIECES_IN_FLIGHT; ++u)
                        if (aa[u]) pp[u] = __fmul_rn(wl.aval[d + u * NGROUPS], pp[u]);
                }
                f(cc, pp, aa);
            }
        }
        if (p0 + THREADS < pe) __syncthreads();                   // lists reused by the next group
    }
}

// One CTA per row.
//   SYMBOLIC (NUMERIC == false): mark the row's columns in a shared-memory
//       bitmap, count them, and -- when `pattern` is given -- keep the bitmap in
//       global memory for the numeric pass (`pitch` words per row).
//   NUMERIC: rebuild the bitmap (FROM_PATTERN == false) or read it back,
//       prefix-sum its popcounts so that rank(j) = prefix[j / 32] +
//       popc(bits below j) is the position of column j in the sorted output row,
//       then walk the products once per window of `val_cap` ranks: each product
//       stores its column and adds its value at its rank in shared memory, and
//       the window is copied to C with 16-byte stores.  The rank carries the
//       row's misalignment (first output index mod 4) so that the shared-memory
//       and the global side of that copy are aligned alike.
// ColT is the shared-memory type of a staged column: 16 bits when N <= 65536
// (a smaller window buffer lets a fourth CTA fit on the SM), else 32.
// Thread t owns WPT consecutive bitmap words per tile of TILE_WORDS words.
template <int THREADS, int MIN_BLOCKS, bool NUMERIC, bool FROM_PATTERN, typename ColT>
__global__ void __launch_bounds__(THREADS, MIN_BLOCKS)
cta_rows_kernel(Csr A, Csr B, Work w, const uint4* __restrict__ rows,
                const uint32_t* __restrict__ n_rows_ptr, const uint4* __restrict__ rows2,
                const uint32_t* __restrict__ n_rows2_ptr, uint32_t cap2, uint32_t* __restrict__ next_row,
                uint32_t pitch, uint32_t tiles, uint32_t val_cap, int vec_ok,
                uint32_t* __restrict__ pattern, const uint32_t* __restrict__ rowC,
                uint32_t* __restrict__ colC, float* __restrict__ valC)
{
    constexpr int NWARPS = THREADS / 32;
    constexpr uint32_t WPT = TILE_WORDS / THREADS;               // 8, 4 or 2
    static_assert(WPT >= 2 && WPT * THREADS == TILE_WORDS, "tile must divide among the threads");
    extern __shared__ uint4 sm4[];
    uint32_t* sm = reinterpret_cast<uint32_t*>(sm4);
    const uint32_t padded = tiles * TILE_WORDS;                  // >= pitch
    // symbolic: bitmap[pitch]; numeric: packed[padded] = {bits, prefix}
    uint32_t* bitmap = sm;
    uint2* packed = reinterpret_cast<uint2*>(sm);
    // Where entry e of the rank table sits.  A thread owns WPT consecutive entries
    // and writes them two at a time with 16-byte stores; with WPT == 8 the lanes
    // of a store are 64 bytes apart and would hit two of the eight 16-byte bank
    // groups, so the 16-byte slot index is XOR-ed with two higher bits.
    auto at = [](uint32_t e) -> uint32_t {
        if constexpr (WPT == 8) {
            const uint32_t slot = e >> 1;
            return ((slot ^ ((slot >> 3) & 3u)) << 1) | (e & 1u);
        } else {
            return e;
        }
    };
    uint32_t* after_map = sm + (NUMERIC ? 2 * padded : pitch);
    WalkLists<THREADS> wl;
    wl.off = after_map;
    wl.aval = reinterpret_cast<float*>(wl.off + WalkLists<THREADS>::CAP);
    wl.n = reinterpret_cast<uint8_t*>(wl.aval + WalkLists<THREADS>::CAP);
    float* vals = reinterpret_cast<float*>(wl.n + WalkLists<THREADS>::CAP);   // [val_cap + 4]
    ColT* cols = reinterpret_cast<ColT*>(vals + val_cap + 4);                 // [val_cap + 4]
    __shared__ uint32_t s_warp[NWARPS];
    __shared__ uint32_t s_n_long;
    __shared__ uint32_t s_next;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // the work items: a first list and, when given, a second one of at most cap2 entries
    const uint32_t n_rows1 = *n_rows_ptr;
    const uint32_t n_rows = n_rows1 + (rows2 ? min(*n_rows2_ptr, cap2) : 0u);
    auto item = [&](uint32_t idx) -> uint4 { return idx < n_rows1 ? rows[idx] : rows2[idx - n_rows1]; };

    // Rows are handed out through a counter (their cost varies by an order of
    // magnitude in the heavy bin, a fixed stride would leave SMs idle), a few at
    // a time where rows are small, so that the next row is known early enough to
    // pull what its prologue reads into L2 while the current row is worked on.
    constexpr uint32_t BATCH = THREADS >= 1024 ? 1 : 4;
    for (;;) {
        __syncthreads();                                          // previous row done with shared memory
        if (threadIdx.x == 0) {
            s_next = atomicAdd(next_row, BATCH);
            s_n_long = 0;
        }
        __syncthreads();
        const uint32_t idx_first = s_next;
        if (idx_first >= n_rows)
            break;
        const uint32_t idx_end = min(idx_first + BATCH, n_rows);
      for (uint32_t idx = idx_first; idx < idx_end; ++idx) {
        if (idx != idx_first) __syncthreads();                    // previous row done with shared memory
        const uint4 d = item(idx);
        const uint32_t i = d.x, pa = d.y, pe = d.z;
        if (i == ALL_WINDOWS)
            continue;                                             // an empty item of the window queue
        const uint32_t out0 = NUMERIC ? rowC[i] : 0;
        if (BATCH > 1 && idx + 1 < idx_end && item(idx + 1).x != ALL_WINDOWS) {
            const uint4 dn = item(idx + 1);
            if ((threadIdx.x & 7) == 0 && dn.y + threadIdx.x < dn.z) {
                prefetch_l2(w.blen + dn.y + threadIdx.x);
                prefetch_l2(w.bq + dn.y + threadIdx.x);
                if (NUMERIC) prefetch_l2(A.val + dn.y + threadIdx.x);
            }
            if (NUMERIC && threadIdx.x == 0) prefetch_l2(rowC + dn.x);
            if (NUMERIC && FROM_PATTERN) {
                const uint32_t* nsrc = pattern + static_cast<size_t>(dn.x) * pitch;
                for (uint32_t x = threadIdx.x * 8; x < pitch; x += THREADS * 8) prefetch_l2(nsrc + x);
            }
        }

        if (!(NUMERIC && FROM_PATTERN)) {
            // ---- pattern: mark every product's column
            const uint32_t n4 = (NUMERIC ? 2 * padded : pitch) / 4;
            for (uint32_t x = threadIdx.x; x < n4; x += THREADS) sm4[x] = make_uint4(0u, 0u, 0u, 0u);
            __syncthreads();
            walk_products<THREADS, false>(A, B, w, pa, pe, wl, &s_n_long, s_warp, [&](const auto& col, const auto&, const auto& act) {
                constexpr int U = sizeof(col) / sizeof(col[0]);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (!act[u]) continue;
                    const uint32_t j = col[u];
                    if (NUMERIC)
                        atomicOr(&packed[at(j >> 5)].x, 1u << (j & 31));
                    else
                        atomicOr(&bitmap[j >> 5], 1u << (j & 31));
                }
            });
            __syncthreads();
        }

        if (!NUMERIC) {
            // ---- count, and keep the bitmap for the numeric pass
            uint32_t* dst = pattern ? pattern + static_cast<size_t>(i) * pitch : nullptr;
            uint32_t c = 0;
            for (uint32_t x = threadIdx.x * 4; x < pitch; x += THREADS * 4) {
                const uint4 b = *reinterpret_cast<const uint4*>(bitmap + x);
                c += __popc(b.x) + __popc(b.y) + __popc(b.z) + __popc(b.w);
                if (dst) *reinterpret_cast<uint4*>(dst + x) = b;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
            if (lane == 0) s_warp[warp] = c;
            __syncthreads();
            if (threadIdx.x == 0) {
                uint32_t total = 0;
#pragma unroll
                for (int v = 0; v < NWARPS; ++v) total += s_warp[v];
                w.cnt[i] = total;
            }
            continue;
        }

        // ---- ranks: prefix[word] = set bits before it (+ the row's misalignment)
        const uint32_t shift = out0 & 3u;
        uint32_t carry = shift;
        const uint32_t* src = FROM_PATTERN ? pattern + static_cast<size_t>(i) * pitch : nullptr;
        for (uint32_t t = 0; t < tiles; ++t) {
            const uint32_t x0 = (t * THREADS + threadIdx.x) * WPT;
            uint32_t bits[WPT];
            if (FROM_PATTERN) {
                if (x0 < pitch) {                                  // pitch is a multiple of 8 >= WPT
                    if constexpr (WPT == 2) {
                        const uint2 v = *reinterpret_cast<const uint2*>(src + x0);
                        bits[0] = v.x; bits[1] = v.y;
                    } else {
#pragma unroll
                        for (uint32_t k = 0; k < WPT; k += 4) {
                            const uint4 v = *reinterpret_cast<const uint4*>(src + x0 + k);
                            bits[k] = v.x; bits[k + 1] = v.y; bits[k + 2] = v.z; bits[k + 3] = v.w;
                        }
                    }
                } else {
#pragma unroll
                    for (uint32_t k = 0; k < WPT; ++k) bits[k] = 0;
                }
            } else {
#pragma unroll
                for (uint32_t k = 0; k < WPT; k += 2) {
                    const uint4 two = *reinterpret_cast<const uint4*>(packed + at(x0 + k));
                    bits[k] = two.x;
                    bits[k + 1] = two.z;
                }
            }
            uint32_t c = 0;
#pragma unroll
            for (uint32_t k = 0; k < WPT; ++k) c += __popc(bits[k]);
            uint32_t tile_total;
            uint32_t run = carry + block_exclusive_scan<THREADS>(c, s_warp, tile_total);
#pragma unroll
            for (uint32_t k = 0; k < WPT; k += 2) {
                const uint32_t r1 = run + __popc(bits[k]);
                *reinterpret_cast<uint4*>(packed + at(x0 + k)) = make_uint4(bits[k], run, bits[k + 1], r1);
                run = r1 + __popc(bits[k + 1]);
            }
            carry += tile_total;
        }
        const uint32_t total = carry - shift;

        // ---- columns and values, one window of ranks at a time: the item's
        // window, or all of them
        const uint32_t r_begin = d.w == ALL_WINDOWS ? 0u : d.w * val_cap;
        const uint32_t r_end = d.w == ALL_WINDOWS ? total : min(total, r_begin + val_cap);
        for (uint32_t r0 = r_begin; r0 < r_end; r0 += val_cap) {
            const uint32_t span = min(val_cap, total - r0);
            const uint32_t lim = span + shift;                    // slots [shift, lim) are this window
            __syncthreads();                                      // ranks written; previous window copied out
            for (uint32_t x = threadIdx.x; x < (lim + 3) / 4; x += THREADS)
                reinterpret_cast<float4*>(vals)[x] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            __syncthreads();
            walk_products<THREADS, true>(A, B, w, pa, pe, wl, &s_n_long, s_warp, [&](const auto& col, const auto& prod, const auto& act) {
                // all rank lookups first, then the stores, then the atomics: the
                // shared-memory round trips of a batch overlap instead of chaining
                constexpr int U = sizeof(col) / sizeof(col[0]);
                uint32_t slot[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const uint32_t j = col[u];
                    const uint2 wp = packed[at(j >> 5)];
                    slot[u] = act[u] ? wp.y + __popc(wp.x & ((1u << (j & 31)) - 1u)) - r0 : 0xffffffffu;
                }
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (slot[u] < lim) cols[slot[u]] = static_cast<ColT>(col[u]);   // slots below `shift`: never copied out
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (slot[u] < lim) atomicAdd(&vals[slot[u]], prod[u]);
            });
            __syncthreads();
            uint32_t* gcol = colC + (out0 + r0 - shift);          // slot s <-> gcol[s]; 16-byte aligned
            float* gval = valC + (out0 + r0 - shift);
            for (uint32_t q = threadIdx.x; q < (lim + 3) / 4; q += THREADS) {
                const uint32_t s0 = q * 4;
                if (vec_ok && s0 >= shift && s0 + 4 <= lim) {
                    if constexpr (sizeof(ColT) == 2) {
                        const uint2 raw = *reinterpret_cast<const uint2*>(cols + s0);
                        *reinterpret_cast<uint4*>(gcol + s0) =
                            make_uint4(raw.x & 0xffffu, raw.x >> 16, raw.y & 0xffffu, raw.y >> 16);
                    } else {
                        *reinterpret_cast<uint4*>(gcol + s0) = *reinterpret_cast<const uint4*>(cols + s0);
                    }
                    *reinterpret_cast<float4*>(gval + s0) = *reinterpret_cast<const float4*>(vals + s0);
                } else {
                    for (uint32_t s = max(s0, shift); s < min(s0 + 4, lim); ++s) {
                        gcol[s] = cols[s];
                        gval[s] = vals[s];
                    }
                }
            }
        }
      }
    }
}

// ------------------------------------------- mid rows, N <= 65536 columns
// The bulk of a sparse product: rows with 33 .. 16383 scalar products whose output
// fits one shared-memory window.  Same two passes and the same bitmap idea as the
// general row kernel above, rebuilt around what bounds it -- the LSU data pipe
// (shared-memory wavefronts: a 32-lane access to random banks takes ~3.5, an
// atomic ~9) and instruction issue:
//
//   * rank table: one 4-byte word per group of 16 columns, {pattern bits 0-15,
//     rank of the group's first column bits 16-28, "group has a column hit by more
//     than one product" bit 31}: a lookup is ONE 4-byte access (8-byte words are
//     served half a warp at a time).  Ranks fit 13 bits because the window does.
//   * accumulation without atomics wherever possible.  The symbolic pass notices
//     when a product's column bit was already set and flags the column's group in a
//     second, small bitmap (128 words per row) that is kept with the row bitmap.
//     In the numeric pass a product of an unflagged group is the only one of its
//     column: it stores its value.  Products of flagged groups (3 % of the columns
//     of a 0.1 % dense product collide) swap themselves into the accumulator with
//     atomicExch and, if they displaced a partial sum, take the slot's content out,
//     add, and put the sum back until nothing was displaced.  fp32 atomicAdd in
//     shared memory is a compare-and-swap loop, the most expensive step per product.
//   * the product walk: 16 lanes per nonzero of A stream that row of B, five
//     chunks of 16 entries in flight (immediate offsets from one base pointer), each
//     chunk skipped as soon as both lane groups of the warp are past their row's
//     end; rows of B of up to 4 entries are done by single threads, rows of 256 and
//     more by the whole CTA.  One ballot-compacted list per 256 nonzeros of A; no
//     scan, no per-piece descriptors.
//   * the next row's kept bitmaps and per-nonzero arrays are loaded into registers
//     while the current row is walked, so a row starts without a trip to HBM.
constexpr int MID_THREADS = 256;
constexpr uint32_t MID_WORDS = 2048;        // bitmap words of 65536 columns
constexpr uint32_t DUP_WORDS = MID_WORDS / 16;   // one bit per group of 16 columns
constexpr uint32_t MID_SHORT = 4;
constexpr uint32_t MID_LONG = 256;
constexpr uint32_t MID_BATCH = 8;           // rows fetched per atomic
constexpr int MID_CHUNKS = 5;               // chunks of 16 entries in flight per lane group
constexpr uint32_t NO_COL = 0xffffffffu;
constexpr uint32_t FAST_MID_CAP = 6208;     // output entries per row: 4 CTAs of 56.5 KB per SM
constexpr uint32_t DUP_FLAG = 0x80000000u;

// physical index of rank-table word `g` (group of 16 columns).  Thread t writes
// words 16 t .. 16 t + 15 with four 16-byte stores; a plain layout would put the
// lanes of one store 64 bytes apart, on two of the eight 16-byte bank groups.  Each
// thread permutes its own four 16-byte slots instead: slot ^= (t >> 1) & 3.
__device__ __forceinline__ uint32_t rank_word(uint32_t g) { return g ^ ((g >> 3) & 12u); }

struct MidEntry {
    uint32_t qs, len;
    float a;
};

// L2 residency hints.  B (tens of MB) is re-read by every row of A and should stay
// in the 126 MB L2; C (GBs, written once) and the kept row bitmaps (written once,
// read once) should not push it out.
struct L2Hints {
    uint64_t keep, stream;
};
__device__ __forceinline__ L2Hints make_l2_hints()
{
    L2Hints h;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(h.keep));
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(h.stream));
    return h;
}
__device__ __forceinline__ uint32_t ld_keep_u32(const uint32_t* p, uint64_t pol)
{
    uint32_t v;
    asm volatile("ld.global.nc.L2::cache_hint.u32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ float ld_keep_f32(const float* p, uint64_t pol)
{
    float v;
    asm volatile("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ void st_stream_v4(void* p, uint4 v, uint64_t pol)
{
    asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ uint4 ld_stream_v4(const void* p, uint64_t pol)
{
    uint4 v;
    asm volatile("ld.global.nc.L2::cache_hint.v4.b32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "l"(pol));
    return v;
}

template <bool NUMERIC>
struct MidSmem {
    uint32_t* table;       // symbolic: bitmap[MID_WORDS] + group flags[DUP_WORDS]; numeric: rank words [2 * MID_WORDS]
    uint32_t* l_qs;        // [256] lists of one block of A's nonzeros: mid rows of B from slot 0 up,
    uint32_t* l_len;       // [256] long rows from slot 255 down
    float* l_a;            // [256]
    uint32_t* vals;        // [val_cap + 4] accumulators (fp32 bit patterns)
    uint16_t* cols;        // [val_cap + 4]
};

// U scalar products of one thread: columns c[] (NO_COL = none), B's values v[], A's value a.
template <bool NUMERIC, int U>
__device__ __forceinline__ void mid_products(const MidSmem<NUMERIC>& sm, const uint32_t (&c)[U],
                                             const float (&v)[U], float a)
{
    if constexpr (!NUMERIC) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (c[u] == NO_COL) continue;
            const uint32_t bit = 1u << (c[u] & 31u);
            const uint32_t old = atomicOr(&sm.table[c[u] >> 5], bit);
            if (old & bit)                                         // second product of this column
                atomicOr(&sm.table[MID_WORDS + (c[u] >> 9)], 1u << ((c[u] >> 4) & 31u));
        }
    } else {
        uint32_t rw[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            rw[u] = c[u] != NO_COL ? sm.table[rank_word(c[u] >> 4)] : 0u;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (c[u] == NO_COL) continue;
            const uint32_t below = (1u << (c[u] & 15u)) - 1u;
            const uint32_t slot = ((rw[u] >> 16) & 0x1fffu) + __popc(rw[u] & below);
            const uint32_t p = __float_as_uint(__fmul_rn(a, v[u]));
            sm.cols[slot] = static_cast<uint16_t>(c[u]);
            if (!(rw[u] & DUP_FLAG)) {
                sm.vals[slot] = p;                                 // the only product of its column
            } else {
                uint32_t* acc = sm.vals + slot;
                uint32_t old = atomicExch(acc, p);
                while (old != 0u) {
                    // displaced a partial sum: take what is there now, add, put back
                    const uint32_t cur = atomicExch(acc, 0u);
                    const float sum = __fadd_rn(__uint_as_float(old), __uint_as_float(cur));
                    old = atomicExch(acc, __float_as_uint(sum));
                }
            }
        }
    }
}

// One row of B, [qs, qs + len), walked by `width` threads of which this is number
// `me`: MID_CHUNKS chunks of `width` entries in flight, then one chunk at a time.
template <bool NUMERIC>
__device__ __forceinline__ void mid_walk_row(const MidSmem<NUMERIC>& sm, const Csr& B, uint32_t qs,
                                             uint32_t len, float a, uint32_t me, uint32_t width, uint64_t keep)
{
    const uint32_t* pc = B.col + qs + me;
    const float* pv = B.val + qs + me;
    uint32_t c[MID_CHUNKS];
    float v[MID_CHUNKS];
#pragma unroll
    for (int u = 0; u < MID_CHUNKS; ++u) {
        const bool on = me + u * width < len;
        c[u] = NO_COL;
        v[u] = 0.0f;
        if (on) {
            c[u] = ld_keep_u32(pc + u * width, keep);
            if (NUMERIC) v[u] = ld_keep_f32(pv + u * width, keep);
        }
    }
    mid_products<NUMERIC, MID_CHUNKS>(sm, c, v, a);
    for (uint32_t q = MID_CHUNKS * width + me; q < len; q += width) {
        const uint32_t c1[1] = {ld_keep_u32(B.col + qs + q, keep)};
        const float v1[1] = {NUMERIC ? ld_keep_f32(B.val + qs + q, keep) : 0.0f};
        mid_products<NUMERIC, 1>(sm, c1, v1, a);
    }
}

template <bool NUMERIC>
__global__ void __launch_bounds__(MID_THREADS, NUMERIC ? 4 : 6)
mid_rows_kernel(Csr A, Csr B, Work w, const uint4* __restrict__ rows,
                const uint32_t* __restrict__ n_rows_ptr, uint32_t* __restrict__ next_row,
                uint32_t pitch, uint32_t val_cap, int vec_ok, uint32_t* __restrict__ pattern,
                uint32_t* __restrict__ dupmap, const uint32_t* __restrict__ rowC,
                uint32_t* __restrict__ colC, float* __restrict__ valC)
{
    extern __shared__ uint4 sm4[];
    MidSmem<NUMERIC> sm;
    sm.table = reinterpret_cast<uint32_t*>(sm4);
    sm.l_qs = sm.table + (NUMERIC ? 2 * MID_WORDS : MID_WORDS + DUP_WORDS);
    sm.l_len = sm.l_qs + 256;
    sm.l_a = reinterpret_cast<float*>(sm.l_len + 256);
    sm.vals = reinterpret_cast<uint32_t*>(sm.l_a + 256);
    sm.cols = reinterpret_cast<uint16_t*>(sm.vals + (NUMERIC ? val_cap + 4 : 0));
    __shared__ uint32_t s_warp[MID_THREADS / 32];
    __shared__ uint32_t s_next, s_n_mid, s_n_long;
    __shared__ uint4 s_desc[MID_BATCH];
    __shared__ uint32_t s_out0[MID_BATCH];

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t sub = tid & 15u, half = tid >> 4;              // lane group of 16 and its index
    const uint32_t n_rows = *n_rows_ptr;
    const bool own_words = tid * 8u < pitch;                      // this thread's 8 bitmap words exist
    const L2Hints l2 = make_l2_hints();

    // what a row needs from global memory before it can start: its kept bitmaps (numeric)
    // and the first 256 of its per-nonzero records
    auto load_inputs = [&](const uint4& d, uint4& p0, uint4& p1, uint32_t& dup, MidEntry& e) {
        if (NUMERIC) {
            p0 = p1 = make_uint4(0u, 0u, 0u, 0u);
            dup = 0;
            if (own_words) {
                const uint4* src = reinterpret_cast<const uint4*>(pattern + static_cast<size_t>(d.x) * pitch + tid * 8u);
                p0 = ld_stream_v4(src, l2.stream);
                p1 = ld_stream_v4(src + 1, l2.stream);
                dup = dupmap[static_cast<size_t>(d.x) * DUP_WORDS + (tid >> 1)];
            }
        }
        e.len = 0; e.qs = 0; e.a = 0.0f;
        if (d.y + tid < d.z) {
            e.qs = w.bq[d.y + tid];
            e.len = w.blen[d.y + tid];
            if (NUMERIC) e.a = A.val[d.y + tid];
        }
    };

    for (;;) {
        __syncthreads();                                          // previous batch done with s_desc
        if (tid == 0) s_next = atomicAdd(next_row, MID_BATCH);
        __syncthreads();
        const uint32_t first = s_next;
        if (first >= n_rows)
            break;
        const uint32_t end = min(first + MID_BATCH, n_rows);
        if (tid < end - first) {
            const uint4 d = rows[first + tid];
            s_desc[tid] = d;
            s_out0[tid] = NUMERIC ? rowC[d.x] : 0u;
        }
        __syncthreads();
        uint4 pat0, pat1;
        uint32_t dupw = 0;
        MidEntry ent;
        load_inputs(s_desc[0], pat0, pat1, dupw, ent);

        for (uint32_t idx = first; idx < end; ++idx) {
            const uint4 d = s_desc[idx - first];
            const uint32_t i = d.x, pa = d.y, pe = d.z;
            const uint32_t out0 = s_out0[idx - first];
            // the next row's inputs travel while this row is worked on
            uint4 npat0 = make_uint4(0u, 0u, 0u, 0u), npat1 = npat0;
            uint32_t ndupw = 0;
            MidEntry nent{0u, 0u, 0.0f};
            if (idx + 1 < end)
                load_inputs(s_desc[idx + 1 - first], npat0, npat1, ndupw, nent);

            const uint32_t shift = out0 & 3u;
            uint32_t total = 0;
            if (tid == 0) {
                s_n_mid = 0;
                s_n_long = 0;
            }
            if constexpr (NUMERIC) {
                // ---- rank table from the kept bitmaps
                const uint32_t bits[8] = {pat0.x, pat0.y, pat0.z, pat0.w, pat1.x, pat1.y, pat1.z, pat1.w};
                uint32_t c = 0;
#pragma unroll
                for (int k = 0; k < 8; ++k) c += __popc(bits[k]);
                uint32_t run = shift + block_exclusive_scan<MID_THREADS>(c, s_warp, total);
                if (own_words) {
                    // this thread's 16 groups are one half of its flag word
                    const uint32_t flags = (tid & 1u) ? dupw >> 16 : dupw & 0xffffu;
                    auto word = [&](uint32_t half_bits, int g) -> uint32_t {
                        const uint32_t o = half_bits | (run << 16) | (((flags >> g) & 1u) << 31);
                        run += __popc(half_bits);
                        return o;
                    };
#pragma unroll
                    for (int k = 0; k < 8; k += 2) {
                        uint4 o;
                        o.x = word(bits[k] & 0xffffu, 2 * k);
                        o.y = word(bits[k] >> 16, 2 * k + 1);
                        o.z = word(bits[k + 1] & 0xffffu, 2 * k + 2);
                        o.w = word(bits[k + 1] >> 16, 2 * k + 3);
                        const uint32_t slot = tid * 4u + (k >> 1);
                        sm4[slot ^ ((slot >> 3) & 3u)] = o;
                    }
                }
                const uint32_t lim4 = (total + shift + 3u) / 4u;
                uint4* vz = reinterpret_cast<uint4*>(sm.vals);
                for (uint32_t x = tid; x < lim4; x += MID_THREADS) vz[x] = make_uint4(0u, 0u, 0u, 0u);
            } else {
                for (uint32_t x = tid; x < (MID_WORDS + DUP_WORDS) / 4; x += MID_THREADS)
                    sm4[x] = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncthreads();

            // ---- the products, 256 nonzeros of A at a time
            for (uint32_t p0 = pa; p0 < pe; p0 += MID_THREADS) {
                MidEntry e = ent;
                if (p0 != pa) {
                    __syncthreads();                              // lists of the previous block consumed
                    if (tid == 0) {
                        s_n_mid = 0;
                        s_n_long = 0;
                    }
                    e.len = 0; e.qs = 0; e.a = 0.0f;
                    if (p0 + tid < pe) {
                        e.qs = w.bq[p0 + tid];
                        e.len = w.blen[p0 + tid];
                        if (NUMERIC) e.a = A.val[p0 + tid];
                    }
                    __syncthreads();
                }
                const bool is_mid = e.len > MID_SHORT && e.len < MID_LONG;
                const bool is_long = e.len >= MID_LONG;
                const uint32_t mm = __ballot_sync(0xffffffffu, is_mid);
                const uint32_t ml = __ballot_sync(0xffffffffu, is_long);
                const uint32_t below = (1u << lane) - 1u;
                if (mm) {
                    uint32_t base = 0;
                    if (lane == 0) base = atomicAdd(&s_n_mid, __popc(mm));
                    base = __shfl_sync(0xffffffffu, base, 0);
                    if (is_mid) {
                        const uint32_t at = base + __popc(mm & below);
                        sm.l_qs[at] = e.qs; sm.l_len[at] = e.len; sm.l_a[at] = e.a;
                    }
                }
                if (ml) {
                    uint32_t base = 0;
                    if (lane == 0) base = atomicAdd(&s_n_long, __popc(ml));
                    base = __shfl_sync(0xffffffffu, base, 0);
                    if (is_long) {
                        const uint32_t at = 255u - (base + __popc(ml & below));
                        sm.l_qs[at] = e.qs; sm.l_len[at] = e.len; sm.l_a[at] = e.a;
                    }
                }
                // short rows of B: this thread alone, straight from its registers
                if (e.len != 0 && e.len <= MID_SHORT) {
                    uint32_t c[MID_SHORT];
                    float v[MID_SHORT];
#pragma unroll
                    for (uint32_t u = 0; u < MID_SHORT; ++u) {
                        const bool on = u < e.len;
                        c[u] = on ? ld_keep_u32(B.col + e.qs + u, l2.keep) : NO_COL;
                        v[u] = (NUMERIC && on) ? ld_keep_f32(B.val + e.qs + u, l2.keep) : 0.0f;
                    }
                    mid_products<NUMERIC, MID_SHORT>(sm, c, v, e.a);
                }
                __syncthreads();
                // rows of B of 5 .. 255 entries: 16 lanes each.  A few entries left over after
                // the last full round of the 16 lane groups are walked by the whole CTA
                // instead (one step each) rather than by a few groups while the others wait.
                const uint32_t n_mid = s_n_mid;
                constexpr uint32_t GROUPS = MID_THREADS / 16;
                const uint32_t left = n_mid % GROUPS;
                const uint32_t n_grouped = (n_mid > GROUPS && left <= GROUPS / 4) ? n_mid - left : n_mid;
                for (uint32_t it = half; it < n_grouped; it += GROUPS)
                    mid_walk_row<NUMERIC>(sm, B, sm.l_qs[it], sm.l_len[it], sm.l_a[it], sub, 16u, l2.keep);
                for (uint32_t it = n_grouped; it < n_mid; ++it)
                    mid_walk_row<NUMERIC>(sm, B, sm.l_qs[it], sm.l_len[it], sm.l_a[it], tid, MID_THREADS, l2.keep);
                // rows of B of 256 entries and more: the whole CTA
                const uint32_t n_long = s_n_long;
                for (uint32_t l = 0; l < n_long; ++l)
                    mid_walk_row<NUMERIC>(sm, B, sm.l_qs[255u - l], sm.l_len[255u - l], sm.l_a[255u - l], tid,
                                          MID_THREADS, l2.keep);
            }
            __syncthreads();

            if constexpr (!NUMERIC) {
                // ---- count, and keep the bitmaps for the numeric pass
                uint32_t c = 0;
                if (own_words) {
                    const uint4 b0 = sm4[tid * 2u], b1 = sm4[tid * 2u + 1u];
                    c = __popc(b0.x) + __popc(b0.y) + __popc(b0.z) + __popc(b0.w) +
                        __popc(b1.x) + __popc(b1.y) + __popc(b1.z) + __popc(b1.w);
                    if (pattern) {
                        uint4* dst = reinterpret_cast<uint4*>(pattern + static_cast<size_t>(i) * pitch + tid * 8u);
                        st_stream_v4(dst, b0, l2.stream);
                        st_stream_v4(dst + 1, b1, l2.stream);
                    }
                }
                if (pattern && tid < DUP_WORDS)
                    dupmap[static_cast<size_t>(i) * DUP_WORDS + tid] = sm.table[MID_WORDS + tid];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
                if (lane == 0) s_warp[warp] = c;
                __syncthreads();
                if (tid == 0) {
                    uint32_t t = 0;
#pragma unroll
                    for (int x = 0; x < MID_THREADS / 32; ++x) t += s_warp[x];
                    w.cnt[i] = t;
                }
            } else {
                // ---- the window goes out with 16-byte stores
                const uint32_t lim = total + shift;
                uint32_t* gcol = colC + (out0 - shift);           // slot s <-> gcol[s]; 16-byte aligned
                uint32_t* gval = reinterpret_cast<uint32_t*>(valC) + (out0 - shift);
                for (uint32_t q = tid; q < (lim + 3u) / 4u; q += MID_THREADS) {
                    const uint32_t s0 = q * 4u;
                    if (vec_ok && s0 >= shift && s0 + 4u <= lim) {
                        const uint2 raw = *reinterpret_cast<const uint2*>(sm.cols + s0);
                        st_stream_v4(gcol + s0, make_uint4(raw.x & 0xffffu, raw.x >> 16, raw.y & 0xffffu, raw.y >> 16),
                                     l2.stream);
                        st_stream_v4(gval + s0, *reinterpret_cast<const uint4*>(sm.vals + s0), l2.stream);
                    } else {
                        for (uint32_t s = max(s0, shift); s < min(s0 + 4u, lim); ++s) {
                            gcol[s] = sm.cols[s];
                            gval[s] = sm.vals[s];
                        }
                    }
                }
            }
            __syncthreads();                                      // shared memory free for the next row
            pat0 = npat0; pat1 = npat1; dupw = ndupw; ent = nent;
        }
    }
}

// --------------------------------------------------------------- row scan
// rowC[0] = 0, rowC[i+1] = sum cnt[0..i]; one CTA of 32 warps.  A warp owns 1024
// consecutive counts per chunk of 32768 and reads / writes them 32 at a time, lane =
// consecutive element, so every global access is one coalesced 128-byte line (a
// thread that owns consecutive elements stores with a 128-byte stride between lanes:
// 20 us for one SM to push 65536 such stores out).
__global__ void __launch_bounds__(1024)
row_scan_kernel(const uint32_t* __restrict__ cnt, uint32_t M, uint32_t* __restrict__ rowC,
                unsigned long long* __restrict__ total_out)
{
    constexpr uint32_t PER = 32;                                  // steps of 32 elements per warp and chunk
    __shared__ unsigned long long s_warp[32];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) rowC[0] = 0;
    unsigned long long carry = 0;
    for (uint32_t base = 0; base < M; base += 1024 * PER) {
        const uint32_t w0 = base + warp * (32 * PER) + lane;
        uint32_t v[PER];
#pragma unroll
        for (uint32_t k = 0; k < PER; ++k) v[k] = w0 + 32 * k < M ? cnt[w0 + 32 * k] : 0u;
        unsigned long long mine = 0;
#pragma unroll
        for (uint32_t k = 0; k < PER; ++k) mine += v[k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
        __syncthreads();                                          // s_warp of the previous chunk read
        if (lane == 0) s_warp[warp] = mine;
        __syncthreads();
        unsigned long long run = carry, chunk_total = 0;
#pragma unroll
        for (uint32_t x = 0; x < 32; ++x) {
            const unsigned long long t = s_warp[x];
            if (x < warp) run += t;
            chunk_total += t;
        }
#pragma unroll
        for (uint32_t k = 0; k < PER; ++k) {
            uint32_t incl = v[k];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= static_cast<uint32_t>(o)) incl += t;
            }
            if (w0 + 32 * k < M) rowC[w0 + 32 * k + 1] = static_cast<uint32_t>(run + incl);
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        carry += chunk_total;
    }
    if (threadIdx.x == 0) *total_out = carry;
}

// ------------------------------------------------------------------- host
struct Plan {
    Csr A, B;
    Work w;
    uint32_t pitch;             // bitmap words per row, a multiple of 8 (rows stay 32-byte aligned)
    unsigned long long* d_total;
    uint32_t* pattern;          // [M][pitch] row bitmaps kept between the passes, or null
    uint32_t* dupmap;           // [M][DUP_WORDS] groups of 16 columns hit more than once (N <= 65536), or null
};

int make_plan(sb200_ctx* ctx, const sb200_csr* A, const sb200_csr* B, Plan* pl)
{
    if (!ctx || !A || !B)
        return SB200_ERR_INVALID_ARG;
    // the workspace below is allocated, and every later launch made, on the context's
    // device whatever device the calling thread had current
    if (cudaSetDevice(ctx->device) != cudaSuccess)
        return SB200_ERR_CUDA;
    if (A->N != B->M)
        return SB200_ERR_INVALID_ARG;
    if (!A->ROW || !B->ROW || (A->NNZ && (!A->COL || !A->V)) || (B->NNZ && (!B->COL || !B->V)))
        return SB200_ERR_INVALID_ARG;
    if (B->N > MAX_COLS)
        return SB200_ERR_TOO_LARGE;
    pl->A = Csr{A->ROW, A->COL, A->V, A->M, A->N};
    pl->B = Csr{B->ROW, B->COL, B->V, B->M, B->N};
    const size_t M = A->M, nnzA = A->NNZ;
    // cnt[M] | prod[M] | bq[nnzA] | blen[nnzA] | list_tiny[M] | counters[8] | total (8 B) | pad |
    // rows_mid[M] (16 B each) | rows_heavy[2M]
    const size_t head_words = (3 * M + 2 * nnzA + 8 + 2 + 3) & ~static_cast<size_t>(3);
    const size_t bytes = head_words * 4 + 3 * M * sizeof(uint4) + 64;
    // what a symbolic pass left in the workspace stays usable if the buffer is not replaced
    const int work_kept = ctx->sp_work_valid;
    const float* before = ctx->d_workspace;
    const int rc = ensure_workspace(ctx, bytes);
    if (rc)
        return rc;
    ctx->sp_work_valid = work_kept && ctx->d_workspace == before;
    uint32_t* base = reinterpret_cast<uint32_t*>(ctx->d_workspace);
    pl->w.cnt = base;
    pl->w.prod = base + M;
    pl->w.bq = base + 2 * M;
    pl->w.blen = base + 2 * M + nnzA;
    pl->w.list_tiny = base + 2 * M + 2 * nnzA;
    pl->w.counters = base + 3 * M + 2 * nnzA;
    uintptr_t tot = reinterpret_cast<uintptr_t>(pl->w.counters + 8);
    tot = (tot + 7) & ~static_cast<uintptr_t>(7);
    pl->d_total = reinterpret_cast<unsigned long long*>(tot);
    uintptr_t desc = (reinterpret_cast<uintptr_t>(base + head_words) + 15) & ~static_cast<uintptr_t>(15);
    pl->w.rows_mid = reinterpret_cast<uint4*>(desc);
    pl->w.rows_heavy = pl->w.rows_mid + M;
    pl->pitch = ((B->N + 31) / 32 + 7) & ~7u;
    if (pl->pitch == 0)
        pl->pitch = 8;
    pl->pattern = nullptr;
    pl->dupmap = nullptr;
    return SB200_OK;
}

constexpr int HEAVY_THREADS = 1024;
constexpr uint32_t HEAVY_VAL_CAP = 1u << 20;  // "as much as fits": one CTA per SM

// Output entries per window of a numeric row kernel with THREADS threads:
// columns + values take what the bitmap leaves of the 227 KB per CTA.  0 when
// not even a small window fits.
template <int THREADS, typename ColT>
uint32_t window_cap(uint32_t pitch, uint32_t want)
{
    const size_t tiles = (pitch + TILE_WORDS - 1) / TILE_WORDS;
    const size_t per_entry = 4 + sizeof(ColT);                  // accumulator + staged column
    const size_t room = 226 * 1024;
    const size_t fixed = tiles * TILE_WORDS * 8 + WalkLists<THREADS>::BYTES + 4 * per_entry;
    if (fixed + 1024 * per_entry > room)
        return 0;
    size_t cap = want;
    if (fixed + cap * per_entry > room)
        cap = (room - fixed) / per_entry;
    return static_cast<uint32_t>(cap) & ~3u;                    // windows start on 16-byte boundaries
}

uint32_t heavy_window_cap(const Plan& pl)
{
    return pl.B.N <= 65536 ? window_cap<HEAVY_THREADS, uint16_t>(pl.pitch, HEAVY_VAL_CAP)
                           : window_cap<HEAVY_THREADS, uint32_t>(pl.pitch, HEAVY_VAL_CAP);
}

// Whether the mid bin of this pass runs on the kernels specialised for N <= 65536
// columns (the numeric one needs the bitmaps and group flags the symbolic one kept).
bool fast_mid_rows(const sb200_ctx* ctx, const Plan& pl, bool numeric, bool from_pattern)
{
    if (pl.B.N > 65536 || !ctx->sp_fast_mid)
        return false;
    return !numeric || (from_pattern && pl.pattern && pl.dupmap);
}

// `reuse`: the per-nonzero and per-row arrays of an earlier call on the same
// operands are still in the workspace; only the bins are rebuilt (rowC given).
int bin_rows(sb200_ctx* ctx, const Plan& pl, const uint32_t* rowC, bool reuse, cudaStream_t stream)
{
    if (cudaMemsetAsync(pl.w.counters, 0, 32, stream) != cudaSuccess)
        return SB200_ERR_CUDA;
    if (pl.A.M == 0)
        return SB200_OK;
    const unsigned blocks = static_cast<unsigned>(ctx->sm_count) * 8;
    const uint32_t heavy_cap = heavy_window_cap(pl);
    // widest output row the mid bin of the numeric pass takes
    const uint32_t cap = fast_mid_rows(ctx, pl, true, pl.pattern != nullptr) ? FAST_MID_CAP : mid_cap(pl.B.N);
    if (reuse && rowC)
        rebin_kernel<<<(pl.A.M + 255) / 256, 256, 0, stream>>>(pl.A, pl.w, rowC, cap, heavy_cap);
    else
        row_products_kernel<<<blocks, 256, 0, stream>>>(pl.A, pl.B.row, pl.w, rowC, cap, heavy_cap);
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

// Row bitmaps are kept when they fit the limit (M * pitch * 4 bytes).
constexpr size_t PATTERN_LIMIT = static_cast<size_t>(2) << 30;

int prepare_pattern(sb200_ctx* ctx, Plan* pl, const sb200_csr* A, const sb200_csr* B)
{
    ctx->sp_valid = 0;
    ctx->sp_work_valid = 0;
    const size_t bitmaps = static_cast<size_t>(A->M) * pl->pitch * 4;
    // N <= 65536: the group flags of the specialised mid-row kernels follow the bitmaps
    const size_t need = bitmaps + (B->N <= 65536 ? static_cast<size_t>(A->M) * DUP_WORDS * 4 : 0);
    if (bitmaps == 0 || need > PATTERN_LIMIT)
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
    pl->dupmap = B->N <= 65536 ? pl->pattern + static_cast<size_t>(A->M) * pl->pitch : nullptr;
    ctx->sp_key = SpPatternKey{A->ROW, A->COL, B->ROW, B->COL, A->M, A->N, B->N, A->NNZ, B->NNZ};
    return SB200_OK;
}

// rows2 / n_rows2 / cap2: an optional second list of work items (the heavy
// bin's per-window items).
template <int THREADS, int MIN_BLOCKS, bool NUMERIC, bool FROM_PATTERN, typename ColT>
int launch_rows(sb200_ctx* ctx, const Plan& pl, const uint4* rows, const uint32_t* n_rows,
                const uint4* rows2, const uint32_t* n_rows2, uint32_t cap2,
                uint32_t* next_row, uint32_t val_cap, const uint32_t* rowC, uint32_t* colC, float* valC,
                cudaStream_t stream)
{
    const uint32_t tiles = (pl.pitch + TILE_WORDS - 1) / TILE_WORDS;
    const size_t padded = static_cast<size_t>(tiles) * TILE_WORDS;
    const size_t lists = WalkLists<THREADS>::BYTES;
    constexpr size_t per_entry = 4 + sizeof(ColT);              // accumulator + staged column
    if (NUMERIC) {
        val_cap = window_cap<THREADS, ColT>(pl.pitch, val_cap);
        if (val_cap == 0)
            return SB200_ERR_TOO_LARGE;
    }
    const size_t smem = NUMERIC ? padded * 8 + lists + (static_cast<size_t>(val_cap) + 4) * per_entry
                                : static_cast<size_t>(pl.pitch) * 4 + lists;
    auto kern = cta_rows_kernel<THREADS, MIN_BLOCKS, NUMERIC, FROM_PATTERN, ColT>;
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
        if (getenv("SB200_VERBOSE"))
            fprintf(stderr, "sb200: cta_rows<%d,%d,%d> smem %zu B, %d CTAs/SM, val_cap %u\n", THREADS,
                    int(NUMERIC), int(FROM_PATTERN), smem, n, val_cap);
    }
    const int per_sm = cached_per_sm;
    const unsigned grid = static_cast<unsigned>(ctx->sm_count) * per_sm;
    if (cudaMemsetAsync(next_row, 0, 4, stream) != cudaSuccess)
        return SB200_ERR_CUDA;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(colC) | reinterpret_cast<uintptr_t>(valC)) & 15) == 0;
    kern<<<grid, THREADS, smem, stream>>>(pl.A, pl.B, pl.w, rows, n_rows, rows2, n_rows2, cap2, next_row,
                                          pl.pitch, tiles, val_cap, vec_ok, pl.pattern, rowC, colC, valC);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

// The mid bin on the kernels specialised for N <= 65536 columns.
template <bool NUMERIC>
int launch_mid_rows(sb200_ctx* ctx, const Plan& pl, const uint32_t* rowC, uint32_t* colC, float* valC,
                    cudaStream_t stream)
{
    const uint32_t val_cap = FAST_MID_CAP;
    const size_t smem = NUMERIC ? 2 * MID_WORDS * 4 + 3 * 256 * 4 + (static_cast<size_t>(val_cap) + 4) * 6
                                : (MID_WORDS + DUP_WORDS) * 4 + 3 * 256 * 4;
    auto kern = mid_rows_kernel<NUMERIC>;
    static thread_local int cached_dev = -1, cached_per_sm = 1;
    if (cached_dev != ctx->device) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
            cudaSuccess) {
            cudaGetLastError();
            return SB200_ERR_CUDA;
        }
        int n = 1;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, MID_THREADS, smem) != cudaSuccess || n < 1)
            n = 1;
        cached_dev = ctx->device;
        cached_per_sm = n;
        if (getenv("SB200_VERBOSE"))
            fprintf(stderr, "sb200: mid_rows<%d> smem %zu B, %d CTAs/SM\n", int(NUMERIC), smem, n);
    }
    uint32_t* next_row = pl.w.counters + 3;
    if (cudaMemsetAsync(next_row, 0, 4, stream) != cudaSuccess)
        return SB200_ERR_CUDA;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(colC) | reinterpret_cast<uintptr_t>(valC)) & 15) == 0;
    kern<<<static_cast<unsigned>(ctx->sm_count) * cached_per_sm, MID_THREADS, smem, stream>>>(
        pl.A, pl.B, pl.w, pl.w.rows_mid, pl.w.counters + 1, next_row, pl.pitch, val_cap, vec_ok, pl.pattern,
        pl.dupmap, rowC, colC, valC);
    ctx->launches += 1;
    return cudaGetLastError() == cudaSuccess ? SB200_OK : SB200_ERR_CUDA;
}

template <bool NUMERIC, bool FROM_PATTERN>
int run_rows(sb200_ctx* ctx, const Plan& pl, const uint32_t* rowC, uint32_t* colC, float* valC,
             cudaStream_t stream)
{
    if (pl.A.M == 0)
        return SB200_OK;
    // heavy rows first: 1024 threads and a large window buffer, one CTA per SM
    const uint4* windows = NUMERIC ? pl.w.rows_heavy + pl.A.M : nullptr;
    int rc;
    if (pl.B.N <= 65536)
        rc = launch_rows<HEAVY_THREADS, 1, NUMERIC, FROM_PATTERN, uint16_t>(
            ctx, pl, pl.w.rows_heavy, pl.w.counters + 2, windows, pl.w.counters + 4, pl.A.M,
            pl.w.counters + 3, HEAVY_VAL_CAP, rowC, colC, valC, stream);
    else
        rc = launch_rows<HEAVY_THREADS, 1, NUMERIC, FROM_PATTERN, uint32_t>(
            ctx, pl, pl.w.rows_heavy, pl.w.counters + 2, windows, pl.w.counters + 4, pl.A.M,
            pl.w.counters + 3, HEAVY_VAL_CAP, rowC, colC, valC, stream);
    if (rc)
        return rc;
    // N <= 65536: the specialised mid-row kernels (the numeric one reads the kept bitmaps)
    if (fast_mid_rows(ctx, pl, NUMERIC, FROM_PATTERN))
        rc = launch_mid_rows<NUMERIC>(ctx, pl, rowC, colC, valC, stream);
    else if constexpr (!NUMERIC)
        rc = launch_rows<ROW_THREADS, 6, false, false, uint32_t>(
            ctx, pl, pl.w.rows_mid, pl.w.counters + 1, nullptr, nullptr, 0, pl.w.counters + 3, 0, rowC, colC,
            valC, stream);
    else if (pl.B.N <= 65536)
        rc = launch_rows<ROW_THREADS, 4, NUMERIC, FROM_PATTERN, uint16_t>(
            ctx, pl, pl.w.rows_mid, pl.w.counters + 1, nullptr, nullptr, 0, pl.w.counters + 3,
            mid_cap(pl.B.N), rowC, colC, valC, stream);
    else
        rc = launch_rows<ROW_THREADS, 3, NUMERIC, FROM_PATTERN, uint32_t>(
            ctx, pl, pl.w.rows_mid, pl.w.counters + 1, nullptr, nullptr, 0, pl.w.counters + 3,
            mid_cap(pl.B.N), rowC, colC, valC, stream);
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
    if ((rc = prepare_pattern(ctx, &pl, A, B)) || (rc = bin_rows(ctx, pl, nullptr, false, stream)))
        return rc;
    if ((rc = run_rows<false, false>(ctx, pl, nullptr, nullptr, nullptr, stream)))
        return rc;
    ctx->sp_valid = pl.pattern != nullptr;
    ctx->sp_work_valid = ctx->sp_valid;
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
    const bool same = same_operands(ctx, A, B);
    if (same) {
        pl.pattern = ctx->d_sp_pattern;
        pl.dupmap = B->N <= 65536 ? pl.pattern + static_cast<size_t>(A->M) * pl.pitch : nullptr;
    }
    if ((rc = bin_rows(ctx, pl, rowC, same && ctx->sp_work_valid, stream)))
        return rc;
    if (same) {
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
    if ((rc = prepare_pattern(ctx, &pl, A, B)) || (rc = bin_rows(ctx, pl, nullptr, false, stream)) ||
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
    if ((rc = bin_rows(ctx, pl, C->ROW, true, stream))) {
        sb200_csr_free(C);
        return rc;
    }
    rc = pl.pattern ? run_rows<true, true>(ctx, pl, C->ROW, C->COL, C->V, stream)
                    : run_rows<true, false>(ctx, pl, C->ROW, C->COL, C->V, stream);
    ctx->sp_valid = 0;
    ctx->sp_work_valid = 0;
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
