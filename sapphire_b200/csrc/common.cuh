// Internal declarations shared by the translation units of libsapphire_b200.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <nvtx3/nvToolsExt.h>

#include "../../include/sapphire_b200.h"

namespace sb200 {

// NVTX range over one ABI call (header-only NVTX: free when no tool is attached).
struct TraceRange {
    explicit TraceRange(const char* name) { nvtxRangePushA(name); }
    ~TraceRange() { nvtxRangePop(); }
    TraceRange(const TraceRange&) = delete;
    TraceRange& operator=(const TraceRange&) = delete;
};

// Codes written to the device status word by a bounded wait that gave up.
enum DeviceFault : unsigned {
    FAULT_NONE = 0,
    FAULT_PRODUCER_WAIT = 0x101,   // TMA producer waiting for a free stage
    FAULT_MMA_WAIT_FULL = 0x102,   // MMA issuer waiting for a filled stage
    FAULT_MMA_WAIT_TMEM = 0x103,   // MMA issuer waiting for a drained accumulator
    FAULT_EPI_WAIT = 0x104,        // epilogue waiting for a finished accumulator
    FAULT_SPLIT_WAIT = 0x105,      // hi/lo split warps waiting for a filled stage
    FAULT_PEER_WAIT = 0x201        // gradient exchange waiting for another rank's announcement
};

struct GemmArgs {
    int mode, transA, transB;
    int64_t M, N, K, batch;
    const float* A; int64_t lda, strideA;
    const float* B; int64_t ldb, strideB;
    const float* C; int64_t ldc, strideC;
    float* D; int64_t ldd, strideD;
    const float* bias;
    float* colsum_out;         // fused column sums of op(B) (tensor-core path, TF32 mode), or null
    float colsum_scale;
    int relu;                  // D = D > 0 ? D : 0 after everything else
    const float* mask;         // [M, N] per batch or null: D = mask > 0 ? D : 0 (ReLU backward gate)
    int64_t ldmask, strideMask;
    // reduce-scatter epilogue: rows [o * rows_per_owner, (o+1) * rows_per_owner) of the product
    // are ADDED into owner[o] (an [rows_per_owner, N] buffer, possibly another GPU's memory)
    // instead of being stored to D; rows_per_owner == 0 switches it off
    float* owner[8];
    int64_t rows_per_owner;
    int owner_store = 0;       // 1: blocks are STORED to owner[o] (a slot per source rank), not added
    // in-place SGD: the accumulator is multiplied by acc_scale (= -lr; 1 = off) before C is
    // added, and the column sums update colsum_out: out -= colsum_lr * (colsum_scale * sum)
    float acc_scale = 1.0f;
    float colsum_lr = 0.0f;
};
constexpr int MAX_OWNERS = 8;

}  // namespace sb200

namespace sb200 {
// Operand arrays the kept sparse row patterns were computed from.
struct SpPatternKey {
    const void *rowA, *colA, *rowB, *colB;
    uint32_t M, K, N, nnzA, nnzB;
};

// One encoded TMA descriptor of the context's cache.  The key is everything
// cuTensorMapEncodeTiled was given, so a hit is valid whatever happened to the
// memory behind `base` in between (a descriptor holds an address and a shape,
// no state).  All key fields are 64-bit: the key is compared with memcmp.
struct TensorMapKey {
    uint64_t base;
    int64_t contig, rows, ld, batches, batch_stride;
    int64_t box_rows;      // rows (3-D map) or chunks (merged 4-D map) per box
    int64_t kind;          // 0: K-major 3-D, 1: MN-major 3-D, 2: MN-major merged 4-D
};
struct alignas(64) TensorMapSlot {
    CUtensorMap map;
    TensorMapKey key;
    uint64_t stamp;        // last use; 0 = empty
};
constexpr int TENSOR_MAP_SLOTS = 64;
// The status allocation: word 0 is the device status word; from SLICE_TICKET_OFFSET on,
// one ticket counter per output tile of a k-sliced GEMM (zero between launches).
constexpr int SLICE_TICKET_OFFSET = 16;
constexpr int SLICE_TICKETS = 240;
constexpr int STATUS_WORDS = SLICE_TICKET_OFFSET + SLICE_TICKETS;
}  // namespace sb200

struct sb200_ctx {
    int device;
    int sm_count;
    int last_path;
    int64_t launches;
    unsigned* d_status;        // device status word
    float* d_workspace;        // scratch for partial column sums / sparse row work
    size_t workspace_bytes;
    int split_explicit_hi;     // 3xTF32: rewrite the high part in shared memory too
    int split_a_tmem;          // 3xTF32: both parts of an [M, K] A tile go to TMEM
    int merge_mn_boxes;        // fetch an MN-major tile with one 4-D TMA box when possible
    int use_cta_pairs;         // large TF32 problems run on the two-CTA (cta_group::2) kernel
    int split_tail_wave;       // a mostly empty last wave of pair tiles goes to the one-CTA kernel
    int k_slices;              // small problems: slices of k on separate SMs, summed by the last to finish
    void* encode_tiled;        // cuTensorMapEncodeTiled, resolved at context creation
    sb200::TensorMapSlot* tmaps;   // [TENSOR_MAP_SLOTS] encoded descriptors, least recently used replaced
    uint64_t tmap_clock;
    int64_t tmap_hits, tmap_misses;
    uint64_t wait_limit_ns;    // bound of every mbarrier wait inside the GEMM kernels
    int test_stall_kb;         // test hook: TMA producers stop after this many k-blocks (< 0: off)
    uint32_t* d_sp_pattern;    // sparse GEMM: row bitmaps kept from the symbolic pass
    size_t sp_pattern_bytes;
    sb200::SpPatternKey sp_key;
    int sp_valid;
    int sp_work_valid;         // ... and its per-row / per-nonzero arrays are still in the workspace
    int sp_fast_mid;           // sparse GEMM: rows of the mid bin run on the kernels specialised for N <= 65536
};

namespace sb200 {

// gemm_tcgen05.cu
bool tcgen05_eligible(const GemmArgs& g);
int launch_gemm_tcgen05(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream);
// gemm_tcgen05_2cta.cu
bool pair_kernel_preferred(const sb200_ctx* ctx, const GemmArgs& g);
int launch_gemm_tcgen05_pair(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream);
// gemm_tcgen05_slices.cu
int k_slices(const sb200_ctx* ctx, const GemmArgs& g);
int launch_gemm_tcgen05_slices(sb200_ctx* ctx, const GemmArgs& g, int split, cudaStream_t stream);
// gemm_simt.cu
int launch_gemm_simt(sb200_ctx* ctx, const GemmArgs& g, cudaStream_t stream);
// lr != 0: out[n] -= lr * (scale * sum) instead of out[n] = scale * sum
int launch_colsum(sb200_ctx* ctx, const float* B, int transB, int64_t K, int64_t N, int64_t ldb,
                  float* out, float scale, cudaStream_t stream, float lr = 0.0f);
// workspace (abi.cu)
int ensure_workspace(sb200_ctx* ctx, size_t bytes);

}  // namespace sb200
