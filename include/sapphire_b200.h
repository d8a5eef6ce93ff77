/*
 * sapphire_b200.h -- C ABI of the B200 (sm_100a) back end for Sapphire's
 * matrix-multiplication path.
 *
 * Everything below the raw-pointer leaf functions of Sapphire's compute
 * interface is replaced by this library; the C++ shims under
 * sapphire_b200/compat/ keep Sapphire's own signatures and forward here.
 * Plain C types only; every function returns an int status (0 = success) and
 * no exception crosses this boundary.  All pointers named "device" are device
 * pointers of the context's GPU; the caller owns every input and output
 * buffer unless stated otherwise.  Work is enqueued on the given stream and
 * the call returns without synchronising, unless stated otherwise.
 *
 * Reference interface citations are paths inside the Sapphire project.
 */
#ifndef SAPPHIRE_B200_H
#define SAPPHIRE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
enum {
    SB200_OK = 0,
    SB200_ERR_INVALID_ARG = 1,   /* NULL pointer, negative size, ld < cols, ...     */
    SB200_ERR_CUDA = 2,          /* a CUDA runtime / driver call failed              */
    SB200_ERR_UNSUPPORTED = 3,   /* valid request this build cannot run              */
    SB200_ERR_DEVICE_TIMEOUT = 4,/* a bounded wait inside a kernel expired           */
    SB200_ERR_ALLOC = 5,         /* device or host allocation failed                 */
    SB200_ERR_TOO_LARGE = 6      /* size beyond a documented limit                   */
};

/* Arithmetic of the dense GEMM.
 *   TF32     operands rounded to TF32 by the tensor core, fp32 accumulate: what
 *            the reference's GPU path asks of cuBLAS
 *            (CUBLAS_COMPUTE_32F_FAST_TF32, Sources/Sapphire/compute/dense/cuda/Gemm.cu:31,49).
 *   TF32X3   each operand split into a TF32 high part and a TF32 low part,
 *            three tensor-core products per k-block; agrees with the
 *            reference's fp32 CPU loop (Sources/Sapphire/compute/dense/naive/NaiveGemm.cpp:20-37)
 *            to about 1e-6 relative.
 */
enum { SB200_MODE_TF32 = 0, SB200_MODE_TF32X3 = 1 };

/* Which kernel family ran; for tests and profiling. */
enum { SB200_PATH_AUTO = 0, SB200_PATH_TCGEN05 = 1, SB200_PATH_SIMT = 2 };

typedef struct sb200_ctx sb200_ctx;

/* Opaque stream handle: a cudaStream_t passed as void* (NULL = the legacy
 * default stream). */
typedef void* sb200_stream;

/*
 * One context per (device, host thread); it owns the per-device workspace,
 * the device status word and a cache of encoded TMA descriptors (64 entries,
 * least recently used replaced, keyed by base address, extents, leading
 * dimension, batch stride and box shape: a GEMM on operands the context has
 * seen before encodes nothing).  Replaces the per (device, thread) cuBLAS
 * handle map of the reference
 * (Sources/Sapphire/compute/dense/cuda/Gemm.cu:24-30,
 *  Sources/Sapphire/util/ResourceManager.cpp:209-214).
 *
 * A context is not thread-safe, and its one workspace is not ordered between
 * streams: calls that share a context must be stream-ordered with respect to
 * each other (one stream per context, or event dependencies between streams).
 * The workspace grows on demand (cudaFree + cudaMalloc, which synchronise the
 * device): its users are the separate column sums of the 3xTF32 and CUDA-core
 * paths, the k-sliced small GEMMs, the sparse product and the dense -> CSR
 * conversion.  Run each kind of call once before a stream capture begins; the
 * same call inside the capture then allocates nothing.
 */
int sb200_ctx_create(int device, sb200_ctx** out);
int sb200_ctx_destroy(sb200_ctx* ctx);

const char* sb200_status_string(int status);

/* Kernel family used by the last sb200_gemm_batched call on this context
 * (SB200_PATH_TCGEN05 or SB200_PATH_SIMT), and a running count of kernels
 * this context has launched. */
int sb200_last_path(const sb200_ctx* ctx);
int64_t sb200_launch_count(const sb200_ctx* ctx);

/* Running counters of a context: kernels launched, TMA descriptors served from
 * the cache, TMA descriptors encoded.  -1 for an unknown counter. */
enum { SB200_COUNTER_LAUNCHES = 0, SB200_COUNTER_TENSOR_MAP_HITS = 1,
       SB200_COUNTER_TENSOR_MAP_MISSES = 2 };
int64_t sb200_ctx_counter(const sb200_ctx* ctx, int which);

/* Tuning knobs of a context (the counterpart of cublasSetMathMode at
 * Sources/Sapphire/compute/dense/cuda/Gemm.cu:31).
 *   SB200_OPT_SPLIT_EXPLICIT_HI  (TF32X3 mode) 0, the default: the high part of
 *       an operand is the raw fp32 word, cut to TF32 by the tensor core; 1: the
 *       high part is rounded to nearest TF32 and rewritten in shared memory.
 *   SB200_OPT_MERGE_MN_BOXES  1, the default: an operand tile whose contiguous
 *       dimension is M or N (extent a multiple of 32) is fetched by one 4-D TMA
 *       box; 0: by one 32 x 32 box per 32-element chunk.
 *   SB200_OPT_CTA_PAIRS  1, the default: TF32 problems with at least one
 *       256 x 256 tile per pair of SMs run on the two-CTA kernel (clusters of two,
 *       tcgen05 cta_group::2); 0: always the one-CTA kernel.
 *   SB200_OPT_SPLIT_TAIL_WAVE  0, the default: one launch per request.  1: when the
 *       256 x 256 tiles of a problem would leave the last wave over the SM pairs
 *       mostly empty (one 4096^3 product: 3.46 waves of work in the time of 4), the
 *       bottom rows of the product run as a second launch of the one-CTA kernel.
 *       Off by default because it measured slower on a power-capped B200 (one
 *       4096^3: 212 us split, 199 us whole): the SMs of a partly empty wave clock
 *       higher, which already buys back most of the quantisation loss.
 *   SB200_OPT_WAIT_LIMIT_US  bound of every wait inside the GEMM kernels in
 *       microseconds (default 2,000,000; at least 100).  A wait that runs out ends
 *       the launch with SB200_ERR_DEVICE_TIMEOUT from sb200_check_device_status --
 *       the counterpart of the reference's CHECK_CUBLAS
 *       (Includes/Sapphire/compute/cudaUtil/CudaParams.cuh:51-58).
 *   SB200_OPT_K_SLICES  1, the default: a TF32 product with few 128 x 64 output
 *       tiles and at least 22 k-blocks of 32 runs as S CTAs per tile, each a slice of
 *       k; the CTA of a tile that finishes last adds the partial tiles in slice
 *       order (bit-reproducible) and runs the epilogue.  0: one CTA per tile.
 *       2 .. 16: that many slices whenever the request is eligible (tests, tuning).
 *   SB200_OPT_SPLIT_A_TMEM  (TF32X3 mode) 1, the default: when A is stored
 *       [M, K] the high and low parts of its tiles are written to tensor memory
 *       and the tensor core reads them from there; 0: both low parts go to
 *       shared memory, as they always do for a transposed A.  Same results.
 *   SB200_OPT_SPGEMM_FAST_MID  1, the default: sparse products with at most 65536
 *       columns run their mid-sized rows (33 .. 16383 scalar products) on the kernels
 *       specialised for that width; 0: on the general row kernel (any width).
 *   SB200_OPT_TEST_STALL_KBLOCKS  test hook, -1 = off, the default: the TMA
 *       producers of the next launches stop after this many k-blocks, so that
 *       every other role's wait runs out and the abort path executes. */
enum { SB200_OPT_SPLIT_EXPLICIT_HI = 1, SB200_OPT_MERGE_MN_BOXES = 2, SB200_OPT_CTA_PAIRS = 3,
       SB200_OPT_SPLIT_TAIL_WAVE = 4, SB200_OPT_WAIT_LIMIT_US = 5,
       SB200_OPT_TEST_STALL_KBLOCKS = 6, SB200_OPT_SPGEMM_FAST_MID = 7,
       SB200_OPT_K_SLICES = 8, SB200_OPT_SPLIT_A_TMEM = 9 };
int sb200_ctx_set_option(sb200_ctx* ctx, int option, int value);

/* Reads (and clears) the device status word after synchronising the stream.
 * Non-zero means a bounded wait in a kernel gave up; the results of that
 * launch are undefined but the context stays usable. */
int sb200_check_device_status(sb200_ctx* ctx, sb200_stream stream);

/*
 * Batched dense GEMM, row-major fp32:
 *
 *     D[b] = (C[b] + bias) + op(A[b]) . op(B[b])          b = 0 .. batch-1
 *
 * op(A) is M x K, op(B) is K x N.  transA = 0: A is stored [M, K] with leading
 * dimension lda >= K; transA = 1: A is stored [K, M], lda >= M.  Likewise
 * transB = 0: B stored [K, N], ldb >= N; transB = 1: B stored [N, K],
 * ldb >= K.  C and D are [M, N] with ldc, ldd >= N.  Batch strides are in
 * elements; a stride of 0 re-reads one matrix for every batch.
 *
 * C may be NULL (zero) and may alias D exactly (same pointer, ld and stride):
 * the reference's entry point is y <- y + a.b
 * (Sources/Sapphire/compute/BasicOps.cpp:183-248; alpha = beta = 1 in
 * Sources/Sapphire/compute/dense/cuda/Gemm.cu:33-34,44-50), so the aliased call
 * is the drop-in for Dense::Cuda::Gemm (Includes/Sapphire/compute/dense/cuda/Gemm.cuh:15-18)
 * and, with strideA or strideB = 0, for GemmMatrixWiseBroadcast (Gemm.cuh:20-25).
 *
 * transA / transB replace the explicit Transpose + Gemm pairs of the Linear
 * backward pass (Sources/Sapphire/operations/Backward/LinearBackward.cpp:49-50, 70-72).
 *
 * bias (device, [N], may be NULL) is added to every row: it replaces the
 * rank-1 Gemm y += ones[B,1].bias[1,N] of
 * Sources/Sapphire/operations/Forward/Linear.cpp:134-135.
 *
 * colsum_out (device, [N], may be NULL): additionally writes
 * colsum_out[n] = colsum_scale * sum_k op(B)[k, n] of batch 0; it replaces the
 * bias-gradient Gemm dB = ones[1,B].dy followed by Scale(1/B)
 * (LinearBackward.cpp:93-97) when this call is dW = x^T.dy.  Requires batch == 1.
 *
 * A single TF32 product with K >= 2048 and so few output tiles that most SMs
 * would idle has its k range cut into slices that run concurrently and add into
 * D; the adds arrive in no fixed order, so the last bits of such a result can
 * differ between runs (the 3xTF32 mode and every other shape are reproducible).
 *
 * path: SB200_PATH_AUTO picks the tcgen05 kernel when the operands satisfy
 * TMA's alignment rules (16-byte aligned base pointers, ld and batch strides
 * multiples of 4 elements) and the SIMT kernel otherwise; the other two
 * values force a family (SB200_ERR_UNSUPPORTED when it cannot run the request).
 */
int sb200_gemm_batched(sb200_ctx* ctx, int mode, int path, int transA, int transB,
                       int64_t M, int64_t N, int64_t K,
                       const float* A, int64_t lda, int64_t strideA,
                       const float* B, int64_t ldb, int64_t strideB,
                       const float* C, int64_t ldc, int64_t strideC,
                       float* D, int64_t ldd, int64_t strideD,
                       const float* bias, float* colsum_out, float colsum_scale,
                       int64_t batch, sb200_stream stream);

/*
 * The same GEMM with the elementwise steps either side of it in a Linear +
 * ReLU stack folded into its epilogue:
 *
 *     D[b] = gate( relu( (C[b] + bias) + op(A[b]) . op(B[b]) ) )
 *
 * relu != 0: the result goes through x > 0 ? x : 0, the forward ReLU that
 * follows a Linear layer (Sources/Sapphire/compute/dense/naive/NaiveBasic.cpp:159-165,
 * device kernel Sources/Sapphire/compute/dense/cuda/kernels/ActivationKernel.cu:11-22).
 * Only the activated tensor is written; its sign pattern equals that of the
 * pre-activation, so it serves as the gate of the backward pass.
 *
 * relu_gate (device, [M, N] per batch with leading dimension ld_gate and batch
 * stride stride_gate, may be NULL): D is kept where relu_gate > 0 and set to 0
 * elsewhere.  With this call as dx = dy . W^T it replaces the ReLUBackward
 * kernel that follows (dx += x > 0 ? dy : 0 into a zeroed buffer,
 * NaiveBasic.cpp:167-174, ActivationBackwardKernel.cu:11-24).  relu_gate must
 * not overlap D.
 *
 * sgd_lr (0 = off): the product updates a weight in place instead of being a
 * gradient that is stored first: D = C - sgd_lr * (op(A) . op(B)), and, where
 * colsum_out is given, colsum_out[n] = colsum_out[n] - sgd_lr * (colsum_scale *
 * sum_k op(B)[k, n]).  With A = x (transA), B = dy, C = D = the weight,
 * colsum_out = the bias and colsum_scale = 1 / batch this is the weight and bias
 * half of the reference's Linear backward unit with its SGD optimizer inside
 * (Sources/Sapphire/operations/Backward/LinearBackward.cpp:53-99: dW = x^T . dy
 * unscaled, dB = (1 / batch) ones . dy;
 * Sources/Sapphire/operations/optimizers/SGD.cpp:22-28: temp = lr * dz, z = z - temp)
 * in one launch, with the same two roundings per element (the product times lr,
 * then the subtraction), so the result equals storing the gradient and running
 * sb200_sgd_update on it bit for bit.  Requires C; not combined with bias, relu or
 * relu_gate.
 *
 * bias, colsum_out and colsum_scale as in sb200_gemm_batched, which is this
 * call with relu = 0, relu_gate = NULL and sgd_lr = 0.
 */
typedef struct sb200_gemm_epilogue {
    const float* bias;
    float* colsum_out;
    float colsum_scale;
    int relu;
    const float* relu_gate;
    int64_t ld_gate;
    int64_t stride_gate;
    float sgd_lr;
} sb200_gemm_epilogue;

int sb200_gemm_batched_ex(sb200_ctx* ctx, int mode, int path, int transA, int transB,
                          int64_t M, int64_t N, int64_t K,
                          const float* A, int64_t lda, int64_t strideA,
                          const float* B, int64_t ldb, int64_t strideB,
                          const float* C, int64_t ldc, int64_t strideC,
                          float* D, int64_t ldd, int64_t strideD,
                          const sb200_gemm_epilogue* epilogue,
                          int64_t batch, sb200_stream stream);

/*
 * GEMM fused with the reduce-scatter that follows it when a Linear layer's
 * weight gradient is computed from row shards (one rank per GPU, each holding
 * a slice of the batch): P = op(A) . op(B) is this rank's partial [M, N]
 * gradient; its rows are cut into n_owners equal blocks and block o is ADDED,
 * tile by tile from the kernel's epilogue, into owners[o], an
 * [M / n_owners, N] buffer (leading dimension ld_out) in the memory of the rank
 * that owns the block -- a pointer into this GPU's memory for the rank itself,
 * a peer mapping (sb200_peer_open) for the others.  The adds are fp32
 * reductions at system scope, so the transfer over NVLink overlaps the tensor
 * core work of the following tiles and no partial gradient is written to this
 * rank's HBM.  Once every rank's call has completed (a stream-ordered barrier
 * across the ranks), owners[rank] on each rank holds its block of the summed
 * gradient; the caller zeroes that buffer before the first rank starts.
 *
 * The reference is single-GPU and has no counterpart; the sum it replaces is the
 * allreduce of the dW = x^T . dy products of
 * Sources/Sapphire/operations/Backward/LinearBackward.cpp:70-72 over the ranks.
 * colsum_out / colsum_scale as in sb200_gemm_batched (this rank's partial bias
 * gradient, local).  Requires M divisible by n_owners (<= 8) with blocks that are
 * multiples of 128 rows, ld_out a multiple of 4, 16-byte aligned buffers and
 * operands the tensor-core kernel accepts (SB200_ERR_UNSUPPORTED otherwise).
 */
int sb200_gemm_reduce_scatter(sb200_ctx* ctx, int mode, int transA, int transB,
                              int64_t M, int64_t N, int64_t K,
                              const float* A, int64_t lda, const float* B, int64_t ldb,
                              float* const* owners, int n_owners, int64_t ld_out,
                              float* colsum_out, float colsum_scale, sb200_stream stream);

/*
 * The same product with its row blocks STORED, not added: block o goes to owners[o]
 * with plain 16-byte stores (full NVLink write rate; fp32 reductions over the links
 * run at a fraction of it).  Each rank passes, for owner o, the address of ITS OWN
 * slot in rank o's buffer (slot index = this rank), so nothing needs zeroing and
 * nothing collides; after a barrier the owner adds its n slots with sb200_sum_blocks
 * in slot order -- a fixed order, so the summed gradient is bit-reproducible, which
 * the adds of sb200_gemm_reduce_scatter (arrival order) are not.
 */
int sb200_gemm_scatter(sb200_ctx* ctx, int mode, int transA, int transB,
                       int64_t M, int64_t N, int64_t K,
                       const float* A, int64_t lda, const float* B, int64_t ldb,
                       float* const* owners, int n_owners, int64_t ld_out,
                       float* colsum_out, float colsum_scale, sb200_stream stream);

/* out[r, c] = blocks[0][r, c] + blocks[1][r, c] + ... + blocks[n_blocks - 1][r, c] (fp32
 * adds in that order) for an [rows, cols] region; block b starts block_stride floats
 * after block b - 1; out may be blocks[0].  cols, the leading dimensions and the
 * stride multiples of 4, 16-byte aligned pointers (SB200_ERR_UNSUPPORTED otherwise).
 * Like the two calls above it has no counterpart in the single-GPU reference. */
int sb200_sum_blocks(sb200_ctx* ctx, float* out, int64_t ld_out, const float* blocks, int n_blocks,
                     int64_t block_stride, int64_t rows, int64_t cols, int64_t ld_block,
                     sb200_stream stream);

/*
 * Device buffers that other processes on the node map into their address space
 * (CUDA IPC): sb200_peer_alloc allocates one and fills a 64-byte handle to send
 * to the other ranks (any byte transport), sb200_peer_open maps a received
 * handle (enabling peer access to the owning GPU on first use) and
 * sb200_peer_close / sb200_peer_free undo the two.  No counterpart in the
 * reference.
 */
int sb200_peer_alloc(sb200_ctx* ctx, size_t bytes, void** ptr, unsigned char* handle64);
int sb200_peer_open(sb200_ctx* ctx, const unsigned char* handle64, void** ptr);
int sb200_peer_close(sb200_ctx* ctx, void* ptr);
int sb200_peer_free(sb200_ctx* ctx, void* ptr);

/*
 * Gradient exchange of a data-parallel step over peer memory, fused with the SGD
 * update: the sum over ranks that the reference, being single-GPU, never needs
 * (its optimizer step is Sources/Sapphire/operations/optimizers/SGD.cpp:22-28; the
 * reduction rule -- weight gradients SUM, bias gradients MEAN -- follows from
 * Sources/Sapphire/operations/Backward/LinearBackward.cpp:72-73, 93-97).
 *
 * A group describes, for each of `world` ranks (one process per GPU, <= 8), three
 * buffers as mapped into THIS process (sb200_peer_alloc / sb200_peer_open; index
 * `rank` = this rank's own): grads[r], rank r's flat gradient bucket of `count`
 * floats; reduced[r], a buffer of `count` floats in which rank r keeps the slice of
 * the summed gradient it owns; flags[r], SB200_DP_FLAG_WORDS 32-bit words, zeroed
 * once before the first step.  All buffers 16-byte aligned.
 *
 * Per training step every rank calls, on its stream, after its backward pass:
 *   sb200_dp_reduce  announces this rank's gradients, waits for every peer's, and
 *                    sums this rank's slice (1 / world of the bucket) over all
 *                    ranks' buckets in fixed rank order (peer loads);
 *   sb200_dp_update  waits for every peer's slice, then
 *                    params <- params - lr * g over all `count` elements, g read
 *                    from the owning rank's slice; elements from n_sum on are
 *                    divided by world first.
 * Both return at once; the waits happen on the GPU and are bounded by
 * SB200_OPT_WAIT_LIMIT_US (a wait that runs out makes sb200_check_device_status
 * return SB200_ERR_DEVICE_TIMEOUT).  The step number lives in the flag words, so the
 * two calls can be captured in a CUDA graph and replayed.  Every rank ends a step
 * with bit-identical parameters.
 */
#define SB200_DP_FLAG_WORDS 32
typedef struct sb200_dp_group {
    int world, rank;
    const float* grads[8];
    float* reduced[8];
    uint32_t* flags[8];
} sb200_dp_group;

int sb200_dp_reduce(sb200_ctx* ctx, const sb200_dp_group* group, int64_t count, sb200_stream stream);

/*
 * A barrier between the ranks' streams over the same kind of flag words (flags[r]: rank
 * r's SB200_DP_FLAG_WORDS words, mapped by every rank, zeroed once; the words it uses are
 * not those of sb200_dp_reduce / sb200_dp_update, one set can serve both): a one-warp
 * kernel announces "this rank's stream has come this far" in every peer's words and
 * waits, bounded by SB200_OPT_WAIT_LIMIT_US, until every peer has announced the same.
 * Work enqueued after it on any rank starts after the work enqueued before it on every
 * rank.  Replaces the one-element all-reduce between a GEMM that writes into peers'
 * buffers (sb200_gemm_reduce_scatter, sb200_gemm_scatter) and the reads that follow.
 * No counterpart in the reference.  Replays from a CUDA graph.
 */
int sb200_peer_barrier(sb200_ctx* ctx, uint32_t* const* flags, int world, int rank, sb200_stream stream);
int sb200_dp_update(sb200_ctx* ctx, const sb200_dp_group* group, float* params, int64_t count,
                    int64_t n_sum, float lr, sb200_stream stream);

/*
 * CSR matrix, device arrays.  Same fields and order as the reference's
 * SparseMatrix (Includes/Sapphire/compute/sparse/SparseMatrix.hpp:28-38):
 * V values, COL column indices, ROW offsets of length M + 1, then NNZ, M, N
 * and padding to 48 bytes, so an array of them can be cast either way.
 */
typedef struct sb200_csr {
    float* V;
    uint32_t* COL;
    uint32_t* ROW;
    uint32_t NNZ;
    uint32_t M;
    uint32_t N;
    uint32_t Padding[3];
} sb200_csr;

/*
 * C = A . B for CSR operands on the device; two passes (symbolic: row sizes,
 * numeric: values), columns ascending inside every row, structural zeros
 * kept.  The callee allocates C->V, C->COL, C->ROW (cudaMalloc) and fills
 * NNZ, M, N; the caller frees them with sb200_csr_free.  The call
 * synchronises the stream once between the passes (it needs nnz(C) on the
 * host to size the output).
 * Replaces Sparse::Cuda::Gemm (Includes/Sapphire/compute/sparse/cuda/SparseGemm.cuh:16-41:
 * "Required memory is automatically allocated", caller frees), one matrix per call.
 * Limit: B->N <= 524288 columns (SB200_ERR_TOO_LARGE beyond): a row's column bitmap and its
 * prefix sums live in shared memory.
 */
int sb200_spgemm_csr(sb200_ctx* ctx, const sb200_csr* A, const sb200_csr* B, sb200_csr* C,
                     sb200_stream stream);

/* The two passes separately, for callers that own the output arrays:
 * symbolic writes rowC[0..M] (device) and returns nnz(C) through *nnzC after
 * synchronising; numeric fills colC / valC (device, nnz(C) entries). */
int sb200_spgemm_csr_symbolic(sb200_ctx* ctx, const sb200_csr* A, const sb200_csr* B,
                              uint32_t* rowC, int64_t* nnzC, sb200_stream stream);
int sb200_spgemm_csr_numeric(sb200_ctx* ctx, const sb200_csr* A, const sb200_csr* B,
                             const uint32_t* rowC, uint32_t* colC, float* valC,
                             sb200_stream stream);

int sb200_csr_free(sb200_csr* C);

/* Copies the three arrays of a device CSR matrix into caller-owned arrays
 * (row: M + 1, col and val: NNZ entries) on the device (to_host = 0) or in
 * host memory (to_host = 1), then synchronises the stream.  One matrix of
 * DeepCopyDeviceToDevice / DeepCopyDeviceToHost
 * (Includes/Sapphire/compute/sparse/Sparse.hpp:49-51, 65-67). */
int sb200_csr_copy_out(const sb200_csr* src, uint32_t* row, uint32_t* col, float* val,
                       int to_host, sb200_stream stream);

/*
 * Dense -> CSR on the device.  `dense` is M x N row-major with row pitch ld >= N
 * (the reference's `paddedN`); an entry is kept when it is not exactly 0.0f;
 * columns ascend inside a row.  The callee allocates out->V / COL / ROW
 * (caller frees with sb200_csr_free); the call synchronises the stream once.
 * Device counterpart of CreateSparseMatrixWithDenseMatrix
 * (Includes/Sapphire/compute/sparse/Sparse.hpp:154-157, declared without a definition).
 */
int sb200_dense_to_csr(sb200_ctx* ctx, const float* dense, uint32_t M, uint32_t N, int64_t ld,
                       sb200_csr* out, sb200_stream stream);

/* CSR -> dense: zero-fills the M x N window of `dense` (row pitch ld >= N) and
 * scatters the entries.  Device counterpart of ConvertSparseMatrixToDenseMatrix
 * (Includes/Sapphire/compute/sparse/Sparse.hpp:159-162). */
int sb200_csr_to_dense(sb200_ctx* ctx, const sb200_csr* src, float* dense, int64_t ld,
                       sb200_stream stream);

/*
 * Column sums for callers that cannot allocate: out[n] = scale * sum_k op(B)[k, n],
 * the bias-gradient part of sb200_gemm_batched on its own (same kernels, same
 * meaning of transB / ldb; B and out are device pointers of the CURRENT device).
 * This entry point has no counterpart in the reference; it exists for callers
 * that must not cause a device allocation -- code running underneath an
 * allocator that assumes it owns the GPU's free memory (Sapphire's
 * ResourceManager pools, a framework's caching allocator), and code on a
 * latency path, since cudaMalloc / cudaFree synchronise the device.  It takes
 * no context (creating one allocates) and calls no cudaMalloc, cudaFree or
 * allocating library routine: its scratch for the per-slice partial sums is a
 * fixed 4 MiB array inside the library image, present on every GPU that loads
 * the library until the process exits.
 *   Limit: N <= SB200_COLSUM_NOALLOC_MAX_N columns (SB200_ERR_TOO_LARGE beyond);
 *   K is unlimited.
 *   The first call on each device looks up the array's device address
 *   (cudaGetSymbolAddress) and the SM count; make that first call before any
 *   stream capture begins.
 *   All calls on a device share the one array.  Nothing needs clearing between
 *   calls (each call overwrites every cell it later reads), but two calls whose
 *   kernels overlap on the GPU -- different streams, no dependency -- race on it:
 *   order them.
 */
#define SB200_COLSUM_NOALLOC_MAX_N 16384
int sb200_colsum_noalloc(const float* B, int transB, int64_t K, int64_t N, int64_t ldb,
                         float* out, float scale, sb200_stream stream);

/* ---- elementwise steps of a Linear training step -------------------------
 * The kernels either side of the GEMMs when Sapphire trains an MLP; same
 * argument meaning as the reference's device leaves.  All pointers are device
 * pointers; "accumulates" means dx is read, added to and written back.
 */

/* out = max(in, 0).  Dense::Cuda::ReLU
 * (Sources/Sapphire/compute/dense/cuda/kernels/ActivationKernel.cu:11-22). */
int sb200_relu(sb200_ctx* ctx, float* out, const float* in, int64_t n, sb200_stream stream);

/* dx += x > 0 ? dy : 0 (accumulates).  ReLUBackward
 * (Sources/Sapphire/compute/dense/cuda/kernels/ActivationBackwardKernel.cu:11-24). */
int sb200_relu_backward(sb200_ctx* ctx, float* dx, const float* dy, const float* x, int64_t n,
                        sb200_stream stream);

/* Row softmax over rows of `unit` elements with max subtraction.  SoftMax
 * (Sources/Sapphire/compute/dense/naive/NaiveBasic.cpp:235-255; device twin
 * ActivationKernel.cu:38-65). */
int sb200_softmax(sb200_ctx* ctx, float* out, const float* in, int64_t total, int unit,
                  sb200_stream stream);

/* dx += J^T dy with the full softmax Jacobian (accumulates).  SoftMaxBackward
 * (Sources/Sapphire/compute/dense/naive/NaiveBasic.cpp:257-281). */
int sb200_softmax_backward(sb200_ctx* ctx, float* dx, const float* dy, const float* y,
                           int64_t total, int unit, sb200_stream stream);

/* loss[i] = -sum_j label[i,j] * log(x[i,j]); x == 0 is replaced by 1.17549e-30;
 * no batch mean.  CrossEntropy
 * (Sources/Sapphire/compute/dense/naive/NaiveCrossEntropy.cpp:15-31). */
int sb200_cross_entropy(sb200_ctx* ctx, float* loss, const float* x, const float* label, int batch,
                        int unit, sb200_stream stream);

/* dx -= label / x (accumulates).  CrossEntropyBackward (NaiveCrossEntropy.cpp:33-51). */
int sb200_cross_entropy_backward(sb200_ctx* ctx, float* dx, const float* x, const float* label,
                                 int batch, int unit, sb200_stream stream);

/*
 * Convolution lowering for the batched GEMM.  x is [N, C, H, W]; the matrix
 * `cols` is [N, C*kh*kw, outR*outC] with
 *     outR = (H + 2 padR - dilR (kh - 1) - 1) / strideR + 1     (outC likewise),
 * row c*kh*kw + (kh*kw - 1 - (fr*kw + fc)) holding filter tap (fr, fc) of
 * channel c (reverse tap order: the GEMM below is then a true convolution, the
 * mode the reference asks of cuDNN) and column orow*outC + ocol the output pixel.
 *
 * sb200_im2col fills cols; taps outside the image read pad_value.  Device
 * counterpart of Dense::Naive::Im2Col
 * (Sources/Sapphire/compute/dense/naive/Convolution.cpp:15-115), which exists on the host
 * only.  The forward convolution of Convolution.cpp:217-253 is then
 *     sb200_gemm_batched(A = filter [Cout, C*kh*kw] with strideA = 0,
 *                        B = cols, C = D = y [N, Cout, outR*outC])
 * -- the broadcast-A case of Compute::Gemm.
 *
 * sb200_col2im adds to every pixel of x the entries of cols that im2col read
 * from it (ascending output-pixel order, like the reference's loop): the input
 * gradient step of Conv2DBackward (Convolution.cpp:117-211, 255-316).
 */
typedef struct sb200_conv_geometry {
    int N, C, H, W;
    int kh, kw;
    int strideR, strideC;
    int padR, padC;
    int dilR, dilC;
} sb200_conv_geometry;

int sb200_im2col(sb200_ctx* ctx, float* cols, const float* x,
                 const sb200_conv_geometry* geometry, float pad_value, sb200_stream stream);
int sb200_col2im(sb200_ctx* ctx, float* x, const float* cols,
                 const sb200_conv_geometry* geometry, sb200_stream stream);

/*
 * SoftMax, CrossEntropy and both their backward passes over [batch, unit] logits
 * as one kernel (one warp per sample), with the arithmetic and operation order
 * of the four separate calls above run on zeroed gradient buffers:
 *     prob  = softmax(logits)                     (written when prob != NULL)
 *     loss  = -sum_j label * log(prob)            (written when loss != NULL)
 *     dlogits = softmax_backward(cross_entropy_backward(prob, label), prob)
 * It replaces the four leaf calls at the end of a classifier's forward pass and
 * the start of its backward pass (NaiveBasic.cpp:235-281,
 * NaiveCrossEntropy.cpp:15-51).  unit <= 1024.  logits, label and prob are dense
 * [batch, unit]; dlogits has row pitch ld_dlogits >= unit, so that it can be
 * written with the 16-byte aligned rows the tensor-core GEMMs of the backward
 * pass want as an operand.
 */
int sb200_softmax_cross_entropy(sb200_ctx* ctx, float* prob, float* loss, float* dlogits,
                                int64_t ld_dlogits, const float* logits, const float* label,
                                int batch, int unit, sb200_stream stream);

/* z <- z - lr * dz as one kernel; the reference runs Scale into a temporary and
 * then Sub (Sources/Sapphire/operations/optimizers/SGD.cpp:22-28). */
int sb200_sgd_update(sb200_ctx* ctx, float* z, const float* dz, float lr, int64_t n,
                     sb200_stream stream);

/* out = in * factor.  Dense::Cuda::Scale
 * (Sources/Sapphire/compute/dense/cuda/kernels/BasicKernel.cu:115-125). */
int sb200_scale(sb200_ctx* ctx, float* out, const float* in, float factor, int64_t n,
                sb200_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* SAPPHIRE_B200_H */
