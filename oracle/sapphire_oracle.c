/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the arithmetic on Sapphire's matrix-multiplication path,
 * used only as the checker for the CUDA kernels (tests, the smoke check and
 * the cpu_baseline leg of the benchmark).  The product library never links
 * or calls anything in this file.
 *
 * Parity status:
 *   dense functions   PINNED.  Every function below is checked bit-for-bit
 *                     against the reference's own compiled CPU code
 *                     (oracle/_ref, built from the reference tree by
 *                     oracle/Makefile) and against fixtures generated from it
 *                     (tests/golden).
 *   orc_im2col/col2im PINNED.  Restated from the reference's host lowering
 *                     (Sources/Sapphire/compute/dense/naive/Convolution.cpp:15-211) and
 *                     checked bit-for-bit against that file itself, compiled
 *                     unmodified against stand-ins for the reference's
 *                     TensorData / CudaDevice headers (oracle/ref_ops_shim.cpp,
 *                     oracle/ref_standins/; the real headers pull in the CUDA
 *                     runtime, cuDNN and the memory pools), and against fixtures
 *                     generated from it (tests/golden/conv_golden.npz).  The
 *                     composition with the Gemm leaf (Conv2D, Conv2DBackward,
 *                     Convolution.cpp:217-316) is pinned the same way.  The tests
 *                     also check that the lowering + Gemm equals a true
 *                     (flipped-kernel) convolution, the mode the reference asks
 *                     of cuDNN (Sources/Sapphire/compute/dense/cuda/Convolution.cu:39).
 *   orc_spgemm_*      PARITY UNPINNED.  The reference declares a CSR sparse
 *                     GEMM (Includes/Sapphire/compute/sparse/naive/SparseGemm.hpp:15-16,
 *                     Includes/Sapphire/compute/sparse/cuda/SparseGemm.cuh:38-41) but ships
 *                     no implementation, no test and no fixture for it.  The
 *                     restatement follows the declared types
 *                     (Includes/Sapphire/compute/sparse/SparseMatrix.hpp:28-38) and
 *                     the output order implied by the reference's device sort
 *                     (ascending column index inside a row,
 *                     Sources/Sapphire/compute/cudaUtil/SparseUtil.cu:69-124).
 *
 * Compile with -ffp-contract=off and without -mfma: the reference is built
 * with -mavx -mavx2 only, so its a*b+c is a rounded multiply followed by a
 * rounded add, and the summation order below is part of the result.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ dense */

/*
 * out += A.B per batch; batch count = totalSize / (M*N); A, B, out dense
 * row-major with leading dimensions K, N, N.  The dot product is summed in
 * ascending k into a fresh fp32 zero and added to out once.
 * Follows Sources/Sapphire/compute/dense/naive/NaiveGemm.cpp:12-38.
 */
void orc_gemm(unsigned totalSize, float* out, const float* A, const float* B,
              unsigned M, unsigned N, unsigned K)
{
    const size_t perOut = (size_t)M * N;
    const size_t batches = perOut ? totalSize / perOut : 0;
    for (size_t b = 0; b < batches; ++b) {
        const float* a = A + b * (size_t)M * K;
        const float* bm = B + b * (size_t)K * N;
        float* o = out + b * perOut;
        for (size_t m = 0; m < M; ++m)
            for (size_t n = 0; n < N; ++n) {
                float dot = 0.0f;
                for (size_t k = 0; k < K; ++k)
                    dot += a[m * K + k] * bm[k * N + n];
                o[m * N + n] += dot;
            }
    }
}

/*
 * The general form the C ABI exposes, restated from what the reference does
 * for each piece:
 *   - transposed operands: the reference first materialises the transpose
 *     (Sources/Sapphire/operations/Backward/LinearBackward.cpp:49-50, 70-72 via
 *     NaiveBasic.cpp:63-84) and then runs the plain loop above, so the value
 *     is the same ascending-k sum over op(A)[m,k] * op(B)[k,n];
 *   - bias: Linear's forward adds the bias with a rank-1 Gemm into a zeroed y
 *     before the main Gemm (Sources/Sapphire/operations/Forward/Linear.cpp:134-136),
 *     i.e. y = (c + bias[n]) + dot;
 *   - leading dimensions / batch strides generalise ld = cols
 *     (NaiveGemm.cpp:16-18); a batch stride of 0 re-reads one matrix for
 *     every batch (Includes/Sapphire/compute/Broadcast.hpp:124-132).
 * C may be NULL (treated as 0) and may alias D.
 */
void orc_gemm_ex(int transA, int transB, long M, long N, long K,
                 const float* A, long lda, long strideA,
                 const float* B, long ldb, long strideB,
                 const float* C, long ldc, long strideC,
                 float* D, long ldd, long strideD,
                 const float* bias, long batch)
{
    for (long b = 0; b < batch; ++b) {
        const float* a = A + b * strideA;
        const float* bm = B + b * strideB;
        const float* c = C ? C + b * strideC : NULL;
        float* d = D + b * strideD;
        for (long m = 0; m < M; ++m)
            for (long n = 0; n < N; ++n) {
                float dot = 0.0f;
                for (long k = 0; k < K; ++k) {
                    const float av = transA ? a[k * lda + m] : a[m * lda + k];
                    const float bv = transB ? bm[n * ldb + k] : bm[k * ldb + n];
                    dot += av * bv;
                }
                float base = c ? c[m * ldc + n] : 0.0f;
                if (bias)
                    base = base + bias[n];
                d[m * ldd + n] = base + dot;
            }
    }
}

/*
 * Bias gradient of a Linear layer: out[n] = scale * sum_k dy[k,n], summed in
 * ascending k from fp32 zero, then scaled.  The reference computes it as
 * Gemm(dB, ones[1,B], dy) into a zeroed dB followed by Scale(dB, 1/B)
 * (Sources/Sapphire/operations/Backward/LinearBackward.cpp:93-97); 1.0f * x is exact.
 */
void orc_colsum(float* out, const float* dy, long rows, long cols, long ld, float scale)
{
    for (long n = 0; n < cols; ++n) {
        float s = 0.0f;
        for (long k = 0; k < rows; ++k)
            s += dy[k * ld + n];
        out[n] = (0.0f + s) * scale;
    }
}

/* Batched 2-D transpose into a fresh buffer; with `broadcast` one input
 * matrix is reused for every batch.  NaiveBasic.cpp:63-84. */
void orc_transpose(float* out, const float* in, unsigned rows, unsigned cols,
                   unsigned batch, int broadcast)
{
    const size_t per = (size_t)rows * cols;
    for (size_t b = 0; b < batch; ++b) {
        const float* src = broadcast ? in : in + b * per;
        float* dst = out + b * per;
        for (size_t i = 0; i < rows; ++i)
            for (size_t j = 0; j < cols; ++j)
                dst[j * rows + i] = src[i * cols + j];
    }
}

/* NaiveBasic.cpp:53-60 */
void orc_scale(float* out, const float* in, float factor, unsigned total)
{
    for (unsigned i = 0; i < total; ++i)
        out[i] = in[i] * factor;
}

/* Elementwise a - b over equal-sized buffers (the no-broadcast case of
 * NaiveBasic.cpp:29-40, which is all the SGD step uses). */
void orc_sub(float* out, const float* a, const float* b, unsigned total)
{
    for (unsigned i = 0; i < total; ++i)
        out[i] = a[i] - b[i];
}

/* NaiveBasic.cpp:159-165 */
void orc_relu(float* out, const float* in, unsigned total)
{
    for (unsigned i = 0; i < total; ++i)
        out[i] = in[i] > 0 ? in[i] : 0;
}

/* dx accumulates.  NaiveBasic.cpp:167-174 */
void orc_relu_backward(float* dx, const float* dy, const float* x, unsigned total)
{
    for (unsigned i = 0; i < total; ++i)
        dx[i] += x[i] > 0.0f ? dy[i] : 0.0f;
}

/* Row softmax with max subtraction; the reference evaluates std::exp(float)
 * twice per element and divides.  NaiveBasic.cpp:235-255 */
void orc_softmax(float* out, const float* in, unsigned total, unsigned unit)
{
    const unsigned rows = unit ? total / unit : 0;
    for (unsigned r = 0; r < rows; ++r) {
        const float* x = in + (size_t)r * unit;
        float* y = out + (size_t)r * unit;
        float hi = -3.402823466e+38f;
        for (unsigned i = 0; i < unit; ++i)
            if (hi < x[i])
                hi = x[i];
        float denom = 0;
        for (unsigned i = 0; i < unit; ++i)
            denom += expf(x[i] - hi);
        for (unsigned i = 0; i < unit; ++i)
            y[i] = expf(x[i] - hi) / denom;
    }
}

/* Full-Jacobian softmax backward, dx accumulates.  NaiveBasic.cpp:257-281 */
void orc_softmax_backward(float* dx, const float* dy, const float* y,
                          unsigned total, unsigned unit)
{
    const unsigned rows = unit ? total / unit : 0;
    for (unsigned r = 0; r < rows; ++r) {
        const size_t o = (size_t)r * unit;
        for (unsigned i = 0; i < unit; ++i) {
            float s = 0.0f;
            for (unsigned j = 0; j < unit; ++j) {
                if (i == j)
                    s += dy[o + j] * (y[o + j] * (1.0f - y[o + j]));
                else
                    s += dy[o + j] * (-y[o + i] * y[o + j]);
            }
            dx[o + i] += s;
        }
    }
}

#define ORC_CE_FLOOR 1.17549e-30f

/* Per-sample -sum label*log(x); x == 0 is replaced by 1.17549e-30; no batch
 * mean.  NaiveCrossEntropy.cpp:15-31 */
void orc_cross_entropy(float* y, const float* x, const float* label, int batch, int unit)
{
    for (int i = 0; i < batch; ++i) {
        float s = 0.0f;
        for (int j = 0; j < unit; ++j) {
            const int idx = i * unit + j;
            const float v = x[idx] == 0.0f ? ORC_CE_FLOOR : x[idx];
            s -= label[idx] * logf(v);
        }
        y[i] = s;
    }
}

/* dx -= label / x.  NaiveCrossEntropy.cpp:33-51 */
void orc_cross_entropy_backward(float* dx, const float* x, const float* label,
                                int batch, int unit)
{
    for (int i = 0; i < batch * unit; ++i) {
        const float v = x[i] == 0.0f ? ORC_CE_FLOOR : x[i];
        dx[i] -= label[i] / v;
    }
}

/* ------------------------------------------------------------ convolution */

static int orc_conv_out(int in, int pad, int dil, int k, int stride)
{
    return (in + 2 * pad - dil * (k - 1) - 1) / stride + 1;
}

/*
 * cols[n][C*kh*kw][outR*outC] from x[n][C][H][W].  Row c*kh*kw + (kh*kw - 1 -
 * (fr*kw + fc)) of the matrix holds filter tap (fr, fc) of channel c -- the
 * taps are stored in reverse, which makes Gemm(filter, cols) a true
 * convolution -- and column orow*outC + ocol the output pixel.  Taps that fall
 * outside the image read `pad`.
 * Follows Sources/Sapphire/compute/dense/naive/Convolution.cpp:15-115.
 */
void orc_im2col(float* cols, const float* x, int N, int C, int H, int W, int kh, int kw,
                int strideR, int strideC, int padR, int padC, int dilR, int dilC, float pad)
{
    const int outR = orc_conv_out(H, padR, dilR, kh, strideR);
    const int outC = orc_conv_out(W, padC, dilC, kw, strideC);
    const long P = (long)outR * outC, taps = (long)kh * kw;
    for (int n = 0; n < N; ++n) {
        const float* xn = x + (long)n * C * H * W;
        float* mn = cols + (long)n * C * taps * P;
        for (int c = 0; c < C; ++c)
            for (int fr = 0; fr < kh; ++fr)
                for (int fc = 0; fc < kw; ++fc) {
                    float* mrow = mn + (c * taps + taps - 1 - ((long)fr * kw + fc)) * P;
                    for (int orow = 0; orow < outR; ++orow)
                        for (int ocol = 0; ocol < outC; ++ocol) {
                            const int r = orow * strideR + fr * dilR - padR;
                            const int q = ocol * strideC + fc * dilC - padC;
                            const int inside = r >= 0 && r < H && q >= 0 && q < W;
                            mrow[(long)orow * outC + ocol] =
                                inside ? xn[((long)c * H + r) * W + q] : pad;
                        }
                }
    }
}

/*
 * The adjoint: x[n][c][r][q] += every entry of cols that im2col would have read
 * from that pixel.  The reference walks (c, orow, ocol, fr, fc) in that nesting
 * and adds in place, so a pixel receives its terms in ascending (orow, ocol)
 * order; fp32 addition order is part of the result.
 * Follows Sources/Sapphire/compute/dense/naive/Convolution.cpp:117-211.
 */
void orc_col2im(float* x, const float* cols, int N, int C, int H, int W, int kh, int kw,
                int strideR, int strideC, int padR, int padC, int dilR, int dilC)
{
    const int outR = orc_conv_out(H, padR, dilR, kh, strideR);
    const int outC = orc_conv_out(W, padC, dilC, kw, strideC);
    const long P = (long)outR * outC, taps = (long)kh * kw;
    for (int n = 0; n < N; ++n) {
        float* xn = x + (long)n * C * H * W;
        const float* mn = cols + (long)n * C * taps * P;
        for (int c = 0; c < C; ++c)
            for (int orow = 0; orow < outR; ++orow)
                for (int ocol = 0; ocol < outC; ++ocol)
                    for (int fr = 0; fr < kh; ++fr)
                        for (int fc = 0; fc < kw; ++fc) {
                            const int r = orow * strideR + fr * dilR - padR;
                            const int q = ocol * strideC + fc * dilC - padC;
                            if (r < 0 || r >= H || q < 0 || q >= W)
                                continue;
                            const long mrow = c * taps + taps - 1 - ((long)fr * kw + fc);
                            xn[((long)c * H + r) * W + q] += mn[mrow * P + (long)orow * outC + ocol];
                        }
    }
}

/* ----------------------------------------------------------------- sparse */

/*
 * CSR x CSR, PARITY UNPINNED (see the header of this file).
 * Row-wise (Gustavson) product C = A.B with
 *   ROW  standard CSR offsets of length M+1 (the reference headers never
 *        state the length; M+1 is assumed),
 *   COL  ascending inside every row,
 *   V    fp32; the products of one output entry are added in the order
 *        (k ascending over A's row, then B's row k in stored order) starting
 *        from the first product,
 *   the structural pattern is kept: an entry whose products cancel to 0.0f
 *   stays in the output.
 *
 * Two calls, like the symbolic/numeric split of the CUDA path:
 *   orc_spgemm_symbolic fills rowC[0..M] and returns nnz(C);
 *   orc_spgemm_numeric  fills colC / valC given rowC.
 * Also returns the number of scalar products through *products.
 */
long orc_spgemm_symbolic(uint32_t M, uint32_t N,
                         const uint32_t* rowA, const uint32_t* colA,
                         const uint32_t* rowB, const uint32_t* colB,
                         uint32_t* rowC, long* products)
{
    uint32_t* mark = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(N ? N : 1));
    if (!mark)
        return -1;
    memset(mark, 0xff, sizeof(uint32_t) * (size_t)(N ? N : 1));
    long nnz = 0, prods = 0;
    rowC[0] = 0;
    for (uint32_t i = 0; i < M; ++i) {
        for (uint32_t p = rowA[i]; p < rowA[i + 1]; ++p) {
            const uint32_t k = colA[p];
            for (uint32_t q = rowB[k]; q < rowB[k + 1]; ++q) {
                const uint32_t j = colB[q];
                ++prods;
                if (mark[j] != i) {
                    mark[j] = i;
                    ++nnz;
                }
            }
        }
        rowC[i + 1] = (uint32_t)nnz;
    }
    free(mark);
    if (products)
        *products = prods;
    return nnz;
}

static int orc_cmp_u32(const void* a, const void* b)
{
    const uint32_t x = *(const uint32_t*)a, y = *(const uint32_t*)b;
    return (x > y) - (x < y);
}

int orc_spgemm_numeric(uint32_t M, uint32_t N,
                       const uint32_t* rowA, const uint32_t* colA, const float* valA,
                       const uint32_t* rowB, const uint32_t* colB, const float* valB,
                       const uint32_t* rowC, uint32_t* colC, float* valC)
{
    const size_t n = N ? N : 1;
    float* acc = (float*)malloc(sizeof(float) * n);
    uint32_t* mark = (uint32_t*)malloc(sizeof(uint32_t) * n);
    if (!acc || !mark) {
        free(acc);
        free(mark);
        return -1;
    }
    memset(mark, 0xff, sizeof(uint32_t) * n);
    for (uint32_t i = 0; i < M; ++i) {
        uint32_t fill = rowC[i];
        for (uint32_t p = rowA[i]; p < rowA[i + 1]; ++p) {
            const uint32_t k = colA[p];
            const float av = valA[p];
            for (uint32_t q = rowB[k]; q < rowB[k + 1]; ++q) {
                const uint32_t j = colB[q];
                const float prod = av * valB[q];
                if (mark[j] != i) {
                    mark[j] = i;
                    acc[j] = prod;
                    colC[fill++] = j;
                } else {
                    acc[j] += prod;
                }
            }
        }
        if (fill != rowC[i + 1]) {
            free(acc);
            free(mark);
            return -2;
        }
        qsort(colC + rowC[i], fill - rowC[i], sizeof(uint32_t), orc_cmp_u32);
        for (uint32_t q = rowC[i]; q < fill; ++q)
            valC[q] = acc[colC[q]];
    }
    free(acc);
    free(mark);
    return 0;
}
