// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// C entry points around the reference's own CPU leaf functions, so that the
// parity tests and the CPU-baseline leg of the benchmark can call the
// unmodified reference arithmetic through ctypes.  The reference sources are
// compiled where they lie (see oracle/Makefile); nothing is copied.  This
// file only forwards arguments.
//
// Reference functions bound here (paths inside the Sapphire project):
//   Sources/Sapphire/compute/dense/naive/NaiveGemm.cpp:12-38      Dense::Naive::Gemm
//   Sources/Sapphire/compute/dense/naive/NaiveBasic.cpp:29-84     Sub, Scale, Transpose
//   Sources/Sapphire/compute/dense/naive/NaiveBasic.cpp:159-174   ReLU, ReLUBackward
//   Sources/Sapphire/compute/dense/naive/NaiveBasic.cpp:235-281   SoftMax, SoftMaxBackward
//   Sources/Sapphire/compute/dense/naive/NaiveCrossEntropy.cpp:15-51
#include <Sapphire/compute/dense/naive/NaiveBasic.hpp>
#include <Sapphire/compute/dense/naive/NaiveCrossEntropy.hpp>
#include <Sapphire/compute/dense/naive/NaiveGemm.hpp>

namespace N = Sapphire::Compute::Dense::Naive;

extern "C" {

void ref_gemm(unsigned totalSize, float* out, const float* A, const float* B,
              unsigned M, unsigned N_, unsigned K)
{
    N::Gemm(totalSize, out, A, B, M, N_, K);
}

void ref_transpose(float* out, const float* in, unsigned rows, unsigned cols,
                   unsigned batch, int broadcast)
{
    N::Transpose(out, in, rows, cols, batch, broadcast != 0);
}

void ref_scale(float* out, const float* in, float factor, unsigned total)
{
    N::Scale(out, in, factor, total);
}

void ref_sub(unsigned total, float* out, const float* a, const float* b,
             unsigned inputStride, int bcA, int bcB)
{
    N::Sub(total, out, a, b, inputStride, bcA != 0, bcB != 0);
}

void ref_relu(float* out, const float* in, unsigned total)
{
    N::ReLU(out, in, total);
}

void ref_relu_backward(float* dx, const float* dy, const float* x, unsigned total)
{
    N::ReLUBackward(dx, dy, x, total);
}

void ref_softmax(float* out, const float* in, unsigned total, unsigned unit)
{
    N::SoftMax(out, in, total, unit);
}

void ref_softmax_backward(float* dx, const float* dy, const float* y,
                          unsigned total, unsigned unit)
{
    N::SoftMaxBackward(dx, dy, y, total, unit);
}

void ref_cross_entropy(float* y, const float* x, const float* label, int batch, int unit)
{
    N::CrossEntropy(y, x, label, batch, unit);
}

void ref_cross_entropy_backward(float* dx, const float* x, const float* label,
                                int batch, int unit)
{
    N::CrossEntropyBackward(dx, x, label, batch, unit);
}

}  // extern "C"
