// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// C entry points around the reference's own host convolution and its Linear backward
// unit, so that the parity tests can pin against them: the restated lowering
// (orc_im2col / orc_col2im and the conv composition in oracle.py), the restated Linear
// backward + SGD of the MLP oracle, and the broadcast planner of the Sapphire-signature
// shims (against the reference's BroadcastWith2Inputs).  Compiled from the reference's
// files where they lie, unmodified (oracle/Makefile, target ref):
//   Sources/Sapphire/compute/dense/naive/Convolution.cpp:15-316  Im2Col, Col2Im, Conv2D, Conv2DBackward
//   Sources/Sapphire/operations/Backward/LinearBackward.cpp:13-99 LinearBackProp
//   Sources/Sapphire/operations/optimizers/SGD.cpp:9-28          Optimizer::SGD
//   Sources/Sapphire/operations/Backward/MathBackward.cpp:13-51  MulBackProp (the file's other
//                                                                units link against stubs below)
//   Sources/Sapphire/compute/dense/naive/NaiveGemm.cpp:12-38     Dense::Naive::Gemm
//   Sources/Sapphire/compute/dense/naive/NaiveBasic.cpp          Dense::Naive::Transpose, Scale, Sub
//   Sources/Sapphire/compute/dense/naive/NaiveInitialize.cpp:34-40 Dense::Naive::Scalar
//   Sources/Sapphire/util/shape.cpp                              Shape
//   Includes/Sapphire/compute/Broadcast.hpp:82-133               BroadcastWith2Inputs
//   Includes/Sapphire/operations/Backward/BackPropWrapper.hpp    (header only)
// The reference's TensorData and CudaDevice headers pull in the CUDA runtime, cuDNN and
// the memory pools, its Model header the whole graph bookkeeping; oracle/ref_standins/
// holds stand-ins with the members these units use (found first on the include path).
// Compute::Gemm, Transpose, Scale, Sub and Initialize::Ones / Zeros, which the units call,
// are defined below as the host branches of Sources/Sapphire/compute/BasicOps.cpp:63-104,
// 183-290 and Sources/Sapphire/compute/Initialize.cpp:47-73 (those files include the CUDA
// kernels' headers and cannot be compiled here): the same shape expansion, the reference's
// own BroadcastWith2Inputs, the reference's own leaf calls.
#include <Sapphire/compute/BasicOps.hpp>
#include <Sapphire/compute/Broadcast.hpp>
#include <Sapphire/compute/dense/naive/Convolution.hpp>
#include <Sapphire/compute/dense/naive/NaiveBasic.hpp>
#include <Sapphire/compute/dense/naive/NaiveGemm.hpp>
#include <Sapphire/compute/dense/naive/NaiveInitialize.hpp>
#include <Sapphire/compute/Initialize.hpp>
#include <Sapphire/Model.hpp>
#include <Sapphire/operations/Backward/LinearBackward.hpp>
#include <Sapphire/operations/Backward/MathBackward.hpp>
#include <Sapphire/operations/optimizers/SGD.hpp>
#include <algorithm>

namespace Sapphire::Compute
{
void Gemm(TensorData& y, const TensorData& a, const TensorData& b)
{
    auto shapeOut = y.GetShape();
    auto shapeA = a.GetShape();
    auto shapeB = b.GetShape();
    shapeOut.Expand(2);
    shapeA.Expand(2);
    shapeB.Expand(2);
    const auto M = shapeOut.Rows();
    const auto N = shapeOut.Cols();
    const auto K = shapeA.Cols();
    const auto maxDim = std::max({ y.GetShape().Dim(), a.GetShape().Dim(), b.GetShape().Dim() });
    shapeOut.Expand(maxDim);
    shapeA.Expand(maxDim);
    shapeB.Expand(maxDim);
    BroadcastWith2Inputs(shapeOut, shapeA, shapeB, shapeOut.Size(), shapeA.Size(), shapeB.Size(),
                         y.HostMutableRawPtr(), a.HostRawPtr(), b.HostRawPtr(), 0, 2,
                         Dense::Naive::Gemm, M, N, K);
}

void Transpose(TensorData& y, const TensorData& x)
{
    const auto inputM = x.Rows();
    const auto inputN = x.Cols();
    const auto broadcast = x.GetNumUnits(2) == 1;
    const auto chunkSize = y.GetShape().Size() / (inputM * inputN);
    Dense::Naive::Transpose(y.HostMutableRawPtr(), x.HostRawPtr(), inputM, inputN, chunkSize, broadcast);
}
void Scale(TensorData& y, const TensorData& x, const float factor)
{
    auto shapeY = y.GetShape();
    Dense::Naive::Scale(y.HostMutableRawPtr(), x.HostRawPtr(), factor, shapeY.Size());
}

namespace
{
// Includes/Sapphire/util/UnitUtils.hpp:38-75 (that header includes the graph bookkeeping):
// how many trailing dimensions all shapes have in common
int MatchingDim(const std::vector<Shape>& shapes)
{
    int curDimFromLast = -1;
    bool match = true;
    while (match) {
        if (shapes.at(0).Dim() + curDimFromLast < 0)
            break;
        const int shapeDim = shapes.at(0).At(curDimFromLast);
        for (const auto& shape : shapes) {
            if (shape.Dim() + curDimFromLast < 0 || shapeDim != shape.At(curDimFromLast)) {
                match = false;
                break;
            }
        }
        if (match)
            curDimFromLast -= 1;
    }
    return -(curDimFromLast + 1);
}
}  // namespace

void Sub(TensorData& y, const TensorData& a, const TensorData& b)
{
    auto shapeOut = y.GetShape();
    auto shapeA = a.GetShape();
    auto shapeB = b.GetShape();
    const auto maxDim = std::max({ y.GetShape().Dim(), a.GetShape().Dim(), b.GetShape().Dim() });
    shapeOut.Expand(maxDim);
    shapeA.Expand(maxDim);
    shapeB.Expand(maxDim);
    const int minRequiredDim = MatchingDim({ shapeOut, shapeA, shapeB });
    BroadcastWith2Inputs(shapeOut, shapeA, shapeB, shapeOut.Size(), shapeA.Size(), shapeB.Size(),
                         y.HostMutableRawPtr(), a.HostRawPtr(), b.HostRawPtr(), 0, minRequiredDim,
                         Dense::Naive::Sub, 0, false, false);
}

// MathBackward.cpp also holds the Add / Dot / Mean units; nothing here runs them
void Add(TensorData&, const TensorData&, const TensorData&)
{
    throw std::runtime_error("Compute::Add is not part of the CPU checker");
}

void Dot(TensorData&, const TensorData&, const TensorData&)
{
    throw std::runtime_error("Compute::Dot is not part of the CPU checker");
}

void MeanBackward(TensorData&, const TensorData&, int)
{
    throw std::runtime_error("Compute::MeanBackward is not part of the CPU checker");
}

namespace Initialize
{
void Ones(TensorUtil::TensorData& data)
{
    Dense::Naive::Scalar(data.HostMutableRawPtr(), 1.0f, data.GetShape());
}

void Zeros(TensorUtil::TensorData& data)
{
    Dense::Naive::Scalar(data.HostMutableRawPtr(), 0.0f, data.GetShape());
}
}  // namespace Initialize
}  // namespace Sapphire::Compute

using Sapphire::Shape;
using Sapphire::TensorUtil::TensorData;
namespace CN = Sapphire::Compute::Dense::Naive;

namespace
{
TensorData wrap(std::initializer_list<int> dims, const float* data)
{
    return TensorData(Shape(std::vector<int>(dims)), const_cast<float*>(data));
}
}  // namespace

extern "C" {

// cols [N, C*kh*kw, P] <- x [N, C, H, W]
void ref_im2col(float* cols, const float* x, int N, int C, int H, int W, int kh, int kw, int strideRow,
                int strideCol, int padRow, int padCol, int dilRow, int dilCol, int outR, int outC, float pad)
{
    TensorData tCols = wrap({ N, C * kh * kw, outR * outC }, cols);
    const TensorData tX = wrap({ N, C, H, W }, x);
    const TensorData tF = wrap({ 1, C, kh, kw }, x);          // only its shape is read
    CN::Im2Col(tCols, tF, tX, strideRow, strideCol, padRow, padCol, dilRow, dilCol, pad);
}

// dx [N, C, H, W] += adjoint of im2col applied to cols, with Col2Im's argument order
// as Conv2DBackward passes it (Convolution.cpp:313-314: strideCol, strideRow)
void ref_col2im(float* dx, const float* cols, int N, int C, int H, int W, int kh, int kw, int strideRow,
                int strideCol, int padRow, int padCol, int dilRow, int dilCol, int outR, int outC)
{
    TensorData tDx = wrap({ N, C, H, W }, dx);
    const TensorData tCols = wrap({ N, C * kh * kw, outR * outC }, cols);
    const TensorData tF = wrap({ 1, C, kh, kw }, cols);       // only its shape is read
    CN::Col2Im(tDx, tCols, tF, strideCol, strideRow, padRow, padCol, dilRow, dilCol);
}

// y [N, Cout, outR, outC] += conv(x, filter [Cout, C, kh, kw])
void ref_conv2d(float* y, const float* x, const float* filt, int N, int C, int H, int W, int Cout, int kh, int kw,
                int strideRow, int strideCol, int padRow, int padCol, int dilRow, int dilCol, int outR, int outC)
{
    TensorData tY = wrap({ N, Cout, outR, outC }, y);
    const TensorData tX = wrap({ N, C, H, W }, x);
    const TensorData tF = wrap({ Cout, C, kh, kw }, filt);
    CN::Conv2D(tY, tX, tF, strideRow, strideCol, padRow, padCol, dilRow, dilCol, Sapphire::CudaDevice());
}

// dx += input gradient, dfilt += filter gradient
void ref_conv2d_backward(float* dx, float* dfilt, const float* dy, const float* x, const float* filt, int N, int C,
                         int H, int W, int Cout, int kh, int kw, int strideRow, int strideCol, int padRow,
                         int padCol, int dilRow, int dilCol, int outR, int outC)
{
    TensorData tDx = wrap({ N, C, H, W }, dx);
    TensorData tDf = wrap({ Cout, C, kh, kw }, dfilt);
    const TensorData tDy = wrap({ N, Cout, outR, outC }, dy);
    const TensorData tX = wrap({ N, C, H, W }, x);
    const TensorData tF = wrap({ Cout, C, kh, kw }, filt);
    CN::Conv2DBackward(tDx, tDf, tDy, tX, tF, strideRow, strideCol, padRow, padCol, dilRow, dilCol,
                       Sapphire::CudaDevice());
}

// y <- y + a.b with the reference's batch / broadcast rules over the leading dimensions
// (Compute::Gemm as restated above: Expand, BroadcastWith2Inputs, Dense::Naive::Gemm)
void ref_compute_gemm(float* y, const int* yShape, int yDim, const float* a, const int* aShape, int aDim,
                      const float* b, const int* bShape, int bDim)
{
    TensorData tY(Shape(std::vector<int>(yShape, yShape + yDim)), y);
    const TensorData tA(Shape(std::vector<int>(aShape, aShape + aDim)), const_cast<float*>(a));
    const TensorData tB(Shape(std::vector<int>(bShape, bShape + bDim)), const_cast<float*>(b));
    Sapphire::Compute::Gemm(tY, tA, tB);
}

// One Linear layer's backward unit with the optimizer inside, as the reference runs it:
// dx [batch, in] += dy . W^T with the pre-update W; W [in, out] and bias [1, out] updated
// in place by SGD with dW = x^T . dy (unscaled) and dB = (1 / batch) ones . dy.
void ref_linear_backprop(float* dx, const float* dy, float* weight, float* bias, const float* x, int batch,
                         int inFeatures, int outFeatures, float learningRate)
{
    Sapphire::Optimizer::SGD sgd(learningRate);
    Sapphire::ModelManager::CurModel().SetOptimizer(&sgd);
    {
        Sapphire::BackProp::LinearBackProp unit(
            "linear", wrap({ batch, inFeatures }, dx), wrap({ batch, outFeatures }, dy),
            wrap({ inFeatures, outFeatures }, weight), wrap({ 1, outFeatures }, bias),
            wrap({ batch, inFeatures }, x), batch);
        unit.InvokeBackPropIfReady(0);
    }
    Sapphire::ModelManager::CurModel().SetOptimizer(nullptr);
}

// The MatMul backward unit: da [batch, M, K] += dy . b^T, db [batch, K, N] += a^T . dy
// (MulBackProp::m_runBackProp: two Transposes, two accumulating Gemms)
void ref_mul_backprop(float* da, float* db, const float* dy, const float* a, const float* b, int batch, int M,
                      int K, int N)
{
    Sapphire::BackProp::MulBackProp unit("mul", wrap({ batch, M, K }, a), wrap({ batch, M, K }, da),
                                         wrap({ batch, K, N }, b), wrap({ batch, K, N }, db),
                                         wrap({ batch, M, N }, dy));
    unit.InvokeBackPropIfReady(0);
}

}  // extern "C"
