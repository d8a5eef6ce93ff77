// TEST INFRASTRUCTURE.  Stand-in for the reference's Sapphire/tensor/TensorData.hpp.
// The real class drags in the CUDA runtime, cuDNN handles and the memory pools
// (Sources/Sapphire/tensor/TensorData.cpp:7-10), none of which the host convolution
// or the Linear backward unit use: they touch the shape, the host pointer, the compute
// mode and the shallow-copy / reshape behaviour of a TensorData.  This class provides exactly those
// members with the reference's semantics -- a handle on a shared, zero-filled host
// buffer of Shape.Size() floats (TensorData.cpp:330: buffers are zeroed on allocation;
// TensorData.hpp:18-213: copies share the buffer; Reshape keeps the data) -- so that
// Convolution.cpp compiles unmodified against it and its own index arithmetic is what
// runs.  The reference's real Shape (Includes/Sapphire/util/Shape.hpp +
// Sources/Sapphire/util/shape.cpp) is used as is.
#ifndef SB200_STANDIN_TENSORDATA_HPP
#define SB200_STANDIN_TENSORDATA_HPP

#include <Sapphire/util/CudaDevice.hpp>
#include <Sapphire/util/Shape.hpp>
#include <cstring>
#include <memory>
#include <stdexcept>

namespace Sapphire::TensorUtil
{
class TensorData
{
public:
    TensorData() = default;

    TensorData(Shape shape, Type type, CudaDevice device)
        : m_shape(std::move(shape)), m_type(type), m_device(std::move(device))
    {
        const auto n = static_cast<size_t>(m_shape.Size());
        m_host = std::shared_ptr<float[]>(new float[n > 0 ? n : 1]);
        std::memset(m_host.get(), 0, (n > 0 ? n : 1) * sizeof(float));
    }

    //! Wraps caller-owned memory (the checker's numpy arrays): no copy, no ownership
    TensorData(Shape shape, float* data)
        : m_shape(std::move(shape)), m_host(std::shared_ptr<float[]>(data, [](float*) {}))
    {
    }

    [[nodiscard]] const Shape& GetShape() const { return m_shape; }
    [[nodiscard]] int Rows() const { return m_shape.Rows(); }
    [[nodiscard]] int Cols() const { return m_shape.Cols(); }
    [[nodiscard]] int GetNumUnits(int requiredDim) const { return m_shape.GetNumUnits(requiredDim); }
    [[nodiscard]] ComputeMode Mode() const { return m_mode; }
    void SetMode(ComputeMode mode) { m_mode = mode; }
    [[nodiscard]] Type GetType() const { return m_type; }
    [[nodiscard]] CudaDevice GetDevice() const { return m_device; }
    [[nodiscard]] CudaDevice GetCudaDevice() const { return m_device; }
    [[nodiscard]] int GetDescriptorKey() const { return -1; }

    void Reshape(const Shape& shape)
    {
        if (shape.Size() != m_shape.Size())
            throw std::runtime_error("TensorData::Reshape - size mismatch");
        m_shape = shape;
    }

    [[nodiscard]] const float* HostRawPtr() const { return m_host.get(); }
    [[nodiscard]] float* HostMutableRawPtr() { return m_host.get(); }

private:
    Shape m_shape;
    Type m_type = Type::Dense;
    CudaDevice m_device;
    ComputeMode m_mode = ComputeMode::Host;
    std::shared_ptr<float[]> m_host;
};
}  // namespace Sapphire::TensorUtil

#endif
