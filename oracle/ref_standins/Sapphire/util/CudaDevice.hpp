// TEST INFRASTRUCTURE.  Stand-in for the reference's Sapphire/util/CudaDevice.hpp, which
// includes <cuda_runtime.h>; the reference's host convolution
// (Sources/Sapphire/compute/dense/naive/Convolution.cpp) only passes a CudaDevice
// through and compares ComputeMode values.  Found first on the include path when that
// file is compiled, unmodified, for the CPU checker (oracle/Makefile, target ref).
#ifndef SB200_STANDIN_CUDADEVICE_HPP
#define SB200_STANDIN_CUDADEVICE_HPP

#include <string>

namespace Sapphire
{
enum class ComputeMode
{
    Host,
    Cuda,
};

class CudaDevice
{
public:
    CudaDevice() = default;
    CudaDevice(int id, std::string name) : m_id(id), m_name(std::move(name)) {}
    [[nodiscard]] int GetID() const { return m_id; }
    [[nodiscard]] std::string Name() const { return m_name; }

private:
    int m_id = -1;
    std::string m_name = "Undefined";
};
}  // namespace Sapphire

#endif
