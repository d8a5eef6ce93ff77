// TEST INFRASTRUCTURE.  Stand-in for the reference's Sapphire/Model.hpp, which brings the
// whole graph bookkeeping (Tensor, TensorDescriptor, Model).  The reference's
// LinearBackProp (Sources/Sapphire/operations/Backward/LinearBackward.cpp:27-99) needs one
// thing of it: ModelManager::CurModel().GetOptimizer(), the optimizer it applies to the
// weight and the bias inside the backward pass.
#ifndef SB200_STANDIN_MODEL_HPP
#define SB200_STANDIN_MODEL_HPP

#include <Sapphire/operations/optimizers/Optimizer.hpp>
#include <stdexcept>

namespace Sapphire
{
class Model
{
public:
    [[nodiscard]] Optimizer::Optimizer* GetOptimizer() const
    {
        if (m_optimizer == nullptr)
            throw std::runtime_error("Model::GetOptimizer() - optimizer was null");
        return m_optimizer;
    }

    void SetOptimizer(Optimizer::Optimizer* optimizer) { m_optimizer = optimizer; }

private:
    Optimizer::Optimizer* m_optimizer = nullptr;
};

class ModelManager
{
public:
    static Model& CurModel()
    {
        static Model model;
        return model;
    }
};
}  // namespace Sapphire

#endif
