// Loss<T>: the interface of upstream's dnn/losses/loss.cuh:7-19.
#pragma once

#include "dnn/core/tensor.cuh"

namespace dnn {

template <typename T>
class Loss {
public:
    virtual ~Loss() = default;
    virtual T compute(const tensor<T>& predictions, const tensor<T>& targets) = 0;
    virtual tensor<T> compute_gradient(const tensor<T>& predictions, const tensor<T>& targets) = 0;
};

}  // namespace dnn
