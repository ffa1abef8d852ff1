// SoftmaxLayer<T>: masked row softmax over attention logits [B,H,T,T].
// Public surface of upstream dnn/layers/softmax_layer.cuh:15-39 (set_mask with a non-owning pointer to a
// [B,1,T,T] or [1,1,T,T] additive mask, forward, backward, name() == "Softmax"); forward throws
// std::runtime_error unless the input is 4-D (dnn/layers/softmax_layer.cu:147-149).
#pragma once

#include <iostream>
#include <optional>
#include <string>

#include "dnn/core/layer.cuh"
#include "dnn/core/tensor.cuh"

namespace dnn {

template <typename T>
class SoftmaxLayer : public Layer<T> {
public:
    explicit SoftmaxLayer(bool training_enabled = false);
    ~SoftmaxLayer() override;

    void set_mask(tensor<T>* mask);  // non-owning; nullptr removes the mask
    tensor<T>* mask() const { return mask_; }

    tensor<T> forward(const tensor<T>& input) override;
    tensor<T> backward(const tensor<T>& grad_output) override;

    void save(std::ostream&) const override {}
    void load(std::istream&) override {}
    std::string name() const override { return "Softmax"; }

private:
    tensor<T>* mask_;
    std::optional<tensor<T>> input_cache_;
};

}  // namespace dnn
