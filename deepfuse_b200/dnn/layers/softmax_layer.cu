#include "dnn/layers/softmax_layer.cuh"

#include <stdexcept>

#include "dnn/core/fp8.cuh"

namespace dnn {

template <typename T>
SoftmaxLayer<T>::SoftmaxLayer(bool training_enabled) : Layer<T>(training_enabled), mask_(nullptr) {}

template <typename T>
SoftmaxLayer<T>::~SoftmaxLayer() = default;

template <typename T>
void SoftmaxLayer<T>::set_mask(tensor<T>* mask) {
    mask_ = mask;
}

template <typename T>
tensor<T> SoftmaxLayer<T>::forward(const tensor<T>& input) {
    const auto& s = input.shape();
    if (s.size() != 4) throw std::runtime_error("SoftmaxLayer expects a 4D input [B, H, T, T]");
    if (s[2] != s[3]) throw std::runtime_error("SoftmaxLayer expects square attention logits [B, H, T, T]");
    if (this->training_enabled_) input_cache_ = input.clone();
    int mask_b = 0;
    const T* mask_ptr = nullptr;
    if (mask_) {
        const auto& ms = mask_->shape();
        if (ms.size() != 4 || ms[1] != 1 || ms[2] != s[2] || ms[3] != s[3] || (ms[0] != s[0] && ms[0] != 1))
            throw std::runtime_error("SoftmaxLayer mask must have shape [B, 1, T, T] or [1, 1, T, T]");
        mask_b = ms[0];
        mask_ptr = mask_->data();
    }
    tensor<T> out(s);
    utils::CHECK_DF8(df8_softmax_masked_f32(input.data(), mask_ptr, mask_b, s[0], s[1], s[2], out.data(), fp8::stream()));
    return out;
}

// Upstream's backward is a placeholder that returns the incoming gradient unchanged
// (softmax_layer.cu:173-182); kept as such.
template <typename T>
tensor<T> SoftmaxLayer<T>::backward(const tensor<T>& grad_output) {
    return grad_output.clone();
}

template class SoftmaxLayer<float>;

}  // namespace dnn
