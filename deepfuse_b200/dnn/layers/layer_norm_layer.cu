#include "dnn/layers/layer_norm_layer.cuh"

#include <stdexcept>

namespace dnn {

template <typename T>
LayerNormLayer<T>::LayerNormLayer(int norm_size, float epsilon, bool affine, bool training_enabled)
    : Layer<T>(training_enabled),
      norm_size_(norm_size),
      epsilon_(epsilon),
      affine_(affine),
      gamma_({norm_size}),
      beta_({norm_size}),
      grad_gamma_({norm_size}),
      grad_beta_({norm_size}),
      row_stats_({2}) {
    if (norm_size <= 0) throw std::invalid_argument("LayerNormLayer: norm_size must be positive");
    gamma_.fill(static_cast<T>(1));
    beta_.fill(static_cast<T>(0));
    grad_gamma_.zero();
    grad_beta_.zero();
}

template <typename T>
tensor<T> LayerNormLayer<T>::forward(const tensor<T>& input) {
    const auto& s = input.shape();
    if (s.empty() || s.back() != norm_size_)
        throw std::runtime_error("LayerNormLayer::forward: the last input dimension must equal norm_size");
    if (this->training_enabled_) input_cache_ = input.clone();
    const int rows = int(input.numel() / size_t(norm_size_));
    tensor<T> out(s);
    utils::CHECK_DF8(df8_layernorm_f32(input.data(), rows, norm_size_, affine_ ? gamma_.data() : nullptr,
                                       affine_ ? beta_.data() : nullptr, epsilon_, out.data(), nullptr, fp8::stream()));
    return out;
}

template <typename T>
void LayerNormLayer<T>::forward_quantized(const float* x, int rows, df8_kind kind, fp8::Quantized& q) {
    const size_t n = size_t(rows) * size_t(norm_size_);
    if (q.codes.numel() != n) q.codes = tensor<uint8_t>({int(n)});
    if (row_stats_.numel() < size_t(2) * size_t(rows)) row_stats_ = tensor<float>({2 * rows});
    q.kind = kind;
    utils::CHECK_DF8(df8_layernorm_quantize_f32(x, rows, norm_size_, affine_ ? gamma_.data() : nullptr,
                                                affine_ ? beta_.data() : nullptr, epsilon_, kind, q.codes.data(),
                                                q.scale.data(), fp8::amax_slot(q.amax.data()), row_stats_.data(),
                                                fp8::stream()));
}

// Upstream's backward returns the incoming gradient unchanged (layer_norm_layer.cu:83-91); kept.
template <typename T>
tensor<T> LayerNormLayer<T>::backward(const tensor<T>& grad_output) {
    return grad_output.clone();
}

template <typename T>
std::vector<tensor<T>*> LayerNormLayer<T>::parameters() {
    if (!affine_) return {};
    return {&gamma_, &beta_};
}

template <typename T>
std::vector<tensor<T>*> LayerNormLayer<T>::gradients() {
    if (!affine_) return {};
    return {&grad_gamma_, &grad_beta_};
}

// Stream layout shared with upstream (layer_norm_layer.cu:102-118): norm_size, gamma, beta, grad_gamma, grad_beta.
template <typename T>
void LayerNormLayer<T>::save(std::ostream& out) const {
    out.write(reinterpret_cast<const char*>(&norm_size_), sizeof(norm_size_));
    gamma_.save(out);
    beta_.save(out);
    grad_gamma_.save(out);
    grad_beta_.save(out);
}

template <typename T>
void LayerNormLayer<T>::load(std::istream& in) {
    in.read(reinterpret_cast<char*>(&norm_size_), sizeof(norm_size_));
    if (!in || norm_size_ <= 0) throw std::runtime_error("LayerNormLayer::load: bad header");
    gamma_.load(in);
    beta_.load(in);
    grad_gamma_.load(in);
    grad_beta_.load(in);
}

template class LayerNormLayer<float>;

}  // namespace dnn
