#include "dnn/layers/transformer_block.cuh"

#include <stdexcept>

namespace dnn {

template <typename T>
TransformerBlock<T>::TransformerBlock(int embed_dim, int num_heads, int mlp_hidden_dim, bool training_enabled)
    : Layer<T>(training_enabled),
      embed_dim_(embed_dim),
      num_heads_(num_heads),
      mlp_hidden_dim_(mlp_hidden_dim),
      norm1_(embed_dim, 1e-5f, true, training_enabled),
      norm2_(embed_dim, 1e-5f, true, training_enabled),
      attn_(embed_dim, num_heads, training_enabled),
      mlp_fc1_(embed_dim, mlp_hidden_dim, training_enabled),
      mlp_fc2_(mlp_hidden_dim, embed_dim, training_enabled),
      x1_({1}) {}

template <typename T>
TransformerBlock<T>::~TransformerBlock() = default;

template <typename T>
void TransformerBlock<T>::set_mask(dnn::tensor<T>* mask) {
    if (!mask || mask->shape().size() != 4 || mask->shape()[1] != 1)
        throw std::invalid_argument("Mask must have shape [B, 1, T, T]");
    attn_.set_mask(mask);
}

template <typename T>
void TransformerBlock<T>::forward_inplace(float* x, int B, int T_len) {
    const int M = B * T_len, E = embed_dim_, F = mlp_hidden_dim_;
    const df8_kind act = fp8::policy().activation_kind;
    if (E % 16 != 0 || F % 16 != 0)
        throw std::runtime_error("TransformerBlock: embed_dim and mlp_hidden_dim must be multiples of 16 on the fp8 path");
    if (x1_.numel() != size_t(M) * E) x1_ = tensor<float>({M, E});
    fp8::PassScope amax_slots;

    // x1 = x + MHA(LN1(x))
    norm1_.forward_quantized(x, M, act, ln_q_);
    attn_.forward_quantized(ln_q_, B, T_len, x, x1_.data());

    // y = x1 + FC2(act(FC1(LN2(x1))))
    norm2_.forward_quantized(x1_.data(), M, act, ln_q_);
    mlp_fc1_.forward_codes_quantized(ln_q_.codes.data(), ln_q_.kind, ln_q_.scale.data(), M,
                                     mlp_gelu_ ? DF8_EPI_GELU : 0, act, hidden_q_);
    mlp_fc2_.forward_codes(hidden_q_.codes.data(), hidden_q_.kind, hidden_q_.scale.data(), M, DF8_EPI_RESIDUAL,
                           x1_.data(), x, nullptr);
}

template <typename T>
void TransformerBlock<T>::decode_inplace(float* x, int B) {
    const int E = embed_dim_, F = mlp_hidden_dim_;
    const df8_kind act = fp8::policy().activation_kind;
    if (x1_.numel() != size_t(B) * E) x1_ = tensor<float>({B, E});
    if (hidden_f32_.numel() != size_t(B) * F) hidden_f32_ = tensor<float>({B, F});
    fp8::PassScope amax_slots;
    norm1_.forward_quantized(x, B, act, ln_q_);
    attn_.decode_quantized(ln_q_, B, x, x1_.data());
    norm2_.forward_quantized(x1_.data(), B, act, ln_q_);
    float* am = fp8::amax_slot(amax_.data());
    mlp_fc1_.forward_codes_skinny(ln_q_.codes.data(), ln_q_.kind, ln_q_.scale.data(), B,
                                  (mlp_gelu_ ? DF8_EPI_GELU : 0) | DF8_EPI_AMAX, nullptr, hidden_f32_.data(), am);
    fp8::quantize_with_amax(hidden_f32_.data(), hidden_f32_.numel(), act, am, hidden_q_);
    mlp_fc2_.forward_codes_skinny(hidden_q_.codes.data(), hidden_q_.kind, hidden_q_.scale.data(), B, DF8_EPI_RESIDUAL,
                                  x1_.data(), x, nullptr);
}

template <typename T>
dnn::tensor<T> TransformerBlock<T>::forward(const dnn::tensor<T>& input) {
    const auto& s = input.shape();
    if (s.size() != 3) throw std::runtime_error("TransformerBlock expects input shape [B, T, E]");
    if (s[2] != embed_dim_) throw std::runtime_error("TransformerBlock: last input dimension must equal embed_dim");
    if (this->training_enabled_) input_cache_ = input.clone();
    dnn::tensor<T> out = input.clone();
    forward_inplace(out.data(), s[0], s[1]);
    if (!out.data() && out.numel())
        throw std::runtime_error("Null device pointer in TransformerBlock::forward output");
    return out;
}

// Training-side; upstream chains the (stub) backward passes of its sublayers
// (transformer_block.cu:96-160).  Not part of the fp8 inference build.
template <typename T>
dnn::tensor<T> TransformerBlock<T>::backward(const dnn::tensor<T>& /*grad_output*/) {
    if (this->training_enabled_ && !input_cache_.has_value())
        throw std::runtime_error("TransformerBlock: input_cache_ is empty in backward().");
    throw std::runtime_error("TransformerBlock::backward: the fp8 inference build has no backward pass");
}

template <typename T>
std::vector<tensor<T>*> TransformerBlock<T>::parameters() {
    std::vector<tensor<T>*> p;
    auto add = [&p](std::vector<tensor<T>*> more) { p.insert(p.end(), more.begin(), more.end()); };
    add(norm1_.parameters());
    add(norm2_.parameters());
    add(attn_.qkv_projection().parameters());
    add(attn_.out_projection().parameters());
    add(mlp_fc1_.parameters());
    add(mlp_fc2_.parameters());
    return p;
}

// Field order of upstream's inline save/load (transformer_block.cuh:37-56).
template <typename T>
void TransformerBlock<T>::save(std::ostream& out) const {
    out.write(reinterpret_cast<const char*>(&embed_dim_), sizeof(embed_dim_));
    out.write(reinterpret_cast<const char*>(&num_heads_), sizeof(num_heads_));
    out.write(reinterpret_cast<const char*>(&mlp_hidden_dim_), sizeof(mlp_hidden_dim_));
    norm1_.save(out);
    norm2_.save(out);
    attn_.save(out);
    mlp_fc1_.save(out);
    mlp_fc2_.save(out);
}

template <typename T>
void TransformerBlock<T>::load(std::istream& in) {
    in.read(reinterpret_cast<char*>(&embed_dim_), sizeof(embed_dim_));
    in.read(reinterpret_cast<char*>(&num_heads_), sizeof(num_heads_));
    in.read(reinterpret_cast<char*>(&mlp_hidden_dim_), sizeof(mlp_hidden_dim_));
    if (!in) throw std::runtime_error("TransformerBlock::load: bad header");
    norm1_.load(in);
    norm2_.load(in);
    attn_.load(in);
    mlp_fc1_.load(in);
    mlp_fc2_.load(in);
}

template class TransformerBlock<float>;

}  // namespace dnn
