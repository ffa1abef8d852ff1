#include "dnn/layers/multi_head_attention.cuh"

#include <cstdlib>

#include <stdexcept>

namespace dnn {

template <typename TT>
MultiHeadAttentionLayer<TT>::MultiHeadAttentionLayer(int embed_dim, int num_heads, bool training_enabled)
    : Layer<TT>(training_enabled),
      embed_dim_(embed_dim),
      num_heads_(num_heads),
      head_dim_(num_heads > 0 ? embed_dim / num_heads : 0),
      use_mask_(false),
      qkv_proj_(embed_dim > 0 ? embed_dim : 1, embed_dim > 0 ? 3 * embed_dim : 1, training_enabled),
      out_proj_(embed_dim > 0 ? embed_dim : 1, embed_dim > 0 ? embed_dim : 1, training_enabled),
      softmax_(training_enabled),
      last_q_({1, 1}),
      last_attn_({1, 1}),
      attn_f32_({1}),
      amax_({2}) {
    if (embed_dim <= 0 || num_heads <= 0) throw std::runtime_error("embed_dim and num_heads must be positive");
    if (embed_dim % num_heads != 0) throw std::runtime_error("embed_dim must be divisible by num_heads");
}

template <typename TT>
MultiHeadAttentionLayer<TT>::~MultiHeadAttentionLayer() = default;

template <typename TT>
void MultiHeadAttentionLayer<TT>::set_mask(tensor<TT>* mask) {
    if (mask && (mask->shape().size() != 4 || mask->shape()[1] != 1))
        throw std::runtime_error("Mask must be 4D tensor with shape [B, 1, T, T]");
    softmax_.set_mask(mask);
    use_mask_ = mask != nullptr;
}

template <typename TT>
void MultiHeadAttentionLayer<TT>::initialize_weights() {
    qkv_proj_.initialize_weights();
    out_proj_.initialize_weights();
}

template <typename TT>
void MultiHeadAttentionLayer<TT>::forward_quantized(const fp8::Quantized& xq, int B, int T, const float* residual,
                                                    float* out) {
    const int M = B * T, E = embed_dim_;
    const df8_kind act = fp8::policy().activation_kind;
    if (attn_f32_.numel() != size_t(M) * E) attn_f32_ = tensor<float>({M, E});

    // QKV projection straight to per-tensor-quantised codes (the fp32 [M,3E] tensor is never written)
    qkv_proj_.forward_codes_quantized(xq.codes.data(), xq.kind, xq.scale.data(), M, 0, act, qkvq_);

    if (kv_) {  // a prefill: keep the keys and values of these positions for the decode steps
        if (B != kv_->batch || kv_len_ + T > kv_->max_len)
            throw std::runtime_error("MultiHeadAttentionLayer: the attached KV cache does not fit this batch / length");
        utils::CHECK_DF8(df8_kv_cache_append(qkvq_.codes.data(), qkvq_.scale.data(), B, T, num_heads_, head_dim_, kv_len_,
                                             kv_->max_len, kv_->k.data(), kv_->v.data(), kv_->row_dq.data(), fp8::stream()));
    }
    int mode = causal_ ? DF8_MASK_CAUSAL : DF8_MASK_NONE;
    const float* mask_ptr = nullptr;
    int mask_b = 0;
    if (tensor<TT>* m = softmax_.mask()) {
        const auto& ms = m->shape();
        if (ms[2] != T || ms[3] != T || (ms[0] != B && ms[0] != 1))
            throw std::runtime_error("Mask must be 4D tensor with shape [B, 1, T, T]");
        mode = DF8_MASK_ADDITIVE;
        mask_ptr = m->data();
        mask_b = ms[0];
    }
    float* am = fp8::amax_slot(amax_.data());
    utils::CHECK_DF8(df8_attention_fp8(qkvq_.codes.data(), qkvq_.kind, qkvq_.scale.data(), B, T, num_heads_, head_dim_,
                                       mode, mask_ptr, mask_b, attn_f32_.data(), am, fp8::stream()));
    fp8::quantize_with_amax(attn_f32_.data(), attn_f32_.numel(), act, am, attnq_);
    out_proj_.forward_codes(attnq_.codes.data(), attnq_.kind, attnq_.scale.data(), M,
                            residual ? DF8_EPI_RESIDUAL : 0, residual, out, nullptr);
}

template <typename TT>
void MultiHeadAttentionLayer<TT>::decode_quantized(const fp8::Quantized& xq, int B, const float* residual, float* out) {
    if (!kv_) throw std::runtime_error("MultiHeadAttentionLayer::decode_quantized: no KV cache attached");
    if (B != kv_->batch || kv_len_ + 1 > kv_->max_len)
        throw std::runtime_error("MultiHeadAttentionLayer::decode_quantized: the KV cache is full or of another batch size");
    const int E = embed_dim_;
    const df8_kind act = fp8::policy().activation_kind;
    if (qkv_f32_.numel() != size_t(B) * 3 * E) qkv_f32_ = tensor<float>({B, 3 * E});
    if (attn_f32_.numel() != size_t(B) * E) attn_f32_ = tensor<float>({B, E});
    // the new token's QKV, quantised per tensor like every QKV tensor of the 8-bit path
    float* am = fp8::amax_slot(amax_.data());
    qkv_proj_.forward_codes_skinny(xq.codes.data(), xq.kind, xq.scale.data(), B, DF8_EPI_AMAX, nullptr, qkv_f32_.data(), am);
    const char* unfused = getenv("DF8_DECODE_UNFUSED");
    if (unfused && unfused[0] == '1') {
        fp8::quantize_with_amax(qkv_f32_.data(), qkv_f32_.numel(), act, am, qkvq_);
        utils::CHECK_DF8(df8_kv_cache_append_pos(qkvq_.codes.data(), qkvq_.scale.data(), B, num_heads_, head_dim_, pos_d_,
                                                 kv_->max_len, kv_->k.data(), kv_->v.data(), kv_->row_dq.data(), fp8::stream()));
        float* amu = fp8::amax_slot(amax_.data() + 1);
        utils::CHECK_DF8(df8_attention_decode_fp8_pos(qkvq_.codes.data(), qkvq_.kind, qkvq_.scale.data(), kv_->k.data(),
                                                      kv_->v.data(), kv_->row_dq.data(), B, num_heads_, head_dim_, kv_len_ + 1,
                                                      pos_d_, kv_->max_len, attn_f32_.data(), amu, fp8::stream()));
        fp8::quantize_with_amax(attn_f32_.data(), attn_f32_.numel(), act, amu, attnq_);
        out_proj_.forward_codes_skinny(attnq_.codes.data(), attnq_.kind, attnq_.scale.data(), B,
                                       residual ? DF8_EPI_RESIDUAL : 0, residual, out, nullptr);
        return;
    }
    // quantise + cache append + attention in one launch (the codes are those of quantize_with_amax)
    float* am2 = fp8::amax_slot(amax_.data() + 1);  // read and written by the same launch: never the slot of `am`
    utils::CHECK_DF8(df8_attention_decode_fused_f32(qkv_f32_.data(), am, act, kv_->k.data(), kv_->v.data(),
                                                    kv_->row_dq.data(), B, num_heads_, head_dim_, kv_len_ + 1, pos_d_,
                                                    kv_->max_len, attn_f32_.data(), am2, fp8::stream()));
    fp8::quantize_with_amax(attn_f32_.data(), attn_f32_.numel(), act, am2, attnq_);
    out_proj_.forward_codes_skinny(attnq_.codes.data(), attnq_.kind, attnq_.scale.data(), B,
                                   residual ? DF8_EPI_RESIDUAL : 0, residual, out, nullptr);
}

template <typename TT>
tensor<TT> MultiHeadAttentionLayer<TT>::forward(const tensor<TT>& input) {
    const auto& shape = input.shape();
    if (shape.size() != 3) throw std::runtime_error("Input tensor must be 3D [B, T, E]");
    if (shape[2] != embed_dim_) throw std::runtime_error("Input tensor's last dimension must equal embed_dim");
    if (this->training_enabled_) input_cache_ = input.clone();
    const int B = shape[0], T = shape[1];
    fp8::quantize(input.data(), input.numel(), fp8::policy().activation_kind, xq_);
    tensor<TT> out(shape);
    forward_quantized(xq_, B, T, nullptr, out.data());
    return out;
}

// Upstream's backward is an identity stub (multi_head_attention.cu:310-319); kept.
template <typename TT>
tensor<TT> MultiHeadAttentionLayer<TT>::backward(const tensor<TT>& grad_output) {
    return grad_output.clone();
}

template <typename TT>
void MultiHeadAttentionLayer<TT>::save(std::ostream& out) const {
    out.write(reinterpret_cast<const char*>(&embed_dim_), sizeof(embed_dim_));
    out.write(reinterpret_cast<const char*>(&num_heads_), sizeof(num_heads_));
    qkv_proj_.save(out);
    out_proj_.save(out);
}

template <typename TT>
void MultiHeadAttentionLayer<TT>::load(std::istream& in) {
    int e = 0, h = 0;
    in.read(reinterpret_cast<char*>(&e), sizeof(e));
    in.read(reinterpret_cast<char*>(&h), sizeof(h));
    if (!in || e <= 0 || h <= 0 || e % h != 0) throw std::runtime_error("MultiHeadAttentionLayer::load: bad header");
    embed_dim_ = e;
    num_heads_ = h;
    head_dim_ = e / h;
    qkv_proj_.load(in);
    out_proj_.load(in);
}

template class MultiHeadAttentionLayer<float>;

}  // namespace dnn
