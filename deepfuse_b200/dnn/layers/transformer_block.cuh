// TransformerBlock<T>: pre-LayerNorm block  x1 = x + MHA(LN1(x));  y = x1 + FC2(act(FC1(LN2(x1)))).
//
// Public surface of upstream dnn/layers/transformer_block.cuh:14-79 (constructor (embed_dim, num_heads,
// mlp_hidden_dim, training_enabled), set_mask([B,1,T,T]), forward([B,T,E]), backward, name() ==
// "TransformerBlock", initialize_all_weights, save/load in upstream's field order).  Wiring follows
// dnn/layers/transformer_block.cu:59-86.  Upstream applies NO activation between FC1 and FC2 (:79-81);
// that remains the default here, and set_mlp_gelu(true) inserts the tanh-GELU of
// dnn/layers/activation_layer.cu:9-20, fused into the FC1 epilogue (the GPT-2 model turns it on).
//
// forward() runs the fused fp8 path: LayerNorm emits fp8 codes directly, both residual additions
// happen inside GEMM epilogues (upstream: separate add kernels, transformer_block.cu:69,86), the QKV
// and FC1 GEMMs emit per-tensor-quantised fp8 codes themselves, and none of the seven
// activation clones upstream keeps (:60-83) is made unless training is enabled.
#pragma once

#include <iostream>
#include <optional>
#include <string>
#include <vector>

#include "dnn/layers/fully_connected_layer.cuh"
#include "dnn/layers/layer_norm_layer.cuh"
#include "dnn/layers/multi_head_attention.cuh"

namespace dnn {

template <typename T>
class TransformerBlock : public Layer<T> {
public:
    TransformerBlock(int embed_dim, int num_heads, int mlp_hidden_dim, bool training_enabled = false);
    ~TransformerBlock() override;

    void set_mask(dnn::tensor<T>* mask);            // additive mask [B, 1, T, T]
    void set_causal(bool causal) { attn_.set_causal(causal); }
    void set_mlp_gelu(bool on) { mlp_gelu_ = on; }  // false reproduces upstream's block
    bool mlp_gelu() const { return mlp_gelu_; }

    dnn::tensor<T> forward(const dnn::tensor<T>& input) override;
    dnn::tensor<T> backward(const dnn::tensor<T>& grad_output) override;
    std::string name() const override { return "TransformerBlock"; }

    void initialize_all_weights() {
        attn_.initialize_weights();
        mlp_fc1_.initialize_weights();
        mlp_fc2_.initialize_weights();
    }

    std::vector<tensor<T>*> parameters() override;

    void save(std::ostream& out) const override;
    void load(std::istream& in) override;

    LayerNormLayer<T>& norm1() { return norm1_; }
    LayerNormLayer<T>& norm2() { return norm2_; }
    MultiHeadAttentionLayer<T>& attention() { return attn_; }
    FullyConnectedLayer<T>& mlp_fc1() { return mlp_fc1_; }
    FullyConnectedLayer<T>& mlp_fc2() { return mlp_fc2_; }

    // In-place variant used by the model loop: x [B*T, E] fp32 is replaced by the block output.
    void forward_inplace(float* x, int B, int T_len);
    // One decode step on x [B, E] (one new token per sequence) against the attention layer's attached KV cache.
    void decode_inplace(float* x, int B);

private:
    int embed_dim_;
    int num_heads_;
    int mlp_hidden_dim_;
    bool mlp_gelu_ = false;
    LayerNormLayer<T> norm1_;
    LayerNormLayer<T> norm2_;
    MultiHeadAttentionLayer<T> attn_;
    FullyConnectedLayer<T> mlp_fc1_;
    FullyConnectedLayer<T> mlp_fc2_;
    std::optional<tensor<T>> input_cache_;
    // reused work buffers
    fp8::Quantized ln_q_, hidden_q_;
    tensor<float> x1_;
    tensor<float> hidden_f32_{{0}}, amax_{{1}};
};

}  // namespace dnn
