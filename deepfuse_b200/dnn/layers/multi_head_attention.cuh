// MultiHeadAttentionLayer<TT>: fused-QKV projection, scaled dot-product attention per head, output
// projection; input and output [B, T, E].
//
// Public surface of upstream dnn/layers/multi_head_attention.cuh:18-66 (constructor (embed_dim, num_heads,
// training_enabled) with its argument checks, forward, backward, set_mask([B,1,T,T]), name() ==
// "MultiHeadAttention", embed_dim/num_heads/head_dim, get_last_attention/get_q_weights/get_last_q,
// initialize_weights, save, load).  Semantics are the intended ones of the class comment (:11-16):
// Q,K,V = column blocks of the QKV projection, heads = column blocks of width D, scores scaled by
// 1/sqrt(D), softmax as SoftmaxLayer, heads merged, output projection.  Upstream's launches compute
// batch-head 0 only and index Q.K^T transposed (dnn/layers/multi_head_attention.cu:262-271); those
// defects are not reproduced.
//
// The whole inner part runs in df8_attention_fp8 on fp8 codes; the [T,T] probability matrix is never
// materialised, so get_last_attention() returns an empty placeholder tensor.
#pragma once

#include <iostream>
#include <optional>
#include <string>

#include "dnn/core/fp8.cuh"
#include "dnn/core/layer.cuh"
#include "dnn/core/tensor.cuh"
#include "dnn/layers/fully_connected_layer.cuh"
#include "dnn/layers/softmax_layer.cuh"

namespace dnn {

template <typename TT>
class MultiHeadAttentionLayer : public Layer<TT> {
public:
    MultiHeadAttentionLayer(int embed_dim, int num_heads, bool training_enabled = false);
    ~MultiHeadAttentionLayer() override;

    tensor<TT> forward(const tensor<TT>& input) override;
    tensor<TT> backward(const tensor<TT>& grad_output) override;

    void set_mask(tensor<TT>* mask);  // optional additive mask [B, 1, T, T]; non-owning
    void set_causal(bool causal) { causal_ = causal; }  // addition: causal masking without a mask tensor

    std::string name() const override { return "MultiHeadAttention"; }
    int embed_dim() const { return embed_dim_; }
    int num_heads() const { return num_heads_; }
    int head_dim() const { return head_dim_; }

    tensor<TT>* get_last_attention() { return &last_attn_; }
    tensor<TT>* get_q_weights() { return qkv_proj_.weights(); }
    tensor<TT>* get_last_q() { return &last_q_; }

    void initialize_weights();
    void save(std::ostream& out) const override;
    void load(std::istream& in) override;

    FullyConnectedLayer<TT>& qkv_projection() { return qkv_proj_; }
    FullyConnectedLayer<TT>& out_projection() { return out_proj_; }

    // fp8 path used by TransformerBlock: `xq` holds the quantised block input [B*T, E];
    // out[B*T, E] = out_proj(attention(qkv_proj(xq))) (+ residual when given), fp32.
    void forward_quantized(const fp8::Quantized& xq, int B, int T, const float* residual, float* out);

    // ---- autoregressive decoding (no upstream counterpart: its forward recomputes the whole sequence) ----
    // A cache of this layer's key and value codes, [B, H, max_len, D] each, with one dequantisation factor per
    // position.  While a cache is attached, forward_quantized() also stores the K / V codes of the positions it
    // sees at rows `kv_len` .. (a prefill), and decode_quantized() runs one step: the new token's QKV (a skinny
    // product), its K / V appended at row `kv_len`, the query against all kv_len + 1 cached positions, the output
    // projection.  The owner (the model) advances kv_len after every layer has seen the positions.
    struct KvCache {
        tensor<uint8_t> k{{0}}, v{{0}};
        tensor<float> row_dq{{0}};
        int batch = 0, max_len = 0;
    };
    void attach_kv_cache(KvCache* cache) { kv_ = cache; }
    void set_kv_len(int len) { kv_len_ = len; }
    // decode_quantized reads the position from this device integer instead of kv_len (null = the host value): a
    // step's launches then do not depend on the position and can be replayed from a CUDA graph
    void set_decode_position(const int* pos_d) { pos_d_ = pos_d; }
    void decode_quantized(const fp8::Quantized& xq, int B, const float* residual, float* out);

private:
    int embed_dim_;
    int num_heads_;
    int head_dim_;
    bool use_mask_;
    bool causal_ = false;
    FullyConnectedLayer<TT> qkv_proj_;
    FullyConnectedLayer<TT> out_proj_;
    SoftmaxLayer<TT> softmax_;  // holds the mask pointer, as upstream does
    tensor<TT> last_q_, last_attn_;
    std::optional<tensor<TT>> input_cache_;
    // reused work buffers
    tensor<float> attn_f32_;
    tensor<float> amax_;
    fp8::Quantized xq_, qkvq_, attnq_;
    KvCache* kv_ = nullptr;
    int kv_len_ = 0;
    const int* pos_d_ = nullptr;
    tensor<float> qkv_f32_{{0}};
};

}  // namespace dnn
