// A caller written the way code against the upstream project's headers is written: include paths, class and
// member names, the layer pipeline of a token-based forward up to the logits (the wiring of upstream
// dnn/models/gpt2.cu:57-83 and :126-142), a tensor subclass that reads the protected members, and
// copy-list-initialisation of a tensor from a shape (upstream's constructor is implicit,
// dnn/core/tensor.cuh:34).  It is only compiled (tests/test_api_compile.py), never run: if it stops compiling,
// the class layer has drifted from the interface it mirrors.
#include <dnn/core/cuda.cuh>
#include <dnn/core/layer.cuh>
#include <dnn/core/tensor.cuh>
#include <dnn/layers/fully_connected_layer.cuh>
#include <dnn/layers/layer_norm_layer.cuh>
#include <dnn/layers/multi_head_attention.cuh>
#include <dnn/layers/softmax_layer.cuh>
#include <dnn/layers/transformer_block.cuh>
#include <dnn/models/gpt2.cuh>
#include <dnn/tokens/positional_encoding.cuh>
#include <dnn/tokens/token_embedding.cuh>

#include <memory>
#include <stdexcept>
#include <vector>

namespace user {

// a subclass that uses the protected members the way a derived tensor type would
struct counted_tensor : dnn::tensor<float> {
    using dnn::tensor<float>::tensor;
    int elements() const { return static_cast<int>(total_size_); }
    const float* raw() const { return data_; }
    int rank() const { return static_cast<int>(shape_.size()); }
};

inline dnn::tensor<float> make_input(int b, int t, int e) {
    dnn::tensor<float> x = std::vector<int>{b, t, e};  // implicit construction from a shape
    x.fill(0.25f).reshape({b * t, e}).reshape({b, t, e});
    return x;
}

// the token pipeline with the dynamic_casts through the layer base classes
inline dnn::tensor<float> logits_of(dnn::TokenEmbedding<float>& emb, dnn::PositionalEncoding<float>& pos,
                                    std::vector<std::unique_ptr<dnn::TransformerBlock<float>>>& blocks,
                                    dnn::FullyConnectedLayer<float>& head, const std::vector<int>& ids, int hidden) {
    const int B = 1, T = static_cast<int>(ids.size());
    dnn::tensor<int> input({B, T});
    input.upload(ids.data());
    auto* embedding_layer = dynamic_cast<dnn::LayerAsymmetric<float, int>*>(&emb);
    if (!embedding_layer) throw std::runtime_error("not a LayerAsymmetric<float, int>");
    dnn::tensor<float> x = embedding_layer->forward(input);
    auto* pos_layer = dynamic_cast<dnn::Layer<float>*>(&pos);
    if (!pos_layer) throw std::runtime_error("not a Layer<float>");
    x = pos_layer->forward(x);
    for (auto& b : blocks) {
        auto* typed = dynamic_cast<dnn::Layer<float>*>(b.get());
        if (!typed) throw std::runtime_error("layer type mismatch");
        x = typed->forward(x);
    }
    x.reshape({B * T, hidden});
    return head.forward(x);
}

int use_everything() {
    dnn::Cuda cuda(0);
    dnn::StreamGuard guard(nullptr);
    counted_tensor c({2, 3});
    dnn::tensor<float> x = make_input(1, 4, 64);
    dnn::tensor<float> y = x.clone();
    y += x;
    dnn::tensor<float> z = x + y;
    dnn::tensoru8 same = (x == y);
    bool eq = x.equals(y) || x.approx_equal(y, 1e-5f);
    dnn::LayerNormLayer<float> ln(64);
    dnn::SoftmaxLayer<float> sm;
    dnn::MultiHeadAttentionLayer<float> mha(64, 2);
    dnn::tensor<float> mask({1, 1, 4, 4});
    mha.set_mask(&mask);
    dnn::tensor<float> a = mha.forward(ln.forward(x));
    dnn::TokenEmbedding<float> emb(100, 64, 16);
    dnn::PositionalEncoding<float> pos(64, 16);
    std::vector<std::unique_ptr<dnn::TransformerBlock<float>>> blocks;
    blocks.push_back(std::make_unique<dnn::TransformerBlock<float>>(64, 2, 128));
    dnn::FullyConnectedLayer<float> head(64, 100);
    dnn::tensor<float> logits = logits_of(emb, pos, blocks, head, {1, 2, 3, 4}, 64);
    dnn::Gpt2<float> model(nullptr, 100, 16, 1, 2, 64, 128);
    dnn::tensor<float> hidden = model.forward(std::vector<int>{1, 2, 3});
    std::vector<dnn::BaseLayer*> layers = model.layers();
    std::vector<dnn::tensor<float>*> params = head.parameters();
    return c.elements() + c.rank() + (c.raw() != nullptr) + int(eq) + z.size() + same.size() + a.size(0) +
           logits.size(1) + hidden.size() + int(layers.size()) + int(params.size()) + (head.name() == "FullyConnected");
}

}  // namespace user
