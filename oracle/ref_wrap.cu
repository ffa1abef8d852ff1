// C wrapper around the UPSTREAM project's own fp32 layers, compiled from the upstream sources where they lie
// (see ref_build.sh; nothing of upstream is copied into this repository).  TEST INFRASTRUCTURE ONLY: it lets a
// GPU test check the CPU oracle against outputs of the reference implementation itself, for the layers whose
// reference kernels are numerically sound: FullyConnectedLayer<float>::forward, SoftmaxLayer<float>::forward
// (T <= 1024), LayerNormLayer<float>::forward on 2-D [rows, C <= 1024] inputs, TokenEmbedding + PositionalEncoding,
// CrossEntropyLoss<float> (dense targets and class indices).
// Upstream's MultiHeadAttention / TransformerBlock / Gpt2 forward are not wrapped: they compute batch-head 0 only.
#include <dnn/core/cuda.cuh>
#include <dnn/core/tensor.cuh>
#include <dnn/layers/fully_connected_layer.cuh>
#include <dnn/layers/layer_norm_layer.cuh>
#include <dnn/layers/softmax_layer.cuh>
#include <dnn/losses/cross_entropy.cuh>
#include <dnn/tokens/positional_encoding.cuh>
#include <dnn/tokens/token_embedding.cuh>

#include <memory>
#include <string>
#include <vector>

namespace {
std::string g_err;
template <typename F>
int guarded(F&& f) {
    try {
        f();
        cudaDeviceSynchronize();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}
std::unique_ptr<dnn::Cuda> g_ctx;
void ensure_ctx() {
    if (!g_ctx) g_ctx = std::make_unique<dnn::Cuda>(0);
}
}  // namespace

extern "C" const char* ref_last_error() { return g_err.c_str(); }

extern "C" int ref_fc_forward(int in_f, int out_f, const float* w, const float* b, const float* x, int M, float* y) {
    return guarded([&] {
        ensure_ctx();
        dnn::FullyConnectedLayer<float> layer(in_f, out_f, false);
        auto p = layer.parameters();
        p[0]->upload(w);
        p[1]->upload(b);
        dnn::tensor<float> in({M, in_f});
        in.upload(x);
        dnn::tensor<float> out = layer.forward(in);
        cudaDeviceSynchronize();
        out.download(y);
    });
}

extern "C" int ref_softmax_forward(int B, int H, int T, const float* x, const float* mask, int mask_b, float* y) {
    return guarded([&] {
        ensure_ctx();
        dnn::SoftmaxLayer<float> layer(false);
        dnn::tensor<float> in({B, H, T, T});
        in.upload(x);
        std::unique_ptr<dnn::tensor<float>> m;
        if (mask) {
            m = std::make_unique<dnn::tensor<float>>(std::vector<int>{mask_b, 1, T, T});
            m->upload(mask);
            layer.set_mask(m.get());
        }
        dnn::tensor<float> out = layer.forward(in);
        cudaDeviceSynchronize();
        out.download(y);
    });
}

extern "C" int ref_layernorm_forward(int rows, int cols, const float* gamma, const float* beta, float eps,
                                     const float* x, float* y) {
    return guarded([&] {
        ensure_ctx();
        dnn::LayerNormLayer<float> layer(cols, eps, true, false);
        auto p = layer.parameters();
        p[0]->upload(gamma);
        p[1]->upload(beta);
        dnn::tensor<float> in({rows, cols});
        in.upload(x);
        dnn::tensor<float> out = layer.forward(in);
        cudaDeviceSynchronize();
        out.download(y);
    });
}

extern "C" int ref_embedding_forward(int V, int E, int max_len, const float* table, const float* bias, const int* ids,
                                     int B, int T, int add_positions, float* y) {
    return guarded([&] {
        ensure_ctx();
        dnn::TokenEmbedding<float> emb(V, E, max_len, false);
        emb.weights()->upload(table);
        emb.bias()->upload(bias);
        dnn::tensor<int> in({B, T});
        in.upload(ids);
        dnn::tensor<float> x = emb.forward(in);
        cudaDeviceSynchronize();
        if (add_positions) {
            dnn::PositionalEncoding<float> pe(E, max_len, false);
            x = pe.forward(x);
            cudaDeviceSynchronize();
        }
        x.download(y);
    });
}

// ---- files written by upstream's own save() code (for the import tests) ---------------------------------

#include <fstream>

extern "C" int ref_tensor_save_f32(const char* path, int ndim, const int* shape, const float* data) {
    return guarded([&] {
        ensure_ctx();
        dnn::tensor<float> t(std::vector<int>(shape, shape + ndim));
        t.upload(data);
        std::ofstream out(path, std::ios::binary);
        t.save(out);
    });
}

extern "C" int ref_fc_save(const char* path, int in_f, int out_f, const float* w, const float* b) {
    return guarded([&] {
        ensure_ctx();
        dnn::FullyConnectedLayer<float> layer(in_f, out_f, false);
        layer.weights()->upload(w);
        layer.bias()->upload(b);
        std::ofstream out(path, std::ios::binary);
        layer.save(out);
    });
}

extern "C" int ref_layernorm_save(const char* path, int n, const float* gamma, const float* beta) {
    return guarded([&] {
        ensure_ctx();
        dnn::LayerNormLayer<float> layer(n, 1e-5f, true, false);
        auto p = layer.parameters();
        p[0]->upload(gamma);
        p[1]->upload(beta);
        std::ofstream out(path, std::ios::binary);
        layer.save(out);
    });
}

extern "C" int ref_embedding_save(const char* path, int V, int E, int max_len, const float* table, const float* bias) {
    return guarded([&] {
        ensure_ctx();
        dnn::TokenEmbedding<float> emb(V, E, max_len, false);
        emb.weights()->upload(table);
        emb.bias()->upload(bias);
        std::ofstream out(path, std::ios::binary);
        emb.save(out);
    });
}

// Upstream's TransformerBlock, Gpt2 and tokenizer are not wrapped: every translation unit that includes
// dnn/tokens/bpe_tokenizer.cuh (gpt2.cuh does) carries the class-static `control_chars_regex`
// (bpe_tokenizer.cuh:56, "[\x00-\x1f\x7f-\x9f]"), whose construction throws std::regex_error under libstdc++ (with
// signed char the range \x7f-\x9f runs backwards) during static initialisation, i.e. a library that contains it
// aborts the process that loads it.  Their on-disk layouts are taken from the source instead
// (transformer_block.cuh:37-56, models/gpt2.cu:144-166).

// CrossEntropyLoss<float>: host logits [B,C]; dense targets [B,C] or class indices [B] (one of the two);
// mean loss to *loss and / or the gradient [B,C] to grad
extern "C" int ref_cross_entropy(int B, int C, const float* logits, const float* targets, const int* idx, float* loss,
                                 float* grad) {
    return guarded([&] {
        ensure_ctx();
        dnn::CrossEntropyLoss<float> ce;
        dnn::tensor<float> x({B, C});
        x.upload(logits);
        if (targets) {
            dnn::tensor<float> t({B, C});
            t.upload(targets);
            if (loss) *loss = ce.compute(x, t);
            if (grad) {
                dnn::tensor<float> g = ce.compute_gradient(x, t);
                cudaDeviceSynchronize();
                g.download(grad);
            }
        } else {
            dnn::tensor<int> t({B});
            t.upload(idx);
            if (loss) *loss = ce.compute(x, t);
            if (grad) {
                dnn::tensor<float> g = ce.compute_gradient(x, t);
                cudaDeviceSynchronize();
                g.download(grad);
            }
        }
    });
}


// FullyConnectedLayer<float> with training enabled: forward(x), backward(dy); host arrays, outputs may be null
extern "C" int ref_fc_backward(int in_f, int out_f, const float* w, const float* b, const float* x, int M, const float* dy,
                               float* dx, float* dw, float* db) {
    return guarded([&] {
        ensure_ctx();
        dnn::FullyConnectedLayer<float> layer(in_f, out_f, true);
        auto p = layer.parameters();
        p[0]->upload(w);
        p[1]->upload(b);
        dnn::tensor<float> in({M, in_f});
        in.upload(x);
        (void)layer.forward(in);
        dnn::tensor<float> g({M, out_f});
        g.upload(dy);
        dnn::tensor<float> gi = layer.backward(g);
        cudaDeviceSynchronize();
        if (dx) gi.download(dx);
        auto grads = layer.gradients();
        if (dw) grads[0]->download(dw);
        if (db) grads[1]->download(db);
    });
}
