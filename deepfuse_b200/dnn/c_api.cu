// C harness over the dnn:: classes (declared in include/df8_dnn.h).  Every function builds and calls
// the C++ objects through their public members and converts exceptions into a return code.
#include "df8_dnn.h"

#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "dnn/core/cuda.cuh"
#include "dnn/core/fp8.cuh"
#include "dnn/layers/fully_connected_layer.cuh"
#include "dnn/layers/layer_norm_layer.cuh"
#include "dnn/layers/multi_head_attention.cuh"
#include "dnn/layers/softmax_layer.cuh"
#include "dnn/layers/transformer_block.cuh"
#include "dnn/losses/cross_entropy.cuh"
#include "dnn/models/gpt2.cuh"
#include "dnn/models/gpt2_column_sharded.cuh"
#include "dnn/tokens/bpe_tokenizer.cuh"
#include "dnn/tokens/positional_encoding.cuh"
#include "dnn/tokens/token_embedding.cuh"
#include "dnn/tokens/vocab_loader.cuh"

#include <fstream>

namespace {

thread_local std::string t_error;
thread_local std::unique_ptr<dnn::Cuda> t_context;

template <typename F>
int guarded(F&& body) {
    try {
        body();
        return 0;
    } catch (const std::invalid_argument& e) {
        t_error = std::string("invalid_argument: ") + e.what();
        return 2;
    } catch (const std::out_of_range& e) {
        t_error = std::string("out_of_range: ") + e.what();
        return 3;
    } catch (const std::exception& e) {
        t_error = std::string("runtime_error: ") + e.what();
        return 1;
    }
}

void sync_stream() { dnn::utils::CHECK_CUDA_EX(cudaStreamSynchronize(dnn::Cuda::stream())); }

struct NamedParam {
    std::string name;
    dnn::tensor<float>* t;
};

}  // namespace

struct dnn_gpt2 {
    std::unique_ptr<dnn::Gpt2<float>> model;
    std::vector<NamedParam> params;
    std::unique_ptr<dnn::tensor<float>> last;  // result of the last forward, kept alive for the caller
    std::unique_ptr<dnn::tensor<int>> ids;
    // dnn_gpt2_serve_step: the logits of the step before the last stay alive while the copy stream reads them
    std::unique_ptr<dnn::tensor<float>> prev;
    std::unique_ptr<dnn::tensor<int>> serve_ids[2];
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_forward = nullptr, ev_copied[2] = {nullptr, nullptr};
    unsigned long long serve_steps = 0;
    ~dnn_gpt2() {
        if (copy_stream) {
            cudaStreamSynchronize(copy_stream);
            cudaStreamDestroy(copy_stream);
        }
        if (ev_forward) cudaEventDestroy(ev_forward);
        for (cudaEvent_t e : ev_copied)
            if (e) cudaEventDestroy(e);
    }

    void index_params() {
        params.clear();
        auto add = [this](const std::string& prefix, dnn::tensor<float>* w, dnn::tensor<float>* b,
                          const char* wn = "weight", const char* bn = "bias") {
            params.push_back({prefix + "." + wn, w});
            params.push_back({prefix + "." + bn, b});
        };
        add("embedding", model->token_embedding().weights(), model->token_embedding().bias());
        for (int i = 0; i < model->num_layers(); ++i) {
            auto& blk = model->block(i);
            const std::string p = "block" + std::to_string(i);
            auto n1 = blk.norm1().parameters();
            auto n2 = blk.norm2().parameters();
            add(p + ".ln1", n1[0], n1[1], "gamma", "beta");
            add(p + ".ln2", n2[0], n2[1], "gamma", "beta");
            add(p + ".qkv", blk.attention().qkv_projection().weights(), blk.attention().qkv_projection().bias());
            add(p + ".out", blk.attention().out_projection().weights(), blk.attention().out_projection().bias());
            add(p + ".fc1", blk.mlp_fc1().weights(), blk.mlp_fc1().bias());
            add(p + ".fc2", blk.mlp_fc2().weights(), blk.mlp_fc2().bias());
        }
        add("final_fc", model->final_fc().weights(), model->final_fc().bias());
    }
};

extern "C" const char* dnn_last_error(void) { return t_error.c_str(); }

extern "C" int dnn_init(int device) {
    return guarded([&] {
        if (!t_context || t_context->id() != device) {
            t_context.reset();
            t_context = std::make_unique<dnn::Cuda>(device);
        }
    });
}

extern "C" int dnn_set_stream(void* stream) {
    return guarded([&] { dnn::Cuda::set_stream(reinterpret_cast<cudaStream_t>(stream)); });
}

extern "C" int dnn_set_fp8_policy(int weight_kind, int activation_kind) {
    return guarded([&] {
        if ((weight_kind != 0 && weight_kind != 1) || (activation_kind != 0 && activation_kind != 1))
            throw std::invalid_argument("fp8 kind must be 0 (e4m3) or 1 (e5m2)");
        dnn::fp8::policy().weight_kind = df8_kind(weight_kind);
        dnn::fp8::policy().activation_kind = df8_kind(activation_kind);
    });
}

extern "C" int dnn_set_host_init(int enabled) {
    return guarded([&] { dnn::fp8::policy().host_init = enabled != 0; });
}

// ---- Gpt2 -------------------------------------------------------------------------------------

extern "C" dnn_gpt2* dnn_gpt2_create(int vocab, int max_seq_len, int layers, int heads, int hidden, int ffn) {
    dnn_gpt2* h = nullptr;
    int rc = guarded([&] {
        auto handle = std::make_unique<dnn_gpt2>();
        handle->model = std::make_unique<dnn::Gpt2<float>>(nullptr, vocab, max_seq_len, layers, heads, hidden, ffn);
        handle->index_params();
        h = handle.release();
    });
    return rc == 0 ? h : nullptr;
}

extern "C" void dnn_gpt2_destroy(dnn_gpt2* m) {
    guarded([&] {
        if (m) sync_stream();
        delete m;
    });
}

extern "C" int dnn_gpt2_set_options(dnn_gpt2* m, int mlp_gelu, int causal) {
    return guarded([&] {
        m->model->set_mlp_gelu(mlp_gelu != 0);
        m->model->set_causal(causal != 0);
    });
}

extern "C" int dnn_gpt2_num_params(dnn_gpt2* m) { return m ? int(m->params.size()) : -1; }

extern "C" int dnn_gpt2_param_info(dnn_gpt2* m, int index, char* name_h, int name_cap, int* shape_h, int* ndim_h) {
    return guarded([&] {
        const NamedParam& p = m->params.at(size_t(index));
        if (name_h && name_cap > 0) std::snprintf(name_h, size_t(name_cap), "%s", p.name.c_str());
        const auto& s = p.t->shape();
        if (ndim_h) *ndim_h = int(s.size());
        if (shape_h)
            for (size_t i = 0; i < s.size() && i < 8; ++i) shape_h[i] = s[i];
    });
}

extern "C" int dnn_gpt2_param_upload(dnn_gpt2* m, int index, const float* data_h) {
    return guarded([&] {
        m->params.at(size_t(index)).t->upload(data_h);
        sync_stream();
    });
}

extern "C" int dnn_gpt2_param_download(dnn_gpt2* m, int index, float* data_h) {
    return guarded([&] { m->params.at(size_t(index)).t->download(data_h); });
}

extern "C" int dnn_gpt2_initialize_on_device(dnn_gpt2* m, unsigned long long seed, float std) {
    return guarded([&] {
        m->model->initialize_on_device(seed, std);
        sync_stream();
    });
}

extern "C" int dnn_gpt2_set_stage_timing(dnn_gpt2* m, int on) {
    return guarded([&] { m->model->set_stage_timing(on != 0); });
}

extern "C" int dnn_gpt2_last_head_ms(dnn_gpt2* m, float* ms_h) {
    return guarded([&] { *ms_h = m->model->last_head_ms(); });
}

extern "C" int dnn_gpt2_prepare(dnn_gpt2* m) {
    return guarded([&] {
        for (int i = 0; i < m->model->num_layers(); ++i) {
            auto& blk = m->model->block(i);
            blk.attention().qkv_projection().quantized_weights();
            blk.attention().out_projection().quantized_weights();
            blk.mlp_fc1().quantized_weights();
            blk.mlp_fc2().quantized_weights();
        }
        m->model->final_fc().quantized_weights();
        sync_stream();
    });
}

namespace {
void stage_ids(dnn_gpt2* m, const int32_t* src, int B, int T, cudaMemcpyKind kind) {
    if (!m->ids || m->ids->shape() != std::vector<int>{B, T}) m->ids = std::make_unique<dnn::tensor<int>>(std::vector<int>{B, T});
    dnn::utils::CHECK_CUDA_EX(cudaMemcpyAsync(m->ids->data(), src, sizeof(int32_t) * size_t(B) * size_t(T), kind,
                                              dnn::Cuda::stream()));
}
}  // namespace

extern "C" int dnn_gpt2_forward_logits(dnn_gpt2* m, const int32_t* ids_d, int B, int T, int check_ids,
                                       float** logits_d) {
    return guarded([&] {
        stage_ids(m, ids_d, B, T, cudaMemcpyDeviceToDevice);
        m->last.reset();  // return the previous result to the pool before allocating the next one
        m->last = std::make_unique<dnn::tensor<float>>(m->model->forward_logits(*m->ids, check_ids != 0));
        *logits_d = m->last->data();
    });
}

extern "C" int dnn_gpt2_forward_logits_host(dnn_gpt2* m, const int32_t* ids_h, int B, int T, float** logits_d) {
    return guarded([&] {
        stage_ids(m, ids_h, B, T, cudaMemcpyHostToDevice);
        m->last.reset();
        m->last = std::make_unique<dnn::tensor<float>>(m->model->forward_logits(*m->ids, false));
        *logits_d = m->last->data();
    });
}

extern "C" int dnn_gpt2_forward_logits_pitched(dnn_gpt2* m, const int32_t* ids, int ids_on_host, int B, int T,
                                               int check_ids, float** logits_d, int* pitch_h) {
    return guarded([&] {
        stage_ids(m, ids, B, T, ids_on_host ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice);
        m->last.reset();
        m->last = std::make_unique<dnn::tensor<float>>(m->model->forward_logits_pitched(*m->ids, check_ids != 0));
        *logits_d = m->last->data();
        if (pitch_h) *pitch_h = m->model->logits_pitch();
    });
}

extern "C" int dnn_gpt2_copy_logits_host(dnn_gpt2* m, float* dst_h) {
    return guarded([&] {
        if (!m->last || m->last->shape().size() != 2) throw std::runtime_error("dnn_gpt2_copy_logits_host: no logits to copy");
        const int rows = m->last->shape()[0], pitch = m->last->shape()[1];
        const int vocab = m->model->vocab_size();
        if (pitch < vocab) throw std::runtime_error("dnn_gpt2_copy_logits_host: the last result is not a logits tensor");
        dnn::utils::CHECK_CUDA_EX(cudaMemcpy2DAsync(dst_h, size_t(vocab) * sizeof(float), m->last->data(),
                                                    size_t(pitch) * sizeof(float), size_t(vocab) * sizeof(float),
                                                    size_t(rows), cudaMemcpyDeviceToHost, dnn::Cuda::stream()));
    });
}

// A serving loop's step: host ids in, the full logits out to (pinned) host memory -- with the device-to-host copy
// of step i on a stream of its own, so that it runs under the forward of step i + 1 (1.65 GB of logits take 29 ms
// over PCIe, a forward 3.3 ms: issued on one stream the two add up).  Two logits tensors and two id buffers alternate.
// dst_h must stay untouched until the next-but-one call or dnn_gpt2_serve_flush.
extern "C" int dnn_gpt2_serve_step(dnn_gpt2* m, const int32_t* ids_h, int B, int T, float* dst_h) {
    return guarded([&] {
        cudaStream_t cs = dnn::Cuda::stream();
        if (!m->copy_stream) {
            dnn::utils::CHECK_CUDA_EX(cudaStreamCreateWithFlags(&m->copy_stream, cudaStreamNonBlocking));
            dnn::utils::CHECK_CUDA_EX(cudaEventCreateWithFlags(&m->ev_forward, cudaEventDisableTiming));
            for (cudaEvent_t& e : m->ev_copied) dnn::utils::CHECK_CUDA_EX(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        }
        const int slot = int(m->serve_steps & 1);
        // the tensor that held the logits two steps ago goes back to the pool: its copy must be over (stream order)
        if (m->serve_steps >= 2) dnn::utils::CHECK_CUDA_EX(cudaStreamWaitEvent(cs, m->ev_copied[slot], 0));
        m->prev.reset();
        m->prev = std::move(m->last);
        auto& ids = m->serve_ids[slot];
        if (!ids || ids->shape() != std::vector<int>{B, T}) ids = std::make_unique<dnn::tensor<int>>(std::vector<int>{B, T});
        dnn::utils::CHECK_CUDA_EX(cudaMemcpyAsync(ids->data(), ids_h, sizeof(int32_t) * size_t(B) * size_t(T), cudaMemcpyHostToDevice, cs));
        m->last = std::make_unique<dnn::tensor<float>>(m->model->forward_logits_pitched(*ids, false));
        dnn::utils::CHECK_CUDA_EX(cudaEventRecord(m->ev_forward, cs));
        dnn::utils::CHECK_CUDA_EX(cudaStreamWaitEvent(m->copy_stream, m->ev_forward, 0));
        const int rows = m->last->shape()[0], pitch = m->last->shape()[1], vocab = m->model->vocab_size();
        dnn::utils::CHECK_CUDA_EX(cudaMemcpy2DAsync(dst_h, size_t(vocab) * sizeof(float), m->last->data(), size_t(pitch) * sizeof(float),
                                        size_t(vocab) * sizeof(float), size_t(rows), cudaMemcpyDeviceToHost, m->copy_stream));
        dnn::utils::CHECK_CUDA_EX(cudaEventRecord(m->ev_copied[slot], m->copy_stream));
        ++m->serve_steps;
    });
}

// The calling thread's stream waits for every copy dnn_gpt2_serve_step has issued (no host synchronisation).
extern "C" int dnn_gpt2_serve_flush(dnn_gpt2* m) {
    return guarded([&] {
        if (!m->copy_stream) return;
        for (cudaEvent_t e : m->ev_copied)
            dnn::utils::CHECK_CUDA_EX(cudaStreamWaitEvent(dnn::Cuda::stream(), e, 0));
    });
}

extern "C" int dnn_gpt2_forward_hidden(dnn_gpt2* m, const int32_t* ids_d, int B, int T, float** hidden_d) {
    return guarded([&] {
        stage_ids(m, ids_d, B, T, cudaMemcpyDeviceToDevice);
        m->last.reset();
        m->last = std::make_unique<dnn::tensor<float>>(m->model->forward_hidden(*m->ids, true));
        *hidden_d = m->last->data();
    });
}

extern "C" int dnn_gpt2_forward_ids(dnn_gpt2* m, const int32_t* ids_h, int T, float* hidden_h) {
    return guarded([&] {
        std::vector<int> ids(ids_h, ids_h + T);
        dnn::tensor<float> hidden = m->model->forward(ids);
        hidden.download(hidden_h);
    });
}

extern "C" int dnn_gpt2_save(dnn_gpt2* m, const char* path) {
    return guarded([&] { m->model->save(path); });
}

extern "C" dnn_gpt2* dnn_gpt2_load(const char* path) {
    dnn_gpt2* h = nullptr;
    int rc = guarded([&] {
        auto handle = std::make_unique<dnn_gpt2>();
        handle->model = dnn::Gpt2<float>::load(path, false);
        handle->index_params();
        h = handle.release();
    });
    return rc == 0 ? h : nullptr;
}

// ---- single layers through their public forward() ------------------------------------------------

extern "C" int dnn_fc_forward(int in_features, int out_features, const float* w_h, const float* b_h,
                              const float* x_h, int M, float* y_h) {
    return guarded([&] {
        dnn::FullyConnectedLayer<float> layer(in_features, out_features);
        auto params = layer.parameters();
        if (w_h) params[0]->upload(w_h);
        if (b_h) params[1]->upload(b_h);
        dnn::tensor<float> x({M, in_features});
        x.upload(x_h);
        dnn::tensor<float> y = layer.forward(x);
        y.download(y_h);
    });
}

// FullyConnectedLayer with training enabled: forward on x_h, then backward on dy_h; all arrays on the host
extern "C" int dnn_fc_backward(int in_features, int out_features, const float* w_h, const float* b_h, const float* x_h,
                               int M, const float* dy_h, float* dx_h, float* dw_h, float* db_h) {
    return guarded([&] {
        dnn::FullyConnectedLayer<float> layer(in_features, out_features, true);
        auto params = layer.parameters();
        if (w_h) params[0]->upload(w_h);
        if (b_h) params[1]->upload(b_h);
        dnn::tensor<float> x({M, in_features});
        x.upload(x_h);
        (void)layer.forward(x);
        dnn::tensor<float> dy({M, out_features});
        dy.upload(dy_h);
        dnn::tensor<float> dx = layer.backward(dy);
        if (dx_h) dx.download(dx_h);
        auto grads = layer.gradients();
        if (dw_h) grads[0]->download(dw_h);
        if (db_h) grads[1]->download(db_h);
    });
}

extern "C" int dnn_layernorm_forward(int rows, int cols, const float* gamma_h, const float* beta_h, float eps,
                                     const float* x_h, float* y_h) {
    return guarded([&] {
        dnn::LayerNormLayer<float> layer(cols, eps, gamma_h != nullptr);
        if (gamma_h) {
            auto p = layer.parameters();
            p[0]->upload(gamma_h);
            if (beta_h) p[1]->upload(beta_h);
        }
        dnn::tensor<float> x({rows, cols});
        x.upload(x_h);
        dnn::tensor<float> y = layer.forward(x);
        y.download(y_h);
    });
}

extern "C" int dnn_softmax_forward(int B, int H, int T, const float* x_h, const float* mask_h, int mask_b,
                                   float* y_h) {
    return guarded([&] {
        dnn::SoftmaxLayer<float> layer;
        dnn::tensor<float> x({B, H, T, T});
        x.upload(x_h);
        std::unique_ptr<dnn::tensor<float>> mask;
        if (mask_h) {
            mask = std::make_unique<dnn::tensor<float>>(std::vector<int>{mask_b, 1, T, T});
            mask->upload(mask_h);
            layer.set_mask(mask.get());
        }
        dnn::tensor<float> y = layer.forward(x);
        y.download(y_h);
    });
}

extern "C" int dnn_mha_forward(int B, int T, int E, int H, const float* wqkv_h, const float* bqkv_h,
                               const float* wo_h, const float* bo_h, const float* x_h, int mask_mode,
                               const float* mask_h, int mask_b, float* y_h) {
    return guarded([&] {
        dnn::MultiHeadAttentionLayer<float> layer(E, H);
        layer.qkv_projection().weights()->upload(wqkv_h);
        layer.qkv_projection().bias()->upload(bqkv_h);
        layer.out_projection().weights()->upload(wo_h);
        layer.out_projection().bias()->upload(bo_h);
        std::unique_ptr<dnn::tensor<float>> mask;
        if (mask_mode == 1) layer.set_causal(true);
        if (mask_mode == 2) {
            mask = std::make_unique<dnn::tensor<float>>(std::vector<int>{mask_b, 1, T, T});
            mask->upload(mask_h);
            layer.set_mask(mask.get());
        }
        dnn::tensor<float> x({B, T, E});
        x.upload(x_h);
        dnn::tensor<float> y = layer.forward(x);
        y.download(y_h);
    });
}

extern "C" int dnn_embedding_forward(int V, int E, int max_len, const float* table_h, const float* bias_h,
                                     const int32_t* ids_h, int B, int T, int add_positions, float* y_h) {
    return guarded([&] {
        dnn::TokenEmbedding<float> emb(V, E, max_len);
        if (table_h) emb.weights()->upload(table_h);
        if (bias_h) emb.bias()->upload(bias_h);
        dnn::tensor<int> ids({B, T});
        ids.upload(ids_h);
        dnn::tensor<float> x = emb.forward(ids);
        if (add_positions) {
            dnn::PositionalEncoding<float> pe(E, max_len);
            x = pe.forward(x);
        }
        x.download(y_h);
    });
}

// One TransformerBlock through its public forward(); params in the order of TransformerBlock::parameters()
// (ln1 g,b; ln2 g,b; qkv W,b; out W,b; fc1 W,b; fc2 W,b), each a host array.
extern "C" int dnn_block_forward(int B, int T, int E, int H, int F, const float* const* params_h, int n_params,
                                 int mlp_gelu, int causal, const float* x_h, float* y_h) {
    return guarded([&] {
        dnn::TransformerBlock<float> block(E, H, F);
        auto params = block.parameters();
        if (int(params.size()) != n_params) throw std::invalid_argument("dnn_block_forward: expected 12 parameter arrays");
        for (int i = 0; i < n_params; ++i) params[size_t(i)]->upload(params_h[i]);
        block.set_mlp_gelu(mlp_gelu != 0);
        block.set_causal(causal != 0);
        dnn::tensor<float> x({B, T, E});
        x.upload(x_h);
        dnn::tensor<float> y = block.forward(x);
        y.download(y_h);
    });
}

// ---- layer streaming ---------------------------------------------------------------------------

extern "C" int dnn_gpt2_enable_streaming(dnn_gpt2* m, int slots, int release_fp32) {
    return guarded([&] {
        m->model->enable_layer_streaming(slots, release_fp32 != 0);
        sync_stream();
    });
}

extern "C" int dnn_gpt2_enable_streaming_sharded(dnn_gpt2* m, int slots, int release_fp32, void* comm) {
    return guarded([&] {
        m->model->enable_layer_streaming(slots, release_fp32 != 0, static_cast<df8_comm*>(comm));
        sync_stream();
    });
}

extern "C" int dnn_gpt2_resize_streaming_slots(dnn_gpt2* m, int slots) {
    return guarded([&] { m->model->resize_streaming_slots(slots); });
}

extern "C" int dnn_gpt2_streaming_traffic(dnn_gpt2* m, unsigned long long* h2d_bytes_h, unsigned long long* gathered_bytes_h) {
    return guarded([&] { m->model->streaming_traffic(h2d_bytes_h, gathered_bytes_h); });
}

extern "C" int dnn_gpt2_time_layer_uploads(dnn_gpt2* m, float* ms_h) {
    return guarded([&] { *ms_h = m->model->time_layer_uploads(); });
}

extern "C" int dnn_gpt2_disable_streaming(dnn_gpt2* m) {
    return guarded([&] { m->model->disable_layer_streaming(); });
}

extern "C" unsigned long long dnn_gpt2_streamed_bytes(dnn_gpt2* m) { return m ? m->model->streamed_bytes() : 0ull; }


// ---- Gpt2ColumnSharded ---------------------------------------------------------------------------

struct dnn_gpt2cs {
    std::unique_ptr<dnn::Gpt2ColumnSharded<float>> model;
    std::vector<NamedParam> params;
    std::unique_ptr<dnn::tensor<float>> last;
    std::unique_ptr<dnn::tensor<int>> ids;

    void index_params() {
        params.clear();
        auto add = [this](const std::string& prefix, dnn::tensor<float>* w, dnn::tensor<float>* b,
                          const char* wn = "weight", const char* bn = "bias") {
            params.push_back({prefix + "." + wn, w});
            params.push_back({prefix + "." + bn, b});
        };
        add("embedding", model->token_embedding().weights(), model->token_embedding().bias());
        for (int i = 0; i < model->num_layers(); ++i) {
            auto& blk = model->block(i);
            const std::string p = "block" + std::to_string(i);
            auto n1 = blk.norm1.parameters();
            auto n2 = blk.norm2.parameters();
            add(p + ".ln1", n1[0], n1[1], "gamma", "beta");
            add(p + ".ln2", n2[0], n2[1], "gamma", "beta");
            add(p + ".qkv", blk.qkv.weights(), blk.qkv.bias());
            add(p + ".out", blk.out.weights(), blk.out.bias());
            add(p + ".fc1", blk.fc1.weights(), blk.fc1.bias());
            add(p + ".fc2", blk.fc2.weights(), blk.fc2.bias());
        }
        add("final_fc", model->final_fc().weights(), model->final_fc().bias());
    }
    void stage_ids(const int32_t* src, int B, int T, cudaMemcpyKind kind) {
        if (!ids || ids->shape() != std::vector<int>{B, T}) ids = std::make_unique<dnn::tensor<int>>(std::vector<int>{B, T});
        dnn::utils::CHECK_CUDA_EX(cudaMemcpyAsync(ids->data(), src, sizeof(int32_t) * size_t(B) * size_t(T), kind,
                                                  dnn::Cuda::stream()));
    }
};

extern "C" dnn_gpt2cs* dnn_gpt2cs_create(void* comm, int vocab, int max_seq_len, int layers, int heads, int hidden,
                                         int ffn) {
    dnn_gpt2cs* h = nullptr;
    int rc = guarded([&] {
        auto handle = std::make_unique<dnn_gpt2cs>();
        handle->model = std::make_unique<dnn::Gpt2ColumnSharded<float>>(static_cast<df8_comm*>(comm), vocab, max_seq_len,
                                                                        layers, heads, hidden, ffn);
        handle->index_params();
        h = handle.release();
    });
    return rc == 0 ? h : nullptr;
}

extern "C" void dnn_gpt2cs_destroy(dnn_gpt2cs* m) {
    guarded([&] {
        if (m) sync_stream();
        delete m;
    });
}

extern "C" int dnn_gpt2cs_set_options(dnn_gpt2cs* m, int mlp_gelu, int causal) {
    return guarded([&] {
        m->model->set_mlp_gelu(mlp_gelu != 0);
        m->model->set_causal(causal != 0);
    });
}

extern "C" int dnn_gpt2cs_vocab_range(dnn_gpt2cs* m, int* begin_h, int* rows_h) {
    return guarded([&] {
        if (begin_h) *begin_h = m->model->vocab_begin();
        if (rows_h) *rows_h = m->model->vocab_rows();
    });
}

extern "C" int dnn_gpt2cs_num_params(dnn_gpt2cs* m) { return m ? int(m->params.size()) : -1; }

extern "C" int dnn_gpt2cs_param_info(dnn_gpt2cs* m, int index, char* name_h, int name_cap, int* shape_h, int* ndim_h) {
    return guarded([&] {
        const NamedParam& p = m->params.at(size_t(index));
        if (name_h && name_cap > 0) std::snprintf(name_h, size_t(name_cap), "%s", p.name.c_str());
        const auto& s = p.t->shape();
        if (ndim_h) *ndim_h = int(s.size());
        if (shape_h)
            for (size_t i = 0; i < s.size() && i < 8; ++i) shape_h[i] = s[i];
    });
}

extern "C" int dnn_gpt2cs_param_upload(dnn_gpt2cs* m, int index, const float* data_h) {
    return guarded([&] {
        m->params.at(size_t(index)).t->upload(data_h);
        sync_stream();
    });
}

extern "C" int dnn_gpt2cs_initialize_on_device(dnn_gpt2cs* m, unsigned long long seed) {
    return guarded([&] {
        m->model->initialize_on_device(seed);
        sync_stream();
    });
}

extern "C" int dnn_gpt2cs_prepare(dnn_gpt2cs* m) {
    return guarded([&] {
        for (int i = 0; i < m->model->num_layers(); ++i) {
            auto& blk = m->model->block(i);
            blk.qkv.quantized_weights();
            blk.out.quantized_weights();
            blk.fc1.quantized_weights();
            blk.fc2.quantized_weights();
        }
        m->model->final_fc().quantized_weights();
        sync_stream();
    });
}

extern "C" int dnn_gpt2cs_forward_logits_shard(dnn_gpt2cs* m, const int32_t* ids_d, int B, int T, int check_ids,
                                               float** logits_d) {
    return guarded([&] {
        m->stage_ids(ids_d, B, T, cudaMemcpyDeviceToDevice);
        m->last.reset();
        m->last = std::make_unique<dnn::tensor<float>>(m->model->forward_logits_shard(*m->ids, check_ids != 0));
        *logits_d = m->last->data();
    });
}

extern "C" int dnn_gpt2cs_forward_logits_shard_pitched(dnn_gpt2cs* m, const int32_t* ids, int ids_on_host, int B, int T,
                                                       int check_ids, float** logits_d, int* pitch_h) {
    return guarded([&] {
        m->stage_ids(ids, B, T, ids_on_host ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice);
        m->last.reset();
        m->last = std::make_unique<dnn::tensor<float>>(m->model->forward_logits_shard_pitched(*m->ids, check_ids != 0));
        *logits_d = m->last->data();
        if (pitch_h) *pitch_h = m->model->logits_pitch();
    });
}

extern "C" int dnn_gpt2cs_forward_hidden(dnn_gpt2cs* m, const int32_t* ids_d, int B, int T, float** hidden_d) {
    return guarded([&] {
        m->stage_ids(ids_d, B, T, cudaMemcpyDeviceToDevice);
        m->last.reset();
        m->last = std::make_unique<dnn::tensor<float>>(m->model->forward_hidden(*m->ids, true));
        *hidden_d = m->last->data();
    });
}

extern "C" unsigned long long dnn_gpt2cs_bytes_pushed(dnn_gpt2cs* m) {
    unsigned long long b = 0;
    guarded([&] { b = m->model->bytes_pushed(); });
    return b;
}

extern "C" int dnn_gpt2cs_forward_logits_shard_host(dnn_gpt2cs* m, const int32_t* ids_h, int B, int T,
                                                    float** logits_d) {
    return guarded([&] {
        m->stage_ids(ids_h, B, T, cudaMemcpyHostToDevice);
        m->last.reset();
        m->last = std::make_unique<dnn::tensor<float>>(m->model->forward_logits_shard(*m->ids, false));
        *logits_d = m->last->data();
    });
}

// ---- the text front end (host-only) ---------------------------------------------------------------------

namespace {
// vocabulary from a JSON file (merges.txt beside it is picked up), or from a binary state stream when
// `state_path` is given instead
std::shared_ptr<dnn::BpeTokenizer> make_tokenizer(const char* vocab_json_path, const char* state_path) {
    auto loader = std::make_shared<dnn::VocabLoader>();
    auto tok = std::make_shared<dnn::BpeTokenizer>(loader);
    if (state_path && state_path[0]) {
        std::ifstream in(state_path, std::ios::binary);
        if (!in) throw std::runtime_error(std::string("cannot open tokenizer state ") + state_path);
        tok->load(in);
    } else {
        loader->load_from_file(vocab_json_path);
    }
    return tok;
}
}  // namespace

extern "C" int dnn_tokenizer_encode(const char* vocab_json_path, const char* state_path, const char* text, int add_special,
                                    int* ids_out, int cap) {
    int n = -1;
    guarded([&] {
        auto tok = make_tokenizer(vocab_json_path, state_path);
        std::vector<int> ids = tok->encode(text, add_special != 0);
        for (int i = 0; i < int(ids.size()) && i < cap; ++i) ids_out[i] = ids[size_t(i)];
        n = int(ids.size());
    });
    return n;
}

extern "C" int dnn_tokenizer_decode(const char* vocab_json_path, const char* state_path, const int* ids, int n,
                                    int skip_special, char* out, int cap) {
    int len = -1;
    guarded([&] {
        auto tok = make_tokenizer(vocab_json_path, state_path);
        std::string s = tok->decode(std::vector<int>(ids, ids + n), skip_special != 0);
        if (int(s.size()) + 1 > cap) throw std::runtime_error("dnn_tokenizer_decode: output buffer too small");
        std::memcpy(out, s.data(), s.size());
        out[s.size()] = 0;
        len = int(s.size());
    });
    return len;
}

extern "C" int dnn_tokenizer_save(const char* vocab_json_path, const char* out_path) {
    return guarded([&] {
        auto tok = make_tokenizer(vocab_json_path, nullptr);
        std::ofstream out(out_path, std::ios::binary);
        if (!out) throw std::runtime_error(std::string("cannot write ") + out_path);
        tok->save(out);
    });
}

// ---- checkpoint files -----------------------------------------------------------------------------------

namespace {
dnn_gpt2* wrap_model(std::unique_ptr<dnn::Gpt2<float>> model) {
    auto handle = std::make_unique<dnn_gpt2>();
    handle->model = std::move(model);
    handle->index_params();
    return handle.release();
}
}  // namespace

extern "C" dnn_gpt2* dnn_gpt2_create_with_tokenizer(const char* vocab_json_path, int vocab, int max_seq_len, int layers,
                                                    int heads, int hidden, int ffn) {
    dnn_gpt2* h = nullptr;
    guarded([&] {
        h = wrap_model(std::make_unique<dnn::Gpt2<float>>(make_tokenizer(vocab_json_path, nullptr), vocab, max_seq_len,
                                                          layers, heads, hidden, ffn));
    });
    return h;
}

extern "C" int dnn_gpt2_save_upstream(dnn_gpt2* m, const char* path) {
    return guarded([&] { m->model->save_upstream(path); });
}

extern "C" dnn_gpt2* dnn_gpt2_load_upstream(const char* path) {
    dnn_gpt2* h = nullptr;
    guarded([&] { h = wrap_model(dnn::Gpt2<float>::load_upstream(path, false)); });
    return h;
}

extern "C" int dnn_gpt2_save_quantized(dnn_gpt2* m, const char* path) {
    return guarded([&] { m->model->save_quantized(path); });
}

extern "C" dnn_gpt2* dnn_gpt2_load_quantized(const char* path) {
    dnn_gpt2* h = nullptr;
    guarded([&] { h = wrap_model(dnn::Gpt2<float>::load_quantized(path)); });
    return h;
}

extern "C" int dnn_gpt2_forward_text(dnn_gpt2* m, const char* text, float* hidden_h, int cap_floats, int* tokens_h) {
    return guarded([&] {
        dnn::tensor<float> hidden = m->model->forward_from_text(text);
        if (tokens_h) *tokens_h = hidden.size(1);
        if (hidden.size() > cap_floats) throw std::runtime_error("dnn_gpt2_forward_text: output buffer too small");
        hidden.download(hidden_h);
    });
}

// Reads one record with the class's own load(), hands the parameters back and writes the record again with the
// class's own save(): what = 0 tensor<float>, 1 FullyConnectedLayer, 2 LayerNormLayer (gamma, beta), 3 TokenEmbedding,
// 4 TransformerBlock (its 12 parameter tensors in the order of dnn_block_forward).  params_h receives the
// parameter tensors one after the other (at most cap_floats floats), *count_h their total length.
extern "C" int dnn_file_roundtrip(int what, const char* in_path, const char* out_path, float* params_h, int cap_floats,
                                  int* count_h) {
    return guarded([&] {
        std::ifstream in(in_path, std::ios::binary);
        if (!in) throw std::runtime_error(std::string("cannot open ") + in_path);
        std::ofstream out(out_path, std::ios::binary);
        if (!out) throw std::runtime_error(std::string("cannot write ") + out_path);
        int used = 0;
        auto take = [&](const dnn::tensor<float>& t) {
            if (used + t.size() > cap_floats) throw std::runtime_error("dnn_file_roundtrip: params_h too small");
            t.download(params_h + used);
            used += t.size();
        };
        dnn::fp8::Policy& pol = dnn::fp8::policy();
        const bool prev = pol.host_init;
        pol.host_init = false;
        try {
            if (what == 0) {
                dnn::tensor<float> t({1});
                t.load(in);
                take(t);
                t.save(out);
            } else if (what == 1) {
                dnn::FullyConnectedLayer<float> fc(1, 1);
                fc.load(in);
                take(*fc.weights());
                take(*fc.bias());
                fc.save(out);
            } else if (what == 2) {
                dnn::LayerNormLayer<float> ln(1);
                ln.load(in);
                for (auto* p : ln.parameters()) take(*p);
                ln.save(out);
            } else if (what == 3) {
                dnn::TokenEmbedding<float> emb(1, 1, 1);
                emb.load(in);
                take(*emb.weights());
                take(*emb.bias());
                emb.save(out);
            } else if (what == 4) {
                dnn::TransformerBlock<float> blk(1, 1, 1);
                blk.load(in);
                for (auto* p : blk.parameters()) take(*p);
                blk.save(out);
            } else {
                throw std::invalid_argument("dnn_file_roundtrip: unknown record kind");
            }
        } catch (...) {
            pol.host_init = prev;
            throw;
        }
        pol.host_init = prev;
        if (count_h) *count_h = used;
    });
}

// ---- autoregressive decoding ----------------------------------------------------------------------------

extern "C" int dnn_gpt2_prefill(dnn_gpt2* m, const int32_t* ids_d, int B, int T, int max_len, float** logits_d) {
    return guarded([&] {
        stage_ids(m, ids_d, B, T, cudaMemcpyDeviceToDevice);
        m->last.reset();
        m->last = std::make_unique<dnn::tensor<float>>(m->model->prefill(*m->ids, max_len, true));
        *logits_d = m->last->data();
    });
}

extern "C" int dnn_gpt2_decode_step(dnn_gpt2* m, const int32_t* next_ids_d, int B, int check_ids, float** logits_d) {
    return guarded([&] {
        stage_ids(m, next_ids_d, B, 1, cudaMemcpyDeviceToDevice);
        m->last.reset();
        m->last = std::make_unique<dnn::tensor<float>>(m->model->decode_step(*m->ids, check_ids != 0));
        *logits_d = m->last->data();
    });
}

extern "C" int dnn_gpt2_end_decode(dnn_gpt2* m) {
    return guarded([&] { m->model->end_decode(); });
}

extern "C" int dnn_gpt2_decode_graph_active(dnn_gpt2* m, int* active) {
    return guarded([&] { *active = m->model->decode_graph_active() ? 1 : 0; });
}

// ---- CrossEntropyLoss ---------------------------------------------------------------------------------------

// logits_d [rows, pitch] (pitch == classes: dense); dense targets [rows, classes] or class indices [rows], one of the
// two; mean loss to *loss_h and / or the gradient [rows, classes] to grad_d (either may be null)
extern "C" int dnn_cross_entropy(const float* logits_d, int rows, int classes, int pitch, const float* targets_d,
                                 const int32_t* idx_d, float* loss_h, float* grad_d) {
    return guarded([&] {
        dnn::CrossEntropyLoss<float> ce;
        dnn::tensor<float> logits({rows, pitch});
        dnn::utils::CHECK_CUDA_EX(cudaMemcpyAsync(logits.data(), logits_d, size_t(rows) * pitch * sizeof(float),
                                             cudaMemcpyDeviceToDevice, dnn::Cuda::stream()));
        std::unique_ptr<dnn::tensor<float>> tg;
        std::unique_ptr<dnn::tensor<int>> idx;
        if (targets_d) {
            if (pitch != classes) throw std::runtime_error("dnn_cross_entropy: dense targets go with dense logits");
            tg = std::make_unique<dnn::tensor<float>>(std::vector<int>{rows, classes});
            dnn::utils::CHECK_CUDA_EX(cudaMemcpyAsync(tg->data(), targets_d, size_t(rows) * classes * sizeof(float),
                                                 cudaMemcpyDeviceToDevice, dnn::Cuda::stream()));
        } else {
            idx = std::make_unique<dnn::tensor<int>>(std::vector<int>{rows});
            dnn::utils::CHECK_CUDA_EX(cudaMemcpyAsync(idx->data(), idx_d, size_t(rows) * sizeof(int), cudaMemcpyDeviceToDevice,
                                                 dnn::Cuda::stream()));
        }
        if (loss_h) {
            if (tg) *loss_h = ce.compute(logits, *tg);
            else if (pitch == classes) *loss_h = ce.compute(logits, *idx);
            else *loss_h = ce.compute_pitched(logits, classes, *idx);
        }
        if (grad_d) {
            dnn::tensor<float> g = tg ? ce.compute_gradient(logits, *tg)
                                      : (pitch == classes ? ce.compute_gradient(logits, *idx)
                                                          : ce.compute_gradient_pitched(logits, classes, *idx));
            dnn::utils::CHECK_CUDA_EX(cudaMemcpyAsync(grad_d, g.data(), size_t(rows) * classes * sizeof(float),
                                                 cudaMemcpyDeviceToDevice, dnn::Cuda::stream()));
            dnn::utils::CHECK_CUDA_EX(cudaStreamSynchronize(dnn::Cuda::stream()));
        }
    });
}
