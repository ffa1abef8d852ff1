#include "dnn/models/gpt2.cuh"

#include <algorithm>
#include <fstream>
#include <random>

#include "dnn/tokens/bpe_tokenizer.cuh"
#include "dnn/tokens/vocab_loader.cuh"

namespace dnn {

template <typename T>
Gpt2<T>::Gpt2(std::shared_ptr<Tokenizer> tokenizer, int vocab_size, int max_seq_len, int num_layers, int num_heads,
              int hidden_dim, int intermediate_dim, T /*learning_rate*/, T /*beta1*/, T /*beta2*/, T /*epsilon*/,
              bool training_enabled)
    : NaturalLanguageModel<T>(std::move(tokenizer), max_seq_len, training_enabled),
      vocab_size_(vocab_size),
      max_seq_len_(max_seq_len),
      hidden_dim_(hidden_dim) {
    token_embedding_ = std::make_unique<TokenEmbedding<T>>(vocab_size, hidden_dim, max_seq_len, training_enabled);
    // (with fp8::policy().host_init off the weights stay zero until initialize_on_device() or an upload fills them)
    if (fp8::policy().host_init) initialize_weights(token_embedding_->weights(), static_cast<T>(0.02f));
    positional_encoding_ = std::make_unique<PositionalEncoding<T>>(hidden_dim, max_seq_len, training_enabled);
    for (int i = 0; i < num_layers; ++i) {
        auto block = std::make_unique<TransformerBlock<T>>(hidden_dim, num_heads, intermediate_dim, training_enabled);
        block->set_mlp_gelu(true);
        transformer_blocks_.push_back(std::move(block));
    }
    final_fc_ = std::make_unique<FullyConnectedLayer<T>>(hidden_dim, vocab_size, training_enabled);
    if (fp8::policy().host_init) initialize_weights(final_fc_->weights(), static_cast<T>(0.02f));
}

template <typename T>
std::string Gpt2<T>::name() const {
    return "Gpt2";
}

// N(0, scale) from a fixed-seed generator (upstream draws from std::random_device, gpt2.cu:204-214).
template <typename T>
void Gpt2<T>::initialize_weights(tensor<T>* weights, T scale) {
    std::mt19937 gen(0x69D72000u + unsigned(weights->numel() % 0xFFFFu));
    std::normal_distribution<float> dist(0.0f, float(scale));
    std::vector<T> host(weights->numel());
    for (auto& v : host) v = static_cast<T>(dist(gen));
    weights->upload(host.data());
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));
}

template <typename T>
void Gpt2<T>::initialize_on_device(uint64_t seed, float std) {
    uint64_t k = seed * 1000ull;
    tensor<T>* emb = token_embedding_->weights();
    fp8::fill_normal(emb->data(), emb->numel(), 0.f, std, ++k);
    emb->bump_version();
    for (auto& b : transformer_blocks_) {
        FullyConnectedLayer<T>* fcs[4] = {&b->attention().qkv_projection(), &b->attention().out_projection(),
                                          &b->mlp_fc1(), &b->mlp_fc2()};
        for (FullyConnectedLayer<T>* fc : fcs) fc->initialize_rows_normal_on_device(std, ++k, 0, 0, fc->out_features());
    }
    final_fc_->initialize_rows_normal_on_device(std, ++k, 0, 0, final_fc_->out_features());
}

template <typename T>
void Gpt2<T>::train_step(const tensor<T>&, const tensor<T>&) {
    throw std::runtime_error("Use token-based train_step for NLP models.");
}

template <typename T>
void Gpt2<T>::train_step(const std::vector<int>&, const std::vector<int>&) {
    throw std::runtime_error("Gpt2::train_step: training (loss, backward, optimiser) is outside the fp8 inference build");
}

template <typename T>
tensor<T> Gpt2<T>::forward(const tensor<T>&) {
    throw std::runtime_error("Use token-based forward for NLP models.");
}

template <typename T>
tensor<T> Gpt2<T>::forward(const std::vector<int>& input_token_ids) {
    tensor<int> ids({1, int(input_token_ids.size())});
    ids.upload(input_token_ids.data());
    return forward_hidden(ids);
}

template <typename T>
tensor<T> Gpt2<T>::forward_hidden(const tensor<int>& ids, bool check_ids) {
    const auto& s = ids.shape();
    if (s.size() != 2) throw std::runtime_error("Gpt2 expects token ids shaped [B, T]");
    const int B = s[0], T_len = s[1];
    if (T_len > positional_encoding_->max_seq_len())
        throw std::runtime_error("Input sequence length exceeds maximum allowed length");
    fp8::PassScope amax_slots;  // one memset for all the pass's amax outputs
    tensor<T> x = token_embedding_->forward_with_positions(ids, positional_encoding_->table().data(), check_ids);
    if (!streamer_) {
        for (auto& block : transformer_blocks_) block->forward_inplace(x.data(), B, T_len);
        return x;
    }
    const int L = int(transformer_blocks_.size());
    for (int l = 0; l < L; ++l) {
        TransformerBlock<T>& blk = *transformer_blocks_[size_t(l)];
        void* slot = nullptr;
        utils::CHECK_DF8(df8_streamer_acquire(streamer_, l, fp8::stream(), &slot));
        const uint8_t* p = static_cast<const uint8_t*>(slot);
        FullyConnectedLayer<T>* fcs[4] = {&blk.attention().qkv_projection(), &blk.attention().out_projection(),
                                          &blk.mlp_fc1(), &blk.mlp_fc2()};
        for (FullyConnectedLayer<T>* fc : fcs) {
            fc->use_external_codes(p);
            p += (fc->weight_code_bytes() + 255) & ~size_t(255);
        }
        blk.forward_inplace(x.data(), B, T_len);
        utils::CHECK_DF8(df8_streamer_release(streamer_, l, fp8::stream()));
        utils::CHECK_DF8(df8_streamer_prefetch(streamer_, (l + stream_slots_) % L));
    }
    return x;
}

template <typename T>
tensor<T> Gpt2<T>::forward_logits(const tensor<int>& ids, bool check_ids) {
    fp8::PassScope amax_slots;
    tensor<T> x = forward_hidden(ids, check_ids);
    const int M = int(x.numel() / size_t(hidden_dim_));
    fp8::quantize(x.data(), x.numel(), fp8::policy().activation_kind, head_q_);
    tensor<T> logits({M, vocab_size_});
    head_gemm(M, logits.data(), vocab_size_);
    return logits;
}

template <typename T>
void Gpt2<T>::head_gemm(int M, float* logits, int pitch) {
    if (stage_timing_) utils::CHECK_CUDA_EX(cudaEventRecord(head_ev_[0], Cuda::stream()));
    final_fc_->forward_codes(head_q_.codes.data(), head_q_.kind, head_q_.scale.data(), M, 0, nullptr, logits, nullptr,
                             pitch);
    if (stage_timing_) utils::CHECK_CUDA_EX(cudaEventRecord(head_ev_[1], Cuda::stream()));
}

template <typename T>
void Gpt2<T>::set_stage_timing(bool on) {
    if (on && !head_ev_[0])
        for (cudaEvent_t& ev : head_ev_) utils::CHECK_CUDA_EX(cudaEventCreate(&ev));
    stage_timing_ = on;
}

template <typename T>
float Gpt2<T>::last_head_ms() const {
    if (!head_ev_[0]) throw std::runtime_error("Gpt2::last_head_ms: stage timing was never switched on");
    utils::CHECK_CUDA_EX(cudaEventSynchronize(head_ev_[1]));
    float ms = 0.f;
    utils::CHECK_CUDA_EX(cudaEventElapsedTime(&ms, head_ev_[0], head_ev_[1]));
    return ms;
}

template <typename T>
tensor<T> Gpt2<T>::forward_logits_pitched(const tensor<int>& ids, bool check_ids) {
    fp8::PassScope amax_slots;
    tensor<T> x = forward_hidden(ids, check_ids);
    const int M = int(x.numel() / size_t(hidden_dim_));
    fp8::quantize(x.data(), x.numel(), fp8::policy().activation_kind, head_q_);
    const int pitch = logits_pitch();
    tensor<T> logits({M, pitch});
    head_gemm(M, logits.data(), pitch);
    return logits;
}

// logits [B, V] of the last position of every sequence of x [B, T_len, E]
template <typename T>
tensor<T> Gpt2<T>::last_rows_logits(const float* x, int B, int T_len) {
    const int E = hidden_dim_;
    tensor<T> last({B, E});
    utils::CHECK_CUDA_EX(cudaMemcpy2DAsync(last.data(), size_t(E) * sizeof(float), x + size_t(T_len - 1) * E,
                                           size_t(T_len) * E * sizeof(float), size_t(E) * sizeof(float), size_t(B),
                                           cudaMemcpyDeviceToDevice, Cuda::stream()));
    fp8::quantize(last.data(), last.numel(), fp8::policy().activation_kind, head_q_);
    tensor<T> logits({B, vocab_size_});
    final_fc_->forward_codes_skinny(head_q_.codes.data(), head_q_.kind, head_q_.scale.data(), B, 0, nullptr, logits.data(),
                                    nullptr);
    return logits;
}

template <typename T>
tensor<T> Gpt2<T>::prefill(const tensor<int>& ids, int max_len, bool check_ids) {
    const auto& s = ids.shape();
    if (s.size() != 2) throw std::runtime_error("Gpt2 expects token ids shaped [B, T]");
    const int B = s[0], T_len = s[1];
    if (max_len <= 0) max_len = max_seq_len_;
    if (T_len < 1 || T_len > max_len || max_len > max_seq_len_ || B < 1 || B > 128)
        throw std::runtime_error("Gpt2::prefill: needs 1 <= T <= max_len <= max_seq_len and 1 <= B <= 128");
    if (streamer_) throw std::runtime_error("Gpt2::prefill: decoding with streamed weights is not supported");
    end_decode();
    for (auto& blk : transformer_blocks_) {
        auto cache = std::make_unique<typename MultiHeadAttentionLayer<T>::KvCache>();
        const int H = blk->attention().num_heads(), D = blk->attention().head_dim();
        cache->k = tensor<uint8_t>({B, H, max_len, D});
        cache->v = tensor<uint8_t>({B, H, max_len, D});
        cache->row_dq = tensor<float>({max_len});
        cache->batch = B;
        cache->max_len = max_len;
        blk->attention().attach_kv_cache(cache.get());
        blk->attention().set_kv_len(0);
        blk->attention().set_causal(true);
        kv_.push_back(std::move(cache));
    }
    fp8::PassScope amax_slots;
    tensor<T> x = token_embedding_->forward_with_positions(ids, positional_encoding_->table().data(), check_ids);
    for (auto& blk : transformer_blocks_) blk->forward_inplace(x.data(), B, T_len);
    kv_len_ = T_len;
    const int pos = T_len;
    utils::CHECK_CUDA_EX(cudaMemcpyAsync(dec_pos_.data(), &pos, sizeof(int), cudaMemcpyHostToDevice, Cuda::stream()));
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));  // `pos` is a local
    for (auto& blk : transformer_blocks_) blk->attention().set_decode_position(dec_pos_.data());
    return last_rows_logits(x.data(), B, T_len);
}

// One decode step on the persistent buffers: every launch reads the position from dec_pos_, so the sequence of
// launches (and every argument) is the same from step to step.
template <typename T>
void Gpt2<T>::decode_body(int B) {
    fp8::PassScope amax_slots;
    const int E = hidden_dim_;
    utils::CHECK_DF8(df8_embed_pe_pos_f32(dec_ids_.data(), B, E, vocab_size_, token_embedding_->weights()->data(),
                                          token_embedding_->bias()->data(), positional_encoding_->table().data(),
                                          dec_pos_.data(), dec_x_.data(), fp8::stream()));
    for (auto& blk : transformer_blocks_) blk->decode_inplace(dec_x_.data(), B);
    fp8::quantize(dec_x_.data(), size_t(B) * E, fp8::policy().activation_kind, head_q_);
    final_fc_->forward_codes_skinny(head_q_.codes.data(), head_q_.kind, head_q_.scale.data(), B, 0, nullptr,
                                    dec_logits_.data(), nullptr);
    utils::CHECK_DF8(df8_position_advance(dec_pos_.data(), fp8::stream()));
}

template <typename T>
tensor<T> Gpt2<T>::decode_step(const tensor<int>& next_ids, bool check_ids) {
    if (kv_.empty()) throw std::runtime_error("Gpt2::decode_step: call prefill first");
    const int B = kv_[0]->batch;
    if (next_ids.numel() != size_t(B)) throw std::runtime_error("Gpt2::decode_step: one token id per sequence of the prefill");
    if (kv_len_ + 1 > kv_[0]->max_len) throw std::runtime_error("Gpt2::decode_step: the KV cache is full");
    cudaStream_t st = Cuda::stream();
    if (check_ids) {  // upstream validates ids on every call (token_embedding.cu:131-138)
        std::vector<int> h(static_cast<size_t>(B), 0);
        utils::CHECK_CUDA_EX(cudaMemcpyAsync(h.data(), next_ids.data(), size_t(B) * sizeof(int), cudaMemcpyDeviceToHost, st));
        utils::CHECK_CUDA_EX(cudaStreamSynchronize(st));
        int bad = 0;
        for (int id : h) bad += (id < 0 || id >= vocab_size_) ? 1 : 0;
        if (bad) throw std::runtime_error("Invalid token ID: " + std::to_string(bad) + " id(s) outside the vocabulary");
    }
    if (dec_ids_.numel() != size_t(B)) {
        dec_ids_ = tensor<int>({B, 1});
        dec_x_ = tensor<T>({B, hidden_dim_});
        dec_logits_ = tensor<T>({B, vocab_size_});
    }
    utils::CHECK_CUDA_EX(cudaMemcpyAsync(dec_ids_.data(), next_ids.data(), size_t(B) * sizeof(int), cudaMemcpyDeviceToDevice, st));
    for (auto& blk : transformer_blocks_) blk->attention().set_kv_len(kv_len_);  // host mirror (bounds checks)

    const char* env = getenv("DF8_DECODE_GRAPH");
    const bool want_graph = dec_graph_ok_ && dec_steps_ >= 1 && st != nullptr && !(env && env[0] == '0');
    if (want_graph && !dec_graph_) {
        // the first step ran eagerly and sized every buffer; capture the second and replay it from then on
        cudaGraph_t graph = nullptr;
        if (cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed) == cudaSuccess) {
            bool body_ok = true;
            try {
                decode_body(B);
            } catch (...) {
                body_ok = false;
            }
            const cudaError_t end = cudaStreamEndCapture(st, &graph);
            if (!(body_ok && end == cudaSuccess && graph && cudaGraphInstantiate(&dec_graph_, graph, 0) == cudaSuccess)) {
                dec_graph_ = nullptr;
                dec_graph_ok_ = false;  // eager from here on
            }
            if (graph) cudaGraphDestroy(graph);
        } else {
            dec_graph_ok_ = false;
        }
        (void)cudaGetLastError();
    }
    if (dec_graph_) utils::CHECK_CUDA_EX(cudaGraphLaunch(dec_graph_, st));
    else decode_body(B);
    ++dec_steps_;
    ++kv_len_;
    return dec_logits_.clone();
}

template <typename T>
void Gpt2<T>::end_decode() {
    for (auto& blk : transformer_blocks_) {
        blk->attention().attach_kv_cache(nullptr);
        blk->attention().set_kv_len(0);
        blk->attention().set_decode_position(nullptr);
    }
    if (!kv_.empty()) utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));  // the caches may still be read
    if (dec_graph_) {
        cudaGraphExecDestroy(dec_graph_);
        dec_graph_ = nullptr;
    }
    dec_graph_ok_ = true;
    dec_steps_ = 0;
    kv_.clear();
    kv_len_ = 0;
}

template <typename T>
Gpt2<T>::~Gpt2() {
    if (dec_graph_) cudaGraphExecDestroy(dec_graph_);
    for (cudaEvent_t ev : head_ev_)
        if (ev) cudaEventDestroy(ev);
    if (streamer_) df8_streamer_destroy(streamer_);
}

template <typename T>
void Gpt2<T>::enable_layer_streaming(int slots, bool release_fp32, df8_comm* comm) {
    if (streamer_ || transformer_blocks_.empty()) return;
    const int L = int(transformer_blocks_.size());
    auto fcs_of = [](TransformerBlock<T>& blk) {
        return std::vector<FullyConnectedLayer<T>*>{&blk.attention().qkv_projection(), &blk.attention().out_projection(),
                                                    &blk.mlp_fc1(), &blk.mlp_fc2()};
    };
    size_t layer_bytes = 0;
    for (FullyConnectedLayer<T>* fc : fcs_of(*transformer_blocks_[0])) layer_bytes += (fc->weight_code_bytes() + 255) & ~size_t(255);
    utils::CHECK_DF8(df8_streamer_create_sharded(layer_bytes, slots, L, comm, &streamer_));
    int n_slots = 0;
    utils::CHECK_DF8(df8_streamer_stats(streamer_, nullptr, nullptr, &n_slots));
    stream_slots_ = n_slots;
    for (int l = 0; l < L; ++l) {
        void* host = nullptr;
        utils::CHECK_DF8(df8_streamer_host_ptr(streamer_, l, &host));
        uint8_t* p = static_cast<uint8_t*>(host);
        for (FullyConnectedLayer<T>* fc : fcs_of(*transformer_blocks_[size_t(l)])) {
            fc->export_weight_codes(p);
            p += (fc->weight_code_bytes() + 255) & ~size_t(255);
            fc->drop_cached_codes();
            if (release_fp32) {
                // keep version(): the cached scale must stay valid
                *fc->weights() = tensor<T>({0, fc->in_features()});
                fc->mark_weights_quantized();
            }
        }
    }
    for (int l = 0; l < stream_slots_; ++l) utils::CHECK_DF8(df8_streamer_prefetch(streamer_, l));
}

template <typename T>
void Gpt2<T>::disable_layer_streaming() {
    if (!streamer_) return;
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));
    for (auto& blk : transformer_blocks_) {
        FullyConnectedLayer<T>* fcs[4] = {&blk->attention().qkv_projection(), &blk->attention().out_projection(),
                                          &blk->mlp_fc1(), &blk->mlp_fc2()};
        for (FullyConnectedLayer<T>* fc : fcs) {
            fc->use_external_codes(nullptr);
            fc->invalidate_quantized_weights();  // re-quantise from the fp32 weights on next use
        }
    }
    df8_streamer_destroy(streamer_);
    streamer_ = nullptr;
}

template <typename T>
void Gpt2<T>::resize_streaming_slots(int slots) {
    if (!streamer_) throw std::runtime_error("Gpt2::resize_streaming_slots: layer streaming is off");
    utils::CHECK_DF8(df8_streamer_resize(streamer_, slots));
    int n_slots = 0;
    utils::CHECK_DF8(df8_streamer_stats(streamer_, nullptr, nullptr, &n_slots));
    stream_slots_ = n_slots;
    for (int l = 0; l < stream_slots_; ++l) utils::CHECK_DF8(df8_streamer_prefetch(streamer_, l));
}

template <typename T>
void Gpt2<T>::streaming_traffic(unsigned long long* h2d_bytes, unsigned long long* gathered_bytes) const {
    if (h2d_bytes) *h2d_bytes = 0;
    if (gathered_bytes) *gathered_bytes = 0;
    if (streamer_) utils::CHECK_DF8(df8_streamer_traffic(streamer_, h2d_bytes, gathered_bytes));
}

template <typename T>
float Gpt2<T>::time_layer_uploads() {
    if (!streamer_) throw std::runtime_error("Gpt2::time_layer_uploads: layer streaming is off");
    float ms = 0.f;
    utils::CHECK_DF8(df8_streamer_time_uploads(streamer_, &ms));
    return ms;
}

template <typename T>
unsigned long long Gpt2<T>::streamed_bytes() const {
    unsigned long long b = 0;
    if (streamer_) df8_streamer_stats(streamer_, &b, nullptr, nullptr);
    return b;
}

template <typename T>
void Gpt2<T>::set_mlp_gelu(bool on) {
    for (auto& b : transformer_blocks_) b->set_mlp_gelu(on);
}

template <typename T>
void Gpt2<T>::set_causal(bool causal) {
    for (auto& b : transformer_blocks_) b->set_causal(causal);
}

template <typename T>
std::vector<BaseLayer*> Gpt2<T>::layers() {
    std::vector<BaseLayer*> all;
    all.push_back(token_embedding_.get());
    all.push_back(positional_encoding_.get());
    for (auto& b : transformer_blocks_) all.push_back(b.get());
    all.push_back(final_fc_.get());
    return all;
}

// Container written here: the four header ints upstream writes (vocab, max_seq_len, layer count, hidden
// dim; gpt2.cu:148-152) followed by the heads and MLP width upstream's loader hard-codes (:179), then each
// layer's own save() stream in execution order.  Upstream's file additionally interleaves the tokenizer
// state and raw layer-name bytes that its own loader cannot read back (:153-187).
template <typename T>
void Gpt2<T>::save(const std::string& path) const {
    std::ofstream out(path, std::ios::binary);
    if (!out) throw std::runtime_error("Failed to open file for saving Gpt2");
    const int num_layers = int(transformer_blocks_.size());
    out.write(reinterpret_cast<const char*>(&vocab_size_), sizeof(int));
    out.write(reinterpret_cast<const char*>(&max_seq_len_), sizeof(int));
    out.write(reinterpret_cast<const char*>(&num_layers), sizeof(int));
    out.write(reinterpret_cast<const char*>(&hidden_dim_), sizeof(int));
    const int heads = transformer_blocks_.empty() ? 0 : transformer_blocks_[0]->attention().num_heads();
    const int ffn = transformer_blocks_.empty() ? 0 : transformer_blocks_[0]->mlp_fc1().out_features();
    out.write(reinterpret_cast<const char*>(&heads), sizeof(int));
    out.write(reinterpret_cast<const char*>(&ffn), sizeof(int));
    token_embedding_->save(out);
    for (const auto& b : transformer_blocks_) b->save(out);
    final_fc_->save(out);
}

template <typename T>
std::unique_ptr<Gpt2<T>> Gpt2<T>::load(const std::string& path, bool training_enabled) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("Failed to open file for loading Gpt2");
    int v = 0, t = 0, l = 0, e = 0, h = 0, f = 0;
    for (int* p : {&v, &t, &l, &e, &h, &f}) in.read(reinterpret_cast<char*>(p), sizeof(int));
    if (!in || v <= 0 || t <= 0 || l < 0 || e <= 0 || h <= 0 || f <= 0)
        throw std::runtime_error("Gpt2::load: bad header");
    auto model = std::make_unique<Gpt2<T>>(nullptr, v, t, l, h, e, f, static_cast<T>(1e-4), static_cast<T>(0.9),
                                           static_cast<T>(0.98), static_cast<T>(1e-8), training_enabled);
    model->token_embedding_->load(in);
    for (auto& b : model->transformer_blocks_) b->load(in);
    model->final_fc_->load(in);
    return model;
}

namespace {

void put_i(std::ostream& out, int v) { out.write(reinterpret_cast<const char*>(&v), sizeof(v)); }
int get_i(std::istream& in, const char* what) {
    int v = 0;
    in.read(reinterpret_cast<char*>(&v), sizeof(v));
    if (!in) throw std::runtime_error(std::string("Gpt2: truncated file while reading ") + what);
    return v;
}
// the raw bytes of a layer's name, as upstream writes them in front of each layer (no length)
void put_name(std::ostream& out, const std::string& name) { out.write(name.data(), std::streamsize(name.size())); }
void expect_name(std::istream& in, const std::string& name) {
    std::string got(name.size(), '\0');
    in.read(&got[0], std::streamsize(got.size()));
    if (!in || got != name) throw std::runtime_error("Gpt2::load_upstream: expected the layer name '" + name + "'");
}
// skips one tensor record (int ndim, int shape[ndim], elements of elem_bytes each)
void skip_tensor(std::istream& in, size_t elem_bytes) {
    const int ndim = get_i(in, "a tensor header");
    if (ndim < 0 || ndim > 8) throw std::runtime_error("Gpt2::load_upstream: bad tensor header");
    size_t n = 1;
    for (int d = 0; d < ndim; ++d) n *= size_t(std::max(0, get_i(in, "a tensor shape")));
    in.seekg(std::streamoff(n * elem_bytes), std::ios::cur);
    if (!in) throw std::runtime_error("Gpt2::load_upstream: truncated tensor");
}
struct HostInitOff {  // constructors leave the weights alone while this lives: they are about to be loaded
    bool prev;
    HostInitOff() : prev(fp8::policy().host_init) { fp8::policy().host_init = false; }
    ~HostInitOff() { fp8::policy().host_init = prev; }
};

}  // namespace

template <typename T>
void Gpt2<T>::save_upstream(const std::string& path) const {
    if (!this->tokenizer_) throw std::runtime_error("Gpt2::save_upstream: the model has no tokenizer (its state is part of the file)");
    std::ofstream out(path, std::ios::binary);
    if (!out) throw std::runtime_error("Failed to open file for saving Gpt2");
    put_i(out, vocab_size_);
    put_i(out, max_seq_len_);
    put_i(out, int(transformer_blocks_.size()));
    put_i(out, hidden_dim_);
    this->tokenizer_->save(out);
    put_name(out, token_embedding_->name());
    token_embedding_->save(out);
    put_name(out, positional_encoding_->name());
    positional_encoding_->save(out);
    for (const auto& b : transformer_blocks_) {
        put_name(out, b->name());
        b->save(out);
    }
    put_name(out, final_fc_->name());
    final_fc_->save(out);
}

template <typename T>
std::unique_ptr<Gpt2<T>> Gpt2<T>::load_upstream(const std::string& path, bool training_enabled) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("Failed to open file for loading Gpt2");
    const int vocab = get_i(in, "the header"), max_seq = get_i(in, "the header");
    const int layers = get_i(in, "the header"), hidden = get_i(in, "the header");
    if (vocab <= 0 || max_seq <= 0 || layers < 0 || hidden <= 0) throw std::runtime_error("Gpt2::load_upstream: bad header");
    auto tokenizer = std::make_shared<BpeTokenizer>(std::make_shared<VocabLoader>());
    tokenizer->load(in);
    // look ahead to the first block's header for the head count and the MLP width
    const std::streampos body = in.tellg();
    expect_name(in, "TokenEmbedding");
    for (int k = 0; k < 3; ++k) get_i(in, "the embedding header");
    skip_tensor(in, sizeof(T));
    skip_tensor(in, sizeof(T));
    expect_name(in, "PositionalEncoding");
    int heads = 1, ffn = hidden;
    if (layers > 0) {
        expect_name(in, "TransformerBlock");
        const int e = get_i(in, "a block header");
        heads = get_i(in, "a block header");
        ffn = get_i(in, "a block header");
        if (e != hidden || heads <= 0 || ffn <= 0 || hidden % heads != 0)
            throw std::runtime_error("Gpt2::load_upstream: the first block does not match the model header");
    }
    in.seekg(body);
    std::unique_ptr<Gpt2<T>> model;
    {
        HostInitOff quiet;
        model = std::make_unique<Gpt2<T>>(tokenizer, vocab, max_seq, layers, heads, hidden, ffn, static_cast<T>(1e-4),
                                          static_cast<T>(0.9), static_cast<T>(0.98), static_cast<T>(1e-8), training_enabled);
    }
    expect_name(in, model->token_embedding_->name());
    model->token_embedding_->load(in);
    expect_name(in, model->positional_encoding_->name());
    model->positional_encoding_->load(in);
    for (auto& b : model->transformer_blocks_) {
        expect_name(in, b->name());
        b->load(in);
    }
    expect_name(in, model->final_fc_->name());
    model->final_fc_->load(in);
    return model;
}

// "DF8Q" 1 | vocab max_seq layers heads hidden ffn | embedding (weights, bias) | per block: ln1, ln2 parameters,
// qkv, out, fc1, fc2 records | head record
template <typename T>
void Gpt2<T>::save_quantized(const std::string& path) {
    std::ofstream out(path, std::ios::binary);
    if (!out) throw std::runtime_error("Failed to open file for saving the quantised Gpt2");
    out.write("DF8Q", 4);
    put_i(out, 1);
    put_i(out, vocab_size_);
    put_i(out, max_seq_len_);
    put_i(out, int(transformer_blocks_.size()));
    put_i(out, transformer_blocks_.empty() ? 1 : transformer_blocks_[0]->attention().num_heads());
    put_i(out, hidden_dim_);
    put_i(out, transformer_blocks_.empty() ? hidden_dim_ : transformer_blocks_[0]->mlp_fc1().out_features());
    token_embedding_->weights()->save(out);
    token_embedding_->bias()->save(out);
    for (auto& b : transformer_blocks_) {
        for (tensor<T>* p : b->norm1().parameters()) p->save(out);
        for (tensor<T>* p : b->norm2().parameters()) p->save(out);
        b->attention().qkv_projection().export_quantized(out);
        b->attention().out_projection().export_quantized(out);
        b->mlp_fc1().export_quantized(out);
        b->mlp_fc2().export_quantized(out);
    }
    final_fc_->export_quantized(out);
    if (!out) throw std::runtime_error("Gpt2::save_quantized: write failed");
}

template <typename T>
std::unique_ptr<Gpt2<T>> Gpt2<T>::load_quantized(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("Failed to open file for loading the quantised Gpt2");
    char magic[4] = {0, 0, 0, 0};
    in.read(magic, 4);
    if (!in || std::string(magic, 4) != "DF8Q" || get_i(in, "the version") != 1)
        throw std::runtime_error("Gpt2::load_quantized: not a quantised Gpt2 file of version 1");
    int cfg[6];
    for (int& v : cfg) v = get_i(in, "the header");
    if (cfg[0] <= 0 || cfg[1] <= 0 || cfg[2] < 0 || cfg[3] <= 0 || cfg[4] <= 0 || cfg[5] <= 0)
        throw std::runtime_error("Gpt2::load_quantized: bad header");
    std::unique_ptr<Gpt2<T>> model;
    {
        HostInitOff quiet;
        model = std::make_unique<Gpt2<T>>(nullptr, cfg[0], cfg[1], cfg[2], cfg[3], cfg[4], cfg[5]);
    }
    model->token_embedding_->weights()->load(in);
    model->token_embedding_->bias()->load(in);
    for (auto& b : model->transformer_blocks_) {
        for (tensor<T>* p : b->norm1().parameters()) p->load(in);
        for (tensor<T>* p : b->norm2().parameters()) p->load(in);
        b->attention().qkv_projection().import_quantized(in);
        b->attention().out_projection().import_quantized(in);
        b->mlp_fc1().import_quantized(in);
        b->mlp_fc2().import_quantized(in);
    }
    model->final_fc_->import_quantized(in);
    return model;
}

template <typename T>
tensor<T> Gpt2<T>::forward_from_text(const std::string& text) {
    if (!this->tokenizer_) throw std::runtime_error("Gpt2::forward_from_text: the model has no tokenizer");
    return forward(this->tokenizer_->encode(text, true));
}

template class Gpt2<float>;

}  // namespace dnn
