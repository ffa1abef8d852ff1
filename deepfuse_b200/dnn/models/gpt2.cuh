// Gpt2<T>: token embedding -> sinusoidal positions -> N pre-LayerNorm transformer blocks -> vocabulary head.
//
// Public surface of upstream dnn/models/gpt2.cuh:20-58: the constructor (tokenizer, vocab_size,
// max_seq_len, num_layers, num_heads, hidden_dim, intermediate_dim, learning_rate, beta1, beta2, epsilon,
// training_enabled) with upstream's defaults, name() == "Gpt2", forward(token ids) returning the hidden
// states [1,T,E] of a single sequence (dnn/models/gpt2.cu:126-142), forward(tensor)/train_step(tensor,
// tensor) throwing "Use token-based ..." (:52-55, :121-124), layers() (:194-202), save/load.
// Wiring as upstream: no final LayerNorm, no mask handed to the blocks.
//
// Additions for batched fp8 inference (upstream's forward is batch-1 and stops before the head; its
// train_step composes the same pieces up to the logits, :66-83):
//   forward_logits(ids [B,T])   -> fp32 logits [B*T, V]   (embedding -> PE -> blocks -> final_fc)
//   forward_hidden(ids [B,T])   -> hidden states [B,T,E]
//   set_mlp_gelu / set_causal   forwarded to every block (GELU is ON by default for this model: GPT-2's MLP
//                               uses it, although upstream's block has no activation)
//   enable_layer_streaming(...) block weights live as fp8 codes in pinned host memory and are uploaded
//                               layer by layer on a side stream while the previous layers compute
#pragma once

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "dnn/layers/fully_connected_layer.cuh"
#include "dnn/layers/transformer_block.cuh"
#include "dnn/models/natural_language_model.cuh"
#include "dnn/tokens/positional_encoding.cuh"
#include "dnn/tokens/token_embedding.cuh"
#include "dnn/tokens/tokenizer.cuh"

namespace dnn {

template <typename T>
class Gpt2 : public NaturalLanguageModel<T> {
public:
    Gpt2(std::shared_ptr<Tokenizer> tokenizer, int vocab_size = 50257, int max_seq_len = 1024, int num_layers = 12,
         int num_heads = 12, int hidden_dim = 768, int intermediate_dim = 3072, T learning_rate = static_cast<T>(1e-4),
         T beta1 = static_cast<T>(0.9), T beta2 = static_cast<T>(0.98), T epsilon = static_cast<T>(1e-8),
         bool training_enabled = false);

    std::string name() const override;

    void train_step(const tensor<T>& input, const tensor<T>& target) override;
    void train_step(const std::vector<int>& input_token_ids, const std::vector<int>& target_token_ids);

    tensor<T> forward(const tensor<T>& input) override;
    tensor<T> forward(const std::vector<int>& input_token_ids);

    void save(const std::string& path) const override;
    static std::unique_ptr<Gpt2<T>> load(const std::string& path, bool training_enabled);
    // Files in the layout upstream's Gpt2::save writes (dnn/models/gpt2.cu:144-166): vocab, max_seq_len, block
    // count, hidden; the tokenizer's state; then, each preceded by the raw bytes of its name(), the token
    // embedding, the (empty) positional encoding, every transformer block and the head.  Upstream's own loader
    // cannot read these files back (:168-192 expects length-prefixed names, reads num_layers - 2 blocks and
    // hard-codes 12 heads / 3072); load_upstream reads what save writes and takes heads and MLP width from the
    // first block's header.  save_upstream needs a tokenizer (its state is part of the file).
    static std::unique_ptr<Gpt2<T>> load_upstream(const std::string& path, bool training_enabled = false);
    void save_upstream(const std::string& path) const;
    // The quantise-once cache: every fully-connected layer as e4m3 codes + scale + bias, the embedding table and
    // the LayerNorm parameters in fp32.  A model loaded from it never holds fp32 weight matrices on the device
    // and computes bit for bit what the model that wrote it computes.
    void save_quantized(const std::string& path);
    static std::unique_ptr<Gpt2<T>> load_quantized(const std::string& path);
    // Token ids of `text` (tokenizer's encode with BOS / EOS) through the token-based forward: hidden states
    // [1,T,E].  (Upstream's NaturalLanguageModel::forward_from_text ends in Gpt2::forward(tensor), which throws.)
    tensor<T> forward_from_text(const std::string& text);

    std::vector<BaseLayer*> layers() override;

    // ---- batched fp8 inference ----
    tensor<T> forward_hidden(const tensor<int>& ids, bool check_ids = true);
    tensor<T> forward_logits(const tensor<int>& ids, bool check_ids = true);
    // The same logits in a row-pitched buffer: a tensor [B*T, logits_pitch()] whose first vocab_size() columns
    // of every row are the logits (the rest is padding with unspecified contents).  Rows of 50257 floats do not
    // start on 16-byte boundaries, which costs the head GEMM one 4-byte store per element; with the pitch
    // rounded up to a multiple of 32 floats its epilogue leaves through TMA stores.
    tensor<T> forward_logits_pitched(const tensor<int>& ids, bool check_ids = true);
    int logits_pitch() const { return (vocab_size_ + 31) / 32 * 32; }
    // Measurement aid: with stage timing on, forward_logits / forward_logits_pitched bracket the vocabulary-head
    // GEMM (the longest single launch of a forward) with two events on the stream; last_head_ms() waits for the
    // second one and returns the launch's duration inside the forward, with the cache state the blocks leave.
    void set_stage_timing(bool on);
    float last_head_ms() const;
    void set_mlp_gelu(bool on);
    void set_causal(bool causal);
    // Every weight matrix <- N(0, std) generated on the device (fp8::fill_normal), biases <- 0; stream numbers
    // seed*1000 + 1, 2, ... in the order embedding, then per block qkv, out, fc1, fc2, then the head.
    void initialize_on_device(uint64_t seed, float std = 0.02f);

    // ---- autoregressive decoding ----
    // prefill(ids [B,T]) runs the forward on a prompt, keeps every layer's key / value codes in a cache sized for
    // `max_len` positions (default: max_seq_len) and returns the logits of the LAST position, [B, V];
    // decode_step(ids [B]) feeds one new token per sequence at the next position and returns its logits [B, V].
    // The blocks' attention is causal from the prefill on (a cached key never sees a later query).  Every tensor
    // that feeds a product is quantised per tensor, as in the batched forward: a step's tensors are [B, .].
    // A prefill opens a decoding session that lasts until end_decode() or the next prefill: the model's parameters
    // and options must not change inside it (from the third step on the launches are replayed from a CUDA graph
    // that holds the buffers' addresses).
    tensor<T> prefill(const tensor<int>& ids, int max_len = 0, bool check_ids = true);
    tensor<T> decode_step(const tensor<int>& next_ids, bool check_ids = true);
    int decode_position() const { return kv_len_; }
    bool decode_graph_active() const { return dec_graph_ != nullptr; }
    void end_decode();

    // Layer streaming (README.md:212-220 sketches `layer->load_weights_to_gpu()`; no such code exists
    // upstream).  The e4m3 codes of every block's four weight matrices move to pinned host memory; the
    // device keeps `slots` layer-sized buffers; during a forward the upload of layer l+slots runs on a side
    // stream while layer l computes.  Scales, biases and LayerNorm parameters stay resident.
    // release_fp32 also frees the blocks' fp32 master weights on the device (weights() then returns
    // empty tensors; re-uploading them requires disabling streaming first).
    // With `comm` (ranks that work on shares of one batch, one process per GPU) each rank uploads 1/world of a
    // layer and an all-gather over NVLink on the copy stream completes the slot; every rank must then run the
    // same sequence of forwards.
    void enable_layer_streaming(int slots = 2, bool release_fp32 = false, df8_comm* comm = nullptr);
    void disable_layer_streaming();
    bool layer_streaming() const { return streamer_ != nullptr; }
    unsigned long long streamed_bytes() const;
    // measurement aids: another number of device slots (all layers resident when slots >= layers), the bytes
    // this rank copied from the host / received from its peers, and the device time of uploading every layer
    // once with nothing else running
    void resize_streaming_slots(int slots);
    void streaming_traffic(unsigned long long* h2d_bytes, unsigned long long* gathered_bytes) const;
    float time_layer_uploads();

    int vocab_size() const { return vocab_size_; }
    int hidden_dim() const { return hidden_dim_; }
    int num_layers() const { return int(transformer_blocks_.size()); }
    TokenEmbedding<T>& token_embedding() { return *token_embedding_; }
    PositionalEncoding<T>& positional_encoding() { return *positional_encoding_; }
    TransformerBlock<T>& block(int i) { return *transformer_blocks_.at(size_t(i)); }
    FullyConnectedLayer<T>& final_fc() { return *final_fc_; }

private:
    void initialize_weights(tensor<T>* weights, T scale);

    int vocab_size_;
    int max_seq_len_;
    int hidden_dim_;
    std::unique_ptr<TokenEmbedding<T>> token_embedding_;
    std::unique_ptr<PositionalEncoding<T>> positional_encoding_;
    std::vector<std::unique_ptr<TransformerBlock<T>>> transformer_blocks_;
    std::unique_ptr<FullyConnectedLayer<T>> final_fc_;
    fp8::Quantized head_q_;
    df8_streamer* streamer_ = nullptr;
    int stream_slots_ = 0;
    std::vector<std::unique_ptr<typename MultiHeadAttentionLayer<T>::KvCache>> kv_;
    int kv_len_ = 0;
    // decode steps: the position lives in device memory, the step's buffers persist, and from the second step on the
    // step's launches are replayed from a CUDA graph captured on the model's stream (a step is ~165 kernels of a few
    // microseconds; issued one by one it is bound by the host).  DF8_DECODE_GRAPH=0 in the environment or the legacy
    // default stream keep the launches eager.
    void decode_body(int B);
    tensor<int> dec_pos_{{1}};
    tensor<int> dec_ids_{{0}};
    tensor<T> dec_x_{{0}}, dec_logits_{{0}};
    cudaGraphExec_t dec_graph_ = nullptr;
    bool dec_graph_ok_ = true;
    int dec_steps_ = 0;
    tensor<T> last_rows_logits(const float* x, int B, int T_len);
    bool stage_timing_ = false;
    cudaEvent_t head_ev_[2] = {nullptr, nullptr};
    void head_gemm(int M, float* logits, int pitch);

public:
    ~Gpt2() override;
};

}  // namespace dnn
