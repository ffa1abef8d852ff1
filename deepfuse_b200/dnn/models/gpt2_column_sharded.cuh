// Gpt2ColumnSharded<T>: the GPT-2 forward with every fully-connected weight matrix split by output columns
// across the ranks of one NCCL communicator (one process per GPU).
//
// Upstream has nothing of the kind: its multi-GPU program runs independent model replicas under a
// tbb::parallel_for (apps/host-multi/main.cpp:157-181) and each FullyConnectedLayer holds its whole [out,in]
// weight (dnn/layers/fully_connected_layer.cu:112-116).  The wiring of a block is upstream's
// (dnn/layers/transformer_block.cu:59-86, models/gpt2.cu:66-83); what is new is where the data lives:
//
//   residual stream x [M,E] fp32      replicated on every rank
//   LayerNorm + quantise              computed redundantly on every rank (cheap, no exchange)
//   QKV projection                    rank r owns the rows {Q_h, K_h, V_h : h in its H/g heads} of the fused
//                                     [3E,E] weight; its [M,3E/g] output is the QKV buffer of those heads, so
//                                     attention runs locally with no exchange.  Per-tensor scale: the
//                                     max|out| pass is all-reduced (one float) before the codes pass.
//   attention output                  [M,E/g] fp32 per rank -> all-reduce(max) -> quantise -> all-gather of
//                                     the codes -> [M,E] on every rank
//   out projection, FC2               rank r owns E/g output columns; the fp32 [M,E/g] results are
//                                     all-gathered and added to the replicated residual stream
//   FC1 (+GELU)                       df8_fc_fp8_column_sharded: max pass -> all-reduce -> codes pass ->
//                                     all-gather of codes
//   vocabulary head                   rank r owns a contiguous block of vocabulary rows; the logits stay
//                                     sharded ([M, V_r] per rank)
//
// With identical weights the result is bit-identical to Gpt2<T>::forward_logits on one GPU (every output
// element sees the same products in the same order; every per-tensor maximum is the maximum over all ranks).
#pragma once

#include <memory>
#include <vector>

#include "dnn/layers/fully_connected_layer.cuh"
#include "dnn/layers/layer_norm_layer.cuh"
#include "dnn/tokens/positional_encoding.cuh"
#include "dnn/tokens/token_embedding.cuh"

namespace dnn {

template <typename T>
class Gpt2ColumnSharded {
public:
    struct Block {
        Block(int E, int Eg, int F, int Fg);
        LayerNormLayer<T> norm1, norm2;
        FullyConnectedLayer<T> qkv;  // E -> 3E/g   rows [Q_r; K_r; V_r]
        FullyConnectedLayer<T> out;  // E -> E/g
        FullyConnectedLayer<T> fc1;  // E -> F/g
        FullyConnectedLayer<T> fc2;  // F -> E/g
    };

    // `comm` stays owned by the caller and must outlive the model.  hidden, ffn and heads must be divisible
    // by the communicator's size (and ffn / size by 32: fp8 output tiles).
    Gpt2ColumnSharded(df8_comm* comm, int vocab_size, int max_seq_len, int num_layers, int num_heads, int hidden_dim,
                      int intermediate_dim);

    // logits of this rank's vocabulary rows: [B*T, vocab_rows()] fp32
    tensor<T> forward_logits_shard(const tensor<int>& ids, bool check_ids = true);
    // hidden states after the last block, [B,T,E], identical on every rank
    tensor<T> forward_hidden(const tensor<int>& ids, bool check_ids = true);

    void set_mlp_gelu(bool on) { mlp_gelu_ = on; }
    void set_causal(bool causal) { causal_ = causal; }
    // Device-side random initialisation of this rank's shards (uniform, the N(0, 0.02) standard deviation),
    // for shapes too large to initialise through the host.
    void initialize_on_device(uint64_t seed, float std = 0.02f);

    int rank() const { return rank_; }
    int world() const { return world_; }
    int vocab_begin() const { return vocab_begin_; }
    int vocab_rows() const { return vocab_rows_; }
    int num_layers() const { return int(blocks_.size()); }
    int hidden_dim() const { return hidden_dim_; }
    Block& block(int i) { return *blocks_.at(size_t(i)); }
    TokenEmbedding<T>& token_embedding() { return *token_embedding_; }
    PositionalEncoding<T>& positional_encoding() { return *positional_encoding_; }
    FullyConnectedLayer<T>& final_fc() { return *final_fc_; }

private:
    void block_forward(Block& b, float* x, int B, int T_len);
    // all-gather `bytes_per_row`-byte rows of the [M, .] shard `local` and lay them out as [M, world * bytes_per_row]
    void gather_columns(const void* local, int M, int bytes_per_row, void* full);

    df8_comm* comm_;
    int rank_ = 0, world_ = 1;
    int vocab_size_, hidden_dim_, ffn_dim_, num_heads_;
    int vocab_begin_ = 0, vocab_rows_ = 0;
    bool mlp_gelu_ = true, causal_ = false;
    std::unique_ptr<TokenEmbedding<T>> token_embedding_;
    std::unique_ptr<PositionalEncoding<T>> positional_encoding_;
    std::vector<std::unique_ptr<Block>> blocks_;
    std::unique_ptr<FullyConnectedLayer<T>> final_fc_;
    // work space, sized on first use
    fp8::Quantized ln_q_, qkvq_, attnq_local_, attnq_, hidden_q_, head_q_;
    tensor<float> attn_f32_{{0}}, y_local_{{0}}, y_full_{{0}}, x1_{{0}};
    tensor<uint8_t> gathered_{{0}}, slice_{{0}};
    tensor<float> amax_;
};

}  // namespace dnn
