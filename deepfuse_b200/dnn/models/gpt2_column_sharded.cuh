// Gpt2ColumnSharded<T>: the GPT-2 forward with every fully-connected weight matrix split by output columns
// across the ranks of one communicator (one process per GPU).
//
// Upstream has nothing of the kind: its multi-GPU program runs independent model replicas under a
// tbb::parallel_for (apps/host-multi/main.cpp:157-181) and each FullyConnectedLayer holds its whole [out,in]
// weight (dnn/layers/fully_connected_layer.cu:112-116).  The wiring of a block is upstream's
// (dnn/layers/transformer_block.cu:59-86, models/gpt2.cu:66-83); what is new is where the data lives.
// With g ranks, M = B*T token rows, E = hidden and F = MLP width:
//
//   residual stream                   SHARDED by columns: rank r holds x[:, r*E/g : (r+1)*E/g] in fp32; the
//                                     out-projection and FC2 GEMMs add their [M, E/g] output slice to it in
//                                     their epilogue, so no fp32 activation ever crosses GPUs
//   LayerNorm + quantise              row statistics of the pieces are exchanged (two floats per row,
//                                     df8_layernorm_shard_*), then max|y| (one float), then each rank quantises
//                                     its columns and the fp8 CODES are gathered: [g][M, E/g] on every rank
//   QKV projection                    rank r owns the rows {Q_h, K_h, V_h : h in its H/g heads} of the fused
//                                     [3E,E] weight; its [M,3E/g] output is the QKV buffer of those heads, so
//                                     attention runs locally.  Per-tensor scale: max|out| pass, maximum over
//                                     ranks (one float), codes pass.
//   attention output                  [M,E/g] fp32 per rank -> maximum over ranks -> quantise -> codes gathered
//   FC1 (+GELU)                       max pass -> maximum over ranks -> codes pass straight into this rank's slab
//                                     of the gathered buffer -> codes gathered: [g][M, F/g]
//   out projection, FC2               read the gathered codes in place as g K-slabs (df8_gemm_fp8_tn_ex), write
//                                     x + out slice
//   vocabulary head                   the last hidden states are quantised like an activation and gathered;
//                                     rank r owns a contiguous block of vocabulary rows; logits stay sharded
//
// Bytes a rank receives per layer: (g-1)/g * M * (3E + F) of fp8 codes plus 2 * 8 * M bytes of row statistics
// (the first version of this model gathered the fp32 out-projection / FC2 slices: M * (E + F) + 8 * M * E).
// Exchanges use peer-mapped buffers and the copy engines (df8_comm_allgather_symm, df8_comm_allreduce_max_p2p),
// NCCL only as the fallback.  With a single rank (no communicator) the model is the unsharded one and
// reproduces dnn::Gpt2 bit for bit; with several ranks the LayerNorm sums are taken in another order, so it
// agrees with dnn::Gpt2 to the extent two roundings of the same 8-bit pipeline do (see the tests).
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
    // the same in a row-pitched buffer [B*T, logits_pitch()] (vocab_rows() rounded up to a multiple of 32 floats:
    // rows then start on 16-byte boundaries and the head GEMM's epilogue leaves through TMA stores)
    tensor<T> forward_logits_shard_pitched(const tensor<int>& ids, bool check_ids = true);
    int logits_pitch() const { return (vocab_rows_ + 31) / 32 * 32; }
    // hidden states after the last block, [B,T,E], gathered onto every rank (fp32; for inspection and tests)
    tensor<T> forward_hidden(const tensor<int>& ids, bool check_ids = true);
    // bytes this rank has pushed to its peers so far (0 with a single rank or on the NCCL fallback)
    unsigned long long bytes_pushed() const;

    void set_mlp_gelu(bool on) { mlp_gelu_ = on; }
    void set_causal(bool causal) { causal_ = causal; }
    // Device-side random initialisation of this rank's shards (N(0, std), the rows Gpt2::initialize_on_device with the
    // same seed gives the unsharded model), for shapes too large to initialise through the host.
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
    // ---- single rank: the unsharded forward on replicated tensors ----
    void block_forward_single(Block& b, float* x, int B, int T_len);
    // ---- several ranks ----
    void ensure_work_space(int M);
    void run_blocks_sharded(const tensor<int>& ids, bool check_ids, int* M_out);  // leaves the hidden states in x_shard_
    void block_forward_sharded(Block& b, int B, int T_len);
    // LayerNorm of the sharded tensor x (this rank's [M, E/g] columns) -> codes of all columns in sym_ln_, scale in ln_scale_
    void layernorm_quantize_sharded(LayerNormLayer<T>& norm, const float* x, int M, int which);
    // per-tensor quantisation of a sharded fp32 tensor [M, E/g] into this rank's slab of `sym`, then gather
    void quantize_gather_sharded(const float* x, int M, float* amax, uint8_t* sym, float* scale);
    void all_max(float* amax);
    int chunks_for(int M) const;
    void head(int M, float* logits, int pitch);

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
    fp8::Quantized ln_q_, qkvq_, attnq_, hidden_q_, head_q_;
    tensor<float> attn_f32_{{0}}, x1_{{0}}, x_shard_{{0}}, x1_shard_{{0}}, row_stats_{{0}};
    tensor<float> amax_, ln_scale_{{2}}, attn_scale_{{2}}, hidden_scale_{{2}};
    // buffers mapped into every peer (df8_comm_symm_alloc; owned by the communicator): fp8 codes of all columns as
    // g slabs [g][M, cols/g], and the LayerNorm row statistics [2][g][M][2]
    // pipelined gathers (several ranks, peer-mapped transport): a gathered tensor travels in row chunks; the producer
    // pushes a chunk as soon as it is quantised and the consuming GEMM runs chunk by chunk behind the tickets
    bool p2p_ = false;
    int chunks_ = 4;  // DF8_SHARD_CHUNKS in the environment; 1 = whole-tensor gathers
    int chunk_min_rows_ = 2048;  // smaller chunks do not fill the GPU (DF8_SHARD_CHUNK_MIN_ROWS)
    unsigned int tickets_ln_[8] = {}, tickets_attn_[8] = {}, tickets_hidden_[8] = {};
    int work_rows_ = 0;
    uint8_t *sym_ln_ = nullptr, *sym_attn_ = nullptr, *sym_hidden_ = nullptr;
    float* sym_stats_ = nullptr;
};

}  // namespace dnn
