#include "dnn/models/gpt2_column_sharded.cuh"

#include <stdexcept>
#include <string>

namespace dnn {

namespace {

__global__ void add_kernel_f32(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                               size_t n4) {
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += size_t(gridDim.x) * blockDim.x) {
        const float4 x = a4[i], y = b4[i];
        o4[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
}

// out = a + b, n a multiple of 4 and the pointers 16-byte aligned (rows of E floats, E % 16 == 0)
void add_f32(const float* a, const float* b, float* out, size_t n) {
    if (n == 0) return;
    add_kernel_f32<<<1184, 256, 0, Cuda::stream()>>>(a, b, out, n / 4);
    utils::CHECK_CUDA_EX(cudaGetLastError());
}

template <typename TensorT>
void ensure(TensorT& t, size_t n) {
    if (t.numel() != n) t = TensorT({int(n)});
}

}  // namespace

template <typename T>
Gpt2ColumnSharded<T>::Block::Block(int E, int Eg, int F, int Fg)
    : norm1(E, 1e-5f), norm2(E, 1e-5f), qkv(E, 3 * Eg), out(E, Eg), fc1(E, Fg), fc2(F, Eg) {}

template <typename T>
Gpt2ColumnSharded<T>::Gpt2ColumnSharded(df8_comm* comm, int vocab_size, int max_seq_len, int num_layers,
                                        int num_heads, int hidden_dim, int intermediate_dim)
    : comm_(comm),
      vocab_size_(vocab_size),
      hidden_dim_(hidden_dim),
      ffn_dim_(intermediate_dim),
      num_heads_(num_heads),
      amax_({1}) {
    if (comm_) utils::CHECK_DF8(df8_comm_rank(comm_, &rank_, &world_));
    if (vocab_size <= 0 || max_seq_len <= 0 || num_layers <= 0 || num_heads <= 0 || hidden_dim <= 0 ||
        intermediate_dim <= 0)
        throw std::invalid_argument("Gpt2ColumnSharded: sizes must be positive");
    if (hidden_dim % num_heads != 0) throw std::runtime_error("embed_dim must be divisible by num_heads");
    if (num_heads % world_ != 0 || hidden_dim % (16 * world_) != 0 || intermediate_dim % (32 * world_) != 0 ||
        (3 * hidden_dim / world_) % 32 != 0)
        throw std::invalid_argument("Gpt2ColumnSharded: heads, hidden_dim / 16 and intermediate_dim / 32 must be "
                                    "divisible by the number of ranks (" + std::to_string(world_) + ")");
    const int Eg = hidden_dim / world_, Fg = intermediate_dim / world_;
    const int per_rank = (vocab_size + world_ - 1) / world_;
    vocab_begin_ = std::min(rank_ * per_rank, vocab_size);
    vocab_rows_ = std::min(per_rank, vocab_size - vocab_begin_);
    if (vocab_rows_ <= 0) throw std::invalid_argument("Gpt2ColumnSharded: more ranks than vocabulary rows");

    token_embedding_ = std::make_unique<TokenEmbedding<T>>(vocab_size, hidden_dim, max_seq_len);
    positional_encoding_ = std::make_unique<PositionalEncoding<T>>(hidden_dim, max_seq_len);
    for (int i = 0; i < num_layers; ++i) {
        blocks_.push_back(std::make_unique<Block>(hidden_dim, Eg, intermediate_dim, Fg));
        if (world_ > 1) {
            Block& b = *blocks_.back();
            b.qkv.set_shard_comm(comm_);
            b.out.set_shard_comm(comm_);
            b.fc1.set_shard_comm(comm_);
            b.fc2.set_shard_comm(comm_);
        }
    }
    final_fc_ = std::make_unique<FullyConnectedLayer<T>>(hidden_dim, vocab_rows_);
    if (world_ > 1) final_fc_->set_shard_comm(comm_);
}

// The shards of the model dnn::Gpt2::initialize_on_device(seed, std) makes: every rank fills its rows of each
// global weight matrix from the same counter-based streams (qkv: the rows of this rank's heads inside the Q, the
// K and the V block of the fused [3E, E] matrix).
template <typename T>
void Gpt2ColumnSharded<T>::initialize_on_device(uint64_t seed, float std) {
    uint64_t k = seed * 1000ull;
    const uint64_t E = uint64_t(hidden_dim_), F = uint64_t(ffn_dim_);
    const int Eg = hidden_dim_ / world_, Fg = ffn_dim_ / world_;
    tensor<T>* emb = token_embedding_->weights();  // replicated
    fp8::fill_normal(emb->data(), emb->numel(), 0.f, std, ++k);
    emb->bump_version();
    for (auto& bp : blocks_) {
        Block& b = *bp;
        ++k;
        for (int part = 0; part < 3; ++part)  // Q, K, V
            b.qkv.initialize_rows_normal_on_device(std, k, (uint64_t(part) * E + uint64_t(rank_) * Eg) * E, part * Eg, Eg);
        b.out.initialize_rows_normal_on_device(std, ++k, uint64_t(rank_) * Eg * E, 0, Eg);
        b.fc1.initialize_rows_normal_on_device(std, ++k, uint64_t(rank_) * Fg * E, 0, Fg);
        b.fc2.initialize_rows_normal_on_device(std, ++k, uint64_t(rank_) * Eg * F, 0, Eg);
    }
    final_fc_->initialize_rows_normal_on_device(std, ++k, uint64_t(vocab_begin_) * E, 0, vocab_rows_);
}

template <typename T>
void Gpt2ColumnSharded<T>::gather_columns(const void* local, int M, int bytes_per_row, void* full) {
    const size_t bytes = size_t(M) * size_t(bytes_per_row);
    if (world_ == 1) {
        utils::CHECK_CUDA_EX(cudaMemcpyAsync(full, local, bytes, cudaMemcpyDeviceToDevice, Cuda::stream()));
        return;
    }
    if (gathered_.numel() < bytes * size_t(world_)) throw std::runtime_error("Gpt2ColumnSharded: gather buffer too small");
    utils::CHECK_DF8(df8_comm_allgather_u8(comm_, static_cast<const uint8_t*>(local), gathered_.data(), bytes,
                                           fp8::stream()));
    utils::CHECK_DF8(df8_interleave_gathered_u8(gathered_.data(), M, bytes_per_row, world_,
                                                static_cast<uint8_t*>(full), fp8::stream()));
}

template <typename T>
void Gpt2ColumnSharded<T>::block_forward(Block& b, float* x, int B, int T_len) {
    const int M = B * T_len, E = hidden_dim_, F = ffn_dim_;
    const int Eg = E / world_, Fg = F / world_, Hg = num_heads_ / world_, D = E / num_heads_;
    const df8_kind act = fp8::policy().activation_kind;
    const df8_stream st = fp8::stream();
    fp8::PassScope amax_slots;
    auto all_max = [&](float* am) {
        if (world_ > 1) utils::CHECK_DF8(df8_comm_allreduce_max_f32(comm_, am, 1, st));
    };
    ensure(qkvq_.codes, size_t(M) * 3 * Eg);
    ensure(attn_f32_, size_t(M) * Eg);
    ensure(attnq_.codes, size_t(M) * E);
    ensure(y_local_, size_t(M) * Eg);
    ensure(y_full_, size_t(M) * E);
    ensure(x1_, size_t(M) * E);
    ensure(hidden_q_.codes, size_t(M) * F);
    ensure(slice_, size_t(M) * Fg);
    ensure(gathered_, size_t(M) * std::max(size_t(F), size_t(E) * 4));

    // ---- x1 = x + out_proj(attention(QKV(LN1(x)))) ----
    b.norm1.forward_quantized(x, M, act, ln_q_);
    {   // QKV of this rank's heads: max|out| over all ranks, then the codes
        const fp8::Quantized& w = b.qkv.quantized_weights();
        float* am = fp8::amax_slot(amax_.data());
        utils::CHECK_DF8(df8_gemm_fp8_tn_amax(ln_q_.codes.data(), ln_q_.kind, ln_q_.scale.data(), w.codes.data(), w.kind,
                                              w.scale.data(), b.qkv.bias()->data(), M, 3 * Eg, E, 0, am, st));
        all_max(am);
        qkvq_.kind = act;
        utils::CHECK_DF8(df8_gemm_fp8_tn_codes(ln_q_.codes.data(), ln_q_.kind, ln_q_.scale.data(), w.codes.data(), w.kind,
                                               w.scale.data(), b.qkv.bias()->data(), M, 3 * Eg, E, 0, act, am,
                                               qkvq_.codes.data(), qkvq_.scale.data(), st));
    }
    {   // attention of the local heads; its output is quantised with the maximum over all heads
        float* am = fp8::amax_slot(amax_.data());
        utils::CHECK_DF8(df8_attention_fp8(qkvq_.codes.data(), qkvq_.kind, qkvq_.scale.data(), B, T_len, Hg, D,
                                           causal_ ? DF8_MASK_CAUSAL : DF8_MASK_NONE, nullptr, 0, attn_f32_.data(), am,
                                           st));
        all_max(am);
        fp8::quantize_with_amax(attn_f32_.data(), size_t(M) * Eg, act, am, attnq_local_);
        gather_columns(attnq_local_.codes.data(), M, Eg, attnq_.codes.data());
        attnq_.kind = act;
    }
    b.out.forward_codes(attnq_.codes.data(), attnq_.kind, attnq_local_.scale.data(), M, 0, nullptr, y_local_.data(),
                        nullptr);
    gather_columns(y_local_.data(), M, Eg * int(sizeof(float)), y_full_.data());
    add_f32(x, y_full_.data(), x1_.data(), size_t(M) * E);

    // ---- x = x1 + FC2(act(FC1(LN2(x1)))) ----
    b.norm2.forward_quantized(x1_.data(), M, act, ln_q_);
    {
        const fp8::Quantized& w = b.fc1.quantized_weights();
        float* am = fp8::amax_slot(amax_.data());
        hidden_q_.kind = act;
        if (world_ > 1) {
            utils::CHECK_DF8(df8_fc_fp8_column_sharded(comm_, ln_q_.codes.data(), ln_q_.kind, ln_q_.scale.data(),
                                                       w.codes.data(), w.kind, w.scale.data(), b.fc1.bias()->data(), M,
                                                       F, E, mlp_gelu_ ? DF8_EPI_GELU : 0, act, slice_.data(),
                                                       gathered_.data(), hidden_q_.codes.data(),
                                                       hidden_q_.scale.data(), am, st));
        } else {
            utils::CHECK_DF8(df8_gemm_fp8_tn_q(ln_q_.codes.data(), ln_q_.kind, ln_q_.scale.data(), w.codes.data(), w.kind,
                                               w.scale.data(), b.fc1.bias()->data(), M, F, E,
                                               mlp_gelu_ ? DF8_EPI_GELU : 0, act, hidden_q_.codes.data(),
                                               hidden_q_.scale.data(), am, st));
        }
    }
    b.fc2.forward_codes(hidden_q_.codes.data(), hidden_q_.kind, hidden_q_.scale.data(), M, 0, nullptr, y_local_.data(),
                        nullptr);
    gather_columns(y_local_.data(), M, Eg * int(sizeof(float)), y_full_.data());
    add_f32(x1_.data(), y_full_.data(), x, size_t(M) * E);
}

template <typename T>
tensor<T> Gpt2ColumnSharded<T>::forward_hidden(const tensor<int>& ids, bool check_ids) {
    const auto& s = ids.shape();
    if (s.size() != 2) throw std::runtime_error("Gpt2ColumnSharded expects token ids shaped [B, T]");
    const int B = s[0], T_len = s[1];
    if (T_len > positional_encoding_->max_seq_len())
        throw std::runtime_error("Input sequence length exceeds maximum allowed length");
    fp8::PassScope amax_slots;
    tensor<T> x = token_embedding_->forward_with_positions(ids, positional_encoding_->table().data(), check_ids);
    for (auto& b : blocks_) block_forward(*b, x.data(), B, T_len);
    return x;
}

template <typename T>
tensor<T> Gpt2ColumnSharded<T>::forward_logits_shard(const tensor<int>& ids, bool check_ids) {
    fp8::PassScope amax_slots;
    tensor<T> x = forward_hidden(ids, check_ids);
    const int M = int(x.numel() / size_t(hidden_dim_));
    fp8::quantize(x.data(), x.numel(), fp8::policy().activation_kind, head_q_);
    tensor<T> logits({M, vocab_rows_});
    final_fc_->forward_codes(head_q_.codes.data(), head_q_.kind, head_q_.scale.data(), M, 0, nullptr, logits.data(),
                             nullptr);
    return logits;
}

template class Gpt2ColumnSharded<float>;

}  // namespace dnn
