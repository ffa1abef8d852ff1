#include "dnn/models/gpt2_column_sharded.cuh"

#include <cstdlib>

#include <stdexcept>
#include <string>

namespace dnn {

namespace {

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
    // the gathered codes are read in place as one K slab per rank; a slab is whole 128-column K blocks
    if (world_ > 1 && ((hidden_dim / world_) % 128 != 0 || (intermediate_dim / world_) % 128 != 0))
        throw std::invalid_argument("Gpt2ColumnSharded: hidden_dim and intermediate_dim must be multiples of 128 x the "
                                    "number of ranks (" + std::to_string(world_) + ")");
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

// ---- single rank ----------------------------------------------------------------------------------

template <typename T>
void Gpt2ColumnSharded<T>::block_forward_single(Block& b, float* x, int B, int T_len) {
    const int M = B * T_len, E = hidden_dim_, F = ffn_dim_;
    const df8_kind act = fp8::policy().activation_kind;
    const df8_stream st = fp8::stream();
    fp8::PassScope amax_slots;
    ensure(x1_, size_t(M) * E);
    ensure(attn_f32_, size_t(M) * E);
    b.norm1.forward_quantized(x, M, act, ln_q_);
    b.qkv.forward_codes_quantized(ln_q_.codes.data(), ln_q_.kind, ln_q_.scale.data(), M, 0, act, qkvq_);
    float* am = fp8::amax_slot(amax_.data());
    utils::CHECK_DF8(df8_attention_fp8(qkvq_.codes.data(), qkvq_.kind, qkvq_.scale.data(), B, T_len, num_heads_,
                                       E / num_heads_, causal_ ? DF8_MASK_CAUSAL : DF8_MASK_NONE, nullptr, 0,
                                       attn_f32_.data(), am, st));
    fp8::quantize_with_amax(attn_f32_.data(), size_t(M) * E, act, am, attnq_);
    b.out.forward_codes(attnq_.codes.data(), attnq_.kind, attnq_.scale.data(), M, DF8_EPI_RESIDUAL, x, x1_.data(), nullptr);
    b.norm2.forward_quantized(x1_.data(), M, act, ln_q_);
    b.fc1.forward_codes_quantized(ln_q_.codes.data(), ln_q_.kind, ln_q_.scale.data(), M, mlp_gelu_ ? DF8_EPI_GELU : 0, act,
                                  hidden_q_);
    b.fc2.forward_codes(hidden_q_.codes.data(), hidden_q_.kind, hidden_q_.scale.data(), M, DF8_EPI_RESIDUAL, x1_.data(), x,
                        nullptr);
    (void)F;
}

// ---- several ranks --------------------------------------------------------------------------------

template <typename T>
void Gpt2ColumnSharded<T>::all_max(float* amax) {
    utils::CHECK_DF8(df8_comm_allreduce_max_p2p(comm_, amax, fp8::stream()));
}

// The buffers every peer writes into are allocated collectively, for the largest M seen so far (a buffer of the
// communicator lives as long as the communicator).
template <typename T>
void Gpt2ColumnSharded<T>::ensure_work_space(int M) {
    const size_t E = size_t(hidden_dim_), F = size_t(ffn_dim_), g = size_t(world_);
    if (M > work_rows_) {
        void* p = nullptr;
        utils::CHECK_DF8(df8_comm_symm_alloc(comm_, size_t(M) * E, &p));
        sym_ln_ = static_cast<uint8_t*>(p);
        utils::CHECK_DF8(df8_comm_symm_alloc(comm_, size_t(M) * E, &p));
        sym_attn_ = static_cast<uint8_t*>(p);
        utils::CHECK_DF8(df8_comm_symm_alloc(comm_, size_t(M) * F, &p));
        sym_hidden_ = static_cast<uint8_t*>(p);
        utils::CHECK_DF8(df8_comm_symm_alloc(comm_, 2 * g * size_t(M) * 2 * sizeof(float), &p));
        sym_stats_ = static_cast<float*>(p);
        work_rows_ = M;
        int enabled = 0;
        utils::CHECK_DF8(df8_comm_p2p_enabled(comm_, &enabled));
        p2p_ = enabled != 0;
        if (const char* e = getenv("DF8_SHARD_CHUNKS")) {  // profiling and tests
            const int n = atoi(e);
            if (n == 1 || n == 2 || n == 4 || n == 8) chunks_ = n;
        }
        if (const char* e = getenv("DF8_SHARD_CHUNK_MIN_ROWS")) {  // tests: small models still exercise the pipeline
            const int n = atoi(e);
            if (n >= 128) chunk_min_rows_ = n;
        }
    }
    ensure(x_shard_, size_t(M) * E / g);
    ensure(x1_shard_, size_t(M) * E / g);
    ensure(attn_f32_, size_t(M) * E / g);
    ensure(row_stats_, size_t(M) * 2);
    ensure(qkvq_.codes, size_t(M) * 3 * E / g);
}

template <typename T>
void Gpt2ColumnSharded<T>::layernorm_quantize_sharded(LayerNormLayer<T>& norm, const float* x, int M, int which) {
    const int Eg = hidden_dim_ / world_;
    const df8_kind act = fp8::policy().activation_kind;
    const df8_stream st = fp8::stream();
    auto params = norm.parameters();  // {gamma, beta}, replicated
    const float* gamma = params.size() > 0 ? params[0]->data() + size_t(rank_) * Eg : nullptr;
    const float* beta = params.size() > 1 ? params[1]->data() + size_t(rank_) * Eg : nullptr;
    // statistics of the row pieces: this rank's [M][2] goes straight into its slot of the gathered array
    float* stats_all = sym_stats_ + size_t(which) * size_t(world_) * size_t(work_rows_) * 2;
    const size_t slot_bytes = size_t(M) * 2 * sizeof(float);
    float* mine = stats_all + size_t(rank_) * size_t(M) * 2;
    utils::CHECK_DF8(df8_layernorm_shard_stats_f32(x, M, Eg, mine, st));
    utils::CHECK_DF8(df8_comm_allgather_symm(comm_, stats_all, 0, slot_bytes, st));
    float* am = fp8::amax_slot(amax_.data());
    utils::CHECK_DF8(df8_layernorm_shard_amax_f32(x, M, Eg, stats_all, world_, gamma, beta, norm.epsilon(),
                                                  row_stats_.data(), am, st));
    all_max(am);
    const int nc = chunks_for(M);
    if (nc == 1) {
        utils::CHECK_DF8(df8_layernorm_shard_quantize_f32(x, M, Eg, row_stats_.data(), gamma, beta, act, am,
                                                          sym_ln_ + size_t(rank_) * size_t(M) * Eg, ln_scale_.data(), st));
        utils::CHECK_DF8(df8_comm_allgather_symm(comm_, sym_ln_, 0, size_t(M) * Eg, st));
        return;
    }
    // row chunks: a chunk is on its way to the peers while the next one is quantised; the consumer (a GEMM over the
    // same row chunk) waits for its ticket
    const int Mc = M / nc;
    for (int c = 0; c < nc; ++c) {
        const size_t off = size_t(rank_) * size_t(M) * Eg + size_t(c) * Mc * Eg;
        utils::CHECK_DF8(df8_layernorm_shard_quantize_f32(x + size_t(c) * Mc * Eg, Mc, Eg, row_stats_.data() + size_t(c) * Mc * 2,
                                                          gamma, beta, act, am, sym_ln_ + off, ln_scale_.data(), st));
        utils::CHECK_DF8(df8_comm_push_symm(comm_, sym_ln_, off, size_t(Mc) * Eg, st, &tickets_ln_[c]));
    }
}

// Row chunks of a pipelined gather: only over the peer-mapped transport, and only when the chunks stay whole GEMM
// tiles (128 rows) and large enough to fill the GPU.
template <typename T>
int Gpt2ColumnSharded<T>::chunks_for(int M) const {
    if (world_ == 1 || !p2p_ || chunks_ <= 1) return 1;
    int nc = chunks_;
    while (nc > 1 && (M % (nc * 128) != 0 || M / nc < chunk_min_rows_)) nc >>= 1;
    return nc;
}

template <typename T>
void Gpt2ColumnSharded<T>::quantize_gather_sharded(const float* x, int M, float* amax, uint8_t* sym, float* scale) {
    const int Eg = hidden_dim_ / world_;
    const df8_kind act = fp8::policy().activation_kind;
    const df8_stream st = fp8::stream();
    all_max(amax);
    const int nc = chunks_for(M);
    if (nc == 1) {
        utils::CHECK_DF8(df8_quantize_f32(x, size_t(M) * Eg, act, amax, sym + size_t(rank_) * size_t(M) * Eg, scale, st));
        utils::CHECK_DF8(df8_comm_allgather_symm(comm_, sym, 0, size_t(M) * Eg, st));
        return;
    }
    const int Mc = M / nc;
    for (int c = 0; c < nc; ++c) {
        const size_t off = size_t(rank_) * size_t(M) * Eg + size_t(c) * Mc * Eg;
        utils::CHECK_DF8(df8_quantize_f32(x + size_t(c) * Mc * Eg, size_t(Mc) * Eg, act, amax, sym + off, scale, st));
        utils::CHECK_DF8(df8_comm_push_symm(comm_, sym, off, size_t(Mc) * Eg, st, &tickets_attn_[c]));
    }
}

template <typename T>
void Gpt2ColumnSharded<T>::block_forward_sharded(Block& b, int B, int T_len) {
    const int M = B * T_len, E = hidden_dim_, F = ffn_dim_, g = world_;
    const int Eg = E / g, Fg = F / g, Hg = num_heads_ / g, D = E / num_heads_;
    const df8_kind act = fp8::policy().activation_kind;
    const df8_stream st = fp8::stream();
    fp8::PassScope amax_slots;
    float* x = x_shard_.data();
    float* x1 = x1_shard_.data();

    const int nc = chunks_for(M), Mc = M / nc;
    // consumers of a chunked gather: wait for the chunk's ticket (the last one also for this rank's own pushes, after
    // which its slab may be rewritten), then work on that row range of the gathered slabs
    auto wait_chunk = [&](const unsigned int* tickets, int c) {
        if (nc > 1) utils::CHECK_DF8(df8_comm_wait_symm(comm_, tickets[c], c == nc - 1 ? 1 : 0, st));
    };

    // ---- x1 = x + out_proj(attention(QKV(LN1(x)))) ----
    layernorm_quantize_sharded(b.norm1, x, M, 0);
    {   // QKV of this rank's heads: max|out| over all ranks, then the codes
        const fp8::Quantized& w = b.qkv.quantized_weights();
        float* am = fp8::amax_slot(amax_.data());
        for (int c = 0; c < nc; ++c) {
            wait_chunk(tickets_ln_, c);
            utils::CHECK_DF8(df8_gemm_fp8_tn_amax_part(sym_ln_ + size_t(c) * Mc * Eg, act, ln_scale_.data(), g, M, w.codes.data(),
                                                       w.kind, w.scale.data(), b.qkv.bias()->data(), Mc, 3 * Eg, E, 0, am, st));
        }
        all_max(am);
        qkvq_.kind = act;
        utils::CHECK_DF8(df8_gemm_fp8_tn_codes_ex(sym_ln_, act, ln_scale_.data(), g, w.codes.data(), w.kind,
                                                  w.scale.data(), b.qkv.bias()->data(), M, 3 * Eg, E, 0, act, am,
                                                  qkvq_.codes.data(), qkvq_.scale.data(), st));
    }
    {   // attention of the local heads; its output is quantised with the maximum over all heads
        float* am = fp8::amax_slot(amax_.data());
        utils::CHECK_DF8(df8_attention_fp8(qkvq_.codes.data(), qkvq_.kind, qkvq_.scale.data(), B, T_len, Hg, D,
                                           causal_ ? DF8_MASK_CAUSAL : DF8_MASK_NONE, nullptr, 0, attn_f32_.data(), am,
                                           st));
        quantize_gather_sharded(attn_f32_.data(), M, am, sym_attn_, attn_scale_.data());
    }
    for (int c = 0; c < nc; ++c) {
        wait_chunk(tickets_attn_, c);
        const size_t r = size_t(c) * Mc * Eg;
        b.out.forward_codes(sym_attn_ + r, act, attn_scale_.data(), Mc, DF8_EPI_RESIDUAL, x + r, x1 + r, nullptr, Eg, g, M);
    }

    // ---- x = x1 + FC2(act(FC1(LN2(x1)))) ----
    layernorm_quantize_sharded(b.norm2, x1, M, 1);
    {
        const fp8::Quantized& w = b.fc1.quantized_weights();
        float* am = fp8::amax_slot(amax_.data());
        const int flags = mlp_gelu_ ? DF8_EPI_GELU : 0;
        for (int c = 0; c < nc; ++c) {
            wait_chunk(tickets_ln_, c);
            utils::CHECK_DF8(df8_gemm_fp8_tn_amax_part(sym_ln_ + size_t(c) * Mc * Eg, act, ln_scale_.data(), g, M, w.codes.data(),
                                                       w.kind, w.scale.data(), b.fc1.bias()->data(), Mc, Fg, E, flags, am, st));
        }
        all_max(am);
        // the codes go straight into this rank's slab of the buffer the peers gather into, a row chunk at a time
        for (int c = 0; c < nc; ++c) {
            const size_t off = size_t(rank_) * size_t(M) * Fg + size_t(c) * Mc * Fg;
            utils::CHECK_DF8(df8_gemm_fp8_tn_codes_part(sym_ln_ + size_t(c) * Mc * Eg, act, ln_scale_.data(), g, M, w.codes.data(),
                                                        w.kind, w.scale.data(), b.fc1.bias()->data(), Mc, Fg, E, flags, act, am,
                                                        sym_hidden_ + off, hidden_scale_.data(), st));
            if (nc > 1) utils::CHECK_DF8(df8_comm_push_symm(comm_, sym_hidden_, off, size_t(Mc) * Fg, st, &tickets_hidden_[c]));
        }
        if (nc == 1) utils::CHECK_DF8(df8_comm_allgather_symm(comm_, sym_hidden_, 0, size_t(M) * Fg, st));
    }
    for (int c = 0; c < nc; ++c) {
        wait_chunk(tickets_hidden_, c);
        b.fc2.forward_codes(sym_hidden_ + size_t(c) * Mc * Fg, act, hidden_scale_.data(), Mc, DF8_EPI_RESIDUAL,
                            x1 + size_t(c) * Mc * Eg, x + size_t(c) * Mc * Eg, nullptr, Eg, g, M);
    }
}

// Embedding (replicated table) -> this rank's columns -> the blocks.  The hidden states stay in x_shard_.
template <typename T>
void Gpt2ColumnSharded<T>::run_blocks_sharded(const tensor<int>& ids, bool check_ids, int* M_out) {
    const auto& s = ids.shape();
    const int B = s[0], T_len = s[1], M = B * T_len, E = hidden_dim_, Eg = E / world_;
    ensure_work_space(M);
    {
        tensor<T> full = token_embedding_->forward_with_positions(ids, positional_encoding_->table().data(), check_ids);
        utils::CHECK_CUDA_EX(cudaMemcpy2DAsync(x_shard_.data(), size_t(Eg) * sizeof(float),
                                               full.data() + size_t(rank_) * Eg, size_t(E) * sizeof(float),
                                               size_t(Eg) * sizeof(float), size_t(M), cudaMemcpyDeviceToDevice,
                                               Cuda::stream()));
    }
    for (auto& b : blocks_) block_forward_sharded(*b, B, T_len);
    *M_out = M;
}

template <typename T>
tensor<T> Gpt2ColumnSharded<T>::forward_hidden(const tensor<int>& ids, bool check_ids) {
    const auto& s = ids.shape();
    if (s.size() != 2) throw std::runtime_error("Gpt2ColumnSharded expects token ids shaped [B, T]");
    const int B = s[0], T_len = s[1];
    if (T_len > positional_encoding_->max_seq_len())
        throw std::runtime_error("Input sequence length exceeds maximum allowed length");
    fp8::PassScope amax_slots;
    if (world_ == 1) {
        tensor<T> x = token_embedding_->forward_with_positions(ids, positional_encoding_->table().data(), check_ids);
        for (auto& b : blocks_) block_forward_single(*b, x.data(), B, T_len);
        return x;
    }
    int M = 0;
    run_blocks_sharded(ids, check_ids, &M);
    // gather the fp32 column slices (NCCL; not on the path of forward_logits_shard) and put them side by side
    const size_t E = size_t(hidden_dim_), Eg = E / size_t(world_);
    tensor<uint8_t> gathered({int(size_t(M) * E * sizeof(float))});
    utils::CHECK_DF8(df8_comm_allgather_u8(comm_, reinterpret_cast<const uint8_t*>(x_shard_.data()), gathered.data(),
                                           size_t(M) * Eg * sizeof(float), fp8::stream()));
    tensor<T> x({B, T_len, hidden_dim_});
    utils::CHECK_DF8(df8_interleave_gathered_u8(gathered.data(), M, int(Eg * sizeof(float)), world_,
                                                reinterpret_cast<uint8_t*>(x.data()), fp8::stream()));
    return x;
}

// logits [M, pitch] of this rank's vocabulary rows from the hidden states of the last forward
template <typename T>
void Gpt2ColumnSharded<T>::head(int M, float* logits, int pitch) {
    const df8_kind act = fp8::policy().activation_kind;
    if (world_ == 1) throw std::logic_error("Gpt2ColumnSharded::head: sharded path only");
    float* am = fp8::amax_slot(amax_.data());
    const int Eg = hidden_dim_ / world_;
    utils::CHECK_DF8(df8_amax_f32(x_shard_.data(), size_t(M) * Eg, am, fp8::stream()));
    quantize_gather_sharded(x_shard_.data(), M, am, sym_ln_, ln_scale_.data());  // tickets in tickets_attn_ when chunked
    const int nc = chunks_for(M), Mc = M / nc;
    for (int c = 0; c < nc; ++c) {
        if (nc > 1) utils::CHECK_DF8(df8_comm_wait_symm(comm_, tickets_attn_[c], c == nc - 1 ? 1 : 0, fp8::stream()));
        final_fc_->forward_codes(sym_ln_ + size_t(c) * Mc * Eg, act, ln_scale_.data(), Mc, 0, nullptr,
                                 logits + size_t(c) * Mc * pitch, nullptr, pitch, world_, M);
    }
}

template <typename T>
tensor<T> Gpt2ColumnSharded<T>::forward_logits_shard_pitched(const tensor<int>& ids, bool check_ids) {
    const auto& s = ids.shape();
    if (s.size() != 2) throw std::runtime_error("Gpt2ColumnSharded expects token ids shaped [B, T]");
    if (s[1] > positional_encoding_->max_seq_len())
        throw std::runtime_error("Input sequence length exceeds maximum allowed length");
    fp8::PassScope amax_slots;
    const int pitch = logits_pitch();
    if (world_ == 1) {
        tensor<T> x = forward_hidden(ids, check_ids);
        const int M = int(x.numel() / size_t(hidden_dim_));
        fp8::quantize(x.data(), x.numel(), fp8::policy().activation_kind, head_q_);
        tensor<T> logits({M, pitch});
        final_fc_->forward_codes(head_q_.codes.data(), head_q_.kind, head_q_.scale.data(), M, 0, nullptr, logits.data(),
                                 nullptr, pitch);
        return logits;
    }
    int M = 0;
    run_blocks_sharded(ids, check_ids, &M);
    tensor<T> logits({M, pitch});
    head(M, logits.data(), pitch);
    return logits;
}

template <typename T>
tensor<T> Gpt2ColumnSharded<T>::forward_logits_shard(const tensor<int>& ids, bool check_ids) {
    const auto& s = ids.shape();
    if (s.size() != 2) throw std::runtime_error("Gpt2ColumnSharded expects token ids shaped [B, T]");
    if (s[1] > positional_encoding_->max_seq_len())
        throw std::runtime_error("Input sequence length exceeds maximum allowed length");
    fp8::PassScope amax_slots;
    if (world_ == 1) {
        tensor<T> x = forward_hidden(ids, check_ids);
        const int M = int(x.numel() / size_t(hidden_dim_));
        fp8::quantize(x.data(), x.numel(), fp8::policy().activation_kind, head_q_);
        tensor<T> logits({M, vocab_rows_});
        final_fc_->forward_codes(head_q_.codes.data(), head_q_.kind, head_q_.scale.data(), M, 0, nullptr, logits.data(),
                                 nullptr);
        return logits;
    }
    int M = 0;
    run_blocks_sharded(ids, check_ids, &M);
    tensor<T> logits({M, vocab_rows_});
    head(M, logits.data(), vocab_rows_);
    return logits;
}

template <typename T>
unsigned long long Gpt2ColumnSharded<T>::bytes_pushed() const {
    unsigned long long b = 0;
    if (comm_ && world_ > 1) utils::CHECK_DF8(df8_comm_bytes_pushed(comm_, &b));
    return b;
}

template class Gpt2ColumnSharded<float>;

}  // namespace dnn
