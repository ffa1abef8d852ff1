#include "dnn/tokens/token_embedding.cuh"

#include <random>
#include <stdexcept>

#include "dnn/core/fp8.cuh"

namespace dnn {

namespace {
int checked_positive(int v, const char* what) {
    if (v <= 0) throw std::invalid_argument(std::string(what) + " must be positive");
    return v;
}
}  // namespace

template <typename T>
TokenEmbedding<T>::TokenEmbedding(int vocab_size, int embedding_dim, int max_seq_len, bool training_enabled)
    : LayerWeightBiasAsymmetric<T, int>(
          tensor<T>({checked_positive(vocab_size, "Vocabulary size"), checked_positive(embedding_dim, "Embedding dimension")}),
          tensor<T>({embedding_dim}), tensor<T>({vocab_size, embedding_dim}), tensor<T>({embedding_dim}),
          training_enabled),
      vocab_size_(vocab_size),
      embedding_dim_(embedding_dim),
      max_seq_len_(checked_positive(max_seq_len, "Maximum sequence length")),
      bad_ids_({1}) {
    if (fp8::policy().host_init) {
        initialize_weights();
    } else {
        this->weights_.zero();
        this->bias_.zero();
    }
    this->grad_weights_.zero();
    this->grad_bias_.zero();
}

// N(0, 0.02) table and zero bias (upstream embedding_init_kernel, token_embedding.cu:11-28, which seeds
// curand from clock64(); here the seed is fixed so runs are reproducible).
template <typename T>
void TokenEmbedding<T>::initialize_weights() {
    std::mt19937 gen(0xE3BED000u + unsigned(vocab_size_) + 131u * unsigned(embedding_dim_));
    std::normal_distribution<float> dist(0.0f, 0.02f);
    std::vector<T> host(this->weights_.numel());
    for (auto& v : host) v = static_cast<T>(dist(gen));
    this->weights_.upload(host.data());
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));
    this->bias_.zero();
}

template <typename T>
tensor<T> TokenEmbedding<T>::forward_with_positions(const tensor<int>& input, const T* pe, bool check_ids) {
    const auto& s = input.shape();
    if (s.size() != 2) throw std::runtime_error("TokenEmbedding input must be 2D [B, T]");
    const int B = s[0], T_len = s[1];
    if (T_len > max_seq_len_) throw std::runtime_error("Input sequence length exceeds maximum allowed length");
    if (this->training_enabled_) input_cache_ = input.clone();
    tensor<T> out({B, T_len, embedding_dim_});
    utils::CHECK_DF8(df8_embed_pe_f32(input.data(), B, T_len, embedding_dim_, vocab_size_, this->weights_.data(),
                                      this->bias_.data(), pe, out.data(), bad_ids_.data(), fp8::stream()));
    if (check_ids) {
        int bad = 0;
        bad_ids_.download(&bad);
        if (bad != 0) throw std::runtime_error("Invalid token ID: " + std::to_string(bad) + " id(s) outside the vocabulary");
    }
    return out;
}

template <typename T>
tensor<T> TokenEmbedding<T>::forward(const tensor<int>& input) {
    return forward_with_positions(input, nullptr, true);
}

// Training-side (upstream embedding_backward_kernel, token_embedding.cu:48-69); not in this build.
template <typename T>
tensor<T> TokenEmbedding<T>::backward(const tensor<T>& /*grad_output*/) {
    throw std::runtime_error("TokenEmbedding::backward: the fp8 inference build has no backward pass");
}

template <typename T>
void TokenEmbedding<T>::save(std::ostream& out) const {
    out.write(reinterpret_cast<const char*>(&vocab_size_), sizeof(vocab_size_));
    out.write(reinterpret_cast<const char*>(&embedding_dim_), sizeof(embedding_dim_));
    out.write(reinterpret_cast<const char*>(&max_seq_len_), sizeof(max_seq_len_));
    this->weights_.save(out);
    this->bias_.save(out);
}

template <typename T>
void TokenEmbedding<T>::load(std::istream& in) {
    in.read(reinterpret_cast<char*>(&vocab_size_), sizeof(vocab_size_));
    in.read(reinterpret_cast<char*>(&embedding_dim_), sizeof(embedding_dim_));
    in.read(reinterpret_cast<char*>(&max_seq_len_), sizeof(max_seq_len_));
    if (!in) throw std::runtime_error("TokenEmbedding::load: bad header");
    this->weights_.load(in);
    this->bias_.load(in);
}

template class TokenEmbedding<float>;

}  // namespace dnn
