// TokenEmbedding<T>: [B,T] int token ids -> [B,T,E] embeddings (+ bias).
// Public surface of upstream dnn/tokens/token_embedding.cuh (constructor (vocab_size, embedding_dim,
// max_seq_len = 1024, training_enabled), forward(tensor<int>), backward, name() == "TokenEmbedding",
// initialize_weights, parameters/gradients, save/load) with upstream's checks: non-positive constructor
// arguments throw std::invalid_argument (dnn/tokens/token_embedding.cu:84-92); a non-2-D input, T above
// max_seq_len or an id outside [0,V) throw std::runtime_error (:120-138).
// Ids are validated on the device by the gather kernel itself (one counter read back) instead of
// upstream's download-and-loop on the host.
#pragma once

#include <iostream>
#include <optional>
#include <string>
#include <vector>

#include "dnn/core/layer.cuh"
#include "dnn/core/tensor.cuh"

namespace dnn {

template <typename T>
class TokenEmbedding : public LayerWeightBiasAsymmetric<T, int> {
public:
    TokenEmbedding(int vocab_size, int embedding_dim, int max_seq_len = 1024, bool training_enabled = false);

    tensor<T> forward(const tensor<int>& input) override;
    tensor<T> backward(const tensor<T>& grad_output) override;
    std::string name() const override { return "TokenEmbedding"; }
    void initialize_weights() override;
    std::vector<tensor<T>*> parameters() override { return {&this->weights_, &this->bias_}; }
    std::vector<tensor<T>*> gradients() override { return {&this->grad_weights_, &this->grad_bias_}; }
    void save(std::ostream& out) const override;
    void load(std::istream& in) override;

    int vocab_size() const { return vocab_size_; }
    int embedding_dim() const { return embedding_dim_; }
    int max_seq_len() const { return max_seq_len_; }

    // Gather + bias + positional table in one kernel; `pe` is a [>=T, E] table or null.
    // When check_ids is true the invalid-id counter is read back (one stream sync) and an id outside
    // [0,V) throws std::runtime_error, as forward() does.
    tensor<T> forward_with_positions(const tensor<int>& input, const T* pe, bool check_ids = true);

private:
    int vocab_size_;
    int embedding_dim_;
    int max_seq_len_;
    std::optional<tensor<int>> input_cache_;
    tensor<int> bad_ids_;
};

}  // namespace dnn
