// NaturalLanguageModel<T>: a model that owns a tokenizer and a [1,1,T,T] attention-mask tensor
// (upstream dnn/models/natural_language_model.cuh:13-86).  As upstream, the mask tensor is filled with
// ones and is never handed to the transformer blocks (:19-24, :56-67): attention is unmasked unless a
// block's set_mask / set_causal is called.
#pragma once

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "dnn/core/cuda.cuh"
#include "dnn/models/model.cuh"
#include "dnn/tokens/tokenizer.cuh"

namespace dnn {

template <typename T>
class NaturalLanguageModel : public TrainingModel<T> {
public:
    NaturalLanguageModel(std::shared_ptr<Tokenizer> tokenizer, int max_seq_len = 1024, bool training_enabled = false)
        : TrainingModel<T>(training_enabled),
          tokenizer_(std::move(tokenizer)),
          max_seq_len_(max_seq_len),
          attention_mask_({1, 1, max_seq_len, max_seq_len}) {
        attention_mask_.fill(static_cast<T>(1.0f));
    }

    tensor<T> forward_from_text(const std::string& text) {
        if (!tokenizer_) throw std::runtime_error("NaturalLanguageModel: no tokenizer");
        return this->forward(to_tensor(tokenizer_->encode(text, true)));
    }

    void train_from_text(const std::string& text) {
        if (!tokenizer_) throw std::runtime_error("NaturalLanguageModel: no tokenizer");
        std::vector<int> tokens = tokenizer_->encode(text, true);
        if (tokens.size() < 2) throw std::runtime_error("NaturalLanguageModel: text too short to train on");
        std::vector<int> in(tokens.begin(), tokens.end() - 1), tgt(tokens.begin() + 1, tokens.end());
        set_attention_mask(int(in.size()));
        this->train_step(to_tensor(in), to_tensor(tgt));
    }

    const Tokenizer* tokenizer() const { return tokenizer_.get(); }

    void set_attention_mask(int seq_len) {
        if (seq_len > max_seq_len_) throw std::runtime_error("Sequence length exceeds maximum context length");
        attention_mask_ = tensor<T>({1, 1, seq_len, seq_len});
        attention_mask_.fill(static_cast<T>(1.0f));
    }
    const tensor<T>& attention_mask() const { return attention_mask_; }

protected:
    std::shared_ptr<Tokenizer> tokenizer_;
    int max_seq_len_;
    tensor<T> attention_mask_;

    tensor<T> to_tensor(const std::vector<int>& ids) const {
        tensor<T> result({1, int(ids.size())});
        std::vector<T> host(ids.begin(), ids.end());
        result.upload(host.data());
        cudaStreamSynchronize(Cuda::stream());  // `host` is pageable and dies at scope exit
        return result;
    }
};

}  // namespace dnn
