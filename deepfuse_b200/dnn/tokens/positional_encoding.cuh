// PositionalEncoding<T>: adds the fixed sinusoidal table to [B,T,E] activations.
// Public surface of upstream dnn/tokens/positional_encoding.cuh (constructor (embed_dim, max_seq_len,
// training_enabled) throwing std::invalid_argument for non-positive arguments, forward, backward,
// name() == "PositionalEncoding").  Table, upstream dnn/tokens/positional_encoding.cu:20-27:
//   div = exp(-2*(i/2)*ln(10000)/E);  PE[pos,i] = sin(pos*div) for even i, cos(pos*div) for odd i.
// The table is computed once on the host in fp32 and uploaded, so that it is identical to the one the
// CPU oracle uses; upstream builds it with device intrinsics and adds it with E threads per block
// (E <= 1024, :94-104), a cap that does not exist here.
#pragma once

#include <optional>
#include <string>

#include "dnn/core/layer.cuh"
#include "dnn/core/tensor.cuh"

namespace dnn {

template <typename T>
class PositionalEncoding : public Layer<T> {
public:
    PositionalEncoding(int embed_dim, int max_seq_len, bool training_enabled = false);
    ~PositionalEncoding() override = default;

    tensor<T> forward(const tensor<T>& input) override;
    tensor<T> backward(const tensor<T>& grad_output) override;
    std::string name() const override { return "PositionalEncoding"; }
    void save(std::ostream&) const override {}
    void load(std::istream&) override {}

    const tensor<T>& table() const { return pos_encoding_; }
    int max_seq_len() const { return max_seq_len_; }

private:
    void initialize_positional_encodings();
    int embed_dim_;
    int max_seq_len_;
    tensor<T> pos_encoding_;
    std::optional<tensor<T>> input_cache_;
};

}  // namespace dnn
