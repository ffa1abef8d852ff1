#include "dnn/tokens/positional_encoding.cuh"

#include <cmath>
#include <stdexcept>
#include <vector>

#include "dnn/core/cuda.cuh"
#include "dnn/utils/common.cuh"

namespace dnn {

namespace {
constexpr int kBlock = 256;

// out[r, :] = in[r, :] + pe[r % T, :]
__global__ void add_table_kernel(const float* __restrict__ in, const float* __restrict__ pe, float* __restrict__ out,
                                 size_t n, int T, int E) {
    for (size_t i = blockIdx.x * size_t(kBlock) + threadIdx.x; i < n; i += size_t(gridDim.x) * kBlock) {
        const size_t row = i / size_t(E);
        const int d = int(i % size_t(E));
        out[i] = in[i] + pe[size_t(row % size_t(T)) * E + d];
    }
}

int positive_or_throw(int v, const char* what) {
    if (v <= 0) throw std::invalid_argument(std::string(what) + " must be positive");
    return v;
}
}  // namespace

template <typename T>
PositionalEncoding<T>::PositionalEncoding(int embed_dim, int max_seq_len, bool training_enabled)
    : Layer<T>(training_enabled),
      embed_dim_(positive_or_throw(embed_dim, "Embedding dimension")),
      max_seq_len_(positive_or_throw(max_seq_len, "Maximum sequence length")),
      pos_encoding_({max_seq_len, embed_dim}) {
    initialize_positional_encodings();
}

template <typename T>
void PositionalEncoding<T>::initialize_positional_encodings() {
    std::vector<T> host(pos_encoding_.numel());
    for (int pos = 0; pos < max_seq_len_; ++pos)
        for (int i = 0; i < embed_dim_; ++i) {
            const float div = std::exp(-2.0f * float(i / 2) * std::log(10000.0f) / float(embed_dim_));
            const float v = (i % 2 == 0) ? std::sin(float(pos) * div) : std::cos(float(pos) * div);
            host[size_t(pos) * embed_dim_ + i] = static_cast<T>(v);
        }
    pos_encoding_.upload(host.data());
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));
}

template <typename T>
tensor<T> PositionalEncoding<T>::forward(const tensor<T>& input) {
    const auto& s = input.shape();
    if (s.size() != 3 || s[2] != embed_dim_)
        throw std::runtime_error("PositionalEncoding expects input shape [B, T, E]");
    if (s[1] > max_seq_len_) throw std::runtime_error("Input sequence length exceeds maximum allowed length");
    if (this->training_enabled_) input_cache_ = input.clone();
    tensor<T> out(s);
    const size_t n = input.numel();
    if (n) {
        const int grid = int(std::min<size_t>((n + kBlock - 1) / kBlock, 148 * 16));
        add_table_kernel<<<grid, kBlock, 0, Cuda::stream()>>>(input.data(), pos_encoding_.data(), out.data(), n, s[1],
                                                             embed_dim_);
        utils::THROW_CUDA_EX();
    }
    return out;
}

// The table is not learned: the gradient passes through unchanged, as upstream returns it.
template <typename T>
tensor<T> PositionalEncoding<T>::backward(const tensor<T>& grad_output) {
    return grad_output.clone();
}

template class PositionalEncoding<float>;

}  // namespace dnn
