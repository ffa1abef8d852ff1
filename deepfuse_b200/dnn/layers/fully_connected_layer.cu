#include "dnn/layers/fully_connected_layer.cuh"

#include <cmath>
#include <random>
#include <stdexcept>
#include <type_traits>
#include <vector>

namespace dnn {

template <typename TT>
FullyConnectedLayer<TT>::FullyConnectedLayer(int in_features, int out_features, bool training_enabled)
    : LayerWeightBias<TT>(tensor<TT>({out_features, in_features}), tensor<TT>({1, out_features, 1, 1}),
                          // gradient buffers: not kept for inference-only layers of models built without host
                          // initialisation (billions of parameters)
                          (training_enabled || fp8::policy().host_init) ? tensor<TT>({out_features, in_features})
                                                                        : tensor<TT>({0}),
                          tensor<TT>({1, out_features, 1, 1}), training_enabled),
      in_features_(in_features),
      out_features_(out_features) {
    if (in_features <= 0 || out_features <= 0)
        throw std::invalid_argument("FullyConnectedLayer: feature counts must be positive");
    if (fp8::policy().host_init) {
        initialize_weights();
    } else {
        this->weights_.zero();
        this->bias_.zero();
    }
    this->grad_weights_.zero();
    this->grad_bias_.zero();
}

template <typename TT>
FullyConnectedLayer<TT>::~FullyConnectedLayer() = default;

// Xavier-uniform weights in [-sqrt(6/(in+out)), +sqrt(6/(in+out))], zero bias — the distribution
// upstream draws (fully_connected_layer.cu:359-385), from a fixed-seed generator instead of
// std::random_device so that a run is reproducible.
template <typename TT>
void FullyConnectedLayer<TT>::initialize_weights() {
    const float limit = std::sqrt(6.0f / float(in_features_ + out_features_));
    std::mt19937 gen(0x5EED0000u + unsigned(in_features_) * 31u + unsigned(out_features_));
    std::uniform_real_distribution<float> dist(-limit, limit);
    std::vector<TT> host(this->weights_.numel());
    for (auto& v : host) v = static_cast<TT>(dist(gen));
    this->weights_.upload(host.data());
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));
    this->bias_.zero();
}

template <typename TT>
void FullyConnectedLayer<TT>::initialize_weights_on_device(float limit, uint64_t seed, uint64_t index_offset) {
    if constexpr (std::is_same<TT, float>::value) {
        fp8::fill_uniform(this->weights_.data(), this->weights_.numel(), limit, seed, index_offset);
        this->weights_.bump_version();
        this->bias_.zero();
    } else {
        throw std::runtime_error("initialize_weights_on_device: float layers only");
    }
}

template <typename TT>
void FullyConnectedLayer<TT>::initialize_rows_normal_on_device(float std, uint64_t seed, uint64_t index_offset,
                                                               int row_begin, int rows) {
    if constexpr (std::is_same<TT, float>::value) {
        if (row_begin < 0 || rows < 0 || row_begin + rows > out_features_)
            throw std::invalid_argument("initialize_rows_normal_on_device: row range outside the weights");
        fp8::fill_normal(this->weights_.data() + size_t(row_begin) * size_t(in_features_),
                         size_t(rows) * size_t(in_features_), 0.f, std, seed, index_offset);
        this->weights_.bump_version();
        this->bias_.zero();
    } else {
        throw std::runtime_error("initialize_rows_normal_on_device: float layers only");
    }
}

namespace {
// rows x cols fp32 -> rows x cols_padded, the new columns zero (zero is the fp8 code 0x00 as well)
tensor<float> pad_columns(const float* src, int rows, int cols, int cols_padded) {
    tensor<float> out({rows, cols_padded});
    out.zero();
    if (rows > 0)
        utils::CHECK_CUDA_EX(cudaMemcpy2DAsync(out.data(), size_t(cols_padded) * sizeof(float), src,
                                               size_t(cols) * sizeof(float), size_t(cols) * sizeof(float), size_t(rows),
                                               cudaMemcpyDeviceToDevice, Cuda::stream()));
    return out;
}
}  // namespace

// The GEMM's TMA loads need a row pitch that is a multiple of 16 bytes, so a layer whose in_features is
// not a multiple of 16 keeps its codes (and quantises its inputs) with the K dimension zero-padded.
template <typename TT>
const fp8::Quantized& FullyConnectedLayer<TT>::quantized_weights() {
    if (wq_version_ != this->weights_.version()) {
        const int kp = padded_in();
        std::optional<tensor<float>> padded;
        const float* src = this->weights_.data();
        size_t n = this->weights_.numel();
        if (kp != in_features_) {
            padded = pad_columns(this->weights_.data(), out_features_, in_features_, kp);
            src = padded->data();
            n = padded->numel();
        }
        if (!shard_comm_) {
            fp8::quantize(src, n, fp8::policy().weight_kind, wq_);
        } else {  // the scale of the whole (sharded) tensor
            // wq_.amax is the layer's own float, not a pre-cleared slot of a PassScope, and inside a scope the
            // library does not clear it either: without this memset a lazy re-quantisation during a forward
            // would take the maximum with whatever the float held (garbage, or the previous weights' maximum)
            utils::CHECK_CUDA_EX(cudaMemsetAsync(wq_.amax.data(), 0, sizeof(float), Cuda::stream()));
            utils::CHECK_DF8(df8_amax_f32(src, n, wq_.amax.data(), fp8::stream()));
            utils::CHECK_DF8(df8_comm_allreduce_max_f32(shard_comm_, wq_.amax.data(), 1, fp8::stream()));
            fp8::quantize_with_amax(src, n, fp8::policy().weight_kind, wq_.amax.data(), wq_);
        }
        wq_version_ = this->weights_.version();
    }
    return wq_;
}

template <typename TT>
void FullyConnectedLayer<TT>::export_weight_codes(uint8_t* dst_h) {
    const fp8::Quantized& w = quantized_weights();
    utils::CHECK_CUDA_EX(cudaMemcpyAsync(dst_h, w.codes.data(), weight_code_bytes(), cudaMemcpyDeviceToHost, Cuda::stream()));
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));
}

// record: int in, out, padded_in, kind; float scale[2], amax; codes [out * padded_in] bytes; bias [out] floats
template <typename TT>
void FullyConnectedLayer<TT>::export_quantized(std::ostream& out) {
    const fp8::Quantized& w = quantized_weights();
    if (w.codes.numel() != weight_code_bytes())
        throw std::runtime_error("FullyConnectedLayer::export_quantized: the weight codes are not resident (layer streaming)");
    const int hdr[4] = {in_features_, out_features_, padded_in(), int(w.kind)};
    out.write(reinterpret_cast<const char*>(hdr), sizeof(hdr));
    float meta[3] = {0.f, 0.f, 0.f};
    utils::CHECK_CUDA_EX(cudaMemcpyAsync(meta, w.scale.data(), 2 * sizeof(float), cudaMemcpyDeviceToHost, Cuda::stream()));
    utils::CHECK_CUDA_EX(cudaMemcpyAsync(meta + 2, w.amax.data(), sizeof(float), cudaMemcpyDeviceToHost, Cuda::stream()));
    std::vector<uint8_t> codes(weight_code_bytes());
    export_weight_codes(codes.data());  // synchronises the stream
    out.write(reinterpret_cast<const char*>(meta), sizeof(meta));
    out.write(reinterpret_cast<const char*>(codes.data()), std::streamsize(codes.size()));
    std::vector<float> bias(static_cast<size_t>(out_features_));
    this->bias_.download(bias.data());
    out.write(reinterpret_cast<const char*>(bias.data()), std::streamsize(bias.size() * sizeof(float)));
}

template <typename TT>
void FullyConnectedLayer<TT>::import_quantized(std::istream& in) {
    if constexpr (!std::is_same<TT, float>::value) {
        throw std::runtime_error("FullyConnectedLayer::import_quantized: float layers only");
    } else {
        int hdr[4] = {0, 0, 0, 0};
        in.read(reinterpret_cast<char*>(hdr), sizeof(hdr));
        if (!in || hdr[0] != in_features_ || hdr[1] != out_features_ || hdr[2] != padded_in() || (hdr[3] != 0 && hdr[3] != 1))
            throw std::runtime_error("FullyConnectedLayer::import_quantized: the record does not match this layer");
        float meta[3];
        in.read(reinterpret_cast<char*>(meta), sizeof(meta));
        std::vector<uint8_t> codes(weight_code_bytes());
        in.read(reinterpret_cast<char*>(codes.data()), std::streamsize(codes.size()));
        std::vector<float> bias(static_cast<size_t>(out_features_));
        in.read(reinterpret_cast<char*>(bias.data()), std::streamsize(bias.size() * sizeof(float)));
        if (!in) throw std::runtime_error("FullyConnectedLayer::import_quantized: truncated record");
        wq_.codes = tensor<uint8_t>({int(codes.size())});
        wq_.codes.upload(codes.data());
        wq_.kind = df8_kind(hdr[3]);
        utils::CHECK_CUDA_EX(cudaMemcpyAsync(wq_.scale.data(), meta, 2 * sizeof(float), cudaMemcpyHostToDevice, Cuda::stream()));
        utils::CHECK_CUDA_EX(cudaMemcpyAsync(wq_.amax.data(), meta + 2, sizeof(float), cudaMemcpyHostToDevice, Cuda::stream()));
        this->bias_.upload(bias.data());
        utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));  // the host buffers die at scope exit
        this->weights_ = tensor<TT>({0, in_features_});  // no fp32 master copy; keep version(): the codes are current
        mark_weights_quantized();
    }
}

template <typename TT>
void FullyConnectedLayer<TT>::drop_cached_codes() {
    quantized_weights();  // make sure the scale is current before the codes go away
    wq_.codes = tensor<uint8_t>({0});
}

template <typename TT>
void FullyConnectedLayer<TT>::forward_codes(const uint8_t* a_codes, df8_kind a_kind, const float* a_scale, int M,
                                            int flags, const float* residual, float* out, float* out_amax, int ldc,
                                            int a_slabs, int a_slab_rows) {
    const fp8::Quantized& w = quantized_weights();
    const uint8_t* w_codes = external_codes_ ? external_codes_ : w.codes.data();
    utils::CHECK_DF8(df8_gemm_fp8_tn_part(a_codes, a_kind, a_scale, a_slabs, a_slab_rows > 0 ? a_slab_rows : M, w_codes, w.kind,
                                          w.scale.data(), this->bias_.data(), residual, M, out_features_, padded_in(), flags,
                                          out, ldc > 0 ? ldc : out_features_, out_amax, fp8::stream()));
}

template <typename TT>
void FullyConnectedLayer<TT>::forward_codes_skinny(const uint8_t* a_codes, df8_kind a_kind, const float* a_scale, int B,
                                                   int flags, const float* residual, float* out, float* out_amax) {
    const fp8::Quantized& w = quantized_weights();
    const uint8_t* w_codes = external_codes_ ? external_codes_ : w.codes.data();
    utils::CHECK_DF8(df8_gemv_fp8_tn(a_codes, a_kind, a_scale, w_codes, w.kind, w.scale.data(), this->bias_.data(), residual,
                                     B, out_features_, padded_in(), flags, out, out_amax, fp8::stream()));
}

template <typename TT>
void FullyConnectedLayer<TT>::forward_codes_quantized(const uint8_t* a_codes, df8_kind a_kind, const float* a_scale,
                                                      int M, int flags, df8_kind out_kind, fp8::Quantized& q) {
    const size_t n = size_t(M) * size_t(out_features_);
    if (q.codes.numel() != n) q.codes = tensor<uint8_t>({int(n)});
    q.kind = out_kind;
    const fp8::Quantized& w = quantized_weights();
    const uint8_t* w_codes = external_codes_ ? external_codes_ : w.codes.data();
    if (out_features_ % 32 == 0) {
        utils::CHECK_DF8(df8_gemm_fp8_tn_q(a_codes, a_kind, a_scale, w_codes, w.kind, w.scale.data(),
                                           this->bias_.data(), M, out_features_, padded_in(), flags, out_kind,
                                           q.codes.data(), q.scale.data(), fp8::amax_slot(q.amax.data()),
                                           fp8::stream()));
        return;
    }
    tensor<float> f32({M, out_features_});
    float* am = fp8::amax_slot(q.amax.data());
    forward_codes(a_codes, a_kind, a_scale, M, flags | DF8_EPI_AMAX, nullptr, f32.data(), am);
    fp8::quantize_with_amax(f32.data(), n, out_kind, am, q);
}

template <typename TT>
tensor<TT> FullyConnectedLayer<TT>::forward(const tensor<TT>& input) {
    const auto& shape = input.shape();
    if (shape.empty() || input.numel() % size_t(in_features_) != 0 || shape.back() != in_features_)
        throw std::runtime_error("FullyConnectedLayer::forward: input's last dimension must be in_features");
    if (this->training_enabled_) input_cache_ = input.clone();
    const int M = int(input.numel() / size_t(in_features_));
    std::vector<int> out_shape(shape.begin(), shape.end() - 1);
    out_shape.push_back(out_features_);
    tensor<TT> output(out_shape);
    if (padded_in() == in_features_) {
        fp8::quantize(input.data(), input.numel(), fp8::policy().activation_kind, xq_);
    } else {
        tensor<float> padded = pad_columns(input.data(), M, in_features_, padded_in());
        fp8::quantize(padded.data(), padded.numel(), fp8::policy().activation_kind, xq_);
    }
    forward_codes(xq_.codes.data(), xq_.kind, xq_.scale.data(), M, 0, nullptr, output.data(), nullptr);
    return output;
}

// Backward pass: upstream's dX = dY W, dW = dY^T X, db = sum_n dY (fc_backward_* kernels,
// fully_connected_layer.cu:43-107, launched at :317-353) as two fp8 products and a column sum.  dY is quantised per
// tensor to e5m2 (gradients want the range), X as in the forward pass (the policy's activation kind), W's cached e4m3
// codes are used transposed; products accumulate in fp32; db is summed in fp32 from the unquantised dY.  Like
// upstream the gradients overwrite grad_weights() / grad_bias(), and the cached forward input is required.
// The contraction lengths (out_features for dX, the row count N for dW) are padded to a multiple of 16 with zero
// codes.
template <typename TT>
tensor<TT> FullyConnectedLayer<TT>::backward(const tensor<TT>& grad_output) {
    if (!this->training_enabled_)
        throw std::runtime_error("FullyConnectedLayer: backward called without input argument in stateless mode");
    if (!input_cache_.has_value()) throw std::runtime_error("FullyConnectedLayer: input_cache_ not set for backward");
    const tensor<TT>& x = *input_cache_;
    const int in_f = in_features_, out_f = out_features_;
    const int N = int(x.numel() / size_t(in_f));
    if (grad_output.numel() != size_t(N) * size_t(out_f))
        throw std::runtime_error("FullyConnectedLayer::backward: grad_output must be [N, out_features] for the cached input");
    if (external_codes_) throw std::runtime_error("FullyConnectedLayer::backward: the weights of this layer are streamed codes");
    std::vector<int> in_shape = x.shape();
    tensor<TT> grad_input(in_shape);
    if (N == 0) return grad_input;
    const df8_stream st = fp8::stream();
    const df8_kind gk = DF8_E5M2, ak = fp8::policy().activation_kind;
    const int Kd = (out_f + 15) / 16 * 16;  // contraction length of dX
    const int Kw = (N + 15) / 16 * 16;      // contraction length of dW
    fp8::PassScope amax_slots;

    // dY: one pass for db and max|dY|, then two layouts of the same codes
    tensor<float> amax({2});
    float* am_dy = fp8::amax_slot(amax.data());
    tensor<float> partial({df8_colsum_partial_floats(out_f)});
    utils::CHECK_DF8(df8_colsum_amax_f32(grad_output.data(), N, out_f, out_f, partial.data(), this->grad_bias_.data(), am_dy, st));
    tensor<float> dy_scale({2}), x_scale({2});
    tensor<uint8_t> dy_t({out_f, Kw});  // dY^T [out, N]
    tensor<uint8_t> dy_c({N, Kd});      // dY   [N, out] with the K padding
    if (Kd == out_f) {  // one read of dY for both layouts
        utils::CHECK_DF8(df8_quantize_both_layouts_f32(grad_output.data(), N, out_f, gk, am_dy, dy_t.data(), Kw, dy_c.data(), Kd,
                                                       dy_scale.data(), st));
    } else {  // transposing the transposed codes back pads the rows with zero codes
        utils::CHECK_DF8(df8_quantize_transpose_f32(grad_output.data(), N, out_f, gk, am_dy, dy_t.data(), Kw, dy_scale.data(), st));
        utils::CHECK_DF8(df8_transpose_u8(dy_t.data(), out_f, N, Kw, dy_c.data(), Kd, st));
    }

    // dX = dY W: the weight codes transposed, [in, out]
    const fp8::Quantized& w = quantized_weights();
    tensor<uint8_t> w_t({in_f, Kd});
    utils::CHECK_DF8(df8_transpose_u8(w.codes.data(), out_f, in_f, padded_in(), w_t.data(), Kd, st));
    utils::CHECK_DF8(df8_gemm_fp8_tn(dy_c.data(), gk, dy_scale.data(), w_t.data(), w.kind, w.scale.data(), nullptr, nullptr, N,
                                     in_f, Kd, 0, grad_input.data(), nullptr, st));

    // dW = dY^T X
    float* am_x = fp8::amax_slot(amax.data() + 1);
    utils::CHECK_DF8(df8_amax_f32(x.data(), x.numel(), am_x, st));
    tensor<uint8_t> x_t({in_f, Kw});
    utils::CHECK_DF8(df8_quantize_transpose_f32(x.data(), N, in_f, ak, am_x, x_t.data(), Kw, x_scale.data(), st));
    utils::CHECK_DF8(df8_gemm_fp8_tn(dy_t.data(), gk, dy_scale.data(), x_t.data(), ak, x_scale.data(), nullptr, nullptr, out_f,
                                     in_f, Kw, 0, this->grad_weights_.data(), nullptr, st));

    return grad_input;
}

// Stream layout shared with upstream (fully_connected_layer.cu:387-401): in, out, weights, bias.
template <typename TT>
void FullyConnectedLayer<TT>::save(std::ostream& out) const {
    out.write(reinterpret_cast<const char*>(&in_features_), sizeof(in_features_));
    out.write(reinterpret_cast<const char*>(&out_features_), sizeof(out_features_));
    this->weights_.save(out);
    this->bias_.save(out);
}

template <typename TT>
void FullyConnectedLayer<TT>::load(std::istream& in) {
    int in_f = 0, out_f = 0;
    in.read(reinterpret_cast<char*>(&in_f), sizeof(in_f));
    in.read(reinterpret_cast<char*>(&out_f), sizeof(out_f));
    if (!in || in_f <= 0 || out_f <= 0) throw std::runtime_error("FullyConnectedLayer::load: bad header");
    in_features_ = in_f;
    out_features_ = out_f;
    this->weights_.load(in);
    this->bias_.load(in);
    this->grad_weights_ = tensor<TT>({out_f, in_f});
    this->grad_bias_ = tensor<TT>({1, out_f, 1, 1});
}

template class FullyConnectedLayer<float>;

}  // namespace dnn
