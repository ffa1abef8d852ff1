// FullyConnectedLayer<TT>: Y[N,out] = X[N,in] . W[out,in]^T + b, on the fp8 tensor-core GEMM.
//
// Public surface of upstream dnn/layers/fully_connected_layer.cuh:22-52 (constructor
// (in_features, out_features, training_enabled), forward, backward, name() == "FullyConnected",
// initialize_weights, save, load, plus weights()/bias()/parameters() from LayerWeightBias), weights
// [out,in] row-major and bias shaped {1,out,1,1} as upstream allocates them
// (dnn/layers/fully_connected_layer.cu:110-151).
//
// forward() quantises the fp32 input per tensor (policy().activation_kind), multiplies it with the
// cached per-tensor e4m3 copy of the weights in df8_gemm_fp8_tn and returns fp32 — in place of
// upstream's one-thread-per-output fp32 kernel (fully_connected_layer.cu:15-41, :199-208).
// The cached weight codes are refreshed whenever the fp32 weight tensor's version() changes.
#pragma once

#include <iostream>
#include <optional>
#include <string>

#include "dnn/core/fp8.cuh"
#include "dnn/core/layer.cuh"
#include "dnn/core/tensor.cuh"

namespace dnn {

template <typename TT>
class FullyConnectedLayer : public LayerWeightBias<TT> {
public:
    FullyConnectedLayer(int in_features, int out_features, bool training_enabled = false);
    ~FullyConnectedLayer() override;

    tensor<TT> forward(const tensor<TT>& input) override;
    tensor<TT> backward(const tensor<TT>& grad_output) override;
    std::string name() const override { return "FullyConnected"; }
    void initialize_weights() override;
    void save(std::ostream& out) const override;
    void load(std::istream& in) override;

    int in_features() const { return in_features_; }
    int out_features() const { return out_features_; }
    // K extent of the fp8 codes: in_features rounded up to a multiple of 16 (zero-padded)
    int padded_in() const { return (in_features_ + 15) / 16 * 16; }

    // ---- fp8 path (additions; upstream has no counterpart) ----
    // Per-tensor quantised weights, refreshed if the fp32 weights changed since the last call.
    const fp8::Quantized& quantized_weights();
    // out[M,out] = epilogue(codes . Wq^T); a_codes is [M, padded_in()]; `flags` are DF8_EPI_* bits;
    // out_amax may be null.  ldc: row pitch of `out` and `residual` in floats (0 = out_features); a_slabs: the
    // columns of a_codes are stored as that many [M, padded_in() / a_slabs] slabs (see df8_gemm_fp8_tn_ex);
    // a_slab_rows: rows per slab when M is only a row range of them (0 = M; see df8_gemm_fp8_tn_part).
    void forward_codes(const uint8_t* a_codes, df8_kind a_kind, const float* a_scale, int M, int flags,
                       const float* residual, float* out, float* out_amax, int ldc = 0, int a_slabs = 1,
                       int a_slab_rows = 0);

    // The same product for the few token rows of a decode step (B <= 128): bound by streaming the weights
    // (df8_gemv_fp8_tn).
    void forward_codes_skinny(const uint8_t* a_codes, df8_kind a_kind, const float* a_scale, int B, int flags,
                              const float* residual, float* out, float* out_amax);

    // q <- per-tensor quantisation (kind out_kind) of epilogue(codes . Wq^T), `flags` = 0 or DF8_EPI_GELU.
    // Uses the two-pass GEMM that never writes the fp32 result when out_features % 32 == 0.
    void forward_codes_quantized(const uint8_t* a_codes, df8_kind a_kind, const float* a_scale, int M, int flags,
                                 df8_kind out_kind, fp8::Quantized& q);

    // Layer streaming: when set, the GEMMs read the weight codes from `codes` (a device slot filled by
    // the streamer) instead of the layer's own cached copy, which may then be dropped; the scale stays
    // resident.  nullptr returns to the cached copy.
    void use_external_codes(const uint8_t* codes) { external_codes_ = codes; }
    // Size in bytes of this layer's weight codes, and a copy of them into HOST memory (synchronises).
    size_t weight_code_bytes() const { return size_t(out_features_) * size_t(padded_in()); }
    void export_weight_codes(uint8_t* dst_h);
    // Frees the device copy of the weight codes (streaming mode keeps them in pinned host memory).
    void drop_cached_codes();
    // The quantise-once cache: this layer's weight codes [out, padded_in()], their {q, dq} scale, the amax they were
    // derived from and the fp32 bias as one binary record; import installs them without the fp32 weights ever
    // being on the device (weights() is then an empty [0, in] tensor, as after release_fp32 in layer streaming).
    void export_quantized(std::ostream& out);
    void import_quantized(std::istream& in);
    // Declares the cached scale current for the present weights tensor / forces a re-quantisation.
    void mark_weights_quantized() { wq_version_ = this->weights_.version(); }
    void invalidate_quantized_weights() { wq_version_ = ~0ull; }
    // Column sharding: this layer holds a row block of a larger weight matrix whose other blocks live on the
    // other ranks of `comm`.  The per-tensor scale must then come from the maximum over ALL blocks, so
    // quantized_weights() all-reduces the local max|w| first (a collective: every rank must quantise).
    void set_shard_comm(df8_comm* comm) {
        shard_comm_ = comm;
        invalidate_quantized_weights();
    }
    // Replaces the weights by uniform values in (-limit, +limit) generated on the device from a counter hash
    // of (seed, element index + index_offset); for models too large to initialise through the host.
    void initialize_weights_on_device(float limit, uint64_t seed, uint64_t index_offset = 0);
    // Rows [row_begin, row_begin + rows) of this layer's weights <- N(0, std) values of the stream `seed` starting at
    // element index_offset (fp8::fill_normal): a shard fills its rows of the global tensor; bias <- 0.
    void initialize_rows_normal_on_device(float std, uint64_t seed, uint64_t index_offset, int row_begin, int rows);

private:
    const uint8_t* external_codes_ = nullptr;
    df8_comm* shard_comm_ = nullptr;
    int in_features_;
    int out_features_;
    std::optional<tensor<TT>> input_cache_;
    fp8::Quantized wq_;
    uint64_t wq_version_ = ~0ull;
    fp8::Quantized xq_;  // reused activation buffer
};

}  // namespace dnn
