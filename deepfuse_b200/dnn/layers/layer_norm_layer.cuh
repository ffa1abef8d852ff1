// LayerNormLayer<T>: normalisation over the last dimension with optional affine parameters.
// Public surface of upstream dnn/layers/layer_norm_layer.cuh:14-42.  Upstream's launch treats
// shape[0] as the row count and shape[1] as the row length (dnn/layers/layer_norm_layer.cu:70-79), which is
// only right for 2-D inputs; this class applies the same per-row formula (:40-62) to rows of
// norm_size taken over the LAST dimension of an input of any rank, which is what the transformer
// block needs for [B,T,E].
#pragma once

#include <iostream>
#include <optional>
#include <string>
#include <vector>

#include "dnn/core/fp8.cuh"
#include "dnn/core/layer.cuh"
#include "dnn/core/tensor.cuh"

namespace dnn {

template <typename T>
class LayerNormLayer : public Layer<T> {
public:
    LayerNormLayer(int norm_size, float epsilon = 1e-5f, bool affine = true, bool training_enabled = false);
    ~LayerNormLayer() override = default;

    tensor<T> forward(const tensor<T>& input) override;
    tensor<T> backward(const tensor<T>& grad_output) override;
    std::vector<tensor<T>*> parameters() override;
    std::vector<tensor<T>*> gradients() override;
    std::string name() const override { return "LayerNorm"; }
    void save(std::ostream& out) const override;
    void load(std::istream& in) override;

    int norm_size() const { return norm_size_; }
    float epsilon() const { return epsilon_; }

    // fp8 path: q <- per-tensor quantisation of LayerNorm(x) without writing the fp32 result.
    void forward_quantized(const float* x, int rows, df8_kind kind, fp8::Quantized& q);

private:
    int norm_size_;
    float epsilon_;
    bool affine_;
    tensor<T> gamma_;
    tensor<T> beta_;
    tensor<T> grad_gamma_;
    tensor<T> grad_beta_;
    std::optional<tensor<T>> input_cache_;
    tensor<float> row_stats_;  // scratch of the fused kernel: (mean, rstd) per row
};

}  // namespace dnn
