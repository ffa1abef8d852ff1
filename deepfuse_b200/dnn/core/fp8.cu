#include "dnn/core/fp8.cuh"

namespace dnn {
namespace fp8 {

Policy& policy() {
    static Policy p;
    return p;
}

void quantize(const float* x, size_t n, df8_kind kind, Quantized& q) {
    if (q.codes.numel() != n) q.codes = tensor<uint8_t>({int(n)});
    q.kind = kind;
    utils::CHECK_DF8(df8_amax_f32(x, n, q.amax.data(), stream()));
    utils::CHECK_DF8(df8_quantize_f32(x, n, kind, q.amax.data(), q.codes.data(), q.scale.data(), stream()));
}

void quantize_with_amax(const float* x, size_t n, df8_kind kind, const float* amax, Quantized& q) {
    if (q.codes.numel() != n) q.codes = tensor<uint8_t>({int(n)});
    q.kind = kind;
    utils::CHECK_DF8(df8_quantize_f32(x, n, kind, amax, q.codes.data(), q.scale.data(), stream()));
}

}  // namespace fp8
}  // namespace dnn
