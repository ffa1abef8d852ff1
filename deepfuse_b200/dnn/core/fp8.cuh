// fp8 execution policy and small helpers shared by the dnn:: layers.
//
// Upstream names the fp8 element kinds only as tensor storage types (dnn/core/tensor.cu:489-498) and has
// no quantised layer; this header is where the new build states how the fp32 layer API maps onto the
// 8-bit kernels: every fully-connected layer keeps its fp32 weights (the API-visible tensors) and a
// cached per-tensor-quantised copy; activations are quantised per tensor right before each GEMM /
// attention call.
#pragma once

#include <cstdint>
#include <vector>

#include "df8.h"
#include "dnn/core/cuda.cuh"
#include "dnn/core/tensor.cuh"
#include "dnn/utils/common.cuh"

namespace dnn {
namespace fp8 {

struct Policy {
    df8_kind weight_kind = DF8_E4M3;
    df8_kind activation_kind = DF8_E4M3;
    // false: layer constructors leave their weights zero instead of drawing them on the host (for models of
    // billions of parameters that are then filled on the device or loaded)
    bool host_init = true;
};

// p[i] = uniform in (-limit, limit) from a counter hash of (seed, i + index_offset), generated on the device
void fill_uniform(float* p, size_t n, float limit, uint64_t seed, uint64_t index_offset = 0);

// p[i] = mean + std * z, z ~ N(0,1) from the counter-based stream `seed` at index i + index_offset (splitmix64 ->
// two uniforms -> Box-Muller in fp32), generated on the device.  Any slice of a tensor can be generated on its
// own, so every rank of a sharded model fills exactly its rows of one global tensor.
void fill_normal(float* p, size_t n, float mean, float std, uint64_t seed, uint64_t index_offset = 0);

// Process-wide policy read by layers at forward time.
Policy& policy();

// Codes + {q, dq} scale + amax of one per-tensor-quantised activation or weight.
struct Quantized {
    tensor<uint8_t> codes;
    tensor<float> scale;  // {q, dq}
    tensor<float> amax;   // 1 element
    df8_kind kind = DF8_E4M3;
    // amax starts at zero: producers take a running maximum into it, and some callers clear it themselves only
    // when no PassScope is open
    explicit Quantized(size_t n = 0)
        : codes({int(n)}), scale({2}), amax({1}) { amax.zero(); }
};

inline df8_stream stream() { return reinterpret_cast<df8_stream>(Cuda::stream()); }

// Amax slots of one forward pass.  Every producer of a per-tensor maximum needs its output float cleared
// first; done call by call that is a memset node in front of five kernels per transformer block.  While a
// PassScope is alive on the thread, amax_slot() hands out consecutive floats of one device array that the
// scope cleared with a single memset, and the kernels library's own per-call clearing is switched off
// (df8_set_amax_preclear).  Scopes nest; only the outermost one does anything.
class PassScope {
public:
    PassScope();
    ~PassScope();
    PassScope(const PassScope&) = delete;
    PassScope& operator=(const PassScope&) = delete;
};

// The float a producer should write max|out| to: a fresh pre-cleared slot inside a PassScope, otherwise
// `own` (the caller's private buffer, cleared by the library call itself).
float* amax_slot(float* own);

// Throws std::runtime_error if a bounded device-side wait of the kernel library has given up since the status
// word was last reset (df8_status_word_check); waits for the device, so callers use it where they synchronise
// anyway (before handing results to the host).
void check_device_status();

// q <- per-tensor quantisation of n fp32 values at x (amax pass + quantise pass).
void quantize(const float* x, size_t n, df8_kind kind, Quantized& q);

// Same, when max|x| is already known on the device (a fused epilogue produced it).
void quantize_with_amax(const float* x, size_t n, df8_kind kind, const float* amax, Quantized& q);

}  // namespace fp8
}  // namespace dnn
