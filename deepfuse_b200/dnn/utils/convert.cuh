// Element conversions between float and the reduced-precision tensor element types, with the names and
// semantics of upstream dnn/utils/convert.cu:5-33 (to_float / to_half), extended to the fp8 codes this build
// stores in tensor<uint8_t>.  Host-callable (the fp8 ones call the CUDA toolkit's cuda_fp8.h conversion).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdint>

namespace dnn {
namespace utils {

inline float to_float(float v) { return v; }
inline float to_float(__half v) { return __half2float(v); }
inline float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
inline __half to_half(float v) { return __float2half(v); }
inline __half to_half(__half v) { return v; }

// fp8 code <-> float (round-to-nearest-even, saturate-to-finite); e5m2 = false selects e4m3
inline uint8_t to_fp8_code(float v, bool e5m2 = false) {
    return __nv_cvt_float_to_fp8(v, __NV_SATFINITE, e5m2 ? __NV_E5M2 : __NV_E4M3);
}
inline float fp8_code_to_float(uint8_t code, bool e5m2 = false) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(code, e5m2 ? __NV_E5M2 : __NV_E4M3)));
}

}  // namespace utils
}  // namespace dnn
