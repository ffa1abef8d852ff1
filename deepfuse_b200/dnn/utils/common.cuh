// Error helpers of the dnn:: API.
//
// Same contract as upstream dnn/utils/common.cuh:20-35: a failed CUDA call becomes a
// std::runtime_error whose text carries "CUDA error at file:line".  Added here: check_df8(), which
// turns a non-zero status of the C-ABI kernel library (include/df8.h) into the same exception type.
#pragma once

#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "df8.h"

namespace dnn {
namespace utils {

inline void check_cuda_error(cudaError_t err, const char* file, int line) {
    if (err != cudaSuccess)
        throw std::runtime_error(std::string("CUDA error at ") + file + ":" + std::to_string(line) + ": " +
                                 cudaGetErrorString(err));
}

inline void check_df8_status(df8_status st, const char* what, const char* file, int line) {
    if (st != DF8_OK)
        throw std::runtime_error(std::string(what) + " failed at " + file + ":" + std::to_string(line) + ": " +
                                 df8_last_error());
}

#define CHECK_CUDA_EX(call) check_cuda_error((call), __FILE__, __LINE__)
#define THROW_CUDA_EX() check_cuda_error(cudaGetLastError(), __FILE__, __LINE__)
#define CHECK_DF8(call) check_df8_status((call), #call, __FILE__, __LINE__)

}  // namespace utils
}  // namespace dnn
