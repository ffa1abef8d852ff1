// Device: a queried cudaDeviceProp, as upstream dnn/core/device.cuh:12-37 exposes it.
#pragma once

#include <cuda_runtime.h>

#include <iostream>
#include <string>

namespace dnn {

class Device {
public:
    explicit Device(int id);

    int id() const { return id_; }
    const cudaDeviceProp& properties() const { return prop_; }
    std::string name() const { return prop_.name; }
    size_t total_memory() const { return prop_.totalGlobalMem; }
    int sm_count() const { return prop_.multiProcessorCount; }
    int compute_major() const { return prop_.major; }
    int compute_minor() const { return prop_.minor; }
    // architecture family by compute capability (10.x is Blackwell)
    std::string architecture() const;
    void dump_info(std::ostream& os = std::cout) const;

private:
    int id_;
    cudaDeviceProp prop_{};
};

}  // namespace dnn
