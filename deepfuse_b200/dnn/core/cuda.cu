#include "dnn/core/cuda.cuh"

#include <iomanip>
#include <mutex>
#include <stdexcept>
#include <string>

namespace dnn {

namespace {
thread_local Cuda* t_current = nullptr;
thread_local cudaStream_t t_stream = cudaStreamLegacy;
}  // namespace

Device::Device(int id) : id_(id) { utils::CHECK_CUDA_EX(cudaGetDeviceProperties(&prop_, id)); }

std::string Device::architecture() const {
    switch (prop_.major) {
        case 7: return prop_.minor >= 5 ? "Turing" : "Volta";
        case 8: return prop_.minor == 9 ? "Ada" : "Ampere";
        case 9: return "Hopper";
        case 10: return "Blackwell";
        case 12: return "Blackwell (consumer)";
        default: return "unknown";
    }
}

void Device::dump_info(std::ostream& os) const {
    os << "Device " << id_ << ": " << prop_.name << " (" << architecture() << ", cc " << prop_.major << "."
       << prop_.minor << "), " << prop_.multiProcessorCount << " SMs, " << std::fixed << std::setprecision(1)
       << double(prop_.totalGlobalMem) / double(1ull << 30) << " GiB\n";
}

Cuda::Cuda(int device_id) : id_(device_id), previous_(t_current) {
    int count = 0;
    utils::CHECK_CUDA_EX(cudaGetDeviceCount(&count));
    if (device_id < 0 || device_id >= count)
        throw std::runtime_error("Invalid CUDA device id " + std::to_string(device_id) + " (" +
                                 std::to_string(count) + " devices)");
    utils::CHECK_CUDA_EX(cudaSetDevice(device_id));
    utils::CHECK_CUDA_EX(cudaFree(nullptr));  // force context creation on this thread
    // keep freed tensor memory in the stream-ordered pool instead of returning it to the driver
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, device_id) == cudaSuccess) {
        unsigned long long keep = ~0ull;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    t_current = this;
}

Cuda::~Cuda() {
    if (t_current == this) t_current = previous_;
}

Cuda& Cuda::current() {
    if (!t_current) throw std::runtime_error("No current Cuda instance on this thread");
    return *t_current;
}

const std::vector<Device>& Cuda::get_devices() {
    static std::vector<Device> devices;
    static std::once_flag once;
    std::call_once(once, [] {
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess) count = 0;
        for (int i = 0; i < count; ++i) devices.emplace_back(i);
    });
    return devices;
}

void Cuda::dump_info(std::ostream& os) const {
    for (const Device& d : get_devices()) d.dump_info(os);
    os << "current device: " << id_ << "\n";
}

void Cuda::set_stream(cudaStream_t stream) { t_stream = stream; }
cudaStream_t Cuda::stream() { return t_stream; }

StreamGuard::StreamGuard(cudaStream_t new_stream) : previous_(Cuda::stream()) { Cuda::set_stream(new_stream); }
StreamGuard::~StreamGuard() { Cuda::set_stream(previous_); }

}  // namespace dnn
