// Cuda: per-host-thread device context, and the thread's current stream.
//
// Public surface of upstream dnn/core/cuda.cuh:23-71 (Cuda(int), id, current, get_devices, dump_info,
// set_stream, stream, StreamGuard) with the same thread-local semantics (dnn/core/cuda.cu:21-99).
// Difference in substance: upstream never hands Cuda::stream() to a launch; here every kernel and
// every tensor allocation of the dnn:: classes is ordered on it.
#pragma once

#include <cuda_runtime.h>

#include <iostream>
#include <vector>

#include "dnn/core/device.cuh"
#include "dnn/utils/common.cuh"

namespace dnn {

class Cuda {
public:
    explicit Cuda(int device_id = 0);
    ~Cuda();
    Cuda(const Cuda&) = delete;
    Cuda& operator=(const Cuda&) = delete;

    int id() const { return id_; }

    // The instance most recently constructed on this thread; throws std::runtime_error if none.
    static Cuda& current();
    static const std::vector<Device>& get_devices();
    void dump_info(std::ostream& os = std::cout) const;

    // Stream multiplexing: the stream every dnn:: launch on this thread is enqueued on.
    // Unset, it is the legacy default stream (as upstream returns, cuda.cu:85-87).
    static void set_stream(cudaStream_t stream);
    static cudaStream_t stream();

private:
    int id_;
    Cuda* previous_;
};

// Scoped replacement of the thread's current stream.
class StreamGuard {
public:
    explicit StreamGuard(cudaStream_t new_stream);
    ~StreamGuard();
    StreamGuard(const StreamGuard&) = delete;
    StreamGuard& operator=(const StreamGuard&) = delete;

private:
    cudaStream_t previous_;
};

}  // namespace dnn
