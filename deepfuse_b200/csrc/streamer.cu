// Layer-streaming weight upload: per-layer byte blobs live in one pinned host arena and are copied,
// layer by layer, into a small ring of device slots on a side stream while earlier layers compute.
//
// The model in the upstream project is apps/host-multi/NVMeLoader_Linux.hpp:38-183: page-aligned pinned
// slots (cudaHostAlloc), one stream per slot, cudaMemcpyAsync host->device, and a (device pointer,
// size, stream) hand-off to the consumer (:90-134).  Upstream fills its slots with a blocking pread
// and never wires the loader into a model; here the arena is filled once (the quantised fp8 weights)
// and the ring is driven by the model's layer loop with events in both directions:
//   copied[slot]  recorded on the copy stream after the upload   -> the compute stream waits on it
//   freed[slot]   recorded on the compute stream after the layer -> the next upload into the slot waits on it
// Nothing here synchronises the host with the device.
#include "df8_internal.cuh"

#include <new>
#include <vector>

struct df8_streamer {
    size_t slot_bytes = 0;
    int n_slots = 0;
    int n_layers = 0;
    int device = 0;
    uint8_t* host_arena = nullptr;  // n_layers * slot_bytes, pinned
    uint8_t* dev_slots = nullptr;   // n_slots * slot_bytes
    cudaStream_t copy_stream = nullptr;
    std::vector<cudaEvent_t> copied, freed;
    std::vector<int> slot_layer;    // which layer each slot holds or is receiving (-1: none)
    std::vector<char> freed_valid;  // freed[slot] has been recorded at least once
    unsigned long long bytes_uploaded = 0;
};

using namespace df8;

extern "C" df8_status df8_streamer_create(size_t slot_bytes, int n_slots, int n_layers, df8_streamer** out) {
    DF8_REQUIRE(out != nullptr, "df8_streamer_create: out is null");
    DF8_REQUIRE(slot_bytes > 0 && n_slots >= 1 && n_layers >= 1, "df8_streamer_create: bad sizes");
    *out = nullptr;
    df8_streamer* s = new (std::nothrow) df8_streamer();
    if (!s) return fail(DF8_ERR_INVALID, "df8_streamer_create: out of host memory");
    s->slot_bytes = (slot_bytes + 255) & ~size_t(255);
    s->n_slots = n_slots < n_layers ? n_slots : n_layers;
    s->n_layers = n_layers;
    auto bail = [&](cudaError_t e, const char* what) {
        df8_status rc = fail(DF8_ERR_CUDA, "df8_streamer_create: %s failed: %s", what, cudaGetErrorString(e));
        if (s->host_arena) cudaFreeHost(s->host_arena);
        if (s->dev_slots) cudaFree(s->dev_slots);
        if (s->copy_stream) cudaStreamDestroy(s->copy_stream);
        for (cudaEvent_t ev : s->copied) cudaEventDestroy(ev);
        for (cudaEvent_t ev : s->freed) cudaEventDestroy(ev);
        delete s;
        return rc;
    };
    cudaError_t e = cudaGetDevice(&s->device);
    if (e != cudaSuccess) return bail(e, "cudaGetDevice");
    e = cudaHostAlloc(reinterpret_cast<void**>(&s->host_arena), s->slot_bytes * size_t(n_layers), cudaHostAllocDefault);
    if (e != cudaSuccess) return bail(e, "cudaHostAlloc");
    e = cudaMalloc(reinterpret_cast<void**>(&s->dev_slots), s->slot_bytes * size_t(s->n_slots));
    if (e != cudaSuccess) return bail(e, "cudaMalloc");
    e = cudaStreamCreateWithFlags(&s->copy_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return bail(e, "cudaStreamCreateWithFlags");
    for (int i = 0; i < s->n_slots; ++i) {
        cudaEvent_t a = nullptr, b = nullptr;
        e = cudaEventCreateWithFlags(&a, cudaEventDisableTiming);
        if (e != cudaSuccess) return bail(e, "cudaEventCreateWithFlags");
        s->copied.push_back(a);
        e = cudaEventCreateWithFlags(&b, cudaEventDisableTiming);
        if (e != cudaSuccess) return bail(e, "cudaEventCreateWithFlags");
        s->freed.push_back(b);
    }
    s->slot_layer.assign(size_t(s->n_slots), -1);
    s->freed_valid.assign(size_t(s->n_slots), 0);
    *out = s;
    return DF8_OK;
}

extern "C" df8_status df8_streamer_destroy(df8_streamer* s) {
    if (!s) return DF8_OK;
    cudaStreamSynchronize(s->copy_stream);
    for (cudaEvent_t ev : s->copied) cudaEventDestroy(ev);
    for (cudaEvent_t ev : s->freed) cudaEventDestroy(ev);
    cudaStreamDestroy(s->copy_stream);
    cudaFree(s->dev_slots);
    cudaFreeHost(s->host_arena);
    delete s;
    return DF8_OK;
}

extern "C" df8_status df8_streamer_host_ptr(df8_streamer* s, int layer, void** host_ptr_h) {
    DF8_REQUIRE(s && host_ptr_h, "df8_streamer_host_ptr: null argument");
    DF8_REQUIRE(layer >= 0 && layer < s->n_layers, "df8_streamer_host_ptr: layer %d out of range", layer);
    *host_ptr_h = s->host_arena + size_t(layer) * s->slot_bytes;
    return DF8_OK;
}

extern "C" df8_status df8_streamer_prefetch(df8_streamer* s, int layer) {
    DF8_REQUIRE(s != nullptr, "df8_streamer_prefetch: null streamer");
    DF8_REQUIRE(layer >= 0 && layer < s->n_layers, "df8_streamer_prefetch: layer %d out of range", layer);
    const int slot = layer % s->n_slots;
    if (s->slot_layer[size_t(slot)] == layer) return DF8_OK;  // already resident or on its way
    if (s->freed_valid[size_t(slot)]) DF8_CUDA_TRY(cudaStreamWaitEvent(s->copy_stream, s->freed[size_t(slot)], 0));
    DF8_CUDA_TRY(cudaMemcpyAsync(s->dev_slots + size_t(slot) * s->slot_bytes,
                                 s->host_arena + size_t(layer) * s->slot_bytes, s->slot_bytes, cudaMemcpyHostToDevice,
                                 s->copy_stream));
    DF8_CUDA_TRY(cudaEventRecord(s->copied[size_t(slot)], s->copy_stream));
    s->slot_layer[size_t(slot)] = layer;
    s->bytes_uploaded += s->slot_bytes;
    return DF8_OK;
}

extern "C" df8_status df8_streamer_acquire(df8_streamer* s, int layer, df8_stream compute_stream, void** dev_ptr_h) {
    DF8_REQUIRE(s && dev_ptr_h, "df8_streamer_acquire: null argument");
    DF8_REQUIRE(layer >= 0 && layer < s->n_layers, "df8_streamer_acquire: layer %d out of range", layer);
    const int slot = layer % s->n_slots;
    if (s->slot_layer[size_t(slot)] != layer) {
        df8_status rc = df8_streamer_prefetch(s, layer);  // not staged ahead of time: upload now (no overlap)
        if (rc != DF8_OK) return rc;
    }
    DF8_CUDA_TRY(cudaStreamWaitEvent(as_stream(compute_stream), s->copied[size_t(slot)], 0));
    *dev_ptr_h = s->dev_slots + size_t(slot) * s->slot_bytes;
    return DF8_OK;
}

extern "C" df8_status df8_streamer_release(df8_streamer* s, int layer, df8_stream compute_stream) {
    DF8_REQUIRE(s != nullptr, "df8_streamer_release: null streamer");
    DF8_REQUIRE(layer >= 0 && layer < s->n_layers, "df8_streamer_release: layer %d out of range", layer);
    const int slot = layer % s->n_slots;
    DF8_REQUIRE(s->slot_layer[size_t(slot)] == layer, "df8_streamer_release: layer %d is not resident", layer);
    DF8_CUDA_TRY(cudaEventRecord(s->freed[size_t(slot)], as_stream(compute_stream)));
    s->freed_valid[size_t(slot)] = 1;
    return DF8_OK;
}

extern "C" df8_status df8_streamer_stats(df8_streamer* s, unsigned long long* bytes_uploaded_h, size_t* slot_bytes_h,
                                         int* n_slots_h) {
    DF8_REQUIRE(s != nullptr, "df8_streamer_stats: null streamer");
    if (bytes_uploaded_h) *bytes_uploaded_h = s->bytes_uploaded;
    if (slot_bytes_h) *slot_bytes_h = s->slot_bytes;
    if (n_slots_h) *n_slots_h = s->n_slots;
    return DF8_OK;
}
