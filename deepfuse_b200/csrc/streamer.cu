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
// Nothing here synchronises the host with the device (except the calls that say so).
//
// Slots are handed out in the order of the uploads (a ring over the execution order, not layer % n_slots):
// with the model's loop acquire(l), release(l), prefetch(l + n_slots) the slot that is refilled is always the
// one that was just released, whatever the ratio of layers to slots.
//
// With several GPUs working on shares of one batch (one process per GPU, the same layer loop on each), every
// rank would pull every layer over its own PCIe link from the same host memory.  A streamer created with a
// communicator uploads only its 1/world share of a layer and completes the slot with an all-gather over
// NVLink on the copy stream, so host->device traffic per rank falls world-fold; every rank must then issue
// the same sequence of prefetch / acquire calls (the all-gather is a collective).
// With DF8_STREAM_P2P=1 in the environment (read when the streamer is created; every rank the same) the slots live
// in a buffer that every rank maps into every other (df8_comm_symm_alloc) and the gather is df8_comm_allgather_symm:
// the copy engines write a rank's share straight into its peers' slots, so no NCCL kernel competes for SMs with the
// forward's persistent kernels.  The writes are one-sided: before a rank pushes into the peers' copies of a slot,
// all ranks meet at a barrier on their copy streams (a one-warp kernel), each after the event that says its own
// readers of the slot's previous occupant are done.  Off by default: faster on two GPUs, but on eight the bounded
// waits of the exchange ran out about once per forward (status word 0x5002) for a reason not yet found.
#include "df8_internal.cuh"

#include <cstdlib>
#include <new>
#include <vector>

struct df8_streamer {
    size_t slot_bytes = 0;   // a layer's blob, padded to a multiple of 256 * world bytes
    size_t part_bytes = 0;   // slot_bytes / world: what this rank uploads itself
    int n_slots = 0;
    int n_layers = 0;
    int device = 0;
    int rank = 0, world = 1;
    df8_comm* comm = nullptr;       // not owned
    uint8_t* host_arena = nullptr;  // n_layers * slot_bytes, pinned
    uint8_t* dev_slots = nullptr;   // n_slots * slot_bytes
    bool use_p2p = false;           // DF8_STREAM_P2P=1: peer-mapped slots and copy-engine pushes instead of ncclAllGather
    bool slots_symm = false;        // dev_slots is a peer-mapped buffer of the communicator (lives as long as it does)
    float* barrier_value = nullptr; // operand of the barrier in front of the one-sided pushes
    cudaStream_t copy_stream = nullptr;
    std::vector<cudaEvent_t> copied, freed;
    std::vector<int> slot_layer;    // which layer each slot holds or is receiving (-1: none)
    std::vector<int> layer_slot;    // the slot a layer is in (-1: not on the device)
    std::vector<char> freed_valid;  // freed[slot] has been recorded since the slot was last filled
    int next_slot = 0;              // ring position of the next upload
    unsigned long long bytes_uploaded = 0;  // bytes that became available on the device (slot_bytes per upload)
    unsigned long long bytes_h2d = 0;       // bytes this rank copied from host memory
    unsigned long long bytes_gathered = 0;  // bytes this rank received from its peers
};

using namespace df8;

namespace {

void destroy_events(df8_streamer* s) {
    for (cudaEvent_t ev : s->copied) cudaEventDestroy(ev);
    for (cudaEvent_t ev : s->freed) cudaEventDestroy(ev);
    s->copied.clear();
    s->freed.clear();
}

df8_status make_slots(df8_streamer* s, int n_slots) {
    s->n_slots = n_slots < s->n_layers ? n_slots : s->n_layers;
    if (s->comm && s->use_p2p) {  // collective: every rank makes its slots at the same point
        void* p = nullptr;
        df8_status rc = df8_comm_symm_alloc(s->comm, s->slot_bytes * size_t(s->n_slots), &p);
        if (rc != DF8_OK) return rc;
        s->dev_slots = static_cast<uint8_t*>(p);
        s->slots_symm = true;
        if (!s->barrier_value) {
            DF8_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&s->barrier_value), sizeof(float)));
            DF8_CUDA_TRY(cudaMemset(s->barrier_value, 0, sizeof(float)));
        }
    } else {
        DF8_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&s->dev_slots), s->slot_bytes * size_t(s->n_slots)));
    }
    for (int i = 0; i < s->n_slots; ++i) {
        cudaEvent_t a = nullptr, b = nullptr;
        DF8_CUDA_TRY(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        s->copied.push_back(a);
        DF8_CUDA_TRY(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        s->freed.push_back(b);
    }
    s->slot_layer.assign(size_t(s->n_slots), -1);
    s->layer_slot.assign(size_t(s->n_layers), -1);
    s->freed_valid.assign(size_t(s->n_slots), 0);
    s->next_slot = 0;
    return DF8_OK;
}

// Uploads `layer` into the ring's next slot (evicting what is there).
df8_status upload(df8_streamer* s, int layer) {
    const int slot = s->next_slot;
    s->next_slot = (s->next_slot + 1) % s->n_slots;
    const int old = s->slot_layer[size_t(slot)];
    if (old >= 0) s->layer_slot[size_t(old)] = -1;
    // the kernels that read the slot's previous occupant must be done
    if (s->freed_valid[size_t(slot)]) DF8_CUDA_TRY(cudaStreamWaitEvent(s->copy_stream, s->freed[size_t(slot)], 0));
    uint8_t* dst = s->dev_slots + size_t(slot) * s->slot_bytes;
    const uint8_t* src = s->host_arena + size_t(layer) * s->slot_bytes;
    const size_t off = size_t(s->rank) * s->part_bytes;
    DF8_CUDA_TRY(cudaMemcpyAsync(dst + off, src + off, s->part_bytes, cudaMemcpyHostToDevice, s->copy_stream));
    if (s->world > 1) {  // in place: this rank's share already sits at its position in the slot
        const df8_stream cs = reinterpret_cast<df8_stream>(s->copy_stream);
        df8_status rc;
        if (s->slots_symm) {
            // every rank's readers of the slot's previous occupant are done before anybody writes into it
            rc = df8_comm_allreduce_max_p2p(s->comm, s->barrier_value, cs);
            if (rc != DF8_OK) return rc;
            rc = df8_comm_allgather_symm(s->comm, s->dev_slots, size_t(slot) * s->slot_bytes, s->part_bytes, cs);
        } else {
            rc = df8_comm_allgather_u8(s->comm, dst + off, dst, s->part_bytes, cs);
        }
        if (rc != DF8_OK) return rc;
    }
    DF8_CUDA_TRY(cudaEventRecord(s->copied[size_t(slot)], s->copy_stream));
    s->slot_layer[size_t(slot)] = layer;
    s->layer_slot[size_t(layer)] = slot;
    s->freed_valid[size_t(slot)] = 0;
    s->bytes_uploaded += s->slot_bytes;
    s->bytes_h2d += s->part_bytes;
    s->bytes_gathered += s->slot_bytes - s->part_bytes;
    return DF8_OK;
}

}  // namespace

extern "C" df8_status df8_streamer_create(size_t slot_bytes, int n_slots, int n_layers, df8_streamer** out) {
    return df8_streamer_create_sharded(slot_bytes, n_slots, n_layers, nullptr, out);
}

extern "C" df8_status df8_streamer_create_sharded(size_t slot_bytes, int n_slots, int n_layers, df8_comm* comm,
                                                  df8_streamer** out) {
    DF8_REQUIRE(out != nullptr, "df8_streamer_create: out is null");
    DF8_REQUIRE(slot_bytes > 0 && n_slots >= 1 && n_layers >= 1, "df8_streamer_create: bad sizes");
    *out = nullptr;
    df8_streamer* s = new (std::nothrow) df8_streamer();
    if (!s) return fail(DF8_ERR_INVALID, "df8_streamer_create: out of host memory");
    if (comm) {
        df8_status rc = df8_comm_rank(comm, &s->rank, &s->world);
        if (rc != DF8_OK) {
            delete s;
            return rc;
        }
        if (s->world > 1) s->comm = comm;
        const char* e = getenv("DF8_STREAM_P2P");
        s->use_p2p = s->comm != nullptr && e && e[0] == '1';
    }
    const size_t unit = size_t(256) * size_t(s->world);
    s->slot_bytes = (slot_bytes + unit - 1) / unit * unit;
    s->part_bytes = s->slot_bytes / size_t(s->world);
    s->n_layers = n_layers;
    auto bail = [&](df8_status rc) {
        if (s->host_arena) cudaFreeHost(s->host_arena);
        if (s->dev_slots && !s->slots_symm) cudaFree(s->dev_slots);
        if (s->barrier_value) cudaFree(s->barrier_value);
        if (s->copy_stream) cudaStreamDestroy(s->copy_stream);
        destroy_events(s);
        delete s;
        return rc;
    };
    auto cuda_bail = [&](cudaError_t e, const char* what) {
        return bail(fail(DF8_ERR_CUDA, "df8_streamer_create: %s failed: %s", what, cudaGetErrorString(e)));
    };
    cudaError_t e = cudaGetDevice(&s->device);
    if (e != cudaSuccess) return cuda_bail(e, "cudaGetDevice");
    e = cudaHostAlloc(reinterpret_cast<void**>(&s->host_arena), s->slot_bytes * size_t(n_layers), cudaHostAllocDefault);
    if (e != cudaSuccess) return cuda_bail(e, "cudaHostAlloc");
    e = cudaStreamCreateWithFlags(&s->copy_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return cuda_bail(e, "cudaStreamCreateWithFlags");
    df8_status rc = make_slots(s, n_slots);
    if (rc != DF8_OK) return bail(rc);
    *out = s;
    return DF8_OK;
}

extern "C" df8_status df8_streamer_destroy(df8_streamer* s) {
    if (!s) return DF8_OK;
    cudaStreamSynchronize(s->copy_stream);
    destroy_events(s);
    cudaStreamDestroy(s->copy_stream);
    if (!s->slots_symm) cudaFree(s->dev_slots);
    if (s->barrier_value) cudaFree(s->barrier_value);
    cudaFreeHost(s->host_arena);
    delete s;
    return DF8_OK;
}

extern "C" df8_status df8_streamer_resize(df8_streamer* s, int n_slots) {
    DF8_REQUIRE(s != nullptr && n_slots >= 1, "df8_streamer_resize: bad argument");
    DF8_CUDA_TRY(cudaDeviceSynchronize());  // nothing may still read or fill the old slots
    destroy_events(s);
    if (!s->slots_symm) DF8_CUDA_TRY(cudaFree(s->dev_slots));  // (a peer-mapped buffer stays with the communicator)
    s->dev_slots = nullptr;
    return make_slots(s, n_slots);
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
    if (s->layer_slot[size_t(layer)] >= 0) return DF8_OK;  // already resident or on its way
    return upload(s, layer);
}

extern "C" df8_status df8_streamer_acquire(df8_streamer* s, int layer, df8_stream compute_stream, void** dev_ptr_h) {
    DF8_REQUIRE(s && dev_ptr_h, "df8_streamer_acquire: null argument");
    DF8_REQUIRE(layer >= 0 && layer < s->n_layers, "df8_streamer_acquire: layer %d out of range", layer);
    if (s->layer_slot[size_t(layer)] < 0) {
        df8_status rc = upload(s, layer);  // not staged ahead of time: upload now (no overlap)
        if (rc != DF8_OK) return rc;
    }
    const int slot = s->layer_slot[size_t(layer)];
    DF8_CUDA_TRY(cudaStreamWaitEvent(as_stream(compute_stream), s->copied[size_t(slot)], 0));
    *dev_ptr_h = s->dev_slots + size_t(slot) * s->slot_bytes;
    return DF8_OK;
}

extern "C" df8_status df8_streamer_release(df8_streamer* s, int layer, df8_stream compute_stream) {
    DF8_REQUIRE(s != nullptr, "df8_streamer_release: null streamer");
    DF8_REQUIRE(layer >= 0 && layer < s->n_layers, "df8_streamer_release: layer %d out of range", layer);
    const int slot = s->layer_slot[size_t(layer)];
    DF8_REQUIRE(slot >= 0, "df8_streamer_release: layer %d is not resident", layer);
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

extern "C" df8_status df8_streamer_traffic(df8_streamer* s, unsigned long long* h2d_bytes_h,
                                           unsigned long long* gathered_bytes_h) {
    DF8_REQUIRE(s != nullptr, "df8_streamer_traffic: null streamer");
    if (h2d_bytes_h) *h2d_bytes_h = s->bytes_h2d;
    if (gathered_bytes_h) *gathered_bytes_h = s->bytes_gathered;
    return DF8_OK;
}

extern "C" df8_status df8_streamer_time_uploads(df8_streamer* s, float* ms_h) {
    DF8_REQUIRE(s && ms_h, "df8_streamer_time_uploads: null argument");
    DF8_CUDA_TRY(cudaDeviceSynchronize());
    cudaEvent_t a = nullptr, b = nullptr;
    DF8_CUDA_TRY(cudaEventCreate(&a));
    DF8_CUDA_TRY(cudaEventCreate(&b));
    df8_status rc = DF8_OK;
    cudaError_t e = cudaEventRecord(a, s->copy_stream);
    for (int l = 0; l < s->n_layers && rc == DF8_OK && e == cudaSuccess; ++l) rc = upload(s, l);
    if (e == cudaSuccess) e = cudaEventRecord(b, s->copy_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->copy_stream);
    if (e == cudaSuccess && rc == DF8_OK) e = cudaEventElapsedTime(ms_h, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (rc != DF8_OK) return rc;
    if (e != cudaSuccess) return fail(DF8_ERR_CUDA, "df8_streamer_time_uploads: %s", cudaGetErrorString(e));
    return DF8_OK;
}
