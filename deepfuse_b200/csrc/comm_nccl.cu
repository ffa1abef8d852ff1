// Collective communication for the column-sharded fully-connected path: NCCL over NVLink / NVSwitch.
//
// The upstream project has no communication backend at all: its "multi-GPU" mode is a tbb::parallel_for
// over independent per-device model replicas that never exchange a byte (apps/host-multi/main.cpp:157-181).
// Splitting one layer's weights across GPUs therefore needs new plumbing.  The library binds NCCL at run
// time (dlopen of libnccl.so.2) so that it loads on machines without NCCL and, inside a process that
// already carries a NCCL (PyTorch's), uses that same copy.
//
// One communicator per process (one process per GPU).  The 128-byte unique id is produced on rank 0 by
// df8_comm_unique_id and handed to the other ranks by whatever channel the host program has
// (torch.distributed, a file, MPI); df8_comm_init_rank is collective.
#include "df8_internal.cuh"

#include <dlfcn.h>

#include <cstring>
#include <mutex>

namespace {

// the handful of NCCL declarations used, so that no NCCL header is needed to build
typedef struct ncclComm* ncclComm_t;
struct ncclUniqueId {
    char internal[128];
};
enum { ncclSuccess = 0 };
enum { ncclUint8 = 1, ncclFloat32 = 7 };  // ncclDataType_t
enum { ncclMax = 2 };                     // ncclRedOp_t

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(ncclUniqueId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*CommAbort)(ncclComm_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    int (*GetVersion)(int*) = nullptr;
    bool ok = false;
};

NcclApi& api() {
    static NcclApi a;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (a.handle) break;
        }
        if (!a.handle) return;
        auto sym = [&](const char* s) { return dlsym(a.handle, s); };
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
        a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(sym("ncclCommAbort"));
        a.AllGather = reinterpret_cast<decltype(a.AllGather)>(sym("ncclAllGather"));
        a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
        a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
        a.GetVersion = reinterpret_cast<decltype(a.GetVersion)>(sym("ncclGetVersion"));
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllGather && a.AllReduce && a.GetErrorString;
    });
    return a;
}

df8_status nccl_fail(const char* what, int rc) {
    const char* text = api().GetErrorString ? api().GetErrorString(rc) : "?";
    return df8::fail(DF8_ERR_COMM, "%s failed: NCCL error %d (%s)", what, rc, text);
}

}  // namespace

struct df8_comm {
    ncclComm_t comm = nullptr;
    int world = 1;
    int rank = 0;
};

using namespace df8;

extern "C" df8_status df8_comm_available(int* version_h) {
    if (!api().ok) return fail(DF8_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
    if (version_h) {
        *version_h = 0;
        if (api().GetVersion) api().GetVersion(version_h);
    }
    return DF8_OK;
}

extern "C" df8_status df8_comm_unique_id(void* id_h) {
    DF8_REQUIRE(id_h != nullptr, "df8_comm_unique_id: id_h is null");
    if (!api().ok) return fail(DF8_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
    ncclUniqueId id;
    int rc = api().GetUniqueId(&id);
    if (rc != ncclSuccess) return nccl_fail("ncclGetUniqueId", rc);
    std::memcpy(id_h, &id, sizeof(id));
    return DF8_OK;
}

extern "C" df8_status df8_comm_init_rank(const void* id_h, int world, int rank, df8_comm** out) {
    DF8_REQUIRE(id_h && out, "df8_comm_init_rank: null argument");
    DF8_REQUIRE(world >= 1 && rank >= 0 && rank < world, "df8_comm_init_rank: bad rank %d of %d", rank, world);
    if (!api().ok) return fail(DF8_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
    ncclUniqueId id;
    std::memcpy(&id, id_h, sizeof(id));
    df8_comm* c = new df8_comm();
    c->world = world;
    c->rank = rank;
    int rc = api().CommInitRank(&c->comm, world, id, rank);
    if (rc != ncclSuccess) {
        delete c;
        return nccl_fail("ncclCommInitRank", rc);
    }
    *out = c;
    return DF8_OK;
}

extern "C" df8_status df8_comm_destroy(df8_comm* c) {
    if (!c) return DF8_OK;
    int rc = c->comm ? api().CommDestroy(c->comm) : ncclSuccess;
    delete c;
    return rc == ncclSuccess ? DF8_OK : nccl_fail("ncclCommDestroy", rc);
}

// Host-initiated abort of a communicator whose peer has gone away: outstanding collectives end with an
// error instead of waiting for ever.  Never called from the data path.
extern "C" df8_status df8_comm_abort(df8_comm* c) {
    if (!c) return DF8_OK;
    int rc = (c->comm && api().CommAbort) ? api().CommAbort(c->comm) : ncclSuccess;
    c->comm = nullptr;
    delete c;
    return rc == ncclSuccess ? DF8_OK : nccl_fail("ncclCommAbort", rc);
}

extern "C" df8_status df8_comm_rank(const df8_comm* c, int* rank_h, int* world_h) {
    DF8_REQUIRE(c != nullptr, "df8_comm_rank: null communicator");
    if (rank_h) *rank_h = c->rank;
    if (world_h) *world_h = c->world;
    return DF8_OK;
}

extern "C" df8_status df8_comm_allgather_u8(df8_comm* c, const uint8_t* send_d, uint8_t* recv_d, size_t bytes_per_rank,
                                            df8_stream stream) {
    DF8_REQUIRE(c && c->comm, "df8_comm_allgather_u8: null communicator");
    DF8_REQUIRE(bytes_per_rank == 0 || (send_d && recv_d), "df8_comm_allgather_u8: null buffer");
    if (bytes_per_rank == 0) return DF8_OK;
    int rc = api().AllGather(send_d, recv_d, bytes_per_rank, ncclUint8, c->comm, as_stream(stream));
    return rc == ncclSuccess ? DF8_OK : nccl_fail("ncclAllGather", rc);
}

extern "C" df8_status df8_comm_allreduce_max_f32(df8_comm* c, float* buf_d, size_t count, df8_stream stream) {
    DF8_REQUIRE(c && c->comm, "df8_comm_allreduce_max_f32: null communicator");
    DF8_REQUIRE(count == 0 || buf_d, "df8_comm_allreduce_max_f32: null buffer");
    if (count == 0) return DF8_OK;
    int rc = api().AllReduce(buf_d, buf_d, count, ncclFloat32, ncclMax, c->comm, as_stream(stream));
    return rc == ncclSuccess ? DF8_OK : nccl_fail("ncclAllReduce", rc);
}
