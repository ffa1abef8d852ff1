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

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

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

// ---- peer-to-peer exchange state ------------------------------------------------------------------------
//
// NCCL moves data with kernels that need SMs of their own and cost ~15-25 us per call on eight GPUs; the
// column-sharded forward issues eleven exchanges per transformer layer, most of them a single float.  The
// exchanges of that path therefore go through buffers every rank has mapped from every other rank (cudaMalloc +
// CUDA IPC handles, exchanged once over NCCL):
//   * large slices travel with the copy engines (cudaMemcpyAsync to the peer mapping on a side stream) straight
//     into the peers' copy of the buffer, and a one-warp kernel then stores this exchange's sequence number into
//     a flag word of every peer; the consumer's stream waits for the flags of all peers with a bounded poll;
//   * one float (a per-tensor maximum) travels inside the flag itself: one kernel per rank stores {sequence,
//     value} into a slot of every peer, polls its own slots (bounded) and reduces.
// Every rank issues the same sequence of exchanges, so a sequence number identifies an exchange on all ranks;
// flags and slots are rings indexed by it, deep enough that no rank can lap another (a rank can be at most one
// exchange ahead: it cannot finish exchange k+1 before every peer has contributed to it).
constexpr int kFlagRing = 64;   // flag words per peer
constexpr int kSlotRing = 64;   // {sequence, value} slots per peer
constexpr int kMaxPeers = 16;

struct Df8SymmBuf {
    uint8_t* local = nullptr;
    size_t bytes = 0;
    void* peer[kMaxPeers] = {};  // peer[r]: rank r's buffer as mapped here (peer[rank] == local)
};

struct Df8PeerPtrs {
    void* p[kMaxPeers];
};

struct df8_comm {
    ncclComm_t comm = nullptr;
    int world = 1;
    int rank = 0;
    // p2p exchange (set up lazily by the first symmetric allocation)
    bool p2p_tried = false, p2p_ok = false;
    std::vector<Df8SymmBuf> symm;
    int ctrl = -1;                    // index in symm of the control buffer: flags [world][kFlagRing] u32, then
                                      // slots [kSlotRing][world] u64
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_ready = nullptr, ev_sent = nullptr;
    uint32_t seq = 0;                 // exchanges of slices issued so far
    uint32_t slot_seq = 0;            // single-float exchanges issued so far
    unsigned long long bytes_pushed = 0;
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

namespace {
// Unmaps the peers' buffers and frees this rank's.  By the time a rank gets here its last exchange has completed,
// i.e. every peer's last write into its buffers has arrived, so nobody writes into memory freed here.
void release_p2p(df8_comm* c) {
    cudaDeviceSynchronize();
    for (Df8SymmBuf& b : c->symm) {
        for (int r = 0; r < c->world && r < kMaxPeers; ++r)
            if (r != c->rank && b.peer[r]) cudaIpcCloseMemHandle(b.peer[r]);
        if (b.local) cudaFree(b.local);
    }
    c->symm.clear();
    if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
    if (c->ev_ready) cudaEventDestroy(c->ev_ready);
    if (c->ev_sent) cudaEventDestroy(c->ev_sent);
    c->copy_stream = nullptr;
    c->ev_ready = c->ev_sent = nullptr;
    (void)cudaGetLastError();
}
}  // namespace

extern "C" df8_status df8_comm_destroy(df8_comm* c) {
    if (!c) return DF8_OK;
    release_p2p(c);
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
    release_p2p(c);
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

// ---- peer-to-peer exchanges (see the comment at df8_comm) -----------------------------------------------

namespace {

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void note_timeout(unsigned int* status, unsigned int code) {
    if (status) {
        atomicCAS(status, 0u, code);
        atomicAdd(status + 1, 1u);
    }
}

constexpr unsigned long long kPeerWaitNs = 2000000000ull;  // a peer that has not answered after 2 s is gone

// After this rank's slices have been copied (stream order): tell every peer, by storing the exchange's sequence
// number into this rank's flag word of the peer's control buffer.
__global__ void signal_peers_kernel(Df8PeerPtrs ctrl, int rank, int world, uint32_t seq) {
    const int p = threadIdx.x;
    if (p < world && p != rank) {
        uint32_t* flags = static_cast<uint32_t*>(ctrl.p[p]);
        st_release_sys_u32(flags + size_t(rank) * kFlagRing + (seq % kFlagRing), seq);
    }
}

// Bounded wait until every peer's flag word for this exchange holds its sequence number.
__global__ void wait_peers_kernel(const uint32_t* flags, int rank, int world, uint32_t seq, unsigned int* status) {
    const int p = threadIdx.x;
    if (p >= world || p == rank) return;
    const uint32_t* f = flags + size_t(p) * kFlagRing + (seq % kFlagRing);
    const unsigned long long t0 = now_ns();
    for (unsigned int spins = 0; ld_acquire_sys_u32(f) != seq; ++spins) {
        if ((spins & 63u) == 63u) {
            if (now_ns() - t0 > kPeerWaitNs) {
                note_timeout(status, 0x5000u + unsigned(p));
                return;
            }
            __nanosleep(200);
        }
    }
}

// One float, maximum over ranks, in place.  {sequence, value} goes into this rank's slot of every peer; the same
// kernel then polls its own slots (bounded) and reduces.  A rank whose peer never answers keeps its own value and
// records the event in the status word.
__global__ void allreduce_max_kernel(float* value, Df8PeerPtrs ctrl, int rank, int world, uint32_t seq,
                                     unsigned int* status) {
    const int p = threadIdx.x;
    const size_t slots_off = size_t(world) * kFlagRing * sizeof(uint32_t);  // slots follow the flags
    const float mine = *value;
    float v = mine;
    if (p < world && p != rank) {
        uint64_t* peer_slots = reinterpret_cast<uint64_t*>(static_cast<uint8_t*>(ctrl.p[p]) + slots_off);
        st_release_sys_u64(peer_slots + size_t(seq % kSlotRing) * world + rank,
                           (uint64_t(seq) << 32) | uint64_t(__float_as_uint(mine)));
        const uint64_t* my_slots = reinterpret_cast<const uint64_t*>(static_cast<uint8_t*>(ctrl.p[rank]) + slots_off);
        const uint64_t* slot = my_slots + size_t(seq % kSlotRing) * world + p;
        const unsigned long long t0 = now_ns();
        uint64_t got = ld_acquire_sys_u64(slot);
        for (unsigned int spins = 0; uint32_t(got >> 32) != seq; ++spins) {
            if ((spins & 63u) == 63u) {
                if (now_ns() - t0 > kPeerWaitNs) {
                    note_timeout(status, 0x5100u + unsigned(p));
                    got = (uint64_t(seq) << 32) | uint64_t(__float_as_uint(mine));
                    break;
                }
                __nanosleep(100);
            }
            got = ld_acquire_sys_u64(slot);
        }
        v = __uint_as_float(uint32_t(got));
    }
    // maxima of non-negative floats (NaN-free by construction: they come from atomicMax on bit patterns)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (p == 0) *value = v;
}

size_t ctrl_bytes(int world) {
    return size_t(world) * kFlagRing * sizeof(uint32_t) + size_t(kSlotRing) * size_t(world) * sizeof(uint64_t);
}

bool p2p_wanted() {
    const char* e = getenv("DF8_COMM_P2P");  // 0: every exchange through NCCL (profiling and tests)
    return !(e && e[0] == '0');
}

// cudaMalloc + map into every peer.  Collective.  On any failure the communicator falls back to NCCL for good.
df8_status symm_alloc(df8_comm* c, size_t bytes, int* index) {
    Df8SymmBuf b;
    b.bytes = bytes;
    DF8_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&b.local), bytes));
    DF8_CUDA_TRY(cudaMemset(b.local, 0, bytes));
    b.peer[c->rank] = b.local;
    bool ok = c->p2p_ok;
    cudaIpcMemHandle_t mine;
    std::memset(&mine, 0, sizeof(mine));
    if (ok && cudaIpcGetMemHandle(&mine, b.local) != cudaSuccess) {
        (void)cudaGetLastError();
        ok = false;
    }
    // handles of all ranks through NCCL (device staging); a rank that failed sends zeros and everybody sees it
    uint8_t *send_d = nullptr, *recv_d = nullptr;
    const size_t hb = sizeof(cudaIpcMemHandle_t) + 8;
    DF8_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&send_d), hb));
    DF8_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&recv_d), hb * size_t(c->world)));
    std::vector<uint8_t> stage(hb, 0), all(hb * size_t(c->world), 0);
    std::memcpy(stage.data(), &mine, sizeof(mine));
    stage[sizeof(mine)] = ok ? 1 : 0;
    DF8_CUDA_TRY(cudaMemcpy(send_d, stage.data(), hb, cudaMemcpyHostToDevice));
    df8_status rc = df8_comm_allgather_u8(c, send_d, recv_d, hb, nullptr);
    if (rc == DF8_OK) {
        DF8_CUDA_TRY(cudaStreamSynchronize(nullptr));
        DF8_CUDA_TRY(cudaMemcpy(all.data(), recv_d, all.size(), cudaMemcpyDeviceToHost));
    }
    cudaFree(send_d);
    cudaFree(recv_d);
    if (rc != DF8_OK) return rc;
    for (int r = 0; r < c->world; ++r) ok = ok && all[size_t(r) * hb + sizeof(mine)] == 1;
    if (ok) {
        for (int r = 0; r < c->world && ok; ++r) {
            if (r == c->rank) continue;
            cudaIpcMemHandle_t h;
            std::memcpy(&h, all.data() + size_t(r) * hb, sizeof(h));
            if (cudaIpcOpenMemHandle(&b.peer[r], h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                (void)cudaGetLastError();
                ok = false;
            }
        }
    }
    // agree on the outcome: one rank that could not map a peer switches everybody to NCCL
    float flag_h = ok ? 0.f : 1.f, *flag_d = nullptr;
    DF8_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&flag_d), sizeof(float)));
    DF8_CUDA_TRY(cudaMemcpy(flag_d, &flag_h, sizeof(float), cudaMemcpyHostToDevice));
    rc = df8_comm_allreduce_max_f32(c, flag_d, 1, nullptr);
    if (rc == DF8_OK) {
        DF8_CUDA_TRY(cudaStreamSynchronize(nullptr));
        DF8_CUDA_TRY(cudaMemcpy(&flag_h, flag_d, sizeof(float), cudaMemcpyDeviceToHost));
    }
    cudaFree(flag_d);
    if (rc != DF8_OK) return rc;
    if (flag_h != 0.f) {
        for (int r = 0; r < c->world; ++r)
            if (r != c->rank && b.peer[r]) {
                cudaIpcCloseMemHandle(b.peer[r]);
                b.peer[r] = nullptr;
            }
        c->p2p_ok = false;
    }
    c->symm.push_back(b);
    *index = int(c->symm.size()) - 1;
    return DF8_OK;
}

df8_status ensure_p2p(df8_comm* c) {
    if (c->p2p_tried) return DF8_OK;
    c->p2p_tried = true;
    c->p2p_ok = p2p_wanted() && c->world <= kMaxPeers;
    DF8_CUDA_TRY(cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
    DF8_CUDA_TRY(cudaEventCreateWithFlags(&c->ev_ready, cudaEventDisableTiming));
    DF8_CUDA_TRY(cudaEventCreateWithFlags(&c->ev_sent, cudaEventDisableTiming));
    return symm_alloc(c, ctrl_bytes(c->world), &c->ctrl);
}

const Df8SymmBuf* find_symm(const df8_comm* c, const void* p, size_t end_offset) {
    const uint8_t* q = static_cast<const uint8_t*>(p);
    for (const Df8SymmBuf& b : c->symm)
        if (q >= b.local && q + end_offset <= b.local + b.bytes) return &b;
    return nullptr;
}

Df8PeerPtrs ctrl_ptrs(const df8_comm* c) {
    Df8PeerPtrs pp = {};
    for (int r = 0; r < c->world; ++r) pp.p[r] = c->symm[size_t(c->ctrl)].peer[r];
    return pp;
}

}  // namespace

extern "C" df8_status df8_comm_symm_alloc(df8_comm* c, size_t bytes, void** local_d_h) {
    DF8_REQUIRE(c && c->comm && local_d_h, "df8_comm_symm_alloc: null argument");
    DF8_REQUIRE(bytes > 0, "df8_comm_symm_alloc: empty buffer");
    df8_status rc = ensure_p2p(c);
    if (rc != DF8_OK) return rc;
    int idx = -1;
    rc = symm_alloc(c, (bytes + 255) & ~size_t(255), &idx);
    if (rc != DF8_OK) return rc;
    *local_d_h = c->symm[size_t(idx)].local;
    return DF8_OK;
}

extern "C" df8_status df8_comm_p2p_enabled(df8_comm* c, int* enabled_h) {
    DF8_REQUIRE(c && enabled_h, "df8_comm_p2p_enabled: null argument");
    *enabled_h = (c->p2p_tried && c->p2p_ok) ? 1 : 0;
    return DF8_OK;
}

extern "C" df8_status df8_comm_allgather_symm(df8_comm* c, void* local_d, size_t offset, size_t bytes_per_rank,
                                              df8_stream stream) {
    DF8_REQUIRE(c && c->comm && local_d, "df8_comm_allgather_symm: null argument");
    if (bytes_per_rank == 0) return DF8_OK;
    const Df8SymmBuf* b = find_symm(c, static_cast<uint8_t*>(local_d) + offset, bytes_per_rank * size_t(c->world));
    DF8_REQUIRE(b != nullptr, "df8_comm_allgather_symm: the region is not inside a buffer of df8_comm_symm_alloc");
    cudaStream_t st = as_stream(stream);
    uint8_t* base = static_cast<uint8_t*>(local_d) + offset;
    const size_t mine = size_t(c->rank) * bytes_per_rank;
    if (!c->p2p_ok) {  // in place through NCCL
        int rc = api().AllGather(base + mine, base, bytes_per_rank, ncclUint8, c->comm, st);
        return rc == ncclSuccess ? DF8_OK : nccl_fail("ncclAllGather", rc);
    }
    unsigned int* status = nullptr;
    df8_status src = status_word_device_ptr(&status);
    if (src != DF8_OK) return src;
    const uint32_t seq = ++c->seq;
    const size_t rel = size_t(base - b->local);
    // this rank's slice is ready when the work already on `stream` is done
    DF8_CUDA_TRY(cudaEventRecord(c->ev_ready, st));
    DF8_CUDA_TRY(cudaStreamWaitEvent(c->copy_stream, c->ev_ready, 0));
    for (int k = 1; k < c->world; ++k) {  // rank r starts with r+1: at any moment the copies form a permutation
        const int p = (c->rank + k) % c->world;
        DF8_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(b->peer[p]) + rel + mine, base + mine, bytes_per_rank,
                                     cudaMemcpyDeviceToDevice, c->copy_stream));
    }
    signal_peers_kernel<<<1, 32, 0, c->copy_stream>>>(ctrl_ptrs(c), c->rank, c->world, seq);
    DF8_LAUNCH_CHECK("signal_peers_kernel");
    DF8_CUDA_TRY(cudaEventRecord(c->ev_sent, c->copy_stream));
    // the consumer side: every peer's slice has landed here; and this rank's slice may be overwritten again
    wait_peers_kernel<<<1, 32, 0, st>>>(reinterpret_cast<const uint32_t*>(c->symm[size_t(c->ctrl)].local), c->rank, c->world,
                                        seq, status);
    DF8_LAUNCH_CHECK("wait_peers_kernel");
    DF8_CUDA_TRY(cudaStreamWaitEvent(st, c->ev_sent, 0));
    c->bytes_pushed += bytes_per_rank * size_t(c->world - 1);
    return DF8_OK;
}

// The two halves of df8_comm_allgather_symm for callers that pipeline a gather in pieces: push one piece of this
// rank's slab (the bytes [local_d + offset, + bytes), to the same place in every peer's copy of the buffer) as soon
// as it is produced; wait for the peers' matching piece only where it is consumed.  Every rank must issue the same
// sequence of pushes.  Pieces of one stream of pushes arrive in order, so waiting for a ticket also covers every
// earlier push of the peers.
extern "C" df8_status df8_comm_push_symm(df8_comm* c, void* local_d, size_t offset, size_t bytes, df8_stream stream,
                                         unsigned int* ticket_h) {
    DF8_REQUIRE(c && c->comm && local_d && ticket_h, "df8_comm_push_symm: null argument");
    DF8_REQUIRE(c->p2p_ok, "df8_comm_push_symm: needs the peer-mapped transport (df8_comm_p2p_enabled)");
    uint8_t* base = static_cast<uint8_t*>(local_d) + offset;
    const Df8SymmBuf* b = find_symm(c, base, bytes);
    DF8_REQUIRE(b != nullptr, "df8_comm_push_symm: the region is not inside a buffer of df8_comm_symm_alloc");
    cudaStream_t st = as_stream(stream);
    const uint32_t seq = ++c->seq;
    *ticket_h = seq;
    if (bytes == 0) return DF8_OK;
    const size_t rel = size_t(base - b->local);
    DF8_CUDA_TRY(cudaEventRecord(c->ev_ready, st));
    DF8_CUDA_TRY(cudaStreamWaitEvent(c->copy_stream, c->ev_ready, 0));
    for (int k = 1; k < c->world; ++k) {
        const int p = (c->rank + k) % c->world;
        DF8_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t*>(b->peer[p]) + rel, base, bytes, cudaMemcpyDeviceToDevice,
                                     c->copy_stream));
    }
    signal_peers_kernel<<<1, 32, 0, c->copy_stream>>>(ctrl_ptrs(c), c->rank, c->world, seq);
    DF8_LAUNCH_CHECK("signal_peers_kernel");
    DF8_CUDA_TRY(cudaEventRecord(c->ev_sent, c->copy_stream));
    c->bytes_pushed += bytes * size_t(c->world - 1);
    return DF8_OK;
}

// `stream` waits (bounded, status word) until every peer's push with this ticket has landed; with own_too != 0 it
// also waits for this rank's own pushes issued so far, after which its slab may be overwritten again.
extern "C" df8_status df8_comm_wait_symm(df8_comm* c, unsigned int ticket, int own_too, df8_stream stream) {
    DF8_REQUIRE(c && c->comm, "df8_comm_wait_symm: null communicator");
    DF8_REQUIRE(c->p2p_ok, "df8_comm_wait_symm: needs the peer-mapped transport (df8_comm_p2p_enabled)");
    DF8_REQUIRE(ticket != 0 && c->seq - ticket < uint32_t(kFlagRing), "df8_comm_wait_symm: ticket %u is not one of the last %d pushes",
                ticket, kFlagRing);
    unsigned int* status = nullptr;
    df8_status src = status_word_device_ptr(&status);
    if (src != DF8_OK) return src;
    cudaStream_t st = as_stream(stream);
    wait_peers_kernel<<<1, 32, 0, st>>>(reinterpret_cast<const uint32_t*>(c->symm[size_t(c->ctrl)].local), c->rank, c->world,
                                        ticket, status);
    DF8_LAUNCH_CHECK("wait_peers_kernel");
    if (own_too) DF8_CUDA_TRY(cudaStreamWaitEvent(st, c->ev_sent, 0));
    return DF8_OK;
}

extern "C" df8_status df8_comm_allreduce_max_p2p(df8_comm* c, float* value_d, df8_stream stream) {
    DF8_REQUIRE(c && c->comm && value_d, "df8_comm_allreduce_max_p2p: null argument");
    df8_status rc = ensure_p2p(c);
    if (rc != DF8_OK) return rc;
    if (!c->p2p_ok) return df8_comm_allreduce_max_f32(c, value_d, 1, stream);
    unsigned int* status = nullptr;
    rc = status_word_device_ptr(&status);
    if (rc != DF8_OK) return rc;
    const uint32_t seq = ++c->slot_seq;
    allreduce_max_kernel<<<1, 32, 0, as_stream(stream)>>>(value_d, ctrl_ptrs(c), c->rank, c->world, seq, status);
    DF8_LAUNCH_CHECK("allreduce_max_kernel");
    return DF8_OK;
}

extern "C" df8_status df8_comm_bytes_pushed(df8_comm* c, unsigned long long* bytes_h) {
    DF8_REQUIRE(c && bytes_h, "df8_comm_bytes_pushed: null argument");
    *bytes_h = c->bytes_pushed;
    return DF8_OK;
}
