// Column-sharded fully-connected layer across the GPUs of one box.
//
// W [out, in] is split on `out` into world_size row blocks; every rank holds the whole quantised input
// [M, in] and its own block of weight codes, computes its [M, out/world] slice of the output, and one
// all-gather of fp8 codes completes the layer.  Because the output is quantised per TENSOR, the ranks
// first agree on max|out| (all-reduce max of one float between the two GEMM passes), so that the codes
// are exactly those a single GPU produces for the unsharded layer.
//
// Upstream has no counterpart: its fully-connected layer always holds the full [out, in] weight
// (dnn/layers/fully_connected_layer.cu:112-116) and its multi-GPU driver runs independent replicas
// (apps/host-multi/main.cpp:157-181).
#include "df8_internal.cuh"

namespace df8 {
namespace {

// gathered [world][M, n] (rank-major, what an all-gather of per-rank slices produces) -> out [M, world*n]
__global__ void __launch_bounds__(256)
interleave_gathered_kernel(const uint4* __restrict__ gathered, int M, int n16, int world, uint4* __restrict__ out) {
    const size_t total = size_t(M) * world * n16;
    for (size_t i = blockIdx.x * size_t(256) + threadIdx.x; i < total; i += size_t(gridDim.x) * 256) {
        const size_t row = i / (size_t(world) * n16);
        const int rem = int(i % (size_t(world) * n16));
        const int r = rem / n16, c = rem % n16;
        out[i] = gathered[(size_t(r) * M + row) * n16 + c];
    }
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_interleave_gathered_u8(const uint8_t* gathered, int M, int cols_per_rank, int world,
                                                 uint8_t* out, df8_stream stream) {
    DF8_REQUIRE(M >= 0 && cols_per_rank >= 0 && world >= 1, "df8_interleave_gathered_u8: bad shape");
    DF8_REQUIRE(cols_per_rank % 16 == 0, "df8_interleave_gathered_u8: cols_per_rank must be a multiple of 16");
    if (M == 0 || cols_per_rank == 0) return DF8_OK;
    DF8_REQUIRE(gathered && out && aligned16(gathered) && aligned16(out), "df8_interleave_gathered_u8: bad buffer");
    const size_t total = size_t(M) * world * (cols_per_rank / 16);
    size_t blocks = (total + 255) / 256;
    const size_t cap = size_t(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    interleave_gathered_kernel<<<int(blocks), 256, 0, as_stream(stream)>>>(
        reinterpret_cast<const uint4*>(gathered), M, cols_per_rank / 16, world, reinterpret_cast<uint4*>(out));
    DF8_LAUNCH_CHECK("interleave_gathered_kernel");
    return DF8_OK;
}

extern "C" df8_status df8_fc_fp8_column_sharded(df8_comm* comm, const uint8_t* a_codes, df8_kind kind_a,
                                                const float* scale_a, const uint8_t* w_shard_codes, df8_kind kind_w,
                                                const float* scale_w, const float* bias_shard, int M, int N, int K,
                                                int flags, df8_kind out_kind, uint8_t* slice_scratch,
                                                uint8_t* gathered_scratch, uint8_t* out_codes, float* out_scale,
                                                float* out_amax, df8_stream stream) {
    DF8_REQUIRE(comm != nullptr, "df8_fc_fp8_column_sharded: null communicator");
    int rank = 0, world = 1;
    df8_status rc = df8_comm_rank(comm, &rank, &world);
    if (rc != DF8_OK) return rc;
    DF8_REQUIRE(N % (32 * world) == 0, "df8_fc_fp8_column_sharded: N=%d must be a multiple of 32 * world (%d)", N, world);
    DF8_REQUIRE(slice_scratch && gathered_scratch && out_codes && out_scale && out_amax,
                "df8_fc_fp8_column_sharded: null buffer");
    const int n = N / world;
    // pass 1: max|.| of this rank's slice; agree on the tensor's maximum
    rc = df8_gemm_fp8_tn_amax(a_codes, kind_a, scale_a, w_shard_codes, kind_w, scale_w, bias_shard, M, n, K, flags,
                              out_amax, stream);
    if (rc != DF8_OK) return rc;
    rc = df8_comm_allreduce_max_f32(comm, out_amax, 1, stream);
    if (rc != DF8_OK) return rc;
    // pass 2: the slice as fp8 codes under the common scale; gather; put the slices side by side
    rc = df8_gemm_fp8_tn_codes(a_codes, kind_a, scale_a, w_shard_codes, kind_w, scale_w, bias_shard, M, n, K, flags,
                               out_kind, out_amax, slice_scratch, out_scale, stream);
    if (rc != DF8_OK) return rc;
    rc = df8_comm_allgather_u8(comm, slice_scratch, gathered_scratch, size_t(M) * size_t(n), stream);
    if (rc != DF8_OK) return rc;
    return df8_interleave_gathered_u8(gathered_scratch, M, n, world, out_codes, stream);
}
