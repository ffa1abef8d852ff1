// Token embedding gather + bias + positional-encoding add in one pass.
//
// Replaces two upstream launches: embedding_forward_kernel (dnn/tokens/token_embedding.cu:31-45,
// launched at :146-154: out[t,d] = E[tok[t],d] + bias[d]) and add_positional_encodings_kernel
// (dnn/tokens/positional_encoding.cu:31-48, launched at :94-104: out[b,t,d] = in[b,t,d] + PE[t,d],
// which caps E at 1024 by using E threads per block).  One warp handles one token row with 128-bit
// accesses; ids outside [0,V) produce a zero row and are counted in `bad_ids` (upstream validates
// ids on the host on every call, token_embedding.cu:131-138; the C++ layer above keeps that
// behaviour by checking the counter or the host copy of the ids).
#include "df8_internal.cuh"

namespace df8 {
namespace {

constexpr int kEmbThreads = 256;

template <bool VEC4>
__global__ void __launch_bounds__(kEmbThreads)
embed_pe_kernel(const int* __restrict__ ids, int rows, int T, int E, int V, const float* __restrict__ table,
                const float* __restrict__ bias, const float* __restrict__ pe, float* __restrict__ out,
                int* __restrict__ bad_ids, const int* __restrict__ pos0) {
    griddep_launch_dependents();
    griddep_wait();
    if (pos0 && pe) pe += size_t(ld_l2_s32(pos0)) * E;  // the sequence's first position, read on the device (decode steps in a graph)
    const int warps_per_block = kEmbThreads / 32;
    const int lane = threadIdx.x & 31;
    for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
        const int id = ids[row];
        const bool ok = id >= 0 && id < V;
        if (!ok && lane == 0 && bad_ids) atomicAdd(bad_ids, 1);
        const int t = row % T;
        const float* e = table + size_t(ok ? id : 0) * E;
        const float* p = pe ? pe + size_t(t) * E : nullptr;
        float* o = out + size_t(row) * E;
        if constexpr (VEC4) {
            for (int i = lane; i < (E >> 2); i += 32) {
                float4 v = ok ? reinterpret_cast<const float4*>(e)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                if (ok && bias) {
                    const float4 b = reinterpret_cast<const float4*>(bias)[i];
                    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
                }
                if (ok && p) {
                    const float4 q = reinterpret_cast<const float4*>(p)[i];
                    v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
                }
                reinterpret_cast<float4*>(o)[i] = v;
            }
        } else {
            for (int i = lane; i < E; i += 32) {
                float v = 0.f;
                if (ok) {
                    v = e[i] + (bias ? bias[i] : 0.f);
                    if (p) v += p[i];
                }
                o[i] = v;
            }
        }
    }
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_embed_pe_f32(const int32_t* ids, int B, int T, int E, int V, const float* table,
                                       const float* bias, const float* pe, float* out, int32_t* bad_ids,
                                       df8_stream stream) {
    DF8_REQUIRE(B >= 0 && T >= 0 && E > 0 && V > 0, "df8_embed_pe_f32: bad shape B=%d T=%d E=%d V=%d", B, T, E, V);
    cudaStream_t st = as_stream(stream);
    if (bad_ids) DF8_CUDA_TRY(cudaMemsetAsync(bad_ids, 0, sizeof(int32_t), st));
    const long rows = long(B) * T;
    if (rows == 0) return DF8_OK;
    DF8_REQUIRE(rows < (1l << 31), "df8_embed_pe_f32: too many tokens");
    DF8_REQUIRE(ids && table && out, "df8_embed_pe_f32: null buffer");
    const int warps_per_block = kEmbThreads / 32;
    long blocks = (rows + warps_per_block - 1) / warps_per_block;
    const long cap = long(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    const bool vec4 = (E % 4 == 0) && aligned16(table) && aligned16(out) && aligned16(bias) && aligned16(pe);
    if (vec4)
        DF8_LAUNCH("embed_pe_kernel", embed_pe_kernel<true>, dim3(unsigned(blocks)), dim3(kEmbThreads), 0, st, ids, int(rows), T,
                   E, V, table, bias, pe, out, bad_ids, static_cast<const int*>(nullptr));
    else
        DF8_LAUNCH("embed_pe_kernel", embed_pe_kernel<false>, dim3(unsigned(blocks)), dim3(kEmbThreads), 0, st, ids, int(rows), T,
                   E, V, table, bias, pe, out, bad_ids, static_cast<const int*>(nullptr));
    return DF8_OK;
}

// One new token per sequence at the position stored in device memory: out[b] = table[ids[b]] + bias + pe_table[*pos_d].
// For a decode step whose launches are replayed from a CUDA graph (the position cannot be a launch argument then).
extern "C" df8_status df8_embed_pe_pos_f32(const int32_t* ids, int B, int E, int V, const float* table, const float* bias,
                                           const float* pe_table, const int32_t* pos_d, float* out, df8_stream stream) {
    DF8_REQUIRE(B >= 0 && E > 0 && V > 0, "df8_embed_pe_pos_f32: bad shape B=%d E=%d V=%d", B, E, V);
    if (B == 0) return DF8_OK;
    DF8_REQUIRE(ids && table && out && pe_table && pos_d, "df8_embed_pe_pos_f32: null buffer");
    const int warps_per_block = kEmbThreads / 32;
    const long blocks = (long(B) + warps_per_block - 1) / warps_per_block;
    const bool vec4 = (E % 4 == 0) && aligned16(table) && aligned16(out) && aligned16(bias) && aligned16(pe_table);
    cudaStream_t st = as_stream(stream);
    if (vec4)
        DF8_LAUNCH("embed_pe_kernel", embed_pe_kernel<true>, dim3(unsigned(blocks)), dim3(kEmbThreads), 0, st, ids, B, 1, E, V, table,
                   bias, pe_table, out, static_cast<int*>(nullptr), pos_d);
    else
        DF8_LAUNCH("embed_pe_kernel", embed_pe_kernel<false>, dim3(unsigned(blocks)), dim3(kEmbThreads), 0, st, ids, B, 1, E, V, table,
                   bias, pe_table, out, static_cast<int*>(nullptr), pos_d);
    return DF8_OK;
}
