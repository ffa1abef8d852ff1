// The autoregressive decode step after a prefill: a cache of the keys and values of every earlier position, and
// the attention of ONE new query per sequence and head against it.
//
// Upstream's Gpt2::forward recomputes the whole sequence for every call (dnn/models/gpt2.cu:126-142) and has no
// cache; its attention semantics (dnn/layers/multi_head_attention.cu:225-301, softmax_layer.cu:26-81:
// p = exp(s - max) / (sum + 1e-6)) are kept.  New here:
//   * the cache holds the fp8 CODES the QKV projection produced, [B, H, T_max, D] per layer for K and for V, plus
//     one dequantisation factor per cached position: the 8-bit path quantises every QKV tensor per tensor, so the
//     positions of a prefill share one scale and every later step brings its own;
//   * a step's attention is bound by reading the cache once from HBM (2 * t * D bytes per sequence and head):
//     no tensor cores, one CTA per (sequence, head), its warps taking keys in turn with an online softmax each
//     and a combine through shared memory.
#include "df8_internal.cuh"

namespace df8 {
namespace {

constexpr int kDecodeWarps = 8;

// qkv [B*Tn, 3E] codes of Tn new positions per sequence -> rows t0 .. t0+Tn-1 of the K and V caches [B,H,Tmax,D]
__global__ void __launch_bounds__(256)
kv_append_kernel(const uint8_t* __restrict__ qkv, int B, int Tn, int H, int D, int t0, int Tmax,
                 uint8_t* __restrict__ kc, uint8_t* __restrict__ vc, const float* __restrict__ scale,
                 float* __restrict__ row_dq, const int* __restrict__ pos) {
    griddep_launch_dependents();
    griddep_wait();
    if (pos) {  // the first new position, read on the device (decode steps replayed from a graph)
        t0 = ld_l2_s32(pos);
        if (t0 < 0 || t0 + Tn > Tmax) return;  // the host keeps its own count and refuses a full cache first
    }
    const int E = H * D, d16 = D / 16;
    const size_t total = size_t(B) * Tn * H * d16;  // 16-byte pieces per cache
    for (size_t i = blockIdx.x * size_t(256) + threadIdx.x; i < total; i += size_t(gridDim.x) * 256) {
        const int c = int(i % d16);
        size_t r = i / d16;
        const int h = int(r % H);
        r /= H;
        const int t = int(r % Tn), b = int(r / Tn);
        const uint8_t* src = qkv + (size_t(b) * Tn + t) * 3 * E + h * D + c * 16;
        const size_t dst = ((size_t(b) * H + h) * Tmax + t0 + t) * D + c * 16;
        *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(src + E);
        *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(src + 2 * E);
    }
    if (blockIdx.x == 0)
        for (int t = threadIdx.x; t < Tn; t += 256) row_dq[t0 + t] = ld_l2_f32(scale + 1);
}

template <int KIND>
__device__ __forceinline__ float dot16(const uint4& k, const float* __restrict__ q) {
    const uint32_t w[4] = {k.x, k.y, k.z, k.w};
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 a = cvt_fp8x2_to_f32x2<KIND>(uint16_t(w[i] & 0xFFFFu));
        const float2 b = cvt_fp8x2_to_f32x2<KIND>(uint16_t(w[i] >> 16));
        s = fmaf(a.x, q[4 * i], s);
        s = fmaf(a.y, q[4 * i + 1], s);
        s = fmaf(b.x, q[4 * i + 2], s);
        s = fmaf(b.y, q[4 * i + 3], s);
    }
    return s;
}

// acc[0..15] += p * (the 16 codes of v)
template <int KIND>
__device__ __forceinline__ void fma16(const uint4& v, float p, float* __restrict__ acc) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 a = cvt_fp8x2_to_f32x2<KIND>(uint16_t(w[i] & 0xFFFFu));
        const float2 b = cvt_fp8x2_to_f32x2<KIND>(uint16_t(w[i] >> 16));
        acc[4 * i] = fmaf(p, a.x, acc[4 * i]);
        acc[4 * i + 1] = fmaf(p, a.y, acc[4 * i + 1]);
        acc[4 * i + 2] = fmaf(p, b.x, acc[4 * i + 2]);
        acc[4 * i + 3] = fmaf(p, b.y, acc[4 * i + 3]);
    }
}

// One CTA per (sequence, head): out[b, h*D : (h+1)*D] = softmax(q . K^T / sqrt(D)) . V over the n_keys cached positions.
// A warp takes 32 keys at a time: every lane scores one key (its row of K is 4 or 8 16-byte loads), then the warp
// accumulates p . V with a lane per (key, 16-byte piece of the value row) -- 32 / (D/16) keys per pass, all loads of a
// block of keys independent of one another -- and folds the partial sums of the lanes that share a piece at the end.
// FUSED: the step's QKV projection arrives as fp32 [B, 3E] with its max|.|; the CTA quantises its own query and
// writes the codes of its own key / value row into position n_keys - 1 of the caches before it attends (the cache
// append and the quantisation pass of the unfused sequence, without their launches).
template <int D, int KIND, bool FUSED>
__global__ void __launch_bounds__(32 * kDecodeWarps)
attention_decode_kernel(const uint8_t* __restrict__ q_codes, const float* __restrict__ q_scale,
                        const float* __restrict__ qkv_f32, const float* __restrict__ qkv_amax, uint8_t* kc, uint8_t* vc,
                        float* row_dq, int H, int n_keys, int Tmax, float* __restrict__ out,
                        float* __restrict__ out_amax, const int* __restrict__ pos) {
    griddep_launch_dependents();
    const int b = blockIdx.x / H, h = blockIdx.x % H;
    // The cached rows come from DRAM (a step's working set exceeds L2) and their loads can only be issued once the
    // position is known: ask L2 for them first, before the wait for the preceding kernel -- they were written by earlier
    // steps, and a prefetch moves nothing the program can see.  n_keys is the host's count (replayed from a graph: the
    // count at capture, a lower bound).
    if (threadIdx.x < 2) {
        const uint8_t* rows = (threadIdx.x == 0 ? kc : vc) + (size_t(b) * H + h) * size_t(Tmax) * D;
        const unsigned int bytes = unsigned(min(n_keys, Tmax)) * unsigned(D);
        for (unsigned int off = 0; off < bytes; off += 16384u) {
            const unsigned int n = min(16384u, bytes - off);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(rows + off), "r"(n) : "memory");
        }
    }
    griddep_wait();
    const int pos_v = pos ? ld_l2_s32(pos) : 0;  // (consumed below, after the other requests are out)
    constexpr int DPL = D / 32;             // output dimensions per lane in the final combine
    constexpr int CH = D / 16, KPI = 32 / CH;  // 16-byte pieces per row, keys per pass of the p . V loop
    const int E = H * D;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ float sq[D];
    __shared__ float sm[kDecodeWarps], sl[kDecodeWarps], sacc[kDecodeWarps][D];
    uint8_t* kbase = kc + (size_t(b) * H + h) * size_t(Tmax) * D;
    uint8_t* vbase = vc + (size_t(b) * H + h) * size_t(Tmax) * D;
    // scores are kept in the log2 domain: s * log2(e) / sqrt(D), the query's scale folded in
    int j_new = -1;
    float dq_new = 0.f;
    if constexpr (!FUSED)
        if (pos) n_keys = min(pos_v + 1, Tmax);  // the new position's own key included
    if constexpr (FUSED) {
        // (the row's values are requested before the maximum is looked at: a warp issues in order, and the scale's
        // divisions would hold these loads back by a memory round trip)
        const float* row = qkv_f32 + size_t(b) * 3 * E + h * D;
        constexpr int kMine = (3 * D + 32 * kDecodeWarps - 1) / (32 * kDecodeWarps);
        float mine[kMine];
#pragma unroll
        for (int u = 0; u < kMine; ++u) {
            const int i = threadIdx.x + u * 32 * kDecodeWarps;
            const int part = i / D, d = i - part * D;
            mine[u] = i < 3 * D ? __ldcg(row + size_t(part) * E + d) : 0.f;
        }
        const float2 sc = scales_from_amax(ld_l2_f32(qkv_amax), fp8_max(KIND));
        if (pos) n_keys = min(pos_v + 1, Tmax);  // the new position's own key included
        const float qs = sc.y * rsqrtf(float(D)) * 1.4426950408889634f;
        j_new = n_keys - 1;
        dq_new = sc.y;
#pragma unroll
        for (int u = 0; u < kMine; ++u) {
            const int i = threadIdx.x + u * 32 * kDecodeWarps;
            if (i >= 3 * D) break;
            const int part = i / D, d = i - part * D;
            const uint16_t c = cvt_f32x2_to_fp8x2<KIND>(__fmul_rn(mine[u], sc.x), 0.f) & 0xffu;
            if (part == 0) sq[d] = cvt_fp8x2_to_f32x2<KIND>(c).x * qs;
            else if (part == 1) kbase[size_t(j_new) * D + d] = uint8_t(c);
            else vbase[size_t(j_new) * D + d] = uint8_t(c);
        }
        if (blockIdx.x == 0 && threadIdx.x == 0) row_dq[j_new] = dq_new;  // later steps read it; this one uses dq_new
    } else {
        const float qs = ld_l2_f32(q_scale + 1) * rsqrtf(float(D)) * 1.4426950408889634f;
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            const uint8_t c = q_codes[size_t(b) * 3 * E + h * D + d];
            sq[d] = cvt_fp8x2_to_f32x2<KIND>(uint16_t(c)).x * qs;
        }
    }
    __syncthreads();  // also orders this CTA's own cache row before the loads below
    const int piece = lane % CH, sub = lane / CH;
    float m = -INFINITY, l = 0.f, acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (int j0 = warp * 32; j0 < n_keys; j0 += kDecodeWarps * 32) {
        const int j = j0 + lane;
        uint4 vv[CH];
#pragma unroll
        for (int it = 0; it < CH; ++it) {
            const int jk = j0 + it * KPI + sub;
            vv[it] = jk < n_keys ? ld_stream_u4(reinterpret_cast<const uint4*>(vbase + size_t(jk) * D + piece * 16))
                                 : make_uint4(0u, 0u, 0u, 0u);
        }
        float s = -INFINITY, dqj = 0.f;
        if (j < n_keys) {
            dqj = (j == j_new) ? dq_new : __ldcg(row_dq + j);
            float dot = 0.f;
            const uint4* krow = reinterpret_cast<const uint4*>(kbase + size_t(j) * D);
#pragma unroll
            for (int c = 0; c < CH; ++c) dot += dot16<KIND>(ld_stream_u4(krow + c), sq + 16 * c);
            s = dot * dqj;
        }
        const float mb = warp_max(s);
        const float m_new = fmaxf(m, mb);
        const float alpha = exp2f(m - m_new);  // 0 for the first block (m = -inf)
        const float p = (j < n_keys) ? exp2f(s - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] *= alpha;
        m = m_new;
        const float pv = p * dqj;  // the value row's scale
#pragma unroll
        for (int it = 0; it < CH; ++it) {
            const float pk = __shfl_sync(0xffffffffu, pv, it * KPI + sub);
            fma16<KIND>(vv[it], pk, acc);
        }
    }
    // lanes that share a piece hold partial sums over different keys
#pragma unroll
    for (int off = CH; off < 32; off <<= 1)
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
    if (lane == 0) {
        sm[warp] = m;
        sl[warp] = l;
    }
    if (lane < CH)
#pragma unroll
        for (int i = 0; i < 16; ++i) sacc[warp][piece * 16 + i] = acc[i];
    __syncthreads();
    if (warp == 0) {
        float mt = -INFINITY;
        for (int w = 0; w < kDecodeWarps; ++w) mt = fmaxf(mt, sm[w]);
        float lt = 0.f, o[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[i] = 0.f;
        for (int w = 0; w < kDecodeWarps; ++w) {
            const float f = (sm[w] == -INFINITY) ? 0.f : exp2f(sm[w] - mt);
            lt += sl[w] * f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[i] = fmaf(sacc[w][lane + 32 * i], f, o[i]);
        }
        // p = exp(s - max) / (sum + 1e-6), as upstream's softmax
        const float inv = 1.f / (lt + 1e-6f);
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const float v = (n_keys > 0) ? o[i] * inv : 0.f;
            out[size_t(b) * E + h * D + lane + 32 * i] = v;
            amax = fmaxf(amax, fabsf(v));
        }
        if (out_amax) {
            amax = warp_max(amax);
            if (lane == 0 && amax > 0.f) atomic_max_nonneg(out_amax, amax);
        }
    }
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_kv_cache_append(const uint8_t* qkv_codes, const float* scale, int B, int Tn, int H, int D,
                                          int t0, int Tmax, uint8_t* k_cache, uint8_t* v_cache, float* row_dq,
                                          df8_stream stream) {
    DF8_REQUIRE(B >= 0 && Tn >= 0 && H > 0 && D > 0 && D % 16 == 0, "df8_kv_cache_append: bad shape");
    DF8_REQUIRE(t0 >= 0 && t0 + Tn <= Tmax, "df8_kv_cache_append: positions %d..%d do not fit a cache of %d", t0, t0 + Tn, Tmax);
    if (B == 0 || Tn == 0) return DF8_OK;
    DF8_REQUIRE(qkv_codes && scale && k_cache && v_cache && row_dq, "df8_kv_cache_append: null buffer");
    DF8_REQUIRE(aligned16(qkv_codes) && aligned16(k_cache) && aligned16(v_cache), "df8_kv_cache_append: buffers must be 16-byte aligned");
    const size_t total = size_t(B) * Tn * H * (D / 16);
    size_t blocks = (total + 255) / 256;
    const size_t cap = size_t(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    DF8_LAUNCH("kv_append_kernel", kv_append_kernel, dim3(unsigned(blocks)), dim3(256), 0, as_stream(stream), qkv_codes, B, Tn,
               H, D, t0, Tmax, k_cache, v_cache, scale, row_dq, static_cast<const int*>(nullptr));
    return DF8_OK;
}

// The same for one new position per sequence whose index is read from device memory.
extern "C" df8_status df8_kv_cache_append_pos(const uint8_t* qkv_codes, const float* scale, int B, int H, int D,
                                              const int32_t* pos_d, int Tmax, uint8_t* k_cache, uint8_t* v_cache,
                                              float* row_dq, df8_stream stream) {
    DF8_REQUIRE(B >= 0 && H > 0 && D > 0 && D % 16 == 0 && Tmax > 0, "df8_kv_cache_append_pos: bad shape");
    if (B == 0) return DF8_OK;
    DF8_REQUIRE(qkv_codes && scale && k_cache && v_cache && row_dq && pos_d, "df8_kv_cache_append_pos: null buffer");
    DF8_REQUIRE(aligned16(qkv_codes) && aligned16(k_cache) && aligned16(v_cache), "df8_kv_cache_append_pos: buffers must be 16-byte aligned");
    const size_t total = size_t(B) * H * (D / 16);
    size_t blocks = (total + 255) / 256;
    const size_t cap = size_t(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    DF8_LAUNCH("kv_append_kernel", kv_append_kernel, dim3(unsigned(blocks)), dim3(256), 0, as_stream(stream), qkv_codes, B, 1, H, D,
               0, Tmax, k_cache, v_cache, scale, row_dq, pos_d);
    return DF8_OK;
}

__global__ void advance_position_kernel(int* pos) {
    griddep_launch_dependents();
    griddep_wait();
    if (threadIdx.x == 0) *pos += 1;
}

extern "C" df8_status df8_position_advance(int32_t* pos_d, df8_stream stream) {
    DF8_REQUIRE(pos_d != nullptr, "df8_position_advance: null argument");
    DF8_LAUNCH("advance_position_kernel", advance_position_kernel, dim3(1), dim3(32), 0, as_stream(stream), pos_d);
    return DF8_OK;
}

extern "C" df8_status df8_attention_decode_fp8(const uint8_t* qkv_codes, df8_kind kind, const float* scale,
                                               const uint8_t* k_cache, const uint8_t* v_cache, const float* row_dq,
                                               int B, int H, int D, int n_keys, int Tmax, float* out, float* out_amax,
                                               df8_stream stream) {
    return df8_attention_decode_fp8_pos(qkv_codes, kind, scale, k_cache, v_cache, row_dq, B, H, D, n_keys, nullptr, Tmax, out,
                                        out_amax, stream);
}

// pos_d != null: the number of keys is *pos_d + 1, read on the device (n_keys is ignored)
extern "C" df8_status df8_attention_decode_fp8_pos(const uint8_t* qkv_codes, df8_kind kind, const float* scale,
                                                   const uint8_t* k_cache, const uint8_t* v_cache, const float* row_dq,
                                                   int B, int H, int D, int n_keys, const int32_t* pos_d, int Tmax,
                                                   float* out, float* out_amax, df8_stream stream) {
    DF8_REQUIRE(kind == DF8_E4M3 || kind == DF8_E5M2, "df8_attention_decode_fp8: unknown fp8 kind %d", int(kind));
    DF8_REQUIRE(B >= 0 && H > 0 && n_keys >= 0 && n_keys <= Tmax, "df8_attention_decode_fp8: bad shape");
    if (D != 64 && D != 128)
        return fail(DF8_ERR_UNSUPPORTED, "df8_attention_decode_fp8: head dimension %d not supported (64 or 128)", D);
    cudaStream_t st = as_stream(stream);
    DF8_CLEAR_AMAX(out_amax, st);
    if (B == 0) return DF8_OK;
    DF8_REQUIRE(qkv_codes && scale && k_cache && v_cache && row_dq && out, "df8_attention_decode_fp8: null buffer");
    DF8_REQUIRE(aligned16(k_cache) && aligned16(v_cache), "df8_attention_decode_fp8: the caches must be 16-byte aligned");
    const dim3 grid(unsigned(B * H)), block(32 * kDecodeWarps);
#define DF8_DECODE(DD, KK)                                                                                                  \
    DF8_LAUNCH("attention_decode_kernel", (attention_decode_kernel<DD, KK, false>), grid, block, 0, st, qkv_codes, scale,        \
               static_cast<const float*>(nullptr), static_cast<const float*>(nullptr), const_cast<uint8_t*>(k_cache),            \
               const_cast<uint8_t*>(v_cache), const_cast<float*>(row_dq), H, n_keys, Tmax, out, out_amax, pos_d)
    if (D == 64 && kind == DF8_E4M3) DF8_DECODE(64, DF8_E4M3);
    else if (D == 64) DF8_DECODE(64, DF8_E5M2);
    else if (kind == DF8_E4M3) DF8_DECODE(128, DF8_E4M3);
    else DF8_DECODE(128, DF8_E5M2);
#undef DF8_DECODE
    return DF8_OK;
}

// The step's attention straight from the fp32 QKV projection [B, 3E] and its max|.|: quantises (per tensor, as
// df8_quantize_f32 with that maximum would), appends the new position's key / value codes and its dequantisation
// factor to the caches, and attends over n_keys positions, the new one (row n_keys - 1, or *pos_d) included.
extern "C" df8_status df8_attention_decode_fused_f32(const float* qkv_f32, const float* qkv_amax, df8_kind kind,
                                                     uint8_t* k_cache, uint8_t* v_cache, float* row_dq, int B, int H, int D,
                                                     int n_keys, const int32_t* pos_d, int Tmax, float* out,
                                                     float* out_amax, df8_stream stream) {
    DF8_REQUIRE(kind == DF8_E4M3 || kind == DF8_E5M2, "df8_attention_decode_fused_f32: unknown fp8 kind %d", int(kind));
    DF8_REQUIRE(B >= 0 && H > 0 && n_keys >= 1 && n_keys <= Tmax, "df8_attention_decode_fused_f32: bad shape");
    if (D != 64 && D != 128)
        return fail(DF8_ERR_UNSUPPORTED, "df8_attention_decode_fused_f32: head dimension %d not supported (64 or 128)", D);
    cudaStream_t st = as_stream(stream);
    DF8_CLEAR_AMAX(out_amax, st);
    if (B == 0) return DF8_OK;
    DF8_REQUIRE(qkv_f32 && qkv_amax && k_cache && v_cache && row_dq && out, "df8_attention_decode_fused_f32: null buffer");
    DF8_REQUIRE(aligned16(k_cache) && aligned16(v_cache), "df8_attention_decode_fused_f32: the caches must be 16-byte aligned");
    const dim3 grid(unsigned(B * H)), block(32 * kDecodeWarps);
    const uint8_t* no_codes = nullptr;
    const float* no_scale = nullptr;
#define DF8_DECODE_FUSED(DD, KK)                                                                                            \
    DF8_LAUNCH("attention_decode_kernel (fused)", (attention_decode_kernel<DD, KK, true>), grid, block, 0, st, no_codes,   \
               no_scale, qkv_f32, qkv_amax, k_cache, v_cache, row_dq, H, n_keys, Tmax, out, out_amax, pos_d)
    if (D == 64 && kind == DF8_E4M3) DF8_DECODE_FUSED(64, DF8_E4M3);
    else if (D == 64) DF8_DECODE_FUSED(64, DF8_E5M2);
    else if (kind == DF8_E4M3) DF8_DECODE_FUSED(128, DF8_E4M3);
    else DF8_DECODE_FUSED(128, DF8_E5M2);
#undef DF8_DECODE_FUSED
    return DF8_OK;
}
