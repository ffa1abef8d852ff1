// Per-tensor amax reduction and fp32 <-> fp8 (e4m3 / e5m2) quantise / dequantise for sm_100a.
//
// All three kernels are HBM-bound streaming kernels: 128-bit coalesced accesses, several
// independent loads in flight per thread, a grid that is a multiple of the SM count, and
// warp-shuffle reductions.  Algorithmic traffic per element: amax 4 B, quantise 4 B + 1 B,
// dequantise 1 B + 4 B.
//
// Upstream has no counterpart kernel (its fp8 tensor instantiations, dnn/core/tensor.cu:489-498,
// are dead code); the conversion follows the CUDA toolkit's cuda_fp8.h semantics
// (round-to-nearest-even, saturate-to-finite), which is what the PTX cvt instructions used
// here implement in hardware.
#include "df8_internal.cuh"

namespace df8 {
namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 8;

// ---- amax ---------------------------------------------------------------------------------

// Grid-stride over float4 chunks, 4 chunks (64 B) in flight per thread per iteration.
__global__ void __launch_bounds__(kThreads) amax_f32_kernel(const float* __restrict__ x, size_t n,
                                                            float* __restrict__ amax_out) {
    griddep_launch_dependents();
    griddep_wait();
    const size_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const size_t stride = size_t(gridDim.x) * kThreads;
    size_t i = size_t(blockIdx.x) * kThreads + threadIdx.x;
    float m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f;
    for (; i + 3 * stride < n4; i += 4 * stride) {
        float4 a = ld_stream_f4(x4 + i);
        float4 b = ld_stream_f4(x4 + i + stride);
        float4 c = ld_stream_f4(x4 + i + 2 * stride);
        float4 d = ld_stream_f4(x4 + i + 3 * stride);
        m0 = fmaxf(m0, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
        m1 = fmaxf(m1, fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
        m2 = fmaxf(m2, fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w))));
        m3 = fmaxf(m3, fmaxf(fmaxf(fabsf(d.x), fabsf(d.y)), fmaxf(fabsf(d.z), fabsf(d.w))));
    }
    for (; i < n4; i += stride) {
        float4 a = ld_stream_f4(x4 + i);
        m0 = fmaxf(m0, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
    }
    // ragged tail (n not a multiple of 4): handled by the first threads of block 0
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) m1 = fmaxf(m1, fabsf(x[(n4 << 2) + threadIdx.x]));

    float m = warp_max(fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
    __shared__ float warp_m[kThreads / 32];
    if ((threadIdx.x & 31) == 0) warp_m[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < kThreads / 32 ? warp_m[threadIdx.x] : 0.f;
        m = warp_max(m);
        if (threadIdx.x == 0 && m > 0.f) atomic_max_nonneg(amax_out, m);
    }
}

// ---- quantise -----------------------------------------------------------------------------

// One float4 in, four packed codes out per thread and step; four independent steps in flight.
// A warp's loads cover 512 contiguous bytes and its stores 128 contiguous bytes.
template <int KIND>
__global__ void __launch_bounds__(kThreads) quantize_f32_kernel(const float* __restrict__ x, size_t n,
                                                                const float* __restrict__ amax_in,
                                                                uint8_t* __restrict__ codes,
                                                                float* __restrict__ scale_out) {
    griddep_launch_dependents();
    griddep_wait();
    const size_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    uint32_t* c4 = reinterpret_cast<uint32_t*>(codes);
    const size_t stride = size_t(gridDim.x) * kThreads;
    size_t i = size_t(blockIdx.x) * kThreads + threadIdx.x;
    if (n4 <= 4 * stride) {
        // a small tensor (a decode step's activations): at most four pieces per thread, all requested before the
        // maximum is looked at -- a warp issues in order, and the scale's divisions would hold the loads back by a
        // memory round trip
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = i + u * stride < n4 ? ld_stream_f4(x4 + i + u * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float2 s = scales_from_amax(ld_l2_f32(amax_in), fp8_max(KIND));
        if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) {
            scale_out[0] = s.x;
            scale_out[1] = s.y;
        }
        const float q = s.x;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i + u * stride < n4)
                c4[i + u * stride] = cvt_f32x4_to_fp8x4<KIND>(__fmul_rn(v[u].x, q), __fmul_rn(v[u].y, q), __fmul_rn(v[u].z, q),
                                                              __fmul_rn(v[u].w, q));
        if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
            const size_t j = (n4 << 2) + threadIdx.x;
            codes[j] = uint8_t(cvt_f32x2_to_fp8x2<KIND>(__fmul_rn(x[j], q), 0.f) & 0xff);
        }
        return;
    }
    const float2 s = scales_from_amax(ld_l2_f32(amax_in), fp8_max(KIND));
    if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) {
        scale_out[0] = s.x;
        scale_out[1] = s.y;
    }
    const float q = s.x;
    for (; i + 3 * stride < n4; i += 4 * stride) {
        float4 a = ld_stream_f4(x4 + i);
        float4 b = ld_stream_f4(x4 + i + stride);
        float4 c = ld_stream_f4(x4 + i + 2 * stride);
        float4 d = ld_stream_f4(x4 + i + 3 * stride);
        c4[i] = cvt_f32x4_to_fp8x4<KIND>(__fmul_rn(a.x, q), __fmul_rn(a.y, q), __fmul_rn(a.z, q), __fmul_rn(a.w, q));
        c4[i + stride] =
            cvt_f32x4_to_fp8x4<KIND>(__fmul_rn(b.x, q), __fmul_rn(b.y, q), __fmul_rn(b.z, q), __fmul_rn(b.w, q));
        c4[i + 2 * stride] =
            cvt_f32x4_to_fp8x4<KIND>(__fmul_rn(c.x, q), __fmul_rn(c.y, q), __fmul_rn(c.z, q), __fmul_rn(c.w, q));
        c4[i + 3 * stride] =
            cvt_f32x4_to_fp8x4<KIND>(__fmul_rn(d.x, q), __fmul_rn(d.y, q), __fmul_rn(d.z, q), __fmul_rn(d.w, q));
    }
    for (; i < n4; i += stride) {
        float4 a = ld_stream_f4(x4 + i);
        c4[i] = cvt_f32x4_to_fp8x4<KIND>(__fmul_rn(a.x, q), __fmul_rn(a.y, q), __fmul_rn(a.z, q), __fmul_rn(a.w, q));
    }
    // ragged tail: fewer than 4 elements, one thread each
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
        const size_t j = (n4 << 2) + threadIdx.x;
        codes[j] = uint8_t(cvt_f32x2_to_fp8x2<KIND>(__fmul_rn(x[j], q), 0.f) & 0xff);
    }
}

// ---- dequantise ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t ld_stream_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

template <int KIND>
__device__ __forceinline__ float4 dequant4(uint32_t w, float dq) {
    float2 lo = cvt_fp8x2_to_f32x2<KIND>(uint16_t(w & 0xffff));
    float2 hi = cvt_fp8x2_to_f32x2<KIND>(uint16_t(w >> 16));
    return make_float4(__fmul_rn(lo.x, dq), __fmul_rn(lo.y, dq), __fmul_rn(hi.x, dq), __fmul_rn(hi.y, dq));
}

// Four packed codes in, one float4 out per thread and step; four independent steps in flight.
template <int KIND>
__global__ void __launch_bounds__(kThreads) dequantize_f32_kernel(const uint8_t* __restrict__ codes, size_t n,
                                                                  const float* __restrict__ scale,
                                                                  float* __restrict__ y) {
    griddep_launch_dependents();
    griddep_wait();
    const float dq = ld_l2_f32(scale + 1);
    const size_t n4 = n >> 2;
    const uint32_t* c4 = reinterpret_cast<const uint32_t*>(codes);
    float4* y4 = reinterpret_cast<float4*>(y);
    const size_t stride = size_t(gridDim.x) * kThreads;
    size_t i = size_t(blockIdx.x) * kThreads + threadIdx.x;
    for (; i + 3 * stride < n4; i += 4 * stride) {
        uint32_t a = ld_stream_u32(c4 + i);
        uint32_t b = ld_stream_u32(c4 + i + stride);
        uint32_t c = ld_stream_u32(c4 + i + 2 * stride);
        uint32_t d = ld_stream_u32(c4 + i + 3 * stride);
        st_stream_f4(y4 + i, dequant4<KIND>(a, dq));
        st_stream_f4(y4 + i + stride, dequant4<KIND>(b, dq));
        st_stream_f4(y4 + i + 2 * stride, dequant4<KIND>(c, dq));
        st_stream_f4(y4 + i + 3 * stride, dequant4<KIND>(d, dq));
    }
    for (; i < n4; i += stride) st_stream_f4(y4 + i, dequant4<KIND>(ld_stream_u32(c4 + i), dq));
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
        const size_t j = (n4 << 2) + threadIdx.x;
        y[j] = __fmul_rn(cvt_fp8x2_to_f32x2<KIND>(uint16_t(codes[j])).x, dq);
    }
}

int grid_for(size_t work_items) {
    const size_t max_grid = size_t(sm_count()) * kCtasPerSm;
    size_t blocks = (work_items + kThreads - 1) / kThreads;
    if (blocks < 1) blocks = 1;
    if (blocks > max_grid) blocks = max_grid;
    return int(blocks);
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_amax_f32(const float* x, size_t n, float* amax_out, df8_stream stream) {
    DF8_REQUIRE(amax_out != nullptr, "df8_amax_f32: amax_out is null");
    DF8_REQUIRE(n == 0 || x != nullptr, "df8_amax_f32: x is null");
    DF8_REQUIRE(aligned16(x), "df8_amax_f32: x must be 16-byte aligned");
    cudaStream_t st = as_stream(stream);
    DF8_CLEAR_AMAX(amax_out, st);
    if (n == 0) return DF8_OK;
    DF8_LAUNCH("amax_f32_kernel", amax_f32_kernel, dim3(unsigned(grid_for(n / 16 + 1))), dim3(kThreads), 0, st, x, n, amax_out);
    return DF8_OK;
}

extern "C" df8_status df8_quantize_f32(const float* x, size_t n, df8_kind kind, const float* amax_in,
                                       uint8_t* codes_out, float* scale_out, df8_stream stream) {
    DF8_REQUIRE(kind == DF8_E4M3 || kind == DF8_E5M2, "df8_quantize_f32: unknown fp8 kind %d", int(kind));
    DF8_REQUIRE(amax_in != nullptr, "df8_quantize_f32: amax_in is null");
    DF8_REQUIRE(n == 0 || (x != nullptr && codes_out != nullptr), "df8_quantize_f32: null buffer");
    DF8_REQUIRE(aligned16(x) && aligned16(codes_out), "df8_quantize_f32: buffers must be 16-byte aligned");
    cudaStream_t st = as_stream(stream);
    const int grid = grid_for(n / 16 + 1);
    if (kind == DF8_E4M3)
        DF8_LAUNCH("quantize_f32_kernel", quantize_f32_kernel<DF8_E4M3>, dim3(unsigned(grid)), dim3(kThreads), 0, st, x, n, amax_in,
                   codes_out, scale_out);
    else
        DF8_LAUNCH("quantize_f32_kernel", quantize_f32_kernel<DF8_E5M2>, dim3(unsigned(grid)), dim3(kThreads), 0, st, x, n, amax_in,
                   codes_out, scale_out);
    return DF8_OK;
}

extern "C" df8_status df8_dequantize_f32(const uint8_t* codes, size_t n, df8_kind kind, const float* scale,
                                         float* y_out, df8_stream stream) {
    DF8_REQUIRE(kind == DF8_E4M3 || kind == DF8_E5M2, "df8_dequantize_f32: unknown fp8 kind %d", int(kind));
    DF8_REQUIRE(scale != nullptr, "df8_dequantize_f32: scale is null");
    DF8_REQUIRE(n == 0 || (codes != nullptr && y_out != nullptr), "df8_dequantize_f32: null buffer");
    DF8_REQUIRE(aligned16(codes) && aligned16(y_out), "df8_dequantize_f32: buffers must be 16-byte aligned");
    if (n == 0) return DF8_OK;
    cudaStream_t st = as_stream(stream);
    const int grid = grid_for(n / 16 + 1);
    if (kind == DF8_E4M3)
        DF8_LAUNCH("dequantize_f32_kernel", dequantize_f32_kernel<DF8_E4M3>, dim3(unsigned(grid)), dim3(kThreads), 0, st, codes, n,
                   scale, y_out);
    else
        DF8_LAUNCH("dequantize_f32_kernel", dequantize_f32_kernel<DF8_E5M2>, dim3(unsigned(grid)), dim3(kThreads), 0, st, codes, n,
                   scale, y_out);
    return DF8_OK;
}
