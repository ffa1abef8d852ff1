// Internal helpers shared by the kernel translation units of libdf8 (not part of the C-ABI).
#pragma once

#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "df8.h"

namespace df8 {

// Records a printf-style message as the calling thread's last error and returns `code`.
df8_status fail(df8_status code, const char* fmt, ...);

// Number of SMs of the current device (cached per device).
int sm_count();

// Device address, on the current device, of the status word that bounded device-side waits write
// when they give up ([0] first code, [1] count).
df8_status status_word_device_ptr(unsigned int** out);

#define DF8_CUDA_TRY(expr)                                                                  \
    do {                                                                                    \
        cudaError_t err__ = (expr);                                                         \
        if (err__ != cudaSuccess)                                                           \
            return ::df8::fail(DF8_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                \
                               cudaGetErrorString(err__), __FILE__, __LINE__);              \
    } while (0)

#define DF8_LAUNCH_CHECK(what)                                                              \
    do {                                                                                    \
        cudaError_t err__ = cudaGetLastError();                                             \
        if (err__ != cudaSuccess)                                                           \
            return ::df8::fail(DF8_ERR_CUDA, "launch of %s failed: %s", what,               \
                               cudaGetErrorString(err__));                                  \
    } while (0)

// Launch through launch_kernel() (programmatic dependent launch allowed); a kernel name with template commas goes
// in parentheses.
#define DF8_LAUNCH(what, kern, grid, block, smem, st, ...)                                  \
    do {                                                                                    \
        cudaError_t err__ = ::df8::launch_kernel(kern, grid, block, smem, st, __VA_ARGS__); \
        if (err__ != cudaSuccess)                                                           \
            return ::df8::fail(DF8_ERR_CUDA, "launch of %s failed: %s", what,               \
                               cudaGetErrorString(err__));                                  \
    } while (0)

// Clears *amax_out on the stream unless the calling thread turned that off (df8_set_amax_preclear).
#define DF8_CLEAR_AMAX(ptr, st)                                                             \
    do {                                                                                    \
        if ((ptr) != nullptr && ::df8::amax_preclear())                                     \
            DF8_CUDA_TRY(cudaMemsetAsync((ptr), 0, sizeof(float), (st)));                   \
    } while (0)

#define DF8_REQUIRE(cond, ...)                                                              \
    do {                                                                                    \
        if (!(cond)) return ::df8::fail(DF8_ERR_INVALID, __VA_ARGS__);                      \
    } while (0)

inline cudaStream_t as_stream(df8_stream s) { return reinterpret_cast<cudaStream_t>(s); }

// Programmatic dependent launch.  Kernels of this library are short (10-100 us) and run back to back on one
// stream, so the gap between two of them (grid drain, launch latency, the next kernel's set-up) is a visible part
// of a forward pass.  Every kernel calls griddep_launch_dependents() on entry and griddep_wait() before its
// first access to global memory; launched through launch_kernel() it may then be scheduled, and run its
// set-up, while the previous kernel of the stream is still finishing.  After an operation that is not such a
// kernel (a memset, a copy, another library's kernel) the attribute has no effect.  DF8_PDL=0 in the
// environment turns the attribute off.
bool pdl_enabled();
bool amax_preclear();

template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__host__ __device__ constexpr float fp8_max(int kind) { return kind == DF8_E4M3 ? 448.0f : 57344.0f; }

// ---- device helpers ---------------------------------------------------------------------

__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }


// Two fp32 -> two fp8 codes, round-to-nearest-even, saturating to the largest finite value.
// The low byte of the result holds `lo`, the high byte `hi`.
template <int KIND>
__device__ __forceinline__ uint16_t cvt_f32x2_to_fp8x2(float lo, float hi) {
    uint16_t r;
    if constexpr (KIND == DF8_E4M3) {
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    } else {
        asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    }
    return r;
}

// Four fp32 -> four packed fp8 codes (byte i holds v[i]).
template <int KIND>
__device__ __forceinline__ uint32_t cvt_f32x4_to_fp8x4(float a, float b, float c, float d) {
    return uint32_t(cvt_f32x2_to_fp8x2<KIND>(a, b)) | (uint32_t(cvt_f32x2_to_fp8x2<KIND>(c, d)) << 16);
}

// Two fp8 codes (low byte = first) -> two fp32 values; exact widening via f16.
template <int KIND>
__device__ __forceinline__ float2 cvt_fp8x2_to_f32x2(uint16_t codes) {
    uint32_t h2;
    if constexpr (KIND == DF8_E4M3) {
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(codes));
    } else {
        asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(codes));
    }
    float lo, hi;
    asm("{.reg .f16 l, h; mov.b32 {l, h}, %2; cvt.f32.f16 %0, l; cvt.f32.f16 %1, h;}"
        : "=f"(lo), "=f"(hi)
        : "r"(h2));
    return make_float2(lo, hi);
}

// q = FP8_MAX / amax and dq = amax / FP8_MAX, each one IEEE fp32 division; both 1 when amax is 0.
__device__ __forceinline__ float2 scales_from_amax(float amax, float fmax) {
    if (!(amax > 0.0f)) return make_float2(1.0f, 1.0f);
    return make_float2(__fdiv_rn(fmax, amax), __fdiv_rn(amax, fmax));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// atomic max for non-negative floats (their bit patterns order like unsigned integers).
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
    atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

// A scalar that an earlier kernel of the stream produced (a max|.|, a scale pair, the decode position), read at L2.
// Kernels launched with the programmatic attribute become resident while their predecessors still run; an L1 line
// that a co-resident kernel filled before the producer's write (neighbouring slots of the max|.| pool share a line)
// would otherwise serve a stale value: L1 is only invalidated when a kernel is launched, not at griddepcontrol.wait.
__device__ __forceinline__ float ld_l2_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_l2_s32(const int* p) {
    int v;
    asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// 128-bit streaming global loads of data touched once, served at L2: never from an L1 line, which may predate the
// producing kernel's write when kernels overlap (see ld_l2_f32).
__device__ __forceinline__ float4 ld_stream_f4(const float4* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_stream_u4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream_f4(float4* p, float4 v) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}
__device__ __forceinline__ void st_stream_u4(uint4* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

}  // namespace df8
