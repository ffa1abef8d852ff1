// Row-wise LayerNorm over the last dimension, plain and fused with the per-tensor fp8 quantiser.
//
// Math (upstream dnn/layers/layer_norm_layer.cu:40-62): mean = sum(x)/C; var = sum((x-mean)^2)/C
// (biased, second pass); y = (x-mean) * rsqrt(var+eps) * gamma + beta.  Upstream computes both sums
// serially in thread 0 and only handles 2-D [rows, C<=1024] inputs (:70-79); here a row is reduced by a
// whole CTA with warp shuffles, any C, and [B,T,E] inputs are rows = B*T.
//
// Because the LayerNorm output always feeds a GEMM, the fused entry point never writes the fp32
// result: pass 1 keeps each row's (mean, rstd) in a small scratch array and reduces max|y| over the
// tensor, pass 2 re-reads x, normalises and emits fp8 codes.  9 bytes of HBM traffic per element
// instead of 13 for LayerNorm -> amax -> quantise as separate kernels.
//
// When the whole activation fits in the GPU's shared memory (rows * C * 4 bytes <= SMs x 200 KB, e.g. 8192 x 768),
// the fused entry point runs ONE co-resident kernel instead: every CTA normalises its rows into shared memory,
// the CTAs meet at a grid-wide barrier once max|y| is complete, and the codes are produced from shared memory.
// x is read once and nothing but the codes is written: 5 bytes per element, one launch.
#include "df8_internal.cuh"
#include "sm100_ptx.cuh"

#include <atomic>
#include <cstdlib>

namespace df8 {
namespace {

constexpr int kLnThreads = 256;
constexpr int kMaxV4 = 4;  // float4 per thread kept in registers: C <= 4096 on the fast path

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();  // protect `red` from the previous reduction's readers
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.f;
    return warp_sum(t);  // every warp computes the same total
}

__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.f;
    return warp_max(t);
}

// MODE 0: write fp32 y (+ optional amax).  MODE 1: stats pass (row stats + amax, no y).
// MODE 2: quantise pass (reads row stats and the scale derived from amax, writes codes).
template <int MODE, int KIND, bool FAST>
__global__ void __launch_bounds__(kLnThreads)
layernorm_kernel(const float* __restrict__ x, int rows, int C, const float* __restrict__ gamma,
                 const float* __restrict__ beta, float eps, float* __restrict__ y, float* __restrict__ amax_out,
                 float2* __restrict__ row_stats, const float* __restrict__ amax_in, uint8_t* __restrict__ codes,
                 float* __restrict__ scale_out) {
    griddep_launch_dependents();
    griddep_wait();
    __shared__ float red[kLnThreads / 32];
    float q = 1.f;
    if constexpr (MODE == 2) {
        const float2 s = scales_from_amax(ld_l2_f32(amax_in), fp8_max(KIND));
        q = s.x;
        if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) {
            scale_out[0] = s.x;
            scale_out[1] = s.y;
        }
    }
    float tile_amax = 0.f;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* xr = x + size_t(row) * C;
        float mean, rstd;
        if constexpr (FAST) {
            // C % 4 == 0 and C <= 4 * kMaxV4 * blockDim: the row lives in registers
            const int c4 = C >> 2;
            float4 v[kMaxV4];
#pragma unroll
            for (int j = 0; j < kMaxV4; ++j) {
                const int i = threadIdx.x + j * kLnThreads;
                v[j] = i < c4 ? reinterpret_cast<const float4*>(xr)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if constexpr (MODE == 2) {
                const float2 st = __ldcg(row_stats + row);  // written by the previous launch: read at L2
                mean = st.x;
                rstd = st.y;
            } else {
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < kMaxV4; ++j) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
                mean = block_sum(s, red) / float(C);
                float sq = 0.f;
#pragma unroll
                for (int j = 0; j < kMaxV4; ++j) {
                    const int i = threadIdx.x + j * kLnThreads;
                    if (i < c4) {
                        const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                        sq += (a * a + b * b) + (c * c + d * d);
                    }
                }
                rstd = rsqrtf(block_sum(sq, red) / float(C) + eps);
                if constexpr (MODE == 1)
                    if (threadIdx.x == 0) row_stats[row] = make_float2(mean, rstd);
            }
#pragma unroll
            for (int j = 0; j < kMaxV4; ++j) {
                const int i = threadIdx.x + j * kLnThreads;
                if (i < c4) {
                    float4 g = make_float4(1.f, 1.f, 1.f, 1.f), b = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (gamma) g = reinterpret_cast<const float4*>(gamma)[i];
                    if (beta) b = reinterpret_cast<const float4*>(beta)[i];
                    float4 o;
                    o.x = fmaf((v[j].x - mean) * rstd, g.x, b.x);
                    o.y = fmaf((v[j].y - mean) * rstd, g.y, b.y);
                    o.z = fmaf((v[j].z - mean) * rstd, g.z, b.z);
                    o.w = fmaf((v[j].w - mean) * rstd, g.w, b.w);
                    if constexpr (MODE == 2) {
                        reinterpret_cast<uint32_t*>(codes + size_t(row) * C)[i] = cvt_f32x4_to_fp8x4<KIND>(
                            __fmul_rn(o.x, q), __fmul_rn(o.y, q), __fmul_rn(o.z, q), __fmul_rn(o.w, q));
                    } else {
                        tile_amax = fmaxf(tile_amax, fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w))));
                        if constexpr (MODE == 0) reinterpret_cast<float4*>(y + size_t(row) * C)[i] = o;
                    }
                }
            }
        } else {
            // any C: three passes over the row (it stays in L1/L2)
            if constexpr (MODE == 2) {
                const float2 st = __ldcg(row_stats + row);  // written by the previous launch: read at L2
                mean = st.x;
                rstd = st.y;
            } else {
                float s = 0.f;
                for (int i = threadIdx.x; i < C; i += blockDim.x) s += xr[i];
                mean = block_sum(s, red) / float(C);
                float sq = 0.f;
                for (int i = threadIdx.x; i < C; i += blockDim.x) {
                    const float d = xr[i] - mean;
                    sq += d * d;
                }
                rstd = rsqrtf(block_sum(sq, red) / float(C) + eps);
                if constexpr (MODE == 1)
                    if (threadIdx.x == 0) row_stats[row] = make_float2(mean, rstd);
            }
            for (int i = threadIdx.x; i < C; i += blockDim.x) {
                const float o = fmaf((xr[i] - mean) * rstd, gamma ? gamma[i] : 1.f, beta ? beta[i] : 0.f);
                if constexpr (MODE == 2) {
                    codes[size_t(row) * C + i] = uint8_t(cvt_f32x2_to_fp8x2<KIND>(__fmul_rn(o, q), 0.f) & 0xff);
                } else {
                    tile_amax = fmaxf(tile_amax, fabsf(o));
                    if constexpr (MODE == 0) y[size_t(row) * C + i] = o;
                }
            }
        }
    }
    if constexpr (MODE != 2) {
        if (amax_out) {
            const float m = block_max(tile_amax, red);
            if (threadIdx.x == 0 && m > 0.f) atomic_max_nonneg(amax_out, m);
        }
    }
}

// Warp-per-row variant for C % 4 == 0 and C <= 128 * V4: a lane keeps V4 float4 of its row in registers, both
// reductions are five shuffles, nothing synchronises the block.  Same MODE meaning as above.
template <int MODE, int KIND, int V4>
__global__ void __launch_bounds__(kLnThreads)
layernorm_rows_kernel(const float* __restrict__ x, int rows, int C, const float* __restrict__ gamma,
                      const float* __restrict__ beta, float eps, float* __restrict__ y, float* __restrict__ amax_out,
                      float2* __restrict__ row_stats, const float* __restrict__ amax_in, uint8_t* __restrict__ codes,
                      float* __restrict__ scale_out) {
    griddep_launch_dependents();
    griddep_wait();
    const int lane = threadIdx.x & 31;
    const int wpb = kLnThreads / 32;
    const int c4 = C >> 2;
    float q = 1.f;
    if constexpr (MODE == 2) {
        const float2 s = scales_from_amax(ld_l2_f32(amax_in), fp8_max(KIND));
        q = s.x;
        if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) {
            scale_out[0] = s.x;
            scale_out[1] = s.y;
        }
    }
    float warp_amax = 0.f;
    for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
        const float4* xr = reinterpret_cast<const float4*>(x + size_t(row) * C);
        float4 v[V4];
#pragma unroll
        for (int j = 0; j < V4; ++j) {
            const int i = lane + 32 * j;
            v[j] = i < c4 ? ld_stream_f4(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float mean, rstd;
        if constexpr (MODE == 2) {
            const float2 st = __ldcg(row_stats + row);  // written by the previous launch: read at L2
            mean = st.x;
            rstd = st.y;
        } else {
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < V4; ++j) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
            mean = warp_sum(s) / float(C);
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < V4; ++j) {
                if (lane + 32 * j < c4) {
                    const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                    sq += (a * a + b * b) + (c * c + d * d);
                }
            }
            rstd = rsqrtf(warp_sum(sq) / float(C) + eps);
            if constexpr (MODE == 1)
                if (lane == 0) row_stats[row] = make_float2(mean, rstd);
        }
#pragma unroll
        for (int j = 0; j < V4; ++j) {
            const int i = lane + 32 * j;
            if (i < c4) {
                float4 g = make_float4(1.f, 1.f, 1.f, 1.f), b = make_float4(0.f, 0.f, 0.f, 0.f);
                if (gamma) g = __ldg(reinterpret_cast<const float4*>(gamma) + i);
                if (beta) b = __ldg(reinterpret_cast<const float4*>(beta) + i);
                float4 o;
                o.x = fmaf((v[j].x - mean) * rstd, g.x, b.x);
                o.y = fmaf((v[j].y - mean) * rstd, g.y, b.y);
                o.z = fmaf((v[j].z - mean) * rstd, g.z, b.z);
                o.w = fmaf((v[j].w - mean) * rstd, g.w, b.w);
                if constexpr (MODE == 2) {
                    reinterpret_cast<uint32_t*>(codes + size_t(row) * C)[i] = cvt_f32x4_to_fp8x4<KIND>(
                        __fmul_rn(o.x, q), __fmul_rn(o.y, q), __fmul_rn(o.z, q), __fmul_rn(o.w, q));
                } else {
                    warp_amax = fmaxf(warp_amax, fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w))));
                    if constexpr (MODE == 0) reinterpret_cast<float4*>(y + size_t(row) * C)[i] = o;
                }
            }
        }
    }
    if constexpr (MODE != 2) {
        if (amax_out) {  // uniform across the block: one atomic per block, not one per warp
            __shared__ float block_amax[kLnThreads / 32];
            const float mx = warp_max(warp_amax);
            if (lane == 0) block_amax[threadIdx.x >> 5] = mx;
            __syncthreads();
            if (threadIdx.x < 32) {
                float m = threadIdx.x < kLnThreads / 32 ? block_amax[threadIdx.x] : 0.f;
                m = warp_max(m);
                if (threadIdx.x == 0 && m > 0.f) atomic_max_nonneg(amax_out, m);
            }
        }
    }
}

// At most 32 rows (a decode step's one token per sequence): ONE CTA, a warp per row with the normalised row kept in
// registers across the block-wide maximum, so statistics, max|y|, scale and codes take one launch and x is read
// once.  Same arithmetic, in the same order, as the two passes of layernorm_rows_kernel (MODE 1 then MODE 2).
template <int KIND, int V4>
__global__ void __launch_bounds__(1024)
layernorm_quantize_one_cta_kernel(const float* __restrict__ x, int rows, int C, const float* __restrict__ gamma,
                                  const float* __restrict__ beta, float eps, float* __restrict__ amax_out,
                                  uint8_t* __restrict__ codes, float* __restrict__ scale_out) {
    griddep_launch_dependents();
    griddep_wait();
    const int lane = threadIdx.x & 31, row = threadIdx.x >> 5;
    const int c4 = C >> 2;
    __shared__ float warp_amax[32];
    __shared__ float4 sgamma[32 * V4], sbeta[32 * V4];
    const float before = ld_l2_f32(amax_out);  // normally 0 (cleared by the caller's convention); kept as a lower bound
    float4 o[V4];
    float4 v[V4];
    float mx = 0.f;
    if (row < rows) {
        const float4* xr = reinterpret_cast<const float4*>(x + size_t(row) * C);
#pragma unroll
        for (int j = 0; j < V4; ++j) {
            const int i = lane + 32 * j;
            v[j] = i < c4 ? ld_stream_f4(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    // gamma and beta to shared memory while the rows are on their way: read where they are needed they would put a
    // memory round trip behind every reduction
    for (int i = threadIdx.x; i < c4; i += blockDim.x) {
        sgamma[i] = gamma ? __ldg(reinterpret_cast<const float4*>(gamma) + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        sbeta[i] = beta ? __ldg(reinterpret_cast<const float4*>(beta) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
    if (row < rows) {
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < V4; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        const float mean = warp_sum(sum) / float(C);
        float sq = 0.f;
#pragma unroll
        for (int j = 0; j < V4; ++j) {
            if (lane + 32 * j < c4) {
                const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                sq += (a * a + b * b) + (c * c + d * d);
            }
        }
        const float rstd = rsqrtf(warp_sum(sq) / float(C) + eps);
#pragma unroll
        for (int j = 0; j < V4; ++j) {
            const int i = lane + 32 * j;
            o[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < c4) {
                const float4 g = sgamma[i], b = sbeta[i];
                o[j].x = fmaf((v[j].x - mean) * rstd, g.x, b.x);
                o[j].y = fmaf((v[j].y - mean) * rstd, g.y, b.y);
                o[j].z = fmaf((v[j].z - mean) * rstd, g.z, b.z);
                o[j].w = fmaf((v[j].w - mean) * rstd, g.w, b.w);
                mx = fmaxf(mx, fmaxf(fmaxf(fabsf(o[j].x), fabsf(o[j].y)), fmaxf(fabsf(o[j].z), fabsf(o[j].w))));
            }
        }
    }
    mx = warp_max(mx);
    if (lane == 0) warp_amax[row] = mx;
    __syncthreads();
    const float amax = fmaxf(before, warp_max(warp_amax[lane]));
    const float2 s = scales_from_amax(amax, fp8_max(KIND));
    if (threadIdx.x == 0) {
        if (amax > 0.f) atomic_max_nonneg(amax_out, amax);
        if (scale_out) {
            scale_out[0] = s.x;
            scale_out[1] = s.y;
        }
    }
    if (row < rows) {
        const float q = s.x;
#pragma unroll
        for (int j = 0; j < V4; ++j) {
            const int i = lane + 32 * j;
            if (i < c4)
                reinterpret_cast<uint32_t*>(codes + size_t(row) * C)[i] = cvt_f32x4_to_fp8x4<KIND>(
                    __fmul_rn(o[j].x, q), __fmul_rn(o[j].y, q), __fmul_rn(o[j].z, q), __fmul_rn(o[j].w, q));
        }
    }
}

template <int KIND>
bool launch_one_cta(const float* x, int rows, int C, const float* gamma, const float* beta, float eps, uint8_t* codes,
                    float* scale_out, float* amax, cudaStream_t st) {
    if (rows > 32 || C > 1024) return false;
    if (const char* e = getenv("DF8_LN_ONE_CTA"))
        if (e[0] == '0') return false;
#define DF8_LN_ONE(V4)                                                                                               \
    (void)launch_kernel((layernorm_quantize_one_cta_kernel<KIND, V4>), dim3(1), dim3(1024), 0, st, x, rows, C, gamma, beta, \
                        eps, amax, codes, scale_out)
    if (C <= 256) DF8_LN_ONE(2);
    else if (C <= 512) DF8_LN_ONE(4);
    else if (C <= 768) DF8_LN_ONE(6);
    else DF8_LN_ONE(8);
#undef DF8_LN_ONE
    return true;
}

template <int MODE, int KIND>
bool launch_rows_kernel(const float* x, int rows, int C, const float* gamma, const float* beta, float eps, float* y,
                        float* amax_out, float2* row_stats, const float* amax_in, uint8_t* codes, float* scale_out,
                        cudaStream_t st) {
    const int wpb = kLnThreads / 32;
    long blocks = (long(rows) + wpb - 1) / wpb;
    const long cap = long(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const int grid = int(blocks);
#define DF8_LN_ROWS(V4)                                                                                           \
    (void)launch_kernel((layernorm_rows_kernel<MODE, KIND, V4>), dim3(unsigned(grid)), dim3(kLnThreads), 0, st, x, rows, C,  \
                        gamma, beta, eps, y, amax_out, row_stats, amax_in, codes, scale_out)
    if (C <= 256) DF8_LN_ROWS(2);
    else if (C <= 512) DF8_LN_ROWS(4);
    else if (C <= 768) DF8_LN_ROWS(6);
    else if (C <= 1024) DF8_LN_ROWS(8);
    else if (C <= 2048) DF8_LN_ROWS(16);
    else if (C <= 4096) DF8_LN_ROWS(32);
    else return false;
#undef DF8_LN_ROWS
    return true;
}

// ---- shared-memory-resident fused LayerNorm + quantise (one launch, grid-wide barrier) ----------------

constexpr int kResThreads = 1024;
constexpr int kResSmemCap = 200 * 1024;
// Arrival counters of the grid barrier.  Every launch uses the same grid (one CTA per SM), so a counter stays a
// multiple of it between launches; consecutive launches take consecutive counters, so launches that overlap on
// a GPU (different streams) do not see each other's arrivals.
constexpr int kResCounters = 64;
constexpr int kResMaxRounds = 32;  // rounds of kResThreads / 32 rows a CTA may hold (checked at launch)
__device__ unsigned int g_ln_grid_counter[kResCounters] = {};

template <int KIND, int V4>
__global__ void __launch_bounds__(kResThreads, 1)
layernorm_quantize_resident_kernel(const float* __restrict__ x, int rows, int C, const float* __restrict__ gamma,
                                   const float* __restrict__ beta, float eps, float* amax, uint8_t* __restrict__ codes,
                                   float* __restrict__ scale_out, int rows_per_cta, int counter_slot,
                                   unsigned int* status) {
    extern __shared__ float4 ybuf[];  // [rows_per_cta][C / 4]: the CTA's rows, raw as they arrive, normalised in place
    __shared__ float block_amax[kResThreads / 32];
    __shared__ uint64_t round_bar[kResMaxRounds];  // one per round of kResThreads / 32 rows: "these rows have landed"
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int nw = kResThreads / 32;
    const int c4 = C >> 2;
    const int r0 = blockIdx.x * rows_per_cta;
    const int nrows = min(rows_per_cta, rows - r0);  // may be <= 0: such a CTA only takes part in the barrier
    const int nrounds = nrows > 0 ? (nrows + nw - 1) / nw : 0;
    if (threadIdx.x == 0) {
        for (int k = 0; k < nrounds; ++k) ptx::mbar_init(ptx::smem_u32(round_bar + k), 1);
        ptx::mbar_fence_init();
    }
    __syncthreads();
    // launched under the previous kernel's tail (when the launch carries the programmatic attribute): CTAs that
    // become resident early wait here, and later at the grid barrier, for the rest of the grid
    griddep_launch_dependents();
    griddep_wait();
    // Every row of the CTA is requested at once, by one thread, as a bulk copy into its place in shared memory: the
    // warps then find their rows there instead of each paying a global-memory round trip per row in turn (two rows
    // per warp at 8192 x 768: the load phase was 5.4 of the kernel's 10 us).
    if (threadIdx.x == 0) {
        const uint32_t row_bytes = uint32_t(C) * 4u;
        for (int k = 0; k < nrounds; ++k) {
            const int first = k * nw, n = min(nw, nrows - first);
            const uint32_t bar = ptx::smem_u32(round_bar + k);
            ptx::mbar_arrive_expect_tx(bar, uint32_t(n) * row_bytes);
            for (int i = 0; i < n; ++i)
                ptx::bulk_load_1d(ptx::smem_u32(ybuf + size_t(first + i) * c4), x + size_t(r0 + first + i) * C, row_bytes, bar);
        }
    }
    const bool affine = gamma != nullptr && beta != nullptr;
    float warp_amax = 0.f;
    for (int lr = warp; lr < nrows; lr += nw) {
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(round_bar + lr / nw), 0)) {
            if (lane == 0 && status) {
                atomicCAS(status, 0u, 0x3100u);
                atomicAdd(status + 1, 1u);
            }
            break;
        }
        float4* yr = ybuf + size_t(lr) * c4;
        float4 v[V4];
#pragma unroll
        for (int j = 0; j < V4; ++j) {
            const int i = lane + 32 * j;
            v[j] = i < c4 ? yr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // the same operations in the same order as layernorm_rows_kernel: the two paths agree bit for bit
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < V4; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        const float mean = warp_sum(sum) / float(C);
        float sq = 0.f;
#pragma unroll
        for (int j = 0; j < V4; ++j) {
            if (lane + 32 * j < c4) {
                const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                sq += (a * a + b * b) + (c * c + d * d);
            }
        }
        const float rstd = rsqrtf(warp_sum(sq) / float(C) + eps);
        if (affine) {  // the usual case, with the parameter loads free to move ahead of the arithmetic
#pragma unroll
            for (int j = 0; j < V4; ++j) {
                const int i = lane + 32 * j;
                if (i < c4) {
                    const float4 g = __ldg(reinterpret_cast<const float4*>(gamma) + i);
                    const float4 b = __ldg(reinterpret_cast<const float4*>(beta) + i);
                    float4 o;
                    o.x = fmaf((v[j].x - mean) * rstd, g.x, b.x);
                    o.y = fmaf((v[j].y - mean) * rstd, g.y, b.y);
                    o.z = fmaf((v[j].z - mean) * rstd, g.z, b.z);
                    o.w = fmaf((v[j].w - mean) * rstd, g.w, b.w);
                    warp_amax = fmaxf(warp_amax, fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w))));
                    yr[i] = o;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < V4; ++j) {
                const int i = lane + 32 * j;
                if (i < c4) {
                    float4 g = make_float4(1.f, 1.f, 1.f, 1.f), b = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (gamma) g = __ldg(reinterpret_cast<const float4*>(gamma) + i);
                    if (beta) b = __ldg(reinterpret_cast<const float4*>(beta) + i);
                    float4 o;
                    o.x = fmaf((v[j].x - mean) * rstd, g.x, b.x);
                    o.y = fmaf((v[j].y - mean) * rstd, g.y, b.y);
                    o.z = fmaf((v[j].z - mean) * rstd, g.z, b.z);
                    o.w = fmaf((v[j].w - mean) * rstd, g.w, b.w);
                    warp_amax = fmaxf(warp_amax, fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w))));
                    yr[i] = o;
                }
            }
        }
    }
    {
        const float mx = warp_max(warp_amax);
        if (lane == 0) block_amax[warp] = mx;
        __syncthreads();
        if (threadIdx.x < 32) {
            float m = block_amax[threadIdx.x];
            m = warp_max(m);
            if (threadIdx.x == 0 && m > 0.f) atomic_max_nonneg(amax, m);
        }
    }
    // ---- grid-wide barrier: max|y| is complete once every CTA has arrived (bounded wait) ----
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int ticket = atomicAdd(&g_ln_grid_counter[counter_slot], 1u);
        const unsigned int target = (ticket / gridDim.x + 1u) * gridDim.x;
        volatile unsigned int* cnt = &g_ln_grid_counter[counter_slot];
        unsigned long long t0 = 0;
        for (unsigned int spins = 0; int(*cnt - target) < 0; ++spins) {
            __nanosleep(64);
            if ((spins & 1023u) == 1023u) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                if (now - t0 > 2000000000ull) {  // a CTA never came: give up, flag it, and finish
                    if (status) {
                        atomicCAS(status, 0u, 0x3000u);
                        atomicAdd(status + 1, 1u);
                    }
                    break;
                }
            }
        }
        __threadfence();
    }
    __syncthreads();
    const float2 sc = scales_from_amax(*reinterpret_cast<volatile float*>(amax), fp8_max(KIND));
    if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) {
        scale_out[0] = sc.x;
        scale_out[1] = sc.y;
    }
    const float q = sc.x;
    for (int lr = warp; lr < nrows; lr += nw) {
        uint32_t* crow = reinterpret_cast<uint32_t*>(codes + size_t(r0 + lr) * C);
#pragma unroll
        for (int j = 0; j < V4; ++j) {
            const int i = lane + 32 * j;
            if (i < c4) {
                const float4 o = ybuf[size_t(lr) * c4 + i];
                crow[i] = cvt_f32x4_to_fp8x4<KIND>(__fmul_rn(o.x, q), __fmul_rn(o.y, q), __fmul_rn(o.z, q),
                                                   __fmul_rn(o.w, q));
            }
        }
    }
}

// Launches the resident kernel if the problem qualifies; returns false (nothing launched) otherwise.
template <int KIND>
bool launch_resident(const float* x, int rows, int C, const float* gamma, const float* beta, float eps, uint8_t* codes,
                     float* scale_out, float* amax, cudaStream_t st) {
    if (const char* e = getenv("DF8_LN_RESIDENT"))
        if (e[0] == '0') return false;
    if (C > 1024 || rows < 1024) return false;
    const int sms = sm_count();
    const int rows_per_cta = (rows + sms - 1) / sms;
    const size_t smem = size_t(rows_per_cta) * size_t(C) * sizeof(float);
    if (smem > size_t(kResSmemCap)) return false;
    if ((rows_per_cta + kResThreads / 32 - 1) / (kResThreads / 32) > kResMaxRounds) return false;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return false;  // bulk copies start on 16-byte boundaries
    unsigned int* status = nullptr;
    if (status_word_device_ptr(&status) != DF8_OK) return false;
    static std::atomic<unsigned int> next_slot{0};
    const int counter_slot = int(next_slot.fetch_add(1u) % unsigned(kResCounters));
    auto launch = [&](auto kern) -> bool {
        // once per device and kernel instantiation (this lambda's body is instantiated per kernel type)
        static std::atomic<bool> configured[64] = {};
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
        if (!configured[dev].load(std::memory_order_acquire)) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kResSmemCap) != cudaSuccess) {
                (void)cudaGetLastError();
                return false;
            }
            configured[dev].store(true, std::memory_order_release);
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(sms));
        cfg.blockDim = dim3(kResThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeCooperative;  // the grid barrier needs every CTA resident
        attr[0].val.cooperative = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        static std::atomic<bool> pdl_refused{false};  // a driver that rejects the combination: plain cooperative launches
        cfg.numAttrs = (pdl_enabled() && !pdl_refused.load()) ? 2 : 1;
        cudaError_t err = cudaLaunchKernelEx(&cfg, kern, x, rows, C, gamma, beta, eps, amax, codes, scale_out,
                                             rows_per_cta, counter_slot, status);
        if (err != cudaSuccess && cfg.numAttrs == 2) {
            (void)cudaGetLastError();
            pdl_refused.store(true);
            cfg.numAttrs = 1;
            err = cudaLaunchKernelEx(&cfg, kern, x, rows, C, gamma, beta, eps, amax, codes, scale_out, rows_per_cta,
                                     counter_slot, status);
        }
        if (err != cudaSuccess) {
            (void)cudaGetLastError();  // e.g. not co-schedulable: the two-kernel path takes over
            return false;
        }
        return true;
    };
    if (C <= 256) return launch(layernorm_quantize_resident_kernel<KIND, 2>);
    if (C <= 512) return launch(layernorm_quantize_resident_kernel<KIND, 4>);
    if (C <= 768) return launch(layernorm_quantize_resident_kernel<KIND, 6>);
    return launch(layernorm_quantize_resident_kernel<KIND, 8>);
}

bool fast_ok(int C, const void* a, const void* b, const void* c, const void* d) {
    return (C % 4 == 0) && C <= 4 * kMaxV4 * kLnThreads && aligned16(a) && aligned16(b) && aligned16(c) &&
           aligned16(d);
}

int ln_grid(int rows) {
    const int cap = sm_count() * 8;
    return rows < cap ? (rows > 0 ? rows : 1) : cap;
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_layernorm_f32(const float* x, int rows, int cols, const float* gamma, const float* beta,
                                        float eps, float* y, float* amax_out, df8_stream stream) {
    DF8_REQUIRE(rows >= 0 && cols > 0, "df8_layernorm_f32: bad shape rows=%d cols=%d", rows, cols);
    cudaStream_t st = as_stream(stream);
    DF8_CLEAR_AMAX(amax_out, st);
    if (rows == 0) return DF8_OK;
    DF8_REQUIRE(x && y, "df8_layernorm_f32: null buffer");
    if (fast_ok(cols, x, y, gamma, beta) &&
        launch_rows_kernel<0, 0>(x, rows, cols, gamma, beta, eps, y, amax_out, nullptr, nullptr, nullptr, nullptr, st)) {
    } else if (fast_ok(cols, x, y, gamma, beta))
        (void)launch_kernel((layernorm_kernel<0, 0, true>), dim3(unsigned(ln_grid(rows))), dim3(kLnThreads), 0, st, x, rows, cols, gamma, beta, eps, y, amax_out,
                                                                          nullptr, nullptr, nullptr, nullptr);
    else
        (void)launch_kernel((layernorm_kernel<0, 0, false>), dim3(unsigned(ln_grid(rows))), dim3(kLnThreads), 0, st, x, rows, cols, gamma, beta, eps, y,
                                                                           amax_out, nullptr, nullptr, nullptr, nullptr);
    DF8_LAUNCH_CHECK("layernorm_kernel");
    return DF8_OK;
}

namespace {
template <int KIND>
df8_status launch_ln_quant(const float* x, int rows, int cols, const float* gamma, const float* beta, float eps,
                           uint8_t* codes, float* scale_out, float* amax_out, float2* row_stats, cudaStream_t st) {
    const int grid = ln_grid(rows);
    const bool fast = fast_ok(cols, x, gamma, beta, nullptr) && (reinterpret_cast<uintptr_t>(codes) & 3u) == 0;
    if (fast && launch_one_cta<KIND>(x, rows, cols, gamma, beta, eps, codes, scale_out, amax_out, st)) {
        DF8_LAUNCH_CHECK("layernorm_quantize_one_cta_kernel");
        return DF8_OK;
    }
    if (fast && launch_resident<KIND>(x, rows, cols, gamma, beta, eps, codes, scale_out, amax_out, st)) return DF8_OK;
    if (fast && cols <= 4096) {
        launch_rows_kernel<1, KIND>(x, rows, cols, gamma, beta, eps, nullptr, amax_out, row_stats, nullptr, nullptr,
                                    nullptr, st);
        launch_rows_kernel<2, KIND>(x, rows, cols, gamma, beta, eps, nullptr, nullptr, row_stats, amax_out, codes,
                                    scale_out, st);
    } else if (fast) {
        (void)launch_kernel((layernorm_kernel<1, KIND, true>), dim3(unsigned(grid)), dim3(kLnThreads), 0, st, x, rows, cols, gamma, beta, eps, nullptr, amax_out,
                                                                    row_stats, nullptr, nullptr, nullptr);
        (void)launch_kernel((layernorm_kernel<2, KIND, true>), dim3(unsigned(grid)), dim3(kLnThreads), 0, st, x, rows, cols, gamma, beta, eps, nullptr, nullptr,
                                                                    row_stats, amax_out, codes, scale_out);
    } else {
        (void)launch_kernel((layernorm_kernel<1, KIND, false>), dim3(unsigned(grid)), dim3(kLnThreads), 0, st, x, rows, cols, gamma, beta, eps, nullptr, amax_out,
                                                                     row_stats, nullptr, nullptr, nullptr);
        (void)launch_kernel((layernorm_kernel<2, KIND, false>), dim3(unsigned(grid)), dim3(kLnThreads), 0, st, x, rows, cols, gamma, beta, eps, nullptr, nullptr,
                                                                     row_stats, amax_out, codes, scale_out);
    }
    DF8_LAUNCH_CHECK("layernorm_kernel (fused quantise)");
    return DF8_OK;
}
}  // namespace

extern "C" df8_status df8_layernorm_quantize_f32(const float* x, int rows, int cols, const float* gamma,
                                                 const float* beta, float eps, df8_kind kind, uint8_t* codes_out,
                                                 float* scale_out, float* amax_out, float* row_stats_scratch,
                                                 df8_stream stream) {
    DF8_REQUIRE(kind == DF8_E4M3 || kind == DF8_E5M2, "df8_layernorm_quantize_f32: unknown fp8 kind %d", int(kind));
    DF8_REQUIRE(rows >= 0 && cols > 0, "df8_layernorm_quantize_f32: bad shape rows=%d cols=%d", rows, cols);
    DF8_REQUIRE(amax_out && scale_out, "df8_layernorm_quantize_f32: amax_out and scale_out are required");
    cudaStream_t st = as_stream(stream);
    DF8_CLEAR_AMAX(amax_out, st);
    DF8_REQUIRE(rows == 0 || (x && codes_out && row_stats_scratch), "df8_layernorm_quantize_f32: null buffer");
    DF8_REQUIRE((reinterpret_cast<uintptr_t>(row_stats_scratch) & 7u) == 0,
                "df8_layernorm_quantize_f32: row_stats_scratch must be 8-byte aligned");
    float2* stats = reinterpret_cast<float2*>(row_stats_scratch);
    return kind == DF8_E4M3
               ? launch_ln_quant<DF8_E4M3>(x, rows, cols, gamma, beta, eps, codes_out, scale_out, amax_out, stats, st)
               : launch_ln_quant<DF8_E5M2>(x, rows, cols, gamma, beta, eps, codes_out, scale_out, amax_out, stats, st);
}

// ---- variant that never allocates -----------------------------------------------------------------
//
// Some callers of the fused LayerNorm + quantise cannot provide the row-statistics scratch buffer
// because they cannot allocate device memory at the point of the call: a serving loop that handed
// every byte of the GPU to its own arena at start-up, a host thread that must not take the
// allocator's lock or the implicit device synchronisation of cudaMalloc / cudaFree, or glue code in
// a language binding that only ever sees the caller's input and output buffers.  For them the
// scratch lives in the library image: a fixed array in device global memory, reserved on every GPU
// that loads the library for as long as the process lives.
namespace {

constexpr int kNoAllocMaxRows = 65536;  // 2 floats per row: 512 KiB of device memory per GPU

static __device__ __align__(256) float g_ln_row_stats[2 * kNoAllocMaxRows];

// Device address of g_ln_row_stats on the current device.  In host code the array's name is only a
// handle for the runtime, not something a kernel may dereference, so the real address is looked up
// once per device (with that device current) and cached.
df8_status ln_static_scratch(float** out) {
    // (host threads that make their first call on a device at the same time all look the address up and store
    // the same value; the atomic only makes that formally race-free)
    static std::atomic<float*> cached[64] = {};
    int dev = 0;
    DF8_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(DF8_ERR_INVALID, "device index %d out of range", dev);
    float* p = cached[dev].load(std::memory_order_acquire);
    if (!p) {
        cudaError_t err = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_ln_row_stats);
        if (err != cudaSuccess)
            return fail(DF8_ERR_CUDA, "cudaGetSymbolAddress(g_ln_row_stats) failed: %s", cudaGetErrorString(err));
        cached[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return DF8_OK;
}

}  // namespace

extern "C" df8_status df8_layernorm_quantize_f32_noalloc(const float* x, int rows, int cols, const float* gamma,
                                                         const float* beta, float eps, df8_kind kind,
                                                         uint8_t* codes_out, float* scale_out, float* amax_out,
                                                         df8_stream stream) {
    DF8_REQUIRE(kind == DF8_E4M3 || kind == DF8_E5M2, "df8_layernorm_quantize_f32_noalloc: unknown fp8 kind %d",
                int(kind));
    DF8_REQUIRE(rows >= 0 && cols > 0, "df8_layernorm_quantize_f32_noalloc: bad shape rows=%d cols=%d", rows, cols);
    if (rows > kNoAllocMaxRows)
        return fail(DF8_ERR_UNSUPPORTED,
                    "df8_layernorm_quantize_f32_noalloc: %d rows exceed the built-in scratch of %d rows; "
                    "use df8_layernorm_quantize_f32 with a caller-provided buffer",
                    rows, kNoAllocMaxRows);
    DF8_REQUIRE(amax_out && scale_out, "df8_layernorm_quantize_f32_noalloc: amax_out and scale_out are required");
    DF8_REQUIRE(rows == 0 || (x && codes_out), "df8_layernorm_quantize_f32_noalloc: null buffer");
    float* stats = nullptr;
    df8_status rc = ln_static_scratch(&stats);
    if (rc != DF8_OK) return rc;
    cudaStream_t st = as_stream(stream);
    // max|LN(x)| is accumulated with atomicMax and must start from zero; the row statistics need no
    // clearing: pass 1 writes the entry of every row before pass 2 reads it.
    DF8_CLEAR_AMAX(amax_out, st);
    float2* stats2 = reinterpret_cast<float2*>(stats);
    return kind == DF8_E4M3
               ? launch_ln_quant<DF8_E4M3>(x, rows, cols, gamma, beta, eps, codes_out, scale_out, amax_out, stats2, st)
               : launch_ln_quant<DF8_E5M2>(x, rows, cols, gamma, beta, eps, codes_out, scale_out, amax_out, stats2, st);
}
