// LayerNorm + per-tensor fp8 quantisation of a tensor whose COLUMNS are split across ranks.
//
// The column-sharded forward keeps the fp32 residual stream sharded: rank r holds columns [r*C/g, (r+1)*C/g) of
// every row.  LayerNorm needs the mean and variance of whole rows, so instead of gathering the fp32 rows (4 bytes
// per element over NVLink) the ranks exchange two floats per row:
//   1. df8_layernorm_shard_stats_f32     {mean_r, M2_r = sum (x - mean_r)^2} of this rank's piece of every row
//   2. (the caller all-gathers the [rows][2] arrays of all ranks)
//   3. df8_layernorm_shard_amax_f32      combines them in rank order (pairwise-update formula for the variance
//                                        of a union: mean = sum n_r mean_r / n, M2 = sum M2_r + n_r (mean_r - mean)^2,
//                                        all n_r equal here), writes {mean, rstd} per row and reduces max|y| over this
//                                        rank's columns
//   4. (the caller takes the maximum over ranks)
//   5. df8_layernorm_shard_quantize_f32  y = (x - mean) * rstd * gamma + beta of this rank's columns -> fp8 codes
//                                        with the scale of the whole tensor
// after which only the CODES (1 byte per element) are gathered.  The formula is upstream's
// (dnn/layers/layer_norm_layer.cu:40-62: biased variance, rsqrtf(var + eps)); only the order of the additions
// differs from a single-GPU row sum, i.e. results agree to fp32 rounding, not bit for bit.
// One warp per row; a row piece is read from L1/L2 on its later passes.
#include "df8_internal.cuh"

namespace df8 {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float row_sum(const float* __restrict__ x, int n, int lane) {
    float s = 0.f;
    const int n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (int i = lane; i < n4; i += 32) {
        const float4 v = x4[i];
        s += (v.x + v.y) + (v.z + v.w);
    }
    for (int i = (n4 << 2) + lane; i < n; i += 32) s += x[i];
    return warp_sum(s);
}

__device__ __forceinline__ float row_m2(const float* __restrict__ x, int n, int lane, float mean) {
    float s = 0.f;
    const int n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (int i = lane; i < n4; i += 32) {
        const float4 v = x4[i];
        const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
        s += (a * a + b * b) + (c * c + d * d);
    }
    for (int i = (n4 << 2) + lane; i < n; i += 32) {
        const float a = x[i] - mean;
        s += a * a;
    }
    return warp_sum(s);
}

__global__ void __launch_bounds__(kThreads)
shard_stats_kernel(const float* __restrict__ x, int rows, int n, float2* __restrict__ partial) {
    griddep_launch_dependents();
    griddep_wait();
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * kThreads) >> 5;
    for (int r = (blockIdx.x * kThreads + threadIdx.x) >> 5; r < rows; r += warps) {
        const float* row = x + size_t(r) * n;
        const float mean = row_sum(row, n, lane) / float(n);
        const float m2 = row_m2(row, n, lane, mean);
        if (lane == 0) partial[r] = make_float2(mean, m2);
    }
}

// partial_all: [world][rows] of {mean_r, M2_r}; every rank holds n columns of the c_total = world * n
__global__ void __launch_bounds__(kThreads)
shard_amax_kernel(const float* __restrict__ x, int rows, int n, const float2* __restrict__ partial_all, int world,
                  const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                  float2* __restrict__ row_stats, float* __restrict__ amax_out) {
    griddep_launch_dependents();
    griddep_wait();
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * kThreads) >> 5;
    float amax = 0.f;
    for (int r = (blockIdx.x * kThreads + threadIdx.x) >> 5; r < rows; r += warps) {
        // every lane combines the ranks' pieces in rank order (identical on all ranks)
        float msum = 0.f;
        for (int k = 0; k < world; ++k) msum += partial_all[size_t(k) * rows + r].x;
        const float mean = msum / float(world);
        float m2 = 0.f;
        for (int k = 0; k < world; ++k) {
            const float2 p = partial_all[size_t(k) * rows + r];
            const float d = p.x - mean;
            m2 += p.y + float(n) * d * d;
        }
        const float rstd = rsqrtf(m2 / (float(n) * float(world)) + eps);
        if (lane == 0) row_stats[r] = make_float2(mean, rstd);
        const float* row = x + size_t(r) * n;
        for (int i = lane; i < n; i += 32) {
            // (explicit intrinsics: the quantise kernel must reproduce exactly these values)
            float y = __fmul_rn(__fsub_rn(row[i], mean), rstd);
            if (gamma) y = __fmaf_rn(y, gamma[i], beta ? beta[i] : 0.f);
            amax = fmaxf(amax, fabsf(y));
        }
    }
    amax = warp_max(amax);
    __shared__ float smax[kThreads / 32];
    if (lane == 0) smax[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = 0.f;
        for (int w = 0; w < kThreads / 32; ++w) m = fmaxf(m, smax[w]);
        if (m > 0.f) atomic_max_nonneg(amax_out, m);
    }
}

template <int KIND>
__global__ void __launch_bounds__(kThreads)
shard_quantize_kernel(const float* __restrict__ x, int rows, int n, const float2* __restrict__ row_stats,
                      const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ amax_in,
                      uint8_t* __restrict__ codes, float* __restrict__ scale_out) {
    griddep_launch_dependents();
    griddep_wait();
    const float2 sc = scales_from_amax(ld_l2_f32(amax_in), fp8_max(KIND));
    if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) {
        scale_out[0] = sc.x;
        scale_out[1] = sc.y;
    }
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * kThreads) >> 5;
    const int n4 = n >> 2;  // n % 4 == 0 (checked by the entry point)
    for (int r = (blockIdx.x * kThreads + threadIdx.x) >> 5; r < rows; r += warps) {
        const float2 st = __ldcg(row_stats + r);
        const float4* row = reinterpret_cast<const float4*>(x + size_t(r) * n);
        uint32_t* out = reinterpret_cast<uint32_t*>(codes + size_t(r) * n);
        for (int i = lane; i < n4; i += 32) {
            const float4 v = row[i];
            float y0 = __fmul_rn(__fsub_rn(v.x, st.x), st.y), y1 = __fmul_rn(__fsub_rn(v.y, st.x), st.y);
            float y2 = __fmul_rn(__fsub_rn(v.z, st.x), st.y), y3 = __fmul_rn(__fsub_rn(v.w, st.x), st.y);
            if (gamma) {
                const float4 g = reinterpret_cast<const float4*>(gamma)[i];
                float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
                if (beta) b = reinterpret_cast<const float4*>(beta)[i];
                y0 = __fmaf_rn(y0, g.x, b.x);
                y1 = __fmaf_rn(y1, g.y, b.y);
                y2 = __fmaf_rn(y2, g.z, b.z);
                y3 = __fmaf_rn(y3, g.w, b.w);
            }
            out[i] = cvt_f32x4_to_fp8x4<KIND>(__fmul_rn(y0, sc.x), __fmul_rn(y1, sc.x), __fmul_rn(y2, sc.x),
                                              __fmul_rn(y3, sc.x));
        }
    }
}

int grid_for_rows(int rows) {
    const int per_block = kThreads / 32;
    const int want = (rows + per_block - 1) / per_block;
    const int cap = sm_count() * 8;
    return want < cap ? (want > 0 ? want : 1) : cap;
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_layernorm_shard_stats_f32(const float* x_shard, int rows, int cols_shard, float* partial_out,
                                                    df8_stream stream) {
    DF8_REQUIRE(rows >= 0 && cols_shard > 0, "df8_layernorm_shard_stats_f32: bad shape rows=%d cols=%d", rows, cols_shard);
    if (rows == 0) return DF8_OK;
    DF8_REQUIRE(x_shard && partial_out, "df8_layernorm_shard_stats_f32: null buffer");
    DF8_REQUIRE(cols_shard % 4 == 0 && aligned16(x_shard) && (reinterpret_cast<uintptr_t>(partial_out) & 7u) == 0,
                "df8_layernorm_shard_stats_f32: cols_shard must be a multiple of 4 and the buffers aligned");
    DF8_LAUNCH("shard_stats_kernel", shard_stats_kernel, dim3(unsigned(grid_for_rows(rows))), dim3(kThreads), 0,
               as_stream(stream), x_shard, rows, cols_shard, reinterpret_cast<float2*>(partial_out));
    return DF8_OK;
}

extern "C" df8_status df8_layernorm_shard_amax_f32(const float* x_shard, int rows, int cols_shard,
                                                   const float* partial_all, int world, const float* gamma_shard,
                                                   const float* beta_shard, float eps, float* row_stats_out,
                                                   float* amax_out, df8_stream stream) {
    DF8_REQUIRE(rows >= 0 && cols_shard > 0 && world >= 1, "df8_layernorm_shard_amax_f32: bad shape");
    DF8_REQUIRE(amax_out != nullptr, "df8_layernorm_shard_amax_f32: amax_out is required");
    cudaStream_t st = as_stream(stream);
    DF8_CLEAR_AMAX(amax_out, st);
    if (rows == 0) return DF8_OK;
    DF8_REQUIRE(x_shard && partial_all && row_stats_out, "df8_layernorm_shard_amax_f32: null buffer");
    DF8_LAUNCH("shard_amax_kernel", shard_amax_kernel, dim3(unsigned(grid_for_rows(rows))), dim3(kThreads), 0, st, x_shard,
               rows, cols_shard, reinterpret_cast<const float2*>(partial_all), world, gamma_shard, beta_shard, eps,
               reinterpret_cast<float2*>(row_stats_out), amax_out);
    return DF8_OK;
}

extern "C" df8_status df8_layernorm_shard_quantize_f32(const float* x_shard, int rows, int cols_shard,
                                                       const float* row_stats, const float* gamma_shard,
                                                       const float* beta_shard, df8_kind kind, const float* amax_in,
                                                       uint8_t* codes_shard_out, float* scale_out, df8_stream stream) {
    DF8_REQUIRE(kind == DF8_E4M3 || kind == DF8_E5M2, "df8_layernorm_shard_quantize_f32: unknown fp8 kind %d", int(kind));
    DF8_REQUIRE(rows >= 0 && cols_shard > 0, "df8_layernorm_shard_quantize_f32: bad shape");
    if (rows == 0) return DF8_OK;
    DF8_REQUIRE(x_shard && row_stats && amax_in && codes_shard_out, "df8_layernorm_shard_quantize_f32: null buffer");
    DF8_REQUIRE(cols_shard % 4 == 0 && aligned16(x_shard) && (reinterpret_cast<uintptr_t>(codes_shard_out) & 3u) == 0 &&
                    (!gamma_shard || aligned16(gamma_shard)) && (!beta_shard || aligned16(beta_shard)),
                "df8_layernorm_shard_quantize_f32: cols_shard must be a multiple of 4 and the buffers aligned");
    const dim3 grid(unsigned(grid_for_rows(rows))), block(kThreads);
    cudaStream_t st = as_stream(stream);
    if (kind == DF8_E4M3) {
        DF8_LAUNCH("shard_quantize_kernel", shard_quantize_kernel<DF8_E4M3>, grid, block, 0, st, x_shard, rows, cols_shard,
                   reinterpret_cast<const float2*>(row_stats), gamma_shard, beta_shard, amax_in, codes_shard_out, scale_out);
    } else {
        DF8_LAUNCH("shard_quantize_kernel", shard_quantize_kernel<DF8_E5M2>, grid, block, 0, st, x_shard, rows, cols_shard,
                   reinterpret_cast<const float2*>(row_stats), gamma_shard, beta_shard, amax_in, codes_shard_out, scale_out);
    }
    return DF8_OK;
}
