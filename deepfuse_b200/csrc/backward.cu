// Helpers of the fully-connected layer's backward pass as fp8 products.
//
// Upstream computes dX = dY W, dW = dY^T X and db = sum_n dY in three scalar kernels
// (dnn/layers/fully_connected_layer.cu:43-107, launched at :317-353).  Here the two products go through the same
// tcgen05 GEMM as the forward pass; it contracts over the contiguous dimension of both operands ("TN"), so
//   dX[n,i] = sum_j dY[n,j] W[j,i]   needs W^T  [in, out]   (codes of the weight matrix, transposed once per update),
//   dW[o,i] = sum_n dY[n,o] X[n,i]   needs dY^T [out, N] and X^T [in, N].
// This file holds what produces those operands and the bias gradient:
//   df8_quantize_transpose_f32  fp32 [rows, cols] -> fp8 codes [cols, ld_t] (quantised with a given max|x|, written
//                               transposed; 4 B read + 1 B written per element, HBM-bound)
//   df8_transpose_u8            codes [rows, ld_in] -> [cols, ld_out]
//   df8_colsum_f32              out[c] = sum_r x[r, c] in a fixed order (two stages, no atomics: the same bits every run)
#include "df8_internal.cuh"

namespace df8 {
namespace {

constexpr int kTile = 64;

// 64 x 64 tile, 256 threads.  Load: a thread reads 4 consecutive floats of 4 rows (coalesced 256-byte row pieces);
// store: 4 threads cover the 64 bytes of one output row.  The tile in shared memory is [col][row + pad] bytes.
template <int KIND, bool QUANT>
__global__ void __launch_bounds__(256)
transpose_kernel(const void* __restrict__ in, long ld_in, int rows, int cols, const float* __restrict__ amax_in,
                 uint8_t* __restrict__ out, long ld_out, float* __restrict__ scale_out, uint8_t* __restrict__ plain,
                 long ld_plain) {
    __shared__ __align__(16) uint8_t tile[kTile][kTile + 16];
    griddep_launch_dependents();
    griddep_wait();
    float q = 1.f;
    if (QUANT) {
        const float2 sc = scales_from_amax(ld_l2_f32(amax_in), fp8_max(KIND));
        q = sc.x;
        if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && scale_out) {
            scale_out[0] = sc.x;
            scale_out[1] = sc.y;
        }
    }
    const int r0 = blockIdx.y * kTile, c0 = blockIdx.x * kTile;
    const int tc = (threadIdx.x & 15) * 4, tr = threadIdx.x >> 4;  // 16 threads across a row piece, 16 rows per pass
    // 128-bit loads / 32-bit stores of a thread's four consecutive elements where the layout allows
    const bool in_vec = QUANT && (ld_in & 3) == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
    const bool plain_vec = plain && (ld_plain & 3) == 0 && (reinterpret_cast<uintptr_t>(plain) & 3u) == 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const int r = r0 + tr + 16 * p;
        const int c = c0 + tc;
        uint8_t code[4] = {0, 0, 0, 0};
        if (r < rows && c < cols) {
            if (QUANT) {
                const float* src = static_cast<const float*>(in) + size_t(r) * ld_in + c;
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (in_vec && c + 3 < cols) {
                    const float4 f = *reinterpret_cast<const float4*>(src);
                    v[0] = f.x, v[1] = f.y, v[2] = f.z, v[3] = f.w;
                } else {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (c + k < cols) v[k] = src[k];
                }
                const uint32_t packed = cvt_f32x4_to_fp8x4<KIND>(__fmul_rn(v[0], q), __fmul_rn(v[1], q), __fmul_rn(v[2], q),
                                                                 __fmul_rn(v[3], q));
#pragma unroll
                for (int k = 0; k < 4; ++k) code[k] = (c + k < cols) ? uint8_t(packed >> (8 * k)) : uint8_t(0);
                if (plain) {  // the same codes in the tensor's own layout
                    uint8_t* dst = plain + size_t(r) * ld_plain + c;
                    if (plain_vec && c + 3 < cols) {
                        *reinterpret_cast<uint32_t*>(dst) = packed;
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            if (c + k < cols) dst[k] = code[k];
                    }
                }
            } else {
                const uint8_t* src = static_cast<const uint8_t*>(in) + size_t(r) * ld_in + c;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (c + k < cols) code[k] = src[k];
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) tile[tc + k][tr + 16 * p] = code[k];
    }
    __syncthreads();
    // output row = input column c0 + oc; its bytes r0 .. r0 + 63 (zero beyond `rows`: they pad the K dimension)
    const int oc = threadIdx.x >> 2, piece = (threadIdx.x & 3) * 16;
    const int c = c0 + oc;
    if (c < cols) {
        uint8_t* dst = out + size_t(c) * ld_out + r0 + piece;
        if (r0 + piece + 16 <= ld_out && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&tile[oc][piece]);
        } else {
            for (int k = 0; k < 16; ++k)
                if (r0 + piece + k < ld_out) dst[k] = tile[oc][piece + k];
        }
    }
}

constexpr int kSumChunks = 32;

// stage 1: grid (cols / 32, kSumChunks); a warp-wide row piece of 32 columns, 8 warps take rows in turn
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const float* __restrict__ x, long ld, int rows, int cols, float* __restrict__ partial,
                      float* __restrict__ amax_out) {
    __shared__ float red[8][32];
    griddep_launch_dependents();
    griddep_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    const int per = (rows + kSumChunks - 1) / kSumChunks;
    const int r_begin = blockIdx.y * per, r_end = min(rows, r_begin + per);
    float s = 0.f, m = 0.f;
    if (c < cols)
        for (int r = r_begin + warp; r < r_end; r += 8) {
            const float v = x[size_t(r) * ld + c];
            s += v;
            m = fmaxf(m, fabsf(v));
        }
    if (amax_out) {  // the same pass also gives max|x| (the tensor is about to be quantised)
        m = warp_max(m);
        if (lane == 0 && m > 0.f) atomic_max_nonneg(amax_out, m);
    }
    red[warp][lane] = s;
    __syncthreads();
    if (warp == 0 && c < cols) {
        float t = red[0][lane];
#pragma unroll
        for (int w = 1; w < 8; ++w) t += red[w][lane];
        partial[size_t(blockIdx.y) * cols + c] = t;
    }
}

__global__ void colsum_final_kernel(const float* __restrict__ partial, int cols, float* __restrict__ out) {
    griddep_launch_dependents();
    griddep_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < cols) {
        float t = 0.f;
        for (int k = 0; k < kSumChunks; ++k) t += __ldcg(partial + size_t(k) * cols + c);
        out[c] = t;
    }
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_quantize_transpose_f32(const float* x_d, int rows, int cols, df8_kind kind, const float* amax_in_d,
                                                 uint8_t* codes_t_d, int ld_t, float* scale_out_d, df8_stream stream) {
    return df8_quantize_both_layouts_f32(x_d, rows, cols, kind, amax_in_d, codes_t_d, ld_t, nullptr, 0, scale_out_d, stream);
}

extern "C" df8_status df8_quantize_both_layouts_f32(const float* x_d, int rows, int cols, df8_kind kind, const float* amax_in_d,
                                                    uint8_t* codes_t_d, int ld_t, uint8_t* codes_d, int ld_c,
                                                    float* scale_out_d, df8_stream stream) {
    DF8_REQUIRE(!codes_d || ld_c >= cols, "df8_quantize_both_layouts_f32: ld_c=%d is smaller than cols=%d", ld_c, cols);
    DF8_REQUIRE(kind == DF8_E4M3 || kind == DF8_E5M2, "df8_quantize_transpose_f32: unknown fp8 kind");
    DF8_REQUIRE(rows >= 0 && cols >= 0 && ld_t >= rows, "df8_quantize_transpose_f32: bad shape rows=%d cols=%d ld_t=%d", rows,
                cols, ld_t);
    if (rows == 0 || cols == 0) return DF8_OK;
    DF8_REQUIRE(x_d && amax_in_d && codes_t_d, "df8_quantize_transpose_f32: null buffer");
    // the tiles cover [0, ld_t) of every output row: columns rows .. ld_t - 1 are written as zero codes
    const dim3 grid{unsigned((cols + kTile - 1) / kTile), unsigned((ld_t + kTile - 1) / kTile)}, block{256};
    cudaStream_t st = as_stream(stream);
    if (kind == DF8_E4M3)
        (void)launch_kernel((transpose_kernel<int(DF8_E4M3), true>), grid, block, 0, st, static_cast<const void*>(x_d), long(cols),
                            rows, cols, amax_in_d, codes_t_d, long(ld_t), scale_out_d, codes_d, long(ld_c));
    else
        (void)launch_kernel((transpose_kernel<int(DF8_E5M2), true>), grid, block, 0, st, static_cast<const void*>(x_d), long(cols),
                            rows, cols, amax_in_d, codes_t_d, long(ld_t), scale_out_d, codes_d, long(ld_c));
    DF8_LAUNCH_CHECK("transpose_kernel (quantise)");
    return DF8_OK;
}

extern "C" df8_status df8_transpose_u8(const uint8_t* in_d, int rows, int cols, int ld_in, uint8_t* out_d, int ld_out,
                                       df8_stream stream) {
    DF8_REQUIRE(rows >= 0 && cols >= 0 && ld_in >= cols && ld_out >= rows,
                "df8_transpose_u8: bad shape rows=%d cols=%d ld_in=%d ld_out=%d", rows, cols, ld_in, ld_out);
    if (rows == 0 || cols == 0) return DF8_OK;
    DF8_REQUIRE(in_d && out_d, "df8_transpose_u8: null buffer");
    const dim3 grid{unsigned((cols + kTile - 1) / kTile), unsigned((ld_out + kTile - 1) / kTile)}, block{256};
    (void)launch_kernel((transpose_kernel<0, false>), grid, block, 0, as_stream(stream), static_cast<const void*>(in_d),
                        long(ld_in), rows, cols, static_cast<const float*>(nullptr), out_d, long(ld_out),
                        static_cast<float*>(nullptr), static_cast<uint8_t*>(nullptr), 0L);
    DF8_LAUNCH_CHECK("transpose_kernel");
    return DF8_OK;
}

extern "C" df8_status df8_colsum_f32(const float* x_d, int rows, int cols, int ld, float* partial_d, float* out_d,
                                     df8_stream stream) {
    return df8_colsum_amax_f32(x_d, rows, cols, ld, partial_d, out_d, nullptr, stream);
}

extern "C" df8_status df8_colsum_amax_f32(const float* x_d, int rows, int cols, int ld, float* partial_d, float* out_d,
                                          float* amax_out_d, df8_stream stream) {
    DF8_REQUIRE(rows >= 0 && cols >= 0 && ld >= cols, "df8_colsum_f32: bad shape rows=%d cols=%d ld=%d", rows, cols, ld);
    cudaStream_t st = as_stream(stream);
    if (amax_out_d) DF8_CLEAR_AMAX(amax_out_d, st);
    if (cols == 0) return DF8_OK;
    DF8_REQUIRE(x_d && partial_d && out_d, "df8_colsum_f32: null buffer");
    (void)launch_kernel(colsum_partial_kernel, dim3(unsigned((cols + 31) / 32), kSumChunks), dim3(256), 0, st, x_d, long(ld), rows,
                        cols, partial_d, amax_out_d);
    DF8_LAUNCH_CHECK("colsum_partial_kernel");
    (void)launch_kernel(colsum_final_kernel, dim3(unsigned((cols + 255) / 256)), dim3(256), 0, st,
                        static_cast<const float*>(partial_d), cols, out_d);
    DF8_LAUNCH_CHECK("colsum_final_kernel");
    return DF8_OK;
}

extern "C" int df8_colsum_partial_floats(int cols) { return kSumChunks * (cols > 0 ? cols : 0); }
