// Stand-alone masked row softmax over attention logits [B,H,T,T] (fp32).
//
// Replaces the launch of softmax_masked_kernel (dnn/layers/softmax_layer.cu:26-81, launched at
// :154-167), same math: x += mask; p = exp(x - rowmax) / (sum + 1e-6); p = 0 where mask < -1e8.
// Upstream uses one block of T threads per row, each thread re-scanning the whole row from shared
// memory for the max and the sum (O(T^2) per row, T <= 1024); here one warp owns a row, keeps it in
// registers when T <= 1024 and reduces with shuffles; longer rows take three passes over global
// memory.  The fused attention kernel does not use this; it exists for SoftmaxLayer::forward.
#include "df8_internal.cuh"

namespace df8 {
namespace {

constexpr int kSmThreads = 256;
constexpr int kMaxPerLane = 32;  // T <= 1024 on the register path

__global__ void __launch_bounds__(kSmThreads)
softmax_masked_kernel(const float* __restrict__ x, const float* __restrict__ mask, int mask_b, long rows, int H, int T,
                      float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int wpb = kSmThreads / 32;
    for (long row = long(blockIdx.x) * wpb + (threadIdx.x >> 5); row < rows; row += long(gridDim.x) * wpb) {
        const int q = int(row % T);
        const long b = row / (long(H) * T);
        const float* xr = x + row * T;
        const float* mr = mask ? mask + ((mask_b > 1 ? b : 0) * T + q) * T : nullptr;
        float* orow = out + row * T;
        if (T <= 32 * kMaxPerLane) {
            float v[kMaxPerLane];
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < kMaxPerLane; ++j) {
                const int i = lane + 32 * j;
                v[j] = i < T ? xr[i] + (mr ? mr[i] : 0.f) : -INFINITY;
                mx = fmaxf(mx, v[j]);
            }
            mx = warp_max(mx);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < kMaxPerLane; ++j) {
                const int i = lane + 32 * j;
                v[j] = i < T ? expf(v[j] - mx) : 0.f;
                sum += v[j];
            }
            sum = warp_sum(sum);
            const float denom = sum + 1e-6f;
#pragma unroll
            for (int j = 0; j < kMaxPerLane; ++j) {
                const int i = lane + 32 * j;
                if (i < T) orow[i] = (mr && mr[i] < -1e8f) ? 0.f : v[j] / denom;
            }
        } else {
            float mx = -INFINITY;
            for (int i = lane; i < T; i += 32) mx = fmaxf(mx, xr[i] + (mr ? mr[i] : 0.f));
            mx = warp_max(mx);
            float sum = 0.f;
            for (int i = lane; i < T; i += 32) sum += expf(xr[i] + (mr ? mr[i] : 0.f) - mx);
            sum = warp_sum(sum);
            const float denom = sum + 1e-6f;
            for (int i = lane; i < T; i += 32)
                orow[i] = (mr && mr[i] < -1e8f) ? 0.f : expf(xr[i] + (mr ? mr[i] : 0.f) - mx) / denom;
        }
    }
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_softmax_masked_f32(const float* x, const float* mask, int mask_b, int B, int H, int T,
                                             float* out, df8_stream stream) {
    DF8_REQUIRE(B >= 0 && H >= 0 && T >= 0, "df8_softmax_masked_f32: bad shape B=%d H=%d T=%d", B, H, T);
    DF8_REQUIRE(!mask || mask_b == 1 || mask_b == B, "df8_softmax_masked_f32: mask must be [B,1,T,T] or [1,1,T,T]");
    const long rows = long(B) * H * T;
    if (rows == 0) return DF8_OK;
    DF8_REQUIRE(x && out, "df8_softmax_masked_f32: null buffer");
    long blocks = (rows + kSmThreads / 32 - 1) / (kSmThreads / 32);
    const long cap = long(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    softmax_masked_kernel<<<int(blocks), kSmThreads, 0, as_stream(stream)>>>(x, mask, mask_b, rows, H, T, out);
    DF8_LAUNCH_CHECK("softmax_masked_kernel");
    return DF8_OK;
}
