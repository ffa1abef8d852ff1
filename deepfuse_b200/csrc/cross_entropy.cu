// Softmax cross-entropy on fp32 logits: per-row loss and the gradient with respect to the logits.
//
// Replaces the launches of cross_entropy_log_softmax_kernel and cross_entropy_gradient_logit_kernel
// (dnn/losses/cross_entropy.cu:12-74, :77-139, launched at :147-153 and :181-187), same math:
//   loss_i  = -sum_j t_ij * (x_ij - max_i - log(sum_j exp(x_ij - max_i) + 1e-7))
//   grad_ij = exp(x_ij - max_i) / (sum_j exp(x_ij - max_i) + 1e-7) - t_ij
// Upstream gives one THREAD a whole row (three serial loops over the classes, 50257 for the GPT-2 head) and wants
// the targets as a dense one-hot matrix the size of the logits.  Here one CTA owns a row: maximum, then the sum of
// exponentials, then the target term, each a strided pass with warp-shuffle + shared-memory reductions; the second and
// third pass find the row (200 KB at 50257 classes) in L2, so the logits cross HBM once.  Targets come either as
// upstream's dense matrix or as one class index per row (no one-hot matrix is ever built: that alone is as many
// bytes as the logits).  Rows may be pitched (the row pitch of Gpt2::forward_logits_pitched).
// HBM-bound: 4 B per logit for the loss, 8 B per logit (+4 with dense targets) for the gradient.
#include "df8_internal.cuh"

#include <atomic>

namespace df8 {
namespace {

constexpr int kCeThreads = 1024;  // one CTA per row; few rows in flight (see run_ce)

// running (maximum, sum of exp(x - maximum)) of the elements seen so far
struct MaxSum {
    float m, s;
};
__device__ __forceinline__ MaxSum merge(MaxSum a, MaxSum b) {
    const float m = fmaxf(a.m, b.m);
    if (m == -INFINITY) return MaxSum{m, 0.f};
    return MaxSum{m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}
__device__ __forceinline__ void absorb4(MaxSum& r, float4 v) {
    const float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
    if (m4 > r.m) {  // rare after the first few elements: rescale what has been summed
        r.s *= __expf(r.m - m4);
        r.m = m4;
    }
    r.s += (__expf(v.x - r.m) + __expf(v.y - r.m)) + (__expf(v.z - r.m) + __expf(v.w - r.m));
}
__device__ __forceinline__ void absorb1(MaxSum& r, float v) {
    if (v > r.m) {
        r.s *= __expf(r.m - v);
        r.m = v;
    }
    r.s += __expf(v - r.m);
}

__device__ __forceinline__ MaxSum block_merge(MaxSum v, MaxSum* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxSum other{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
        v = merge(v, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    MaxSum r = lane < kCeThreads / 32 ? red[lane] : MaxSum{-INFINITY, 0.f};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxSum other{__shfl_xor_sync(0xffffffffu, r.m, o), __shfl_xor_sync(0xffffffffu, r.s, o)};
        r = merge(r, other);
    }
    __syncthreads();
    return r;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = lane < kCeThreads / 32 ? red[lane] : 0.f;
    r = warp_sum(r);
    __syncthreads();
    return r;
}

// One pass over the row gives the maximum and the sum of exponentials together (each thread keeps a running pair and
// rescales its sum when its maximum grows; pairs are merged across the block): the logits cross HBM once for the
// loss.  The gradient reads the row a second time, from L2: run_ce keeps the rows in flight (2 CTAs per SM) well
// inside L2, where a grid of one CTA per row had 240 MB of rows in flight and read every row from HBM twice.
// VEC: rows start on 16-byte boundaries (base aligned, pitch a multiple of 4 floats): 128-bit accesses over the
// whole groups of a row, the up-to-three loose floats at its end one by one.
template <bool GRAD, bool VEC>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(const float* __restrict__ logits, long ld, const float* __restrict__ targets, long ldt,
                     const int* __restrict__ target_idx, int rows, int C, float* __restrict__ row_loss,
                     float* __restrict__ grad, long ldg, unsigned int* __restrict__ bad_index) {
    __shared__ MaxSum red_ms[kCeThreads / 32];
    __shared__ float red[kCeThreads / 32];
    griddep_launch_dependents();
    griddep_wait();
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* x = logits + size_t(row) * ld;
        const int c4 = VEC ? C >> 2 : 0;
        MaxSum r{-INFINITY, 0.f};
        if (VEC) {
            const float4* x4 = reinterpret_cast<const float4*>(x);
#pragma unroll 4
            for (int i = threadIdx.x; i < c4; i += kCeThreads) absorb4(r, ld_stream_f4(x4 + i));
        }
        for (int i = 4 * c4 + threadIdx.x; i < C; i += kCeThreads) absorb1(r, x[i]);
        r = block_merge(r, red_ms);
        const float mx = r.m, s = r.s;
        int t = -1;
        if (target_idx) {
            t = target_idx[row];
            if (t < 0 || t >= C) {  // recorded for the host (upstream's one-hot helper would write out of bounds)
                if (threadIdx.x == 0 && bad_index) atomicAdd(bad_index, 1u);
                t = -1;
            }
        }
        if (!GRAD) {
            const float lse = logf(s + 1e-7f);
            float total = 0.f;
            if (target_idx) {
                if (threadIdx.x == 0 && t >= 0) total = x[t] - mx - lse;
            } else {
                const float* tr = targets + size_t(row) * ldt;
                for (int i = threadIdx.x; i < C; i += kCeThreads) {
                    const float tv = tr[i];
                    if (tv != 0.f) total += tv * (x[i] - mx - lse);
                }
                total = block_sum(total, red);
            }
            if (threadIdx.x == 0) row_loss[row] = -total;
        } else {
            const float inv = 1.f / (s + 1e-7f);
            float* g = grad + size_t(row) * ldg;
            const float* tr = targets ? targets + size_t(row) * ldt : nullptr;
            const bool gvec = VEC && !tr && (ldg & 3) == 0 && (reinterpret_cast<uintptr_t>(grad) & 15u) == 0;
            if (gvec) {
                const float4* x4 = reinterpret_cast<const float4*>(x);
                float4* g4 = reinterpret_cast<float4*>(g);
#pragma unroll 4
                for (int i = threadIdx.x; i < c4; i += kCeThreads) {
                    const float4 v = ld_stream_f4(x4 + i);
                    float4 o;
                    o.x = expf(v.x - mx) * inv;
                    o.y = expf(v.y - mx) * inv;
                    o.z = expf(v.z - mx) * inv;
                    o.w = expf(v.w - mx) * inv;
                    const int d = t - 4 * i;  // the target class, if it lies in this group
                    if (d == 0) o.x -= 1.f;
                    else if (d == 1) o.y -= 1.f;
                    else if (d == 2) o.z -= 1.f;
                    else if (d == 3) o.w -= 1.f;
                    st_stream_f4(g4 + i, o);
                }
                for (int i = 4 * c4 + threadIdx.x; i < C; i += kCeThreads) g[i] = expf(x[i] - mx) * inv - (i == t ? 1.f : 0.f);
            } else {
                for (int i = threadIdx.x; i < C; i += kCeThreads) {
                    const float p = expf(x[i] - mx) * inv;
                    const float tv = tr ? tr[i] : (i == t ? 1.f : 0.f);
                    g[i] = p - tv;
                }
            }
        }
    }
}

// Gradient with the row held in shared memory between the two passes (rows of up to ~56 K classes: the GPT-2
// vocabulary's 50257 floats are 196 KB): the logits cross HBM once and the gradient once, whatever L2 does with 1.65 GB
// of gradient stores streaming through it.  One CTA per SM; class-index targets, rows on 16-byte boundaries.
__global__ void __launch_bounds__(kCeThreads, 1)
cross_entropy_grad_smem_kernel(const float* __restrict__ logits, long ld, const int* __restrict__ target_idx, int rows,
                               int C, float* __restrict__ grad, long ldg, unsigned int* __restrict__ bad_index) {
    extern __shared__ float4 row4[];  // ceil(C / 4) groups
    __shared__ MaxSum red_ms[kCeThreads / 32];
    griddep_launch_dependents();
    griddep_wait();
    const int c4 = C >> 2;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* x = logits + size_t(row) * ld;
        const float4* x4 = reinterpret_cast<const float4*>(x);
        MaxSum r{-INFINITY, 0.f};
#pragma unroll 4
        for (int i = threadIdx.x; i < c4; i += kCeThreads) {
            const float4 v = ld_stream_f4(x4 + i);
            row4[i] = v;
            absorb4(r, v);
        }
        float* tail = reinterpret_cast<float*>(row4 + c4);
        for (int i = 4 * c4 + threadIdx.x; i < C; i += kCeThreads) {
            const float v = x[i];
            tail[i - 4 * c4] = v;
            absorb1(r, v);
        }
        r = block_merge(r, red_ms);  // its barriers also make the row visible to every thread
        const float mx = r.m, inv = 1.f / (r.s + 1e-7f);
        int t = target_idx[row];
        if (t < 0 || t >= C) {
            if (threadIdx.x == 0 && bad_index) atomicAdd(bad_index, 1u);
            t = -1;
        }
        float* g = grad + size_t(row) * ldg;
        const bool gvec = (ldg & 3) == 0 && (reinterpret_cast<uintptr_t>(grad) & 15u) == 0;
        if (gvec) {
            float4* g4 = reinterpret_cast<float4*>(g);
#pragma unroll 4
            for (int i = threadIdx.x; i < c4; i += kCeThreads) {
                const float4 v = row4[i];
                float4 o;
                o.x = expf(v.x - mx) * inv;
                o.y = expf(v.y - mx) * inv;
                o.z = expf(v.z - mx) * inv;
                o.w = expf(v.w - mx) * inv;
                const int d = t - 4 * i;
                if (d == 0) o.x -= 1.f;
                else if (d == 1) o.y -= 1.f;
                else if (d == 2) o.z -= 1.f;
                else if (d == 3) o.w -= 1.f;
                st_stream_f4(g4 + i, o);
            }
        } else {
            const float* rowf = reinterpret_cast<const float*>(row4);
            for (int i = threadIdx.x; i < 4 * c4; i += kCeThreads) g[i] = expf(rowf[i] - mx) * inv - (i == t ? 1.f : 0.f);
        }
        for (int i = 4 * c4 + threadIdx.x; i < C; i += kCeThreads) g[i] = expf(tail[i - 4 * c4] - mx) * inv - (i == t ? 1.f : 0.f);
        __syncthreads();  // the next row overwrites the buffer
    }
}

constexpr int kCeSmemCap = 224 * 1024;

__device__ unsigned int g_ce_bad_index = 0;

df8_status run_ce(bool want_grad, const float* logits, int ld, const float* targets, int ldt, const int* target_idx, int rows,
                  int classes, float* row_loss, float* grad, int ldg, cudaStream_t st) {
    unsigned int* bad = nullptr;
    DF8_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&bad), g_ce_bad_index));
    const bool vec = aligned16(logits) && ld % 4 == 0;
    const int sms = sm_count();
    const int grid = rows < sms * 2 ? rows : sms * 2;  // rows in flight: 2 per SM (60 MB at 50257 classes, inside L2)
    const dim3 g{unsigned(grid)}, b{kCeThreads};
    if (want_grad && vec && target_idx && !targets && size_t((classes + 3) / 4) * 16 <= size_t(kCeSmemCap)) {
        static std::atomic<bool> configured[64] = {};
        int dev = 0;
        DF8_CUDA_TRY(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && !configured[dev].load()) {
            DF8_CUDA_TRY(cudaFuncSetAttribute(cross_entropy_grad_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kCeSmemCap));
            configured[dev].store(true);
        }
        const size_t smem = size_t((classes + 3) / 4) * 16;
        (void)launch_kernel(cross_entropy_grad_smem_kernel, dim3(unsigned(rows < sms ? rows : sms)), b, smem, st, logits, long(ld),
                            target_idx, rows, classes, grad, long(ldg), bad);
        DF8_LAUNCH_CHECK("cross_entropy_grad_smem_kernel");
        return DF8_OK;
    }
    if (want_grad) {
        if (vec) (void)launch_kernel((cross_entropy_kernel<true, true>), g, b, 0, st, logits, long(ld), targets, long(ldt), target_idx, rows, classes, row_loss, grad, long(ldg), bad);
        else (void)launch_kernel((cross_entropy_kernel<true, false>), g, b, 0, st, logits, long(ld), targets, long(ldt), target_idx, rows, classes, row_loss, grad, long(ldg), bad);
    } else {
        if (vec) (void)launch_kernel((cross_entropy_kernel<false, true>), g, b, 0, st, logits, long(ld), targets, long(ldt), target_idx, rows, classes, row_loss, grad, long(ldg), bad);
        else (void)launch_kernel((cross_entropy_kernel<false, false>), g, b, 0, st, logits, long(ld), targets, long(ldt), target_idx, rows, classes, row_loss, grad, long(ldg), bad);
    }
    DF8_LAUNCH_CHECK("cross_entropy_kernel");
    return DF8_OK;
}

}  // namespace
}  // namespace df8

using namespace df8;

extern "C" df8_status df8_cross_entropy_f32(const float* logits_d, int ld, const float* targets_d, int ldt,
                                            const int* target_idx_d, int rows, int classes, float* row_loss_d,
                                            df8_stream stream) {
    DF8_REQUIRE(rows >= 0 && classes > 0 && ld >= classes, "df8_cross_entropy_f32: bad shape rows=%d classes=%d ld=%d", rows,
                classes, ld);
    DF8_REQUIRE((targets_d != nullptr) != (target_idx_d != nullptr),
                "df8_cross_entropy_f32: give dense targets or class indices, one of the two");
    DF8_REQUIRE(!targets_d || ldt >= classes, "df8_cross_entropy_f32: ldt=%d is smaller than classes=%d", ldt, classes);
    if (rows == 0) return DF8_OK;
    DF8_REQUIRE(logits_d && row_loss_d, "df8_cross_entropy_f32: null buffer");
    return run_ce(false, logits_d, ld, targets_d, ldt, target_idx_d, rows, classes, row_loss_d, nullptr, 0, as_stream(stream));
}

extern "C" df8_status df8_cross_entropy_grad_f32(const float* logits_d, int ld, const float* targets_d, int ldt,
                                                 const int* target_idx_d, int rows, int classes, float* grad_d, int ldg,
                                                 df8_stream stream) {
    DF8_REQUIRE(rows >= 0 && classes > 0 && ld >= classes && ldg >= classes,
                "df8_cross_entropy_grad_f32: bad shape rows=%d classes=%d ld=%d ldg=%d", rows, classes, ld, ldg);
    DF8_REQUIRE((targets_d != nullptr) != (target_idx_d != nullptr),
                "df8_cross_entropy_grad_f32: give dense targets or class indices, one of the two");
    DF8_REQUIRE(!targets_d || ldt >= classes, "df8_cross_entropy_grad_f32: ldt=%d is smaller than classes=%d", ldt, classes);
    if (rows == 0) return DF8_OK;
    DF8_REQUIRE(logits_d && grad_d, "df8_cross_entropy_grad_f32: null buffer");
    return run_ce(true, logits_d, ld, targets_d, ldt, target_idx_d, rows, classes, nullptr, grad_d, ldg, as_stream(stream));
}

extern "C" df8_status df8_cross_entropy_bad_indices(unsigned int* count_h, int reset) {
    DF8_REQUIRE(count_h != nullptr, "df8_cross_entropy_bad_indices: null argument");
    unsigned int* bad = nullptr;
    DF8_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&bad), g_ce_bad_index));
    DF8_CUDA_TRY(cudaMemcpy(count_h, bad, sizeof(unsigned int), cudaMemcpyDeviceToHost));
    if (reset) DF8_CUDA_TRY(cudaMemset(bad, 0, sizeof(unsigned int)));
    return DF8_OK;
}
