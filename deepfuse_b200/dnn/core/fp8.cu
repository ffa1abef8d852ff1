#include "dnn/core/fp8.cuh"

namespace dnn {
namespace fp8 {

Policy& policy() {
    static Policy p;
    return p;
}

namespace {
// splitmix64 of (seed, index) -> uniform in (-limit, limit)
__global__ void fill_uniform_kernel(float* w, size_t n, float limit, uint64_t seed, uint64_t offset) {
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
        uint64_t z = seed * 0x9E3779B97F4A7C15ull + (i + offset + 1) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        const float u = float(uint32_t(z >> 40)) * (1.0f / 16777216.0f);  // [0, 1)
        w[i] = (2.0f * u - 1.0f) * limit;
    }
}
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float u01(uint64_t bits) { return (float(bits >> 40) + 0.5f) * (1.0f / 16777216.0f); }

__global__ void fill_normal_kernel(float* w, size_t n, float mean, float stddev, uint64_t seed, uint64_t offset) {
    const uint64_t base = seed * 0xD1342543DE82EF95ull;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
        const uint64_t idx = uint64_t(i) + offset;
        const float r = sqrtf(-2.0f * logf(u01(mix64(base + 2 * idx))));
        w[i] = mean + stddev * (r * cosf(6.28318530718f * u01(mix64(base + 2 * idx + 1))));
    }
}
}  // namespace

void fill_normal(float* p, size_t n, float mean, float std, uint64_t seed, uint64_t index_offset) {
    if (n == 0) return;
    fill_normal_kernel<<<1184, 256, 0, Cuda::stream()>>>(p, n, mean, std, seed, index_offset);
    utils::CHECK_CUDA_EX(cudaGetLastError());
}

void fill_uniform(float* p, size_t n, float limit, uint64_t seed, uint64_t index_offset) {
    if (n == 0) return;
    fill_uniform_kernel<<<1184, 256, 0, Cuda::stream()>>>(p, n, limit, seed, index_offset);
    utils::CHECK_CUDA_EX(cudaGetLastError());
}

namespace {
constexpr int kPoolFloats = 4096;
struct PassState {
    int depth = 0;
    int next = 0;
    int prev_preclear = 1;
    float* pool = nullptr;  // of the device the scope was opened on; never freed (16 KB per device and thread)
};
thread_local PassState g_pass;
thread_local float* g_pools[64] = {};

void clear_pool() {
    utils::CHECK_CUDA_EX(cudaMemsetAsync(g_pass.pool, 0, kPoolFloats * sizeof(float), Cuda::stream()));
    g_pass.next = 0;
}
}  // namespace

PassScope::PassScope() {
    if (g_pass.depth++ > 0) return;
    int dev = 0;
    utils::CHECK_CUDA_EX(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {  // no pool for such a device: behave as if no scope were open
        g_pass.pool = nullptr;
        return;
    }
    if (!g_pools[dev]) utils::CHECK_CUDA_EX(cudaMalloc(&g_pools[dev], kPoolFloats * sizeof(float)));
    g_pass.pool = g_pools[dev];
    clear_pool();
    g_pass.prev_preclear = df8_set_amax_preclear(0);
}

PassScope::~PassScope() {
    if (--g_pass.depth > 0) return;
    if (g_pass.pool) df8_set_amax_preclear(g_pass.prev_preclear);
    g_pass.pool = nullptr;
}

float* amax_slot(float* own) {
    if (g_pass.depth == 0 || !g_pass.pool) return own;
    // every slot handed out so far has been consumed by kernels already on the stream, so a full pool is
    // simply cleared again
    if (g_pass.next == kPoolFloats) clear_pool();
    return g_pass.pool + g_pass.next++;
}

void check_device_status() { utils::CHECK_DF8(df8_status_word_check()); }

void quantize(const float* x, size_t n, df8_kind kind, Quantized& q) {
    if (q.codes.numel() != n) q.codes = tensor<uint8_t>({int(n)});
    q.kind = kind;
    float* am = amax_slot(q.amax.data());
    utils::CHECK_DF8(df8_amax_f32(x, n, am, stream()));
    utils::CHECK_DF8(df8_quantize_f32(x, n, kind, am, q.codes.data(), q.scale.data(), stream()));
}

void quantize_with_amax(const float* x, size_t n, df8_kind kind, const float* amax, Quantized& q) {
    if (q.codes.numel() != n) q.codes = tensor<uint8_t>({int(n)});
    q.kind = kind;
    utils::CHECK_DF8(df8_quantize_f32(x, n, kind, amax, q.codes.data(), q.scale.data(), stream()));
}

}  // namespace fp8
}  // namespace dnn
