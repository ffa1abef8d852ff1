// The status word written by bounded device-side waits, and its host accessors.
#include "df8_internal.cuh"

#include <atomic>

namespace df8 {

__device__ unsigned int g_status_word[4];  // [0] first timeout code, [1] number of timeouts

df8_status status_word_device_ptr(unsigned int** out) {
    static std::atomic<unsigned int*> cached[64] = {};
    int dev = 0;
    DF8_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(DF8_ERR_INVALID, "device index %d out of range", dev);
    unsigned int* p = cached[dev].load(std::memory_order_acquire);
    if (!p) {
        // the symbol's name is a host-side stand-in: its device address must be looked up per device
        DF8_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status_word));
        cached[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return DF8_OK;
}

}  // namespace df8

using namespace df8;

extern "C" df8_status df8_status_word_read(unsigned int* code_h, unsigned int* count_h) {
    unsigned int w[4] = {0, 0, 0, 0};
    DF8_CUDA_TRY(cudaMemcpyFromSymbol(w, g_status_word, sizeof(w)));
    if (code_h) *code_h = w[0];
    if (count_h) *count_h = w[1];
    return DF8_OK;
}

extern "C" df8_status df8_status_word_reset(void) {
    unsigned int w[4] = {0, 0, 0, 0};
    DF8_CUDA_TRY(cudaMemcpyToSymbol(g_status_word, w, sizeof(w)));
    return DF8_OK;
}

extern "C" df8_status df8_status_word_check(void) {
    unsigned int w[4] = {0, 0, 0, 0};
    DF8_CUDA_TRY(cudaMemcpyFromSymbol(w, g_status_word, sizeof(w)));
    if (w[0] == 0 && w[1] == 0) return DF8_OK;
    return fail(DF8_ERR_TIMEOUT, "a bounded device-side wait gave up: first code 0x%x, %u event(s); results since the "
                                 "last df8_status_word_reset() are not valid", w[0], w[1]);
}
