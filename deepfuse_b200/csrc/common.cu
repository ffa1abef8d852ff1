// Error reporting and device queries shared by every entry point of libdf8.
//
// The upstream project reports CUDA failures by throwing std::runtime_error from
// utils::check_cuda_error (dnn/utils/common.cuh:20-35).  No exception may cross a C boundary, so
// the C-ABI records the message per thread and returns a status code; the C++ `dnn::` classes
// above turn a non-zero status back into the exception types upstream throws.
#include "df8_internal.cuh"

#include <cstdlib>
#include <mutex>

namespace df8 {

namespace {
thread_local char g_last_error[512] = "";
}

df8_status fail(df8_status code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

namespace {
thread_local bool g_amax_preclear = true;
}
bool amax_preclear() { return g_amax_preclear; }

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("DF8_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

int sm_count() {
    static int cached[64];
    static std::once_flag once;
    std::call_once(once, [] {
        for (int& c : cached) c = 0;
    });
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace df8

extern "C" const char* df8_last_error(void) { return df8::g_last_error; }

extern "C" int df8_set_amax_preclear(int enabled) {
    const int before = df8::g_amax_preclear ? 1 : 0;
    df8::g_amax_preclear = enabled != 0;
    return before;
}

extern "C" const char* df8_version(void) { return "df8 0.1 (sm_100a)"; }
