// Host-side plumbing of the voyager_b200 C ABI: error text, launch accounting, device queries.
#include <atomic>
#include <cstdarg>
#include <cstring>

#include "vq_common.cuh"

namespace {
thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};
struct DevInfo {
    int sms = 0;
    int smem_optin = 0;
};
DevInfo g_dev[64];
DevInfo& dev_info() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) d = 0;
    DevInfo& i = g_dev[d];
    if (i.sms == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d) == cudaSuccess && v > 0) i.sms = v;
        else i.sms = 148;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, d) == cudaSuccess && v > 0)
            i.smem_optin = v;
        else i.smem_optin = 48 * 1024;
    }
    return i;
}
}  // namespace

int vq_set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}
void vq_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
int vq_sm_count() { return dev_info().sms; }
int vq_max_smem_optin() { return dev_info().smem_optin; }

FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    f.d = d;
    uint32_t s = 0;
    while ((1ull << s) < d) ++s;
    f.s = s;
    f.m = (uint32_t)(((1ull << 32) * ((1ull << s) - d)) / d + 1);
    if (d == 1) { f.m = 0; f.s = 0; }
    return f;
}

extern "C" {

int vq_version(void) { return VQ_ABI_VERSION; }
const char* vq_last_error(void) { return g_error; }
uint64_t vq_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

// Host-only self check of the index-division constants (callable without a GPU).
int vq_selftest_fastdiv(uint32_t d, uint32_t n) {
    if (d == 0 || d >= (1u << 31) || n >= (1u << 31)) return -1;
    FastDiv f = make_fastdiv(d);
    return fd_div(n, f) == n / d ? 0 : 1;
}

}  // extern "C"
