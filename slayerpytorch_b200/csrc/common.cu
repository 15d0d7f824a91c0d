// Error reporting and device queries shared by all entry points.
#include <stdarg.h>

#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace sb200 {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

void clear_error() { g_err[0] = '\0'; }

int sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int reserve_dynamic_smem(const void *func, size_t bytes)
{
    if (bytes <= 48 * 1024) return SLAYER_B200_OK;
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, size_t> granted;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
    std::lock_guard<std::mutex> lock(mu);
    size_t &have = granted[std::make_pair(func, dev)];
    if (have >= bytes) return SLAYER_B200_OK;
    cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) {
        set_error("cannot reserve %zu bytes of dynamic shared memory: %s", bytes, cudaGetErrorString(e));
        return SLAYER_B200_ECUDA;
    }
    have = bytes;
    return SLAYER_B200_OK;
}

}  // namespace sb200

extern "C" int slayer_b200_abi_version(void) { return 1; }

extern "C" const char *slayer_b200_last_error(void) { return sb200::g_err; }
