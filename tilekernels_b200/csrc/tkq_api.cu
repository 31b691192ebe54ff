// Library-wide host helpers: error text, launch check, per-device SM count.
#include <cstdio>
#include <cstring>

#include <mutex>

#include "tkq_common.cuh"
#include "tkq_launch.cuh"

namespace tkq {

static thread_local char g_error[256] = "no error";

int set_error(int code, const char* msg) {
    std::snprintf(g_error, sizeof(g_error), "%s", msg);
    return code;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return 0;
    std::snprintf(g_error, sizeof(g_error), "%s: %s", what, cudaGetErrorString(e));
    return static_cast<int>(e);
}

int device_sm_count() {
    static int cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64 && cache[dev] > 0) return cache[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < 64) cache[dev] = n;
    return n;
}

static int current_device() {
    int dev = 0;
    return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}

int cached_occupancy(const void* kernel, int threads, int dyn_smem) {
    struct Entry {
        const void* kernel;
        int device, threads, smem, occ;
    };
    static Entry table[512];
    static int used = 0;
    static std::mutex mu;
    const int dev = current_device();
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
        if (table[i].kernel == kernel && table[i].device == dev && table[i].threads == threads && table[i].smem == dyn_smem)
            return table[i].occ;
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, threads, dyn_smem) != cudaSuccess || occ < 1) {
        cudaGetLastError();
        occ = 1;
    }
    if (used < 512) table[used++] = Entry{kernel, dev, threads, dyn_smem, occ};
    return occ;
}

int ensure_dynamic_smem(const void* kernel, int bytes) {
    struct Entry {
        const void* kernel;
        int device, bytes;
    };
    static Entry table[512];
    static int used = 0;
    static std::mutex mu;
    const int dev = current_device();
    std::lock_guard<std::mutex> lock(mu);
    int slot = -1;
    for (int i = 0; i < used; ++i)
        if (table[i].kernel == kernel && table[i].device == dev) {
            if (table[i].bytes >= bytes) return 0;
            slot = i;
            break;
        }
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return set_error(static_cast<int>(e), "cudaFuncSetAttribute(max dynamic shared memory) failed");
    }
    if (slot >= 0) table[slot].bytes = bytes;
    else if (used < 512) table[used++] = Entry{kernel, dev, bytes};  // a full table only costs the repeated call
    return 0;
}

}  // namespace tkq

extern "C" int tkq_version(void) { return 200; }

extern "C" const char* tkq_last_error_string(void) { return tkq::g_error; }
