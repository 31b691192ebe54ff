// Host-side launch geometry helpers.
#pragma once

#include <algorithm>

#include "tkq_common.cuh"

namespace tkq {

// Grid for a grid-stride kernel: enough blocks to fill every SM at the kernel's
// own occupancy (whole waves over the SM count), never more than the work needs.
// The occupancy query is cached per kernel instance and block size.
// Resident blocks per SM of `kernel` at this block size on the current device (cached per device; tkq_api.cu).
int cached_occupancy(const void* kernel, int threads, int dyn_smem);

// Raises the kernel's dynamic shared-memory limit to at least `bytes` on the current device.  The attribute
// belongs to the (device, kernel) pair, so the cache that avoids repeating the call is keyed by both.
// Returns 0 or the code set_error recorded.
int ensure_dynamic_smem(const void* kernel, int bytes);

template <class Kernel>
int grid_size(Kernel kernel, int threads, int64_t blocks_of_work, int dyn_smem, int sm_limit = 0) {
    const int occ = cached_occupancy(reinterpret_cast<const void*>(kernel), threads, dyn_smem);
    int sms = device_sm_count();
    if (sm_limit > 0) sms = std::min(sms, sm_limit);
    const int64_t resident = static_cast<int64_t>(sms) * occ;
    return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks_of_work, resident)));
}

// Splits `chunks` per-thread chunks of a row over a block: K chunks per thread
// (1, 2 or 4) and a block size that is a multiple of 32, at most max_threads.
inline bool row_shape(int64_t chunks, int max_threads, int* k_out, int* threads_out) {
    for (int k = 1; k <= 4; k *= 2) {
        const int64_t t = (chunks + k - 1) / k;
        if (t <= max_threads) {
            *k_out = k;
            *threads_out = static_cast<int>(std::max<int64_t>(32, (t + 31) / 32 * 32));
            return true;
        }
    }
    return false;
}

}  // namespace tkq
