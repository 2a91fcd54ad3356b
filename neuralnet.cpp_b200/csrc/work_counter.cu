// Work counters for kernels whose CTAs draw their work items from a counter in global memory.
//
// One pair {next item, CTAs that have left} per stream that launches such kernels: kernels of one stream never overlap,
// kernels of different streams may.  A launch finds its pair at zero and leaves it at zero (the CTA that leaves last
// resets it), so no launch needs a memset of its own.  The pairs live in a file-scope device array: nothing is allocated.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace nnb {

constexpr int WORK_STREAMS = 64;
__device__ unsigned int g_work_counters[WORK_STREAMS][8];       // 32 bytes apart

int work_counter_pair(cudaStream_t s, unsigned int** out)
{
    struct Table { std::mutex mu; unsigned int* base = nullptr; int used = 0; cudaStream_t streams[WORK_STREAMS]; };
    static Table tables[64];
    Table& t = tables[current_device_slot()];
    std::lock_guard<std::mutex> lock(t.mu);
    if (!t.base) NNB_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&t.base), g_work_counters));
    int i = 0;
    while (i < t.used && t.streams[i] != s) ++i;
    if (i == t.used) {
        NNB_ARG_CHECK(t.used < WORK_STREAMS, "more than 64 distinct streams have launched work-drawing kernels on this device");
        t.streams[t.used++] = s;
    }
    *out = t.base + 8 * i;
    return 0;
}

}  // namespace nnb
