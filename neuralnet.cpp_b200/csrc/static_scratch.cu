// A bias-gradient entry point for callers that cannot provide scratch memory.
//
// nnb200_bias_grad needs a caller-allocated buffer for its per-chunk partial sums.  Some hosts of
// this library have nowhere to get one: the reference's CudaBackend allocates op *outputs* only
// and has no hook through which a kernel could ask for workspace, and services that fix their
// device-memory budget at start-up (or run inside latency-critical loops) must not call cudaMalloc,
// which synchronises the whole device.  For them the partial sums live in a file-scope device
// array that every GPU loading the library holds from load to exit.
#include "kernels.h"
#include "nnb200.h"

namespace nnb {

// 1 MiB per GPU.  Enough for e.g. 8192 rows x 4096 columns (64 chunks of 128 rows x 4096).
static __device__ __align__(256) float g_bias_grad_scratch[NNB200_BIAS_GRAD_STATIC_MAX_FLOATS];

constexpr int kMaxDevices = 64;
static std::atomic<float*> g_scratch_addr[kMaxDevices];     // zero-initialised; two threads that race here store the same address

// In host code the array's name is only a handle for the runtime, not an address a kernel can use:
// the device address is looked up once per device, with that device current, and cached.
static int static_scratch(float** out)
{
    int dev = 0;
    NNB_CUDA_CHECK(cudaGetDevice(&dev));
    NNB_ARG_CHECK(dev >= 0 && dev < kMaxDevices, "device ordinal out of range");
    float* addr = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!addr) {
        void* p = nullptr;
        NNB_CUDA_CHECK(cudaGetSymbolAddress(&p, g_bias_grad_scratch));
        addr = static_cast<float*>(p);
        g_scratch_addr[dev].store(addr, std::memory_order_release);
    }
    *out = addr;
    return 0;
}

}  // namespace nnb

using namespace nnb;

extern "C" int nnb200_bias_grad_static(const void* g, long long ldg, float* out, int rows, int cols, int dtype,
                                       void* stream)
{
    NNB_ARG_CHECK(dtype == 0 || dtype == 1, "dtype must be 0 (fp32) or 1 (bf16)");
    NNB_ARG_CHECK(rows >= 0 && cols >= 0, "negative shape");
    NNB_ARG_CHECK(rows == 0 || cols == 0 || (g && out), "null gradient or output pointer");
    NNB_ARG_CHECK(ldg >= cols, "the row stride is shorter than a row (rows would overlap)");
    if (colsum_scratch_floats(rows, cols) > static_cast<size_t>(NNB200_BIAS_GRAD_STATIC_MAX_FLOATS)) {
        fprintf(stderr,
                "nnb200_bias_grad_static: %d x %d needs %zu scratch floats, the built-in buffer holds %d; "
                "use nnb200_bias_grad with caller scratch\n",
                rows, cols, colsum_scratch_floats(rows, cols), NNB200_BIAS_GRAD_STATIC_MAX_FLOATS);
        return -1;
    }
    float* scratch = nullptr;
    NNB_TRY(static_scratch(&scratch));
    // Every partial the second stage reads is written by the first stage of the same call, so the
    // buffer needs no clearing between calls even though it keeps the previous call's contents.
    if (dtype == 1)
        return colsum_accumulate<bf16>(static_cast<const bf16*>(g), ldg, nullptr, nullptr, nullptr, nullptr, 0, out, scratch,
                                       rows, cols, to_stream(stream));
    return colsum_accumulate<float>(static_cast<const float*>(g), ldg, nullptr, nullptr, nullptr, nullptr, 0, out, scratch,
                                    rows, cols, to_stream(stream));
}
