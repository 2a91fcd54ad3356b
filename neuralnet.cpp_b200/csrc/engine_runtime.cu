// Device runtime behind the C++ drop-in engine: device selection, one compute stream, stream-ordered
// memory from the device's default pool, and blocking host<->device copies.  It is the counterpart of
// the reference's CudaBackend::initialize / CudaBuffer::allocate / upload_blocking / download_blocking /
// sync_stream (backend/cuda_backend.hpp:66-125, 207-337), behind plain C entry points so that the
// engine headers need no CUDA header.  Unlike the reference (cudaMalloc + cudaFree around every op
// output, each a device-wide synchronisation) blocks come from and return to a pool in stream order:
// an op's output can be released while kernels that read it are still queued.
#include <cstdlib>
#include <cstring>

#include "kernels.h"
#include "nnb200.h"

namespace {
struct Runtime {
    bool ready = false;
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t t0 = nullptr, t1 = nullptr;          // nnb200_rt_timer_start / _stop
};
Runtime g_rt;
}  // namespace

extern "C" {

int nnb200_rt_init(int device, char* name_out, size_t name_len, size_t* total_mem, int* sm_count)
{
    if (!g_rt.ready) {
        int count = 0;
        NNB_CUDA_CHECK(cudaGetDeviceCount(&count));
        if (count <= 0) { fprintf(stderr, "nnb200_rt_init: no CUDA device\n"); return -2; }
        if (device < 0) {                                    // one process per GPU: the launcher's local rank picks it
            const char* lr = std::getenv("LOCAL_RANK");
            device = lr ? std::atoi(lr) : 0;
            if (device >= count) {                           // never wrap: two replicas on one GPU would fight over its SMs and TMEM
                fprintf(stderr, "nnb200_rt_init: LOCAL_RANK %d but only %d CUDA device(s): start one process per GPU\n", device, count);
                return -1;
            }
        }
        if (device < 0) { fprintf(stderr, "nnb200_rt_init: negative LOCAL_RANK\n"); return -1; }
        if (device >= count) { fprintf(stderr, "nnb200_rt_init: device %d of %d\n", device, count); return -1; }
        NNB_CUDA_CHECK(cudaSetDevice(device));
        NNB_CUDA_CHECK(cudaStreamCreateWithFlags(&g_rt.stream, cudaStreamNonBlocking));
        cudaMemPool_t pool;
        NNB_CUDA_CHECK(cudaDeviceGetDefaultMemPool(&pool, device));
        unsigned long long keep = ~0ull;                     // never hand freed blocks back to the driver
        NNB_CUDA_CHECK(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
        NNB_TRY(nnb200_set_handle_stream(g_rt.stream));
        g_rt.device = device;
        g_rt.ready = true;
    }
    cudaDeviceProp prop;
    NNB_CUDA_CHECK(cudaGetDeviceProperties(&prop, g_rt.device));
    if (name_out && name_len) { std::strncpy(name_out, prop.name, name_len - 1); name_out[name_len - 1] = 0; }
    if (total_mem) *total_mem = prop.totalGlobalMem;
    if (sm_count) *sm_count = prop.multiProcessorCount;
    return 0;
}

int nnb200_rt_device(void) { return g_rt.ready ? g_rt.device : -1; }
void* nnb200_rt_stream(void) { return g_rt.stream; }

int nnb200_rt_alloc(size_t bytes, void** out)
{
    if (!g_rt.ready || !out) return -1;
    *out = nullptr;
    if (bytes == 0) return 0;
    NNB_CUDA_CHECK(cudaMallocAsync(out, bytes, g_rt.stream));
    return 0;
}

int nnb200_rt_free(void* p)
{
    if (!p) return 0;
    if (!g_rt.ready) return -1;
    NNB_CUDA_CHECK(cudaFreeAsync(p, g_rt.stream));
    return 0;
}

int nnb200_rt_upload(void* dst, const void* host_src, size_t bytes)
{
    if (!g_rt.ready) return -1;
    if (bytes == 0) return 0;
    NNB_CUDA_CHECK(cudaMemcpyAsync(dst, host_src, bytes, cudaMemcpyHostToDevice, g_rt.stream));
    NNB_CUDA_CHECK(cudaStreamSynchronize(g_rt.stream));
    return 0;
}

int nnb200_rt_download(void* host_dst, const void* src, size_t bytes)
{
    if (!g_rt.ready) return -1;
    if (bytes == 0) return 0;
    NNB_CUDA_CHECK(cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, g_rt.stream));
    NNB_CUDA_CHECK(cudaStreamSynchronize(g_rt.stream));
    return 0;
}

int nnb200_rt_copy(void* dst, const void* src, size_t bytes)
{
    if (!g_rt.ready) return -1;
    if (bytes == 0) return 0;
    NNB_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, g_rt.stream));
    return 0;
}

int nnb200_rt_zero(void* dst, size_t bytes)
{
    if (!g_rt.ready) return -1;
    if (bytes == 0) return 0;
    NNB_CUDA_CHECK(cudaMemsetAsync(dst, 0, bytes, g_rt.stream));
    return 0;
}

// One pair of CUDA events on the runtime's stream: _start records the first, _stop records the second, waits for it
// and returns the device time between the two in milliseconds (what a driver program times a run of steps with).
int nnb200_rt_timer_start(void)
{
    if (!g_rt.ready) return -1;
    if (!g_rt.t0) { NNB_CUDA_CHECK(cudaEventCreate(&g_rt.t0)); NNB_CUDA_CHECK(cudaEventCreate(&g_rt.t1)); }
    NNB_CUDA_CHECK(cudaEventRecord(g_rt.t0, g_rt.stream));
    return 0;
}
int nnb200_rt_timer_stop(float* host_ms)
{
    if (!g_rt.ready || !g_rt.t0 || !host_ms) return -1;
    NNB_CUDA_CHECK(cudaEventRecord(g_rt.t1, g_rt.stream));
    NNB_CUDA_CHECK(cudaEventSynchronize(g_rt.t1));
    NNB_CUDA_CHECK(cudaEventElapsedTime(host_ms, g_rt.t0, g_rt.t1));
    return 0;
}

int nnb200_rt_sync(void)
{
    if (!g_rt.ready) return -1;
    NNB_CUDA_CHECK(cudaStreamSynchronize(g_rt.stream));
    return 0;
}

}  // extern "C"
