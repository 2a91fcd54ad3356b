// Shared helpers for the sm_100a kernels: error convention, small math, warp/block reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <climits>
#include <cstdint>
#include <cstdio>

// Error convention of the C ABI (the one cuda/cuda_kernels.cu:24-55 of the reference uses):
// 0 = success, positive = cudaError_t, -1 = shape/argument error; a message goes to stderr.
#define NNB_CUDA_CHECK(call)                                                                  \
    do {                                                                                      \
        cudaError_t err__ = (call);                                                           \
        if (err__ != cudaSuccess) {                                                           \
            fprintf(stderr, "nnb200: CUDA error at %s:%d: %s\n", __FILE__, __LINE__,          \
                    cudaGetErrorString(err__));                                               \
            return static_cast<int>(err__);                                                   \
        }                                                                                     \
    } while (0)

// after every kernel launch: counts it (the host-side launch counter the benchmark reports) and
// surfaces launch-configuration errors
#define NNB_LAUNCH_CHECK()                                                                    \
    do {                                                                                      \
        ++nnb::g_launches;                                                                    \
        NNB_CUDA_CHECK(cudaGetLastError());                                                   \
    } while (0)

#define NNB_ARG_CHECK(cond, msg)                                                              \
    do {                                                                                      \
        if (!(cond)) {                                                                        \
            fprintf(stderr, "nnb200: %s: %s\n", __func__, msg);                               \
            return -1;                                                                        \
        }                                                                                     \
    } while (0)

#define NNB_TRY(call)                                                                         \
    do {                                                                                      \
        int rc__ = (call);                                                                    \
        if (rc__ != 0) return rc__;                                                           \
    } while (0)

namespace nnb {

extern unsigned long long g_launches;   // kernels launched by this library since the last reset

using bf16 = __nv_bfloat16;

static inline cudaStream_t to_stream(void* s) { return static_cast<cudaStream_t>(s); }

constexpr int kSmCount = 148;   // B200: 2 dies x 74 SMs; grids are sized in multiples of this

__host__ __device__ constexpr inline long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

#ifdef __CUDACC__
// 1 / (1 + e^-x) for the bf16 paths: one exponential and one reciprocal instruction, both flushing denormals (the
// non-flushing forms of __expf and __fdividef cost several range-fixing instructions each); 0 for x < -88, 1 for x > 88.
// The activation kernels and the GEMM epilogues that replace them use this one function, so they agree bit for bit.
__device__ __forceinline__ float sigmoid_fast(float x)
{
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return r;
}
#endif

// Per-device caches.  A process may drive several GPUs (one after the other or from several threads), and function
// attributes, SM counts and occupancy figures belong to the device that is current when they are set or read.
inline int current_device_slot()
{
    int dev = 0;
    cudaGetDevice(&dev);
    return dev & 63;
}
// SMs of the current device
inline int device_sm_count()
{
    static std::atomic<int> cache[64];
    const int dev = current_device_slot();
    int v = cache[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        v = kSmCount;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) { cudaGetLastError(); v = kSmCount; }
        cache[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}
// Runs `f` (returning cudaError_t) once per device: the opt-in to more than 48 KB of dynamic shared memory and the like.
struct PerDeviceOnce {
    std::atomic<unsigned long long> done{0};
    template <typename F> int run(F f)
    {
        const unsigned long long bit = 1ull << current_device_slot();
        if (done.load(std::memory_order_acquire) & bit) return 0;
        const cudaError_t e = f();
        if (e != cudaSuccess) {
            fprintf(stderr, "nnb200: CUDA error setting up a kernel: %s\n", cudaGetErrorString(e));
            return static_cast<int>(e);
        }
        done.fetch_or(bit, std::memory_order_release);
        return 0;
    }
};

// number of blocks for a grid-stride kernel: enough to fill the machine, never more than the work
static inline int grid_for(long long work_items, int per_block, int blocks_per_sm = 8)
{
    long long need = ceil_div(work_items, per_block);
    long long cap = static_cast<long long>(kSmCount) * blocks_per_sm;
    if (need < 1) need = 1;
    return static_cast<int>(need < cap ? need : cap);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// block-wide sum for up to 1024 threads; `red` is 32 floats of shared memory; result on all threads
__device__ __forceinline__ float block_sum(float v, float* red)
{
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : 0.f;
    return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* red)
{
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : -INFINITY;
    return warp_max(r);
}

// 16-byte vector of T
template <typename T> struct Vec16;
template <> struct alignas(16) Vec16<float> { static constexpr int N = 4; float v[4]; };
template <> struct alignas(16) Vec16<bf16>  { static constexpr int N = 8; bf16 v[8]; };

template <typename T> __device__ __forceinline__ Vec16<T> ld16(const T* p)
{
    Vec16<T> r;
    *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
    return r;
}
template <typename T> __device__ __forceinline__ void st16(T* p, const Vec16<T>& r)
{
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

}  // namespace nnb
