// The engine primitives of the reference C ABI (cuda/cuda_kernels.h:27-165), fp32, rebuilt as
// vectorised / coalesced sm_100a kernels.  Same symbols, argument meaning and error convention, so
// the reference CudaBackend links against this library unchanged.
#include "kernels.h"
#include "nnb200.h"

namespace nnb {

static cudaStream_t g_handle_stream = nullptr;   // stream used by cuda_matmul_with_handle

// ---------------------------------------------------------------- elementwise
template <typename F>
__global__ void map1_kernel(const float* __restrict__ a, float* __restrict__ out, size_t n, F f)
{
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t n4 = n / 4;
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (aligned) {
        for (size_t v = i; v < n4; v += stride) {
            float4 x = reinterpret_cast<const float4*>(a)[v];
            x.x = f(x.x); x.y = f(x.y); x.z = f(x.z); x.w = f(x.w);
            reinterpret_cast<float4*>(out)[v] = x;
        }
        for (size_t k = n4 * 4 + i; k < n; k += stride) out[k] = f(a[k]);
    } else {
        for (; i < n; i += stride) out[i] = f(a[i]);
    }
}
template <typename F>
__global__ void map2_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                            size_t n, F f)
{
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t n4 = n / 4;
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                           reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (aligned) {
        for (size_t v = i; v < n4; v += stride) {
            float4 x = reinterpret_cast<const float4*>(a)[v];
            const float4 y = reinterpret_cast<const float4*>(b)[v];
            x.x = f(x.x, y.x); x.y = f(x.y, y.y); x.z = f(x.z, y.z); x.w = f(x.w, y.w);
            reinterpret_cast<float4*>(out)[v] = x;
        }
        for (size_t k = n4 * 4 + i; k < n; k += stride) out[k] = f(a[k], b[k]);
    } else {
        for (; i < n; i += stride) out[i] = f(a[i], b[i]);
    }
}

__device__ __forceinline__ float apply_unary(unsigned op, float x)
{
    switch (op) {
        case 0: return -x;
        case 1: return expf(x);
        case 2: return logf(x);
        case 3: return sqrtf(x);
        case 4: return 1.0f / sqrtf(x);
        case 5: return fabsf(x);
        default: return tanhf(x);
    }
}
__device__ __forceinline__ float apply_binary(unsigned op, float a, float b)
{
    switch (op) {
        case 0: return a + b;
        case 1: return a - b;
        case 2: return a * b;
        case 3: return a / b;
        case 4: return fmaxf(a, b);
        default: return fminf(a, b);
    }
}
__device__ __forceinline__ bool apply_cmp(unsigned c, float a, float b)
{
    switch (c) {
        case 0: return a < b;
        case 1: return a <= b;
        case 2: return a > b;
        case 3: return a >= b;
        case 4: return a == b;
        default: return a != b;
    }
}

template <typename F> static int launch_map1(const float* a, float* out, size_t n, F f, cudaStream_t s)
{
    if (n == 0) return 0;
    map1_kernel<<<grid_for(static_cast<long long>(n / 4 + 1), 256), 256, 0, s>>>(a, out, n, f);
    NNB_LAUNCH_CHECK();
    return 0;
}
template <typename F> static int launch_map2(const float* a, const float* b, float* out, size_t n, F f, cudaStream_t s)
{
    if (n == 0) return 0;
    map2_kernel<<<grid_for(static_cast<long long>(n / 4 + 1), 256), 256, 0, s>>>(a, b, out, n, f);
    NNB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- reductions
// per-row reduce: one warp per row, coalesced, shuffle tree.  mode 0 sum, 1 max, 2 min
__global__ void reduce_row_kernel(const float* __restrict__ A, float* __restrict__ out, unsigned rows, unsigned cols,
                                  unsigned mode)
{
    const unsigned warps_per_block = blockDim.x >> 5, lane = threadIdx.x & 31;
    for (unsigned r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < rows; r += gridDim.x * warps_per_block) {
        const float* row = A + static_cast<size_t>(r) * cols;
        float acc = (mode == 0) ? 0.f : (mode == 1 ? -INFINITY : INFINITY);
        for (unsigned c = lane; c < cols; c += 32) {
            const float v = row[c];
            acc = (mode == 0) ? acc + v : (mode == 1 ? fmaxf(acc, v) : fminf(acc, v));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, acc, o);
            acc = (mode == 0) ? acc + other : (mode == 1 ? fmaxf(acc, other) : fminf(acc, other));
        }
        if (lane == 0) out[r] = acc;
    }
}

// per-column reduce: a block owns 32 columns; 32x8 threads read whole 128-byte row segments
// (coalesced, unlike a thread-per-column walk down a stride-`cols` column) and fold 8 row lanes in smem.
__global__ void reduce_col_kernel(const float* __restrict__ A, float* __restrict__ out, unsigned rows, unsigned cols,
                                  unsigned mode)
{
    __shared__ float part[8][33];
    const unsigned tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const unsigned c = blockIdx.x * 32 + tx;
    float acc = (mode == 0) ? 0.f : (mode == 1 ? -INFINITY : INFINITY);
    if (c < cols)
        for (unsigned r = ty; r < rows; r += 8) {
            const float v = A[static_cast<size_t>(r) * cols + c];
            acc = (mode == 0) ? acc + v : (mode == 1 ? fmaxf(acc, v) : fminf(acc, v));
        }
    part[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && c < cols) {
        for (int k = 1; k < 8; ++k) {
            const float v = part[k][tx];
            acc = (mode == 0) ? acc + v : (mode == 1 ? fmaxf(acc, v) : fminf(acc, v));
        }
        out[c] = acc;
    }
}

__global__ void broadcast_kernel(const float* __restrict__ A, const float* __restrict__ vec, float* __restrict__ out,
                                 unsigned rows, unsigned cols, unsigned op, int by_row)
{
    const size_t n = static_cast<size_t>(rows) * cols;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const unsigned r = static_cast<unsigned>(i / cols), c = static_cast<unsigned>(i - static_cast<size_t>(r) * cols);
        out[i] = apply_binary(op, A[i], by_row ? vec[r] : vec[c]);
    }
}

// ---------------------------------------------------------------- layout
__global__ void transpose_kernel(const float* __restrict__ A, float* __restrict__ out, unsigned R, unsigned C)
{
    __shared__ float tile[32][33];
    const unsigned bx = blockIdx.x * 32, by = blockIdx.y * 32;
    for (unsigned j = threadIdx.y; j < 32; j += 8) {
        const unsigned r = by + j, c = bx + threadIdx.x;
        if (r < R && c < C) tile[j][threadIdx.x] = A[static_cast<size_t>(r) * C + c];
    }
    __syncthreads();
    for (unsigned j = threadIdx.y; j < 32; j += 8) {
        const unsigned c = bx + j, r = by + threadIdx.x;
        if (r < R && c < C) out[static_cast<size_t>(c) * R + r] = tile[threadIdx.x][j];
    }
}

// (M, B*N) <-> (B*M, N): whole rows of N contiguous floats move, so every access is coalesced
__global__ void rearrange3d_kernel(const float* __restrict__ A, float* __restrict__ out, unsigned M, unsigned B,
                                   unsigned N, unsigned inverse)
{
    const size_t total = static_cast<size_t>(M) * B * N;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const unsigned n = static_cast<unsigned>(i % N);
        const size_t rest = i / N;
        if (!inverse) {   // out index (b, m, n) <- in (m, b, n)
            const unsigned m = static_cast<unsigned>(rest % M), b = static_cast<unsigned>(rest / M);
            out[i] = A[(static_cast<size_t>(m) * B + b) * N + n];
        } else {          // out index (m, b, n) <- in (b, m, n)
            const unsigned b = static_cast<unsigned>(rest % B), m = static_cast<unsigned>(rest / B);
            out[i] = A[(static_cast<size_t>(b) * M + m) * N + n];
        }
    }
}

// ---------------------------------------------------------------- gather / scatter
__global__ void gather_kernel(const float* __restrict__ table, const float* __restrict__ idx, float* __restrict__ out,
                              unsigned vocab, unsigned D, unsigned num)
{
    const unsigned warps = (gridDim.x * blockDim.x) >> 5, lane = threadIdx.x & 31;
    for (unsigned i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < num; i += warps) {
        const float f = idx[i];
        const bool ok = f > -1.0f && f < static_cast<float>(vocab);
        const float* src = table + static_cast<size_t>(ok ? static_cast<unsigned>(f) : 0u) * D;
        float* dst = out + static_cast<size_t>(i) * D;
        for (unsigned c = lane; c < D; c += 32) dst[c] = ok ? src[c] : 0.f;
    }
}

// Deterministic scatter-add: thread (row v, column c) walks the index list in ascending i and adds
// the matching rows in that order, which is the order of the sequential CPU loop
// (cpu_engine.hpp:203-214 of the reference), so the fp32 result is bit-identical to it.  The
// index list is staged through shared memory.  Cost is O(vocab * num) index compares; the fused
// training step uses the sorted-segment kernel in embedding.cu instead.
__global__ void scatter_add_ordered_kernel(float* __restrict__ dst, const float* __restrict__ idx,
                                           const float* __restrict__ grad, unsigned vocab, unsigned D, unsigned num)
{
    __shared__ float sidx[1024];
    const unsigned v = blockIdx.x;
    float acc[4];
    const unsigned c0 = threadIdx.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[k] = 0.f;
    for (unsigned cbase = 0; cbase < D; cbase += blockDim.x * 4) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const unsigned c = cbase + c0 + k * blockDim.x;
            acc[k] = (c < D) ? dst[static_cast<size_t>(v) * D + c] : 0.f;
        }
        for (unsigned base = 0; base < num; base += 1024) {
            __syncthreads();
            for (unsigned t = threadIdx.x; t < 1024 && base + t < num; t += blockDim.x) sidx[t] = idx[base + t];
            __syncthreads();
            const unsigned lim = min(1024u, num - base);
            for (unsigned t = 0; t < lim; ++t) {
                const float f = sidx[t];
                if (f > -1.0f && static_cast<unsigned>(f) == v) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const unsigned c = cbase + c0 + k * blockDim.x;
                        if (c < D) acc[k] += grad[static_cast<size_t>(base + t) * D + c];
                    }
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const unsigned c = cbase + c0 + k * blockDim.x;
            if (c < D) dst[static_cast<size_t>(v) * D + c] = acc[k];
        }
    }
}

}  // namespace nnb

using namespace nnb;

extern "C" {

int nnb200_set_handle_stream(void* stream)
{
    g_handle_stream = to_stream(stream);
    return 0;
}

int cuda_matmul(const float* A, const float* B, float* C, std::size_t A_rows, std::size_t A_cols, std::size_t B_rows,
                std::size_t B_cols, int transA, int transB, void* stream)
{
    const long long M = transA ? A_cols : A_rows, K = transA ? A_rows : A_cols;
    const long long K2 = transB ? B_cols : B_rows, N = transB ? B_rows : B_cols;
    if (K != K2) return -1;
    // op(A)[m][k]: A[m*A_cols + k] or A[k*A_cols + m];  op(B)[k][n]: B[k*B_cols + n] or B[n*B_cols + k]
    return sgemm_strided(A, B, C, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
                         transA ? 1 : static_cast<long long>(A_cols), transA ? static_cast<long long>(A_cols) : 1,
                         transB ? static_cast<long long>(B_cols) : 1, transB ? 1 : static_cast<long long>(B_cols),
                         N, 1, 0, 0, 0, 1.0f, nullptr, nullptr, nullptr, 0, to_stream(stream));
}

int cuda_matmul_with_handle(const float* A, const float* B, float* C, std::size_t A_rows, std::size_t A_cols,
                            std::size_t B_rows, std::size_t B_cols, int transA, int transB, void* handle_ptr)
{
    (void)handle_ptr;   // no library handle is needed; the stream is the one set by nnb200_set_handle_stream
    return cuda_matmul(A, B, C, A_rows, A_cols, B_rows, B_cols, transA, transB, g_handle_stream);
}

int cuda_batched_matmul(const float* A, const float* B, float* C, std::size_t A_rows, std::size_t A_cols,
                        std::size_t B_rows, std::size_t B_cols, unsigned int batch, int transA, int transB, void* stream)
{
    if (batch == 0 || A_rows % batch || B_rows % batch) return -1;
    const long long a_rpb = A_rows / batch, b_rpb = B_rows / batch;
    const long long M = transA ? A_cols : a_rpb, K = transA ? a_rpb : A_cols;
    const long long K2 = transB ? B_cols : b_rpb, N = transB ? b_rpb : B_cols;
    if (K != K2) return -1;
    for (unsigned b0 = 0; b0 < batch; b0 += 65535) {
        const unsigned nb = batch - b0 < 65535 ? batch - b0 : 65535;
        NNB_TRY(sgemm_strided(A + b0 * a_rpb * A_cols, B + b0 * b_rpb * B_cols, C + b0 * M * N, static_cast<int>(M),
                              static_cast<int>(N), static_cast<int>(K), transA ? 1 : static_cast<long long>(A_cols),
                              transA ? static_cast<long long>(A_cols) : 1, transB ? static_cast<long long>(B_cols) : 1,
                              transB ? 1 : static_cast<long long>(B_cols), N, static_cast<int>(nb), a_rpb * A_cols,
                              b_rpb * B_cols, M * N, 1.0f, nullptr, nullptr, nullptr, 0, to_stream(stream)));
    }
    return 0;
}

int cuda_elementwise_unary(const float* A, float* out, unsigned int count, unsigned int op, void* stream)
{
    if (op > 6) return -1;
    return launch_map1(A, out, count, [op] __device__(float x) { return apply_unary(op, x); }, to_stream(stream));
}

int cuda_elementwise_binary(const float* A, const float* B, float* out, unsigned int count, unsigned int op, void* stream)
{
    if (op > 5) return -1;
    return launch_map2(A, B, out, count, [op] __device__(float a, float b) { return apply_binary(op, a, b); },
                       to_stream(stream));
}

int cuda_elementwise_binary_scalar(const float* A, float* out, unsigned int count, unsigned int op, float scalar,
                                   int scalar_first, void* stream)
{
    if (op > 5) return -1;
    if (scalar_first)
        return launch_map1(A, out, count, [op, scalar] __device__(float x) { return apply_binary(op, scalar, x); },
                           to_stream(stream));
    return launch_map1(A, out, count, [op, scalar] __device__(float x) { return apply_binary(op, x, scalar); },
                       to_stream(stream));
}

int cuda_axpy(const float* A, const float* B, float* out, unsigned int count, float scalar, void* stream)
{
    return launch_map2(A, B, out, count, [scalar] __device__(float a, float b) { return a + scalar * b; },
                       to_stream(stream));
}

int cuda_elementwise_select_scalar_cond(const float* A, const float* then_v, float* out, unsigned int count,
                                        unsigned int cmp, float scalar_b, float scalar_else, void* stream)
{
    if (cmp > 5) return -1;
    return launch_map2(A, then_v, out, count,
                       [cmp, scalar_b, scalar_else] __device__(float a, float t) {
                           return apply_cmp(cmp, a, scalar_b) ? t : scalar_else;
                       },
                       to_stream(stream));
}

int cuda_reduce_row(const float* A, float* out, unsigned int rows, unsigned int cols, unsigned int mode, void* stream)
{
    if (mode > 2) return -1;
    if (rows == 0) return 0;
    reduce_row_kernel<<<grid_for(rows, 8), 256, 0, to_stream(stream)>>>(A, out, rows, cols, mode);
    NNB_LAUNCH_CHECK();
    return 0;
}

int cuda_reduce_col(const float* A, float* out, unsigned int rows, unsigned int cols, unsigned int mode, void* stream)
{
    if (mode > 2) return -1;
    if (cols == 0) return 0;
    reduce_col_kernel<<<static_cast<unsigned>(ceil_div(cols, 32)), 256, 0, to_stream(stream)>>>(A, out, rows, cols, mode);
    NNB_LAUNCH_CHECK();
    return 0;
}

int cuda_broadcast_row(const float* A, const float* vec, float* out, unsigned int rows, unsigned int cols,
                       unsigned int op, void* stream)
{
    if (op > 5) return -1;
    if (static_cast<size_t>(rows) * cols == 0) return 0;
    broadcast_kernel<<<grid_for(static_cast<long long>(rows) * cols, 256), 256, 0, to_stream(stream)>>>(A, vec, out, rows,
                                                                                                      cols, op, 1);
    NNB_LAUNCH_CHECK();
    return 0;
}

int cuda_broadcast_col(const float* A, const float* vec, float* out, unsigned int rows, unsigned int cols,
                       unsigned int op, void* stream)
{
    if (op > 5) return -1;
    if (static_cast<size_t>(rows) * cols == 0) return 0;
    broadcast_kernel<<<grid_for(static_cast<long long>(rows) * cols, 256), 256, 0, to_stream(stream)>>>(A, vec, out, rows,
                                                                                                      cols, op, 0);
    NNB_LAUNCH_CHECK();
    return 0;
}

int cuda_transpose(const float* A, float* out, unsigned int R, unsigned int C, void* stream)
{
    if (static_cast<size_t>(R) * C == 0) return 0;
    dim3 grid(static_cast<unsigned>(ceil_div(C, 32)), static_cast<unsigned>(ceil_div(R, 32)));
    if (grid.y > 65535) return -1;
    transpose_kernel<<<grid, dim3(32, 8), 0, to_stream(stream)>>>(A, out, R, C);
    NNB_LAUNCH_CHECK();
    return 0;
}

int cuda_rearrange_3d(const float* A, float* out, unsigned int M, unsigned int B, unsigned int N, unsigned int inverse,
                      void* stream)
{
    const long long total = static_cast<long long>(M) * B * N;
    if (total == 0) return 0;
    rearrange3d_kernel<<<grid_for(total, 256), 256, 0, to_stream(stream)>>>(A, out, M, B, N, inverse);
    NNB_LAUNCH_CHECK();
    return 0;
}

int cuda_gather(const float* table, const float* indices, float* out, unsigned int vocab, unsigned int D,
                unsigned int num, void* stream)
{
    if (static_cast<size_t>(num) * D == 0) return 0;
    gather_kernel<<<grid_for(num, 8), 256, 0, to_stream(stream)>>>(table, indices, out, vocab, D, num);
    NNB_LAUNCH_CHECK();
    return 0;
}

int cuda_scatter_add(float* dst, const float* indices, const float* grad, unsigned int vocab, unsigned int D,
                     unsigned int num, void* stream)
{
    if (static_cast<size_t>(num) * D == 0 || vocab == 0) return 0;
    scatter_add_ordered_kernel<<<vocab, 128, 0, to_stream(stream)>>>(dst, indices, grad, vocab, D, num);
    NNB_LAUNCH_CHECK();
    return 0;
}

}  // extern "C"
