// Engine primitives the reference CudaEngine leaves unimplemented (cuda_engine.hpp:213-261, 461-469),
// in the reference's own layouts, fp32: the five fused two-pass attention primitives, the two fused
// cross-entropy primitives and the ExprSpec interpreter.  They make the unchanged reference Layer /
// Loss code run on the GPU one primitive at a time (the strict drop-in); the fused training step in
// gpt_step.cu is the fast path.  Semantics follow the CPU engine line by line:
//   batched_matmul_reduce / _softmax_denom / _softmax_apply / _softmax_backward_q / _kv
//                                   cpu_engine.hpp:426-915
//   col_softmax_denom / col_softmax_sparse_forward          cpu_engine.hpp:922-1006
//   eval_expr / eval_expr_reduce                            cpu_engine.hpp:1298-1659
#include "kernels.h"
#include "nnb200.h"

namespace nnb {

struct BmmDims {
    int batch, M, N, K, transA, transB;
    float alpha;
};
// A_b(i,k), B_b(k,j) exactly as the CPU engine indexes them (cpu_engine.hpp:452-469)
__device__ __forceinline__ float a_at(const float* __restrict__ A, const BmmDims& d, int b, int i, int k)
{
    const size_t base = static_cast<size_t>(b) * d.M * d.K;
    return d.transA ? A[base + static_cast<size_t>(k) * d.M + i] : A[base + static_cast<size_t>(i) * d.K + k];
}
__device__ __forceinline__ float b_at(const float* __restrict__ B, const BmmDims& d, int b, int k, int j)
{
    const size_t base = static_cast<size_t>(b) * d.K * d.N;
    return d.transB ? B[base + static_cast<size_t>(j) * d.K + k] : B[base + static_cast<size_t>(k) * d.N + j];
}
__device__ __forceinline__ float dot_ab(const float* __restrict__ A, const float* __restrict__ B, const BmmDims& d, int b, int i, int j)
{
    float s = 0.f;
    for (int k = 0; k < d.K; ++k) s += a_at(A, d, b, i, k) * b_at(B, d, b, k, j);
    return s;
}
__device__ __forceinline__ float combine(int op, float acc, float v) { return op == 1 ? fmaxf(acc, v) : (op == 2 ? fminf(acc, v) : acc + v); }

// one warp per output entry; lanes stride over the reduced index.  op: 0 Sum, 1 Max, 2 Min
__global__ void bmm_reduce_kernel(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ mask,
                                  float* __restrict__ out, BmmDims d, int op, int reduce_cols)
{
    const int lane = threadIdx.x & 31;
    const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int outer = reduce_cols ? d.M : d.N, inner = reduce_cols ? d.N : d.M;
    if (w >= static_cast<long long>(d.batch) * outer) return;
    const int b = static_cast<int>(w / outer), o = static_cast<int>(w % outer);
    const float init = op == 1 ? -3.402823466e38f : (op == 2 ? 3.402823466e38f : 0.f);   // lowest() / max() / 0
    float acc = init;
    for (int t = lane; t < inner; t += 32) {
        const int i = reduce_cols ? o : t, j = reduce_cols ? t : o;
        const float mv = mask ? mask[static_cast<size_t>(i) * d.N + j] : 0.f;
        if (op != 1 && mv == -INFINITY) continue;                       // masked entries skipped for Sum / Min
        acc = combine(op, acc, d.alpha * dot_ab(A, B, d, b, i, j) + mv);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc = combine(op, acc, __shfl_xor_sync(0xffffffffu, acc, s));
    if (lane == 0) out[w] = acc;
}

__global__ void bmm_denom_kernel(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ row_max,
                                 const float* __restrict__ mask, float* __restrict__ out, BmmDims d)
{
    const int lane = threadIdx.x & 31;
    const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (w >= static_cast<long long>(d.batch) * d.M) return;
    const int b = static_cast<int>(w / d.M), i = static_cast<int>(w % d.M);
    const float mval = row_max[w];
    float acc = 0.f;
    for (int j = lane; j < d.N; j += 32) {
        const float mv = mask ? mask[static_cast<size_t>(i) * d.N + j] : 0.f;
        if (mv == -INFINITY) continue;
        acc += expf(d.alpha * dot_ab(A, B, d, b, i, j) + mv - mval);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[w] = acc;
}

// softmax weight of (i, j): exp(alpha*s + mask - m_i) / l_i, zero where the mask is -inf
__device__ __forceinline__ float weight_ij(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ mask,
                                           const BmmDims& d, int b, int i, int j, float mval, float inv_l)
{
    const float mv = mask ? mask[static_cast<size_t>(i) * d.N + j] : 0.f;
    if (mv == -INFINITY) return 0.f;
    return expf(d.alpha * dot_ab(A, B, d, b, i, j) + mv - mval) * inv_l;
}

constexpr int kChunk = 128;   // keys / queries whose weights a warp stages in shared memory at a time

// O[(b*M+i)*D + c] = sum_j W_ij V[(b*N+j)*D + c]
__global__ void __launch_bounds__(128)
bmm_apply_kernel(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ V,
                 const float* __restrict__ row_max, const float* __restrict__ denom, const float* __restrict__ mask,
                 float* __restrict__ out, BmmDims d, int D)
{
    __shared__ float sw[4][kChunk];
    const int lane = threadIdx.x & 31, wl = threadIdx.x >> 5;
    const long long w = static_cast<long long>(blockIdx.x) * 4 + wl;
    if (w >= static_cast<long long>(d.batch) * d.M) return;
    const int b = static_cast<int>(w / d.M), i = static_cast<int>(w % d.M);
    const float mval = row_max[w], inv_l = 1.0f / denom[w];
    for (int c0 = 0; c0 < D; c0 += 32 * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j0 = 0; j0 < d.N; j0 += kChunk) {
            __syncwarp();
            for (int t = lane; t < kChunk; t += 32) sw[wl][t] = (j0 + t < d.N) ? weight_ij(A, B, mask, d, b, i, j0 + t, mval, inv_l) : 0.f;
            __syncwarp();
            const int lim = min(kChunk, d.N - j0);
            for (int t = 0; t < lim; ++t) {
                const float wv = sw[wl][t];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int c = c0 + u * 32 + lane;
                    if (c < D) acc[u] += wv * V[(static_cast<size_t>(b) * d.N + j0 + t) * D + c];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = c0 + u * 32 + lane;
            if (c < D) out[static_cast<size_t>(w) * D + c] = acc[u];
        }
    }
}

// R_i = sum_j W_ij P_ij ; gradQ[(b*K+k)*M + i] = alpha * sum_j W_ij (P_ij - R_i) B_b(k, j)
__global__ void __launch_bounds__(128)
bmm_backward_q_kernel(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ P,
                      const float* __restrict__ row_max, const float* __restrict__ denom, const float* __restrict__ mask,
                      float* __restrict__ grad_q, float* __restrict__ r_out, BmmDims d)
{
    __shared__ float sw[4][kChunk];
    const int lane = threadIdx.x & 31, wl = threadIdx.x >> 5;
    const long long w = static_cast<long long>(blockIdx.x) * 4 + wl;
    if (w >= static_cast<long long>(d.batch) * d.M) return;
    const int b = static_cast<int>(w / d.M), i = static_cast<int>(w % d.M);
    const float mval = row_max[w], inv_l = 1.0f / denom[w];
    const float* prow = P + static_cast<size_t>(w) * d.N;
    float rv = 0.f;
    for (int j = lane; j < d.N; j += 32) rv += weight_ij(A, B, mask, d, b, i, j, mval, inv_l) * prow[j];
    rv = warp_sum(rv);
    if (lane == 0) r_out[w] = rv;
    for (int k0 = 0; k0 < d.K; k0 += 32 * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j0 = 0; j0 < d.N; j0 += kChunk) {
            __syncwarp();
            for (int t = lane; t < kChunk; t += 32)
                sw[wl][t] = (j0 + t < d.N) ? weight_ij(A, B, mask, d, b, i, j0 + t, mval, inv_l) * (prow[j0 + t] - rv) : 0.f;
            __syncwarp();
            const int lim = min(kChunk, d.N - j0);
            for (int t = 0; t < lim; ++t) {
                const float tv = sw[wl][t];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int k = k0 + u * 32 + lane;
                    if (k < d.K) acc[u] += tv * b_at(B, d, b, k, j0 + t);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int k = k0 + u * 32 + lane;
            if (k < d.K) grad_q[(static_cast<size_t>(b) * d.K + k) * d.M + i] = d.alpha * acc[u];
        }
    }
}

// gradK[(b*K+k)*N + j] = alpha * sum_i W_ij (P_ij - R_i) A_b(i, k) ; gradV[(b*K+k)*N + j] = sum_i W_ij G[(b*M+i)*D + k]
// (the reference sizes gradV by K and reads the first K columns of G, cpu_engine.hpp:870-908)
__global__ void __launch_bounds__(128)
bmm_backward_kv_kernel(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ P,
                       const float* __restrict__ G, const float* __restrict__ R, const float* __restrict__ row_max,
                       const float* __restrict__ denom, const float* __restrict__ mask, float* __restrict__ grad_k,
                       float* __restrict__ grad_v, BmmDims d, int D)
{
    __shared__ float sw[4][kChunk], st[4][kChunk];
    const int lane = threadIdx.x & 31, wl = threadIdx.x >> 5;
    const long long w = static_cast<long long>(blockIdx.x) * 4 + wl;
    if (w >= static_cast<long long>(d.batch) * d.N) return;
    const int b = static_cast<int>(w / d.N), j = static_cast<int>(w % d.N);
    for (int k0 = 0; k0 < d.K; k0 += 32 * 4) {
        float ak[4] = {0.f, 0.f, 0.f, 0.f}, av[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i0 = 0; i0 < d.M; i0 += kChunk) {
            __syncwarp();
            for (int t = lane; t < kChunk; t += 32) {
                float wv = 0.f, tv = 0.f;
                if (i0 + t < d.M) {
                    const size_t ri = static_cast<size_t>(b) * d.M + i0 + t;
                    wv = weight_ij(A, B, mask, d, b, i0 + t, j, row_max[ri], 1.0f / denom[ri]);
                    tv = wv * (P[ri * d.N + j] - R[ri]);
                }
                sw[wl][t] = wv; st[wl][t] = tv;
            }
            __syncwarp();
            const int lim = min(kChunk, d.M - i0);
            for (int t = 0; t < lim; ++t) {
                const float wv = sw[wl][t], tv = st[wl][t];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int k = k0 + u * 32 + lane;
                    if (k < d.K) {
                        ak[u] += tv * a_at(A, d, b, i0 + t, k);
                        av[u] += wv * G[(static_cast<size_t>(b) * d.M + i0 + t) * D + k];
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int k = k0 + u * 32 + lane;
            if (k < d.K) {
                grad_k[(static_cast<size_t>(b) * d.K + k) * d.N + j] = d.alpha * ak[u];
                grad_v[(static_cast<size_t>(b) * d.K + k) * d.N + j] = av[u];
            }
        }
    }
}

// ---------------------------------------------------------------- cross-entropy, (classes, tokens) layout
// a block owns 32 token columns; 8 row lanes walk the classes, so every access is a coalesced 128-byte row piece
__global__ void __launch_bounds__(256)
col_softmax_denom_kernel(const float* __restrict__ logits, const float* __restrict__ col_max, float* __restrict__ out, int C, int N)
{
    __shared__ float red[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5, n = blockIdx.x * 32 + tx;
    float acc = 0.f;
    if (n < N) { const float mx = col_max[n]; for (int r = ty; r < C; r += 8) acc += expf(logits[static_cast<size_t>(r) * N + n] - mx); }
    red[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && n < N) { for (int k = 1; k < 8; ++k) acc += red[k][tx]; out[n] = acc; }
}

__global__ void __launch_bounds__(256)
col_softmax_sparse_kernel(const float* __restrict__ logits, const float* __restrict__ labels, const float* __restrict__ mask,
                          float* __restrict__ grad, float* __restrict__ loss_vec, int C, int N, int vocab, float inv_nv)
{
    __shared__ float red[8][33];
    __shared__ float smax[32], sden[32];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5, n = blockIdx.x * 32 + tx;
    const bool in = n < N;
    const float lf = in ? labels[n] : 0.f;
    const long long lbl = lf >= 0.f ? static_cast<long long>(lf) : 0;
    const bool valid = in && (!mask || mask[n] >= 0.5f) && lbl < vocab;
    float mx = -INFINITY;
    if (valid) for (int r = ty; r < C; r += 8) mx = fmaxf(mx, logits[static_cast<size_t>(r) * N + n]);
    red[ty][tx] = mx;
    __syncthreads();
    if (ty == 0) { for (int k = 1; k < 8; ++k) mx = fmaxf(mx, red[k][tx]); smax[tx] = mx; }
    __syncthreads();
    mx = smax[tx];
    float den = 0.f;
    if (valid) for (int r = ty; r < C; r += 8) den += expf(logits[static_cast<size_t>(r) * N + n] - mx);
    __syncthreads();
    red[ty][tx] = den;
    __syncthreads();
    if (ty == 0) { for (int k = 1; k < 8; ++k) den += red[k][tx]; sden[tx] = den; }
    __syncthreads();
    den = sden[tx];
    if (in) {
        for (int r = ty; r < C; r += 8) {
            float g = 0.f;
            if (valid) { g = inv_nv * expf(logits[static_cast<size_t>(r) * N + n] - mx) / den; if (r == lbl) g -= inv_nv; }
            grad[static_cast<size_t>(r) * N + n] = g;
        }
        if (ty == 0) loss_vec[n] = valid ? logits[static_cast<size_t>(lbl) * N + n] - mx - logf(den) : 0.f;
    }
}

static int check_bmm(const BmmDims& d) { return (d.batch > 0 && d.M > 0 && d.N > 0 && d.K > 0) ? 0 : -1; }

}  // namespace nnb

using namespace nnb;

extern "C" {

int nnb200_batched_matmul(const float* A, const float* B, float* C, size_t A_rows, size_t A_cols, size_t B_rows, size_t B_cols,
                          unsigned int batch, int transA, int transB, float alpha, void* stream)
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
                              b_rpb * B_cols, M * N, alpha, nullptr, nullptr, nullptr, 0, to_stream(stream)));
    }
    return 0;
}

int nnb200_bmm_reduce(const float* A, const float* B, const float* mask, float* out, int batch, int M, int N, int K, int op,
                      int transA, int transB, float alpha, int reduce_cols, void* stream)
{
    const BmmDims d{batch, M, N, K, transA, transB, alpha};
    if (check_bmm(d) || op < 0 || op > 2) return -1;
    const long long warps = static_cast<long long>(batch) * (reduce_cols ? M : N);
    bmm_reduce_kernel<<<static_cast<unsigned>(ceil_div(warps * 32, 256)), 256, 0, to_stream(stream)>>>(A, B, mask, out, d, op, reduce_cols);
    NNB_LAUNCH_CHECK();
    return 0;
}

int nnb200_bmm_softmax_denom(const float* A, const float* B, const float* row_max, const float* mask, float* out, int batch,
                             int M, int N, int K, int transA, int transB, float alpha, void* stream)
{
    const BmmDims d{batch, M, N, K, transA, transB, alpha};
    if (check_bmm(d)) return -1;
    bmm_denom_kernel<<<static_cast<unsigned>(ceil_div(static_cast<long long>(batch) * M * 32, 256)), 256, 0, to_stream(stream)>>>(A, B, row_max, mask, out, d);
    NNB_LAUNCH_CHECK();
    return 0;
}

int nnb200_bmm_softmax_apply(const float* A, const float* B, const float* V, const float* row_max, const float* denom,
                             const float* mask, float* out, int batch, int M, int N, int K, int D, int transA, int transB,
                             float alpha, void* stream)
{
    const BmmDims d{batch, M, N, K, transA, transB, alpha};
    if (check_bmm(d) || D <= 0) return -1;
    bmm_apply_kernel<<<static_cast<unsigned>(ceil_div(static_cast<long long>(batch) * M, 4)), 128, 0, to_stream(stream)>>>(A, B, V, row_max, denom, mask, out, d, D);
    NNB_LAUNCH_CHECK();
    return 0;
}

int nnb200_bmm_softmax_backward_q(const float* A, const float* B, const float* P, const float* row_max, const float* denom,
                                  const float* mask, float* grad_q, float* r_out, int batch, int M, int N, int K, int transA,
                                  int transB, float alpha, void* stream)
{
    const BmmDims d{batch, M, N, K, transA, transB, alpha};
    if (check_bmm(d)) return -1;
    bmm_backward_q_kernel<<<static_cast<unsigned>(ceil_div(static_cast<long long>(batch) * M, 4)), 128, 0, to_stream(stream)>>>(A, B, P, row_max, denom, mask, grad_q, r_out, d);
    NNB_LAUNCH_CHECK();
    return 0;
}

int nnb200_bmm_softmax_backward_kv(const float* A, const float* B, const float* P, const float* G, const float* R,
                                   const float* row_max, const float* denom, const float* mask, float* grad_k, float* grad_v,
                                   int batch, int M, int N, int K, int D, int transA, int transB, float alpha, void* stream)
{
    const BmmDims d{batch, M, N, K, transA, transB, alpha};
    if (check_bmm(d) || D < K) return -1;
    bmm_backward_kv_kernel<<<static_cast<unsigned>(ceil_div(static_cast<long long>(batch) * N, 4)), 128, 0, to_stream(stream)>>>(A, B, P, G, R, row_max, denom, mask, grad_k, grad_v, d, D);
    NNB_LAUNCH_CHECK();
    return 0;
}

int nnb200_col_softmax_denom(const float* logits, const float* col_max, float* out, int classes, int tokens, void* stream)
{
    if (classes <= 0 || tokens <= 0) return -1;
    col_softmax_denom_kernel<<<static_cast<unsigned>(ceil_div(tokens, 32)), 256, 0, to_stream(stream)>>>(logits, col_max, out, classes, tokens);
    NNB_LAUNCH_CHECK();
    return 0;
}

int nnb200_col_softmax_sparse_forward(const float* logits, const float* labels, const float* mask, float* grad, float* loss_vec,
                                      int classes, int tokens, int vocab_size, float inv_num_valid, void* stream)
{
    if (classes <= 0 || tokens <= 0) return -1;
    if (vocab_size > classes) { fprintf(stderr, "nnb200_col_softmax_sparse_forward: vocab_size > classes\n"); return -1; }
    col_softmax_sparse_kernel<<<static_cast<unsigned>(ceil_div(tokens, 32)), 256, 0, to_stream(stream)>>>(logits, labels, mask, grad, loss_vec, classes, tokens, vocab_size, inv_num_valid);
    NNB_LAUNCH_CHECK();
    return 0;
}

}  // extern "C"
