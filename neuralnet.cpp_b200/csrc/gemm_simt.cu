// fp32 SIMT GEMM with arbitrary strides: the check-mode contraction (fp32 in, fp32 accumulate in
// ascending k) behind cuda_matmul / cuda_batched_matmul and the fp32 mode of the training step.
// It is deliberately simple; the fast path is the tcgen05 kernel in gemm_tcgen05.cu.
#include "kernels.h"

namespace nnb {

constexpr int ST_BM = 64, ST_BN = 64, ST_BK = 16;

// C[b][m*ldc + n] = alpha * sum_k A[b][m*sam + k*sak] * B[b][n*sbn + k*sbk]
//                   (+ bias_n[n]) (+ bias_m[m]) (+ residual[b][m*ldc + n]) (+ C if accumulate)
__global__ void __launch_bounds__(256)
sgemm_strided_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                     int M, int N, int K, long long sam, long long sak, long long sbn, long long sbk, long long ldc,
                     long long batch_a, long long batch_b, long long batch_c,
                     float alpha, const float* __restrict__ bias_n, const float* __restrict__ bias_m,
                     const float* __restrict__ residual, int accumulate)
{
    __shared__ float As[ST_BK][ST_BM + 4];
    __shared__ float Bs[ST_BK][ST_BN + 4];
    const int b = blockIdx.z;
    A += static_cast<long long>(b) * batch_a;
    B += static_cast<long long>(b) * batch_b;
    C += static_cast<long long>(b) * batch_c;
    if (residual) residual += static_cast<long long>(b) * batch_c;
    const int m0 = blockIdx.y * ST_BM, n0 = blockIdx.x * ST_BN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += ST_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            int mm, kk;
            if (sak == 1) { mm = e >> 4; kk = e & 15; } else { mm = e & 63; kk = e >> 6; }
            const int gm = m0 + mm, gk = k0 + kk;
            As[kk][mm] = (gm < M && gk < K) ? A[gm * sam + gk * sak] : 0.f;
            int nn;
            if (sbk == 1) { nn = e >> 4; kk = e & 15; } else { nn = e & 63; kk = e >> 6; }
            const int gn = n0 + nn, gk2 = k0 + kk;
            Bs[kk][nn] = (gn < N && gk2 < K) ? B[gn * sbn + gk2 * sbk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < ST_BK; ++kk) {
            float a[4], bb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; bb[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = alpha * acc[i][j];
            if (bias_n) v += bias_n[gn];
            if (bias_m) v += bias_m[gm];
            const long long o = gm * ldc + gn;
            if (residual) v += residual[o];
            if (accumulate) v += C[o];
            C[o] = v;
        }
    }
}

int sgemm_strided(const float* A, const float* B, float* C, int M, int N, int K,
                  long long sam, long long sak, long long sbn, long long sbk, long long ldc,
                  int batch, long long batch_a, long long batch_b, long long batch_c,
                  float alpha, const float* bias_n, const float* bias_m, const float* residual,
                  int accumulate, cudaStream_t stream)
{
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    NNB_ARG_CHECK(batch <= 65535, "batch too large for one launch");
    dim3 grid(static_cast<unsigned>(ceil_div(N, ST_BN)), static_cast<unsigned>(ceil_div(M, ST_BM)), batch);
    NNB_ARG_CHECK(grid.y <= 65535, "M too large for one launch");
    sgemm_strided_kernel<<<grid, 256, 0, stream>>>(A, B, C, M, N, K, sam, sak, sbn, sbk, ldc, batch_a, batch_b,
                                                   batch_c, alpha, bias_n, bias_m, residual, accumulate);
    NNB_LAUNCH_CHECK();
    return 0;
}

}  // namespace nnb

extern "C" int nnb200_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major,
                               float alpha, const float* bias_n, const float* residual, int accumulate,
                               void* stream)
{
    // A is (M,K) with K contiguous (a_mn_major=0) or stored (K,M) with M contiguous (1);
    // B is (N,K) with K contiguous (b_mn_major=0) or stored (K,N) with N contiguous (1).
    return nnb::sgemm_strided(A, B, C, M, N, K, a_mn_major ? 1 : lda, a_mn_major ? lda : 1,
                              b_mn_major ? 1 : ldb, b_mn_major ? ldb : 1, ldc, 1, 0, 0, 0, alpha, bias_n,
                              nullptr, residual, accumulate, nnb::to_stream(stream));
}
