// Fused causal / document-masked / ALiBi attention, SIMT fp32-accumulate version.
//
// This is the check-mode path (fp32 in, fp32 math) and the path for head sizes the tensor-core
// kernel does not tile.  It computes exactly what AttentionBase::forward/backward compute
// (compute_layer.hpp:1133-1412) with the mask of build_attention_mask (:2081-2128):
//   s_ij = q_i.k_j / sqrt(dk) - slope_h*(i-j)   where j <= i and doc_i == doc_j, else -inf
//   O_i = sum_j softmax_j(s_ij) v_j
// without materialising the (B*H*S, S) score, mask and probability matrices.
// Layout: qkv is (tokens, 3*d) row-major, q | k | v side by side, head h at columns h*dk.. of each;
// out / dout are (tokens, d); lse and dvec are (B*H*S) with index (b*H + h)*S + i.
#include "kernels.h"

namespace nnb {

__device__ __forceinline__ float alibi_slope(int h, int H)
{
    // m_h = 2^(-8h/H), h from 0 (compute_layer.hpp:2179-2187)
    return powf(2.0f, -8.0f * static_cast<float>(h) / static_cast<float>(H));
}

template <typename T, int DK>
__global__ void __launch_bounds__(128)
attn_fwd_simt_kernel(const T* __restrict__ qkv, T* __restrict__ out, float* __restrict__ lse,
                     const int* __restrict__ doc, int B, int S, int H, int alibi, float scale)
{
    __shared__ float qs[4][DK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = static_cast<long long>(blockIdx.x) * 4 + warp;      // (b*H + h)*S + i
    if (row >= static_cast<long long>(B) * H * S) return;
    const int i = static_cast<int>(row % S), h = static_cast<int>((row / S) % H), b = static_cast<int>(row / S / H);
    const int d = H * DK, ld = 3 * d;
    const T* qp = qkv + (static_cast<size_t>(b) * S + i) * ld + h * DK;
    for (int c = lane; c < DK; c += 32) qs[warp][c] = to_f32(qp[c]);
    __syncwarp();
    const float slope = alibi ? alibi_slope(h, H) : 0.f;
    const int my_doc = doc ? doc[b * S + i] : 0;
    const T* kbase = qkv + static_cast<size_t>(b) * S * ld + d + h * DK;
    const T* vbase = kbase + d;
    float m = -INFINITY;
    for (int j = lane; j <= i; j += 32) {
        if (doc && doc[b * S + j] != my_doc) continue;
        const T* kp = kbase + static_cast<size_t>(j) * ld;
        float s = 0.f;
#pragma unroll 8
        for (int c = 0; c < DK; ++c) s += qs[warp][c] * to_f32(kp[c]);
        s = scale * s - slope * static_cast<float>(i - j);
        m = fmaxf(m, s);
    }
    m = warp_max(m);
    float l = 0.f, o[DK];
#pragma unroll
    for (int c = 0; c < DK; ++c) o[c] = 0.f;
    for (int j = lane; j <= i; j += 32) {
        if (doc && doc[b * S + j] != my_doc) continue;
        const T* kp = kbase + static_cast<size_t>(j) * ld;
        const T* vp = vbase + static_cast<size_t>(j) * ld;
        float s = 0.f;
#pragma unroll 8
        for (int c = 0; c < DK; ++c) s += qs[warp][c] * to_f32(kp[c]);
        s = scale * s - slope * static_cast<float>(i - j);
        const float p = expf(s - m);
        l += p;
#pragma unroll
        for (int c = 0; c < DK; ++c) o[c] += p * to_f32(vp[c]);
    }
    l = warp_sum(l);
    const float inv_l = 1.0f / l;
    T* op = out + (static_cast<size_t>(b) * S + i) * d + h * DK;
#pragma unroll
    for (int c = 0; c < DK; ++c) {
        const float v = warp_sum(o[c]);
        if (lane == (c & 31)) op[c] = from_f32<T>(v * inv_l);
    }
    if (lane == 0) lse[row] = m + logf(l);
}

// dvec[row] = sum_c dout[i][h*dk+c] * out[i][h*dk+c]  (= R_i = sum_j W_ij P_ij of the reference's
// backward_q primitive, cpu_engine.hpp:767-783)
template <typename T>
__global__ void attn_dvec_kernel(const T* __restrict__ out, const T* __restrict__ dout, float* __restrict__ dvec,
                                 int B, int S, int H, int dk)
{
    const int lane = threadIdx.x & 31;
    const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (row >= static_cast<long long>(B) * H * S) return;
    const int i = static_cast<int>(row % S), h = static_cast<int>((row / S) % H), b = static_cast<int>(row / S / H);
    const size_t off = (static_cast<size_t>(b) * S + i) * (H * dk) + h * dk;
    float s = 0.f;
    for (int c = lane; c < dk; c += 32) s += to_f32(out[off + c]) * to_f32(dout[off + c]);
    s = warp_sum(s);
    if (lane == 0) dvec[row] = s;
}

// Vectorised variant: a warp walks a whole token row (all heads) with 16-byte loads; the lanes that
// share a head fold their partial dot products with shuffles.  Needs dk a multiple of the vector
// width with dk/width a power of two <= 32.
template <typename T>
__global__ void __launch_bounds__(256)
attn_dvec_vec_kernel(const T* __restrict__ out, const T* __restrict__ dout, float* __restrict__ dvec, int B, int S,
                     int H, int dk)
{
    constexpr int VN = Vec16<T>::N;
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int d = H * dk, nvec = d / VN, L = dk / VN;
    const int nvec_pad = (nvec + 31) & ~31;
    const long long ntok = static_cast<long long>(B) * S;
    for (long long t = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); t < ntok; t += static_cast<long long>(gridDim.x) * wpb) {
        const int b = static_cast<int>(t / S), i = static_cast<int>(t % S);
        for (int v = lane; v < nvec_pad; v += 32) {
            float sacc = 0.f;
            if (v < nvec) {
                const Vec16<T> ov = ld16(out + t * d + v * VN), gv = ld16(dout + t * d + v * VN);
#pragma unroll
                for (int k = 0; k < VN; ++k) sacc += to_f32(ov.v[k]) * to_f32(gv.v[k]);
            }
            for (int off = L >> 1; off > 0; off >>= 1) sacc += __shfl_xor_sync(0xffffffffu, sacc, off);
            if (v < nvec && (lane & (L - 1)) == 0) dvec[(static_cast<size_t>(b) * H + v / L) * S + i] = sacc;
        }
    }
}

template <typename T>
static int launch_dvec(const T* out, const T* dout, float* dvec, int B, int S, int H, int dk, cudaStream_t s)
{
    constexpr int VN = Vec16<T>::N;
    const long long rows = static_cast<long long>(B) * H * S;
    const int L = dk / VN;
    const bool vec = (dk % VN) == 0 && L >= 1 && L <= 32 && (L & (L - 1)) == 0 &&
                     ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(dout)) & 15) == 0;
    if (vec) attn_dvec_vec_kernel<T><<<grid_for(static_cast<long long>(B) * S, 8), 256, 0, s>>>(out, dout, dvec, B, S, H, dk);
    else attn_dvec_kernel<T><<<static_cast<unsigned>(ceil_div(rows * 32, 256)), 256, 0, s>>>(out, dout, dvec, B, S, H, dk);
    NNB_LAUNCH_CHECK();
    return 0;
}

// dQ: one warp per query row, lanes over keys
template <typename T, int DK>
__global__ void __launch_bounds__(128)
attn_bwd_dq_simt_kernel(const T* __restrict__ qkv, const T* __restrict__ dout, const float* __restrict__ lse,
                        const float* __restrict__ dvec, T* __restrict__ dqkv, const int* __restrict__ doc, int B, int S,
                        int H, int alibi, float scale)
{
    __shared__ float qs[4][DK], gs[4][DK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = static_cast<long long>(blockIdx.x) * 4 + warp;
    if (row >= static_cast<long long>(B) * H * S) return;
    const int i = static_cast<int>(row % S), h = static_cast<int>((row / S) % H), b = static_cast<int>(row / S / H);
    const int d = H * DK, ld = 3 * d;
    const T* qp = qkv + (static_cast<size_t>(b) * S + i) * ld + h * DK;
    const T* gp = dout + (static_cast<size_t>(b) * S + i) * d + h * DK;
    for (int c = lane; c < DK; c += 32) { qs[warp][c] = to_f32(qp[c]); gs[warp][c] = to_f32(gp[c]); }
    __syncwarp();
    const float slope = alibi ? alibi_slope(h, H) : 0.f;
    const int my_doc = doc ? doc[b * S + i] : 0;
    const float L = lse[row], Dv = dvec[row];
    const T* kbase = qkv + static_cast<size_t>(b) * S * ld + d + h * DK;
    const T* vbase = kbase + d;
    float dq[DK];
#pragma unroll
    for (int c = 0; c < DK; ++c) dq[c] = 0.f;
    for (int j = lane; j <= i; j += 32) {
        if (doc && doc[b * S + j] != my_doc) continue;
        const T* kp = kbase + static_cast<size_t>(j) * ld;
        const T* vp = vbase + static_cast<size_t>(j) * ld;
        float s = 0.f, dp = 0.f;
#pragma unroll 8
        for (int c = 0; c < DK; ++c) { s += qs[warp][c] * to_f32(kp[c]); dp += gs[warp][c] * to_f32(vp[c]); }
        s = scale * s - slope * static_cast<float>(i - j);
        const float ds = expf(s - L) * (dp - Dv);
#pragma unroll
        for (int c = 0; c < DK; ++c) dq[c] += ds * to_f32(kp[c]);
    }
    T* dqp = dqkv + (static_cast<size_t>(b) * S + i) * ld + h * DK;
#pragma unroll
    for (int c = 0; c < DK; ++c) {
        const float v = warp_sum(dq[c]);
        if (lane == (c & 31)) dqp[c] = from_f32<T>(scale * v);
    }
}

// dK, dV: one warp per key row, lanes over the queries that see it
template <typename T, int DK>
__global__ void __launch_bounds__(128)
attn_bwd_dkv_simt_kernel(const T* __restrict__ qkv, const T* __restrict__ dout, const float* __restrict__ lse,
                         const float* __restrict__ dvec, T* __restrict__ dqkv, const int* __restrict__ doc, int B, int S,
                         int H, int alibi, float scale)
{
    __shared__ float ks[4][DK], vs[4][DK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = static_cast<long long>(blockIdx.x) * 4 + warp;
    if (row >= static_cast<long long>(B) * H * S) return;
    const int j = static_cast<int>(row % S), h = static_cast<int>((row / S) % H), b = static_cast<int>(row / S / H);
    const int d = H * DK, ld = 3 * d;
    const T* kp = qkv + (static_cast<size_t>(b) * S + j) * ld + d + h * DK;
    for (int c = lane; c < DK; c += 32) { ks[warp][c] = to_f32(kp[c]); vs[warp][c] = to_f32(kp[d + c]); }
    __syncwarp();
    const float slope = alibi ? alibi_slope(h, H) : 0.f;
    const int my_doc = doc ? doc[b * S + j] : 0;
    const long long row0 = (static_cast<long long>(b) * H + h) * S;
    float dk[DK], dv[DK];
#pragma unroll
    for (int c = 0; c < DK; ++c) { dk[c] = 0.f; dv[c] = 0.f; }
    for (int i = j + lane; i < S; i += 32) {
        if (doc && doc[b * S + i] != my_doc) continue;
        const T* qp = qkv + (static_cast<size_t>(b) * S + i) * ld + h * DK;
        const T* gp = dout + (static_cast<size_t>(b) * S + i) * d + h * DK;
        float s = 0.f, dp = 0.f;
#pragma unroll 8
        for (int c = 0; c < DK; ++c) { s += to_f32(qp[c]) * ks[warp][c]; dp += to_f32(gp[c]) * vs[warp][c]; }
        s = scale * s - slope * static_cast<float>(i - j);
        const float p = expf(s - lse[row0 + i]);
        const float ds = p * (dp - dvec[row0 + i]);
#pragma unroll
        for (int c = 0; c < DK; ++c) { dk[c] += ds * to_f32(qp[c]); dv[c] += p * to_f32(gp[c]); }
    }
    T* dkp = dqkv + (static_cast<size_t>(b) * S + j) * ld + d + h * DK;
#pragma unroll
    for (int c = 0; c < DK; ++c) {
        const float a = warp_sum(dk[c]), bsum = warp_sum(dv[c]);
        if (lane == (c & 31)) { dkp[c] = from_f32<T>(scale * a); dkp[d + c] = from_f32<T>(bsum); }
    }
}

template <typename T, int DK>
static int fwd_dk(const T* qkv, T* out, float* lse, const int* doc, int B, int S, int H, int alibi, cudaStream_t s)
{
    const long long rows = static_cast<long long>(B) * H * S;
    attn_fwd_simt_kernel<T, DK><<<static_cast<unsigned>(ceil_div(rows, 4)), 128, 0, s>>>(
        qkv, out, lse, doc, B, S, H, alibi, 1.0f / sqrtf(static_cast<float>(DK)));
    NNB_LAUNCH_CHECK();
    return 0;
}
template <typename T, int DK>
static int bwd_dk(const T* qkv, const T* out, const T* dout, const float* lse, float* dvec, T* dqkv, const int* doc,
                  int B, int S, int H, int alibi, cudaStream_t s)
{
    const long long rows = static_cast<long long>(B) * H * S;
    const float scale = 1.0f / sqrtf(static_cast<float>(DK));
    NNB_TRY(launch_dvec<T>(out, dout, dvec, B, S, H, DK, s));
    const unsigned grid = static_cast<unsigned>(ceil_div(rows, 4));
    attn_bwd_dq_simt_kernel<T, DK><<<grid, 128, 0, s>>>(qkv, dout, lse, dvec, dqkv, doc, B, S, H, alibi, scale);
    NNB_LAUNCH_CHECK();
    attn_bwd_dkv_simt_kernel<T, DK><<<grid, 128, 0, s>>>(qkv, dout, lse, dvec, dqkv, doc, B, S, H, alibi, scale);
    NNB_LAUNCH_CHECK();
    return 0;
}

#define DISPATCH_DK(dk, CALL)                                                         \
    switch (dk) {                                                                     \
        case 8: { constexpr int DKC = 8; return CALL; }                               \
        case 16: { constexpr int DKC = 16; return CALL; }                             \
        case 32: { constexpr int DKC = 32; return CALL; }                             \
        case 64: { constexpr int DKC = 64; return CALL; }                             \
        case 128: { constexpr int DKC = 128; return CALL; }                           \
        default: fprintf(stderr, "nnb200: attention head size %d unsupported (8,16,32,64,128)\n", dk); return -1; \
    }

template <typename T>
int attention_fwd_simt(const T* qkv, T* out, float* lse, const int* doc, int B, int S, int H, int dk, int alibi,
                       cudaStream_t s)
{
    if (static_cast<long long>(B) * S * H == 0) return 0;
    DISPATCH_DK(dk, (fwd_dk<T, DKC>(qkv, out, lse, doc, B, S, H, alibi, s)));
}
template <typename T>
int attention_bwd_simt(const T* qkv, const T* out, const T* dout, const float* lse, float* dvec, T* dqkv,
                       const int* doc, int B, int S, int H, int dk, int alibi, cudaStream_t s)
{
    if (static_cast<long long>(B) * S * H == 0) return 0;
    DISPATCH_DK(dk, (bwd_dk<T, DKC>(qkv, out, dout, lse, dvec, dqkv, doc, B, S, H, alibi, s)));
}

int attention_dvec_bf16(const bf16* out, const bf16* dout, float* dvec, int B, int S, int H, int dk, cudaStream_t s)
{
    return launch_dvec<bf16>(out, dout, dvec, B, S, H, dk, s);
}

template int attention_fwd_simt<float>(const float*, float*, float*, const int*, int, int, int, int, int, cudaStream_t);
template int attention_fwd_simt<bf16>(const bf16*, bf16*, float*, const int*, int, int, int, int, int, cudaStream_t);
template int attention_bwd_simt<float>(const float*, const float*, const float*, const float*, float*, float*,
                                       const int*, int, int, int, int, int, cudaStream_t);
template int attention_bwd_simt<bf16>(const bf16*, const bf16*, const bf16*, const float*, float*, bf16*, const int*,
                                      int, int, int, int, int, cudaStream_t);

}  // namespace nnb
