// Memory-bound kernels of the fused GPT training step, token-major layout: every activation is a
// row-major (tokens, features) matrix, row i = b*seq + t.  Each kernel is templated on the
// activation type (float = fp32 check mode, bf16 = tensor-core mode); statistics, reductions and
// parameter gradients are always fp32.  They restate, fused, what the reference composes from
// engine primitives:
//   RMSNorm / LayerNorm      compute_layer.hpp:541-654, 722-800
//   QuickGeLU / SwiGLU       compute_layer.hpp:256-339, 360-458
//   softmax cross-entropy    compute_loss.hpp:229-309 + cpu_engine.hpp:948-1006
//   AdamW / clip / Muon      compute_optimizer.hpp:90-140, 252-304, 388-412, 517-590
#include "kernels.h"
#include "tc_ptx.cuh"

namespace nnb {

constexpr float kNormEps = 1e-5f;     // compute_layer.hpp:495,687
constexpr float kGeluBeta = 1.702f;   // compute_layer.hpp:259

__device__ __forceinline__ float sigmoidf_ref(float x) { return 1.0f / (1.0f + expf(-x)); }
// bf16 mode rounds every activation to 8 mantissa bits anyway: use the fast exp / reciprocal there
template <typename T> __device__ __forceinline__ float sigmoid_t(float x)
{
    if constexpr (sizeof(T) == 2) return sigmoid_fast(x);
    else return sigmoidf_ref(x);
}
template <typename T> __device__ __forceinline__ float exp_t(float x)
{
    if constexpr (sizeof(T) == 2) return __expf(x);
    else return expf(x);
}
// N consecutive floats (N a multiple of 4, p 16-byte aligned) with 16-byte loads: a per-lane slice of a parameter vector
template <int N> __device__ __forceinline__ void ld_f32x(const float* __restrict__ p, float* out)
{
#pragma unroll
    for (int k = 0; k < N; k += 4) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(p + k));
        out[k] = t.x; out[k + 1] = t.y; out[k + 2] = t.z; out[k + 3] = t.w;
    }
}

// the same from shared (or any generic) memory: ld_f32x reads through the read-only global path and must not be given
// a shared-memory address
template <int N> __device__ __forceinline__ void ld_f32x_generic(const float* p, float* out)
{
#pragma unroll
    for (int k = 0; k < N; k += 4) {
        const float4 t = *reinterpret_cast<const float4*>(p + k);
        out[k] = t.x; out[k + 1] = t.y; out[k + 2] = t.z; out[k + 3] = t.w;
    }
}
// tells the compiler that a 16-byte register vector may have changed: values derived from it before are not kept alive
// across this point (a row held packed is converted again in a second pass instead of being kept twice)
template <typename V> __device__ __forceinline__ void forget_derived(V& v)
{
    static_assert(sizeof(V) == 16, "16-byte vectors only");
    uint4& w = reinterpret_cast<uint4&>(v);
    asm volatile("" : "+r"(w.x), "+r"(w.y), "+r"(w.z), "+r"(w.w));
}

// ======================================================================================
// normalisation: one warp per token row
// ======================================================================================
template <typename T, bool LAYER>
__global__ void __launch_bounds__(256)
norm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                T* __restrict__ y, float* __restrict__ rinv_out, float* __restrict__ mean_out, int rows, int d)
{
    constexpr int VN = Vec16<T>::N;
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const bool vec = (d % VN) == 0;
    const float inv_d = 1.0f / static_cast<float>(d);
    for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
        const T* xr = x + static_cast<size_t>(r) * d;
        T* yr = y + static_cast<size_t>(r) * d;
        float mean = 0.f;
        if (LAYER) {
            float s = 0.f;
            if (vec) for (int c = lane * VN; c < d; c += 32 * VN) { auto v = ld16(xr + c);
#pragma unroll
                for (int k = 0; k < VN; ++k) s += to_f32(v.v[k]); }
            else for (int c = lane; c < d; c += 32) s += to_f32(xr[c]);
            mean = warp_sum(s) * inv_d;
        }
        float ss = 0.f;
        if (vec) for (int c = lane * VN; c < d; c += 32 * VN) { auto v = ld16(xr + c);
#pragma unroll
            for (int k = 0; k < VN; ++k) { const float t = to_f32(v.v[k]) - mean; ss += t * t; } }
        else for (int c = lane; c < d; c += 32) { const float t = to_f32(xr[c]) - mean; ss += t * t; }
        const float rinv = 1.0f / sqrtf(warp_sum(ss) * inv_d + kNormEps);
        if (lane == 0) { rinv_out[r] = rinv; if (LAYER) mean_out[r] = mean; }
        if (vec) for (int c = lane * VN; c < d; c += 32 * VN) {
            auto v = ld16(xr + c); Vec16<T> o;
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                float n = (to_f32(v.v[k]) - mean) * rinv;
                n = n * gamma[c + k];
                if (LAYER) n += beta[c + k];
                o.v[k] = from_f32<T>(n);
            }
            st16(yr + c, o);
        } else for (int c = lane; c < d; c += 32) {
            float n = (to_f32(xr[c]) - mean) * rinv * gamma[c];
            if (LAYER) n += beta[c];
            yr[c] = from_f32<T>(n);
        }
    }
}

// dx = norm-backward(g) [+ add]; `add` is the gradient arriving over the residual connection
template <typename T, bool LAYER>
__global__ void __launch_bounds__(256)
norm_bwd_dx_kernel(const T* __restrict__ g, const T* __restrict__ x, const float* __restrict__ gamma,
                   const float* __restrict__ rinv_in, const float* __restrict__ mean_in, const T* __restrict__ add,
                   T* __restrict__ dx, int rows, int d)
{
    constexpr int VN = Vec16<T>::N;
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const bool vec = (d % VN) == 0;
    const float inv_d = 1.0f / static_cast<float>(d);
    for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
        const size_t off = static_cast<size_t>(r) * d;
        const float rinv = rinv_in[r], mean = LAYER ? mean_in[r] : 0.f;
        float s_g = 0.f, s_gn = 0.f;
        if (vec) for (int c = lane * VN; c < d; c += 32 * VN) {
            auto gv = ld16(g + off + c); auto xv = ld16(x + off + c);
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                const float gg = to_f32(gv.v[k]) * gamma[c + k];
                const float n = (to_f32(xv.v[k]) - mean) * rinv;
                s_g += gg; s_gn += gg * n;
            }
        } else for (int c = lane; c < d; c += 32) {
            const float gg = to_f32(g[off + c]) * gamma[c];
            const float n = (to_f32(x[off + c]) - mean) * rinv;
            s_g += gg; s_gn += gg * n;
        }
        const float m_gn = warp_sum(s_gn) * inv_d;
        const float m_g = LAYER ? warp_sum(s_g) * inv_d : 0.f;
        if (vec) for (int c = lane * VN; c < d; c += 32 * VN) {
            auto gv = ld16(g + off + c); auto xv = ld16(x + off + c); Vec16<T> o, av;
            if (add) av = ld16(add + off + c);
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                const float gg = to_f32(gv.v[k]) * gamma[c + k];
                const float n = (to_f32(xv.v[k]) - mean) * rinv;
                float v = (gg - m_g - n * m_gn) * rinv;
                if (add) v += to_f32(av.v[k]);
                o.v[k] = from_f32<T>(v);
            }
            st16(dx + off + c, o);
        } else for (int c = lane; c < d; c += 32) {
            const float gg = to_f32(g[off + c]) * gamma[c];
            const float n = (to_f32(x[off + c]) - mean) * rinv;
            float v = (gg - m_g - n * m_gn) * rinv;
            if (add) v += to_f32(add[off + c]);
            dx[off + c] = from_f32<T>(v);
        }
    }
}

// Register-resident variants for d == 32 * NV * (elements per 16 bytes): a lane keeps its NV vectors of
// the row and of gamma/beta in registers, so every activation is read once and the parameters once per warp.
template <typename T, bool LAYER, int NV>
__global__ void __launch_bounds__(256, 3)
norm_fwd_reg_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                    T* __restrict__ y, float* __restrict__ rinv_out, float* __restrict__ mean_out, int rows)
{
    constexpr int VN = Vec16<T>::N, D = 32 * NV * VN;
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    // the first row is requested before the parameters, and every next row before the current one is reduced
    const int stride = gridDim.x * wpb;
    int r = blockIdx.x * wpb + (threadIdx.x >> 5);
    Vec16<T> nx[NV];
    if (r < rows) {
#pragma unroll
        for (int v = 0; v < NV; ++v) nx[v] = ld16(x + static_cast<size_t>(r) * D + (v * 32 + lane) * VN);
    }
    float gm[NV][VN], bt[NV][VN];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        ld_f32x<VN>(gamma + (v * 32 + lane) * VN, gm[v]);
        if (LAYER) ld_f32x<VN>(beta + (v * 32 + lane) * VN, bt[v]);
    }
    const float inv_d = 1.0f / static_cast<float>(D);
    for (; r < rows; r += stride) {
        float xv[NV][VN];
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
            for (int k = 0; k < VN; ++k) xv[v][k] = to_f32(nx[v].v[k]);
        if (r + stride < rows) {
#pragma unroll
            for (int v = 0; v < NV; ++v) nx[v] = ld16(x + static_cast<size_t>(r + stride) * D + (v * 32 + lane) * VN);
        }
        float mean = 0.f;
        if (LAYER) {
            float sm = 0.f;
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
                for (int k = 0; k < VN; ++k) sm += xv[v][k];
            mean = warp_sum(sm) * inv_d;
        }
        float ss = 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
            for (int k = 0; k < VN; ++k) { const float t = xv[v][k] - mean; ss += t * t; }
        const float rinv = 1.0f / sqrtf(warp_sum(ss) * inv_d + kNormEps);
        if (lane == 0) { rinv_out[r] = rinv; if (LAYER) mean_out[r] = mean; }
        T* yr = y + static_cast<size_t>(r) * D;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            Vec16<T> o;
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                float n = (xv[v][k] - mean) * rinv * gm[v][k];
                if (LAYER) n += bt[v][k];
                o.v[k] = from_f32<T>(n);
            }
            st16(yr + (v * 32 + lane) * VN, o);
        }
    }
}

// Wide rows (d = 32 * NV * elements per 16 bytes, NV up to 16: 4096 bf16 columns): a warp per row with the row held in
// registers as fp32, all its loads in flight at once, and the parameters in shared memory; every activation is read
// once.  Blocks of four warps, three per SM: twelve rows (96 KB at 4096 bf16 columns) in flight per SM.
template <typename T, bool LAYER, int NV>
__global__ void __launch_bounds__(128, 3)
norm_fwd_wide_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                     T* __restrict__ y, float* __restrict__ rinv_out, float* __restrict__ mean_out, int rows)
{
    constexpr int VN = Vec16<T>::N, D = 32 * NV * VN;
    extern __shared__ __align__(16) float norm_params[];            // gamma[D], then beta[D] for LayerNorm
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int stride = gridDim.x * wpb;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { norm_params[i] = gamma[i]; if (LAYER) norm_params[D + i] = beta[i]; }
    __syncthreads();
    const float inv_d = 1.0f / static_cast<float>(D);
    for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += stride) {
        float xv[NV][VN];
        {
            Vec16<T> xr[NV];
#pragma unroll
            for (int v = 0; v < NV; ++v) xr[v] = ld16(x + static_cast<size_t>(r) * D + (v * 32 + lane) * VN);
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
                for (int k = 0; k < VN; ++k) xv[v][k] = to_f32(xr[v].v[k]);
        }
        float mean = 0.f;
        if (LAYER) {
            float sm = 0.f;
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
                for (int k = 0; k < VN; ++k) sm += xv[v][k];
            mean = warp_sum(sm) * inv_d;
        }
        float ss = 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
            for (int k = 0; k < VN; ++k) { const float t = xv[v][k] - mean; ss += t * t; }
        const float rinv = 1.0f / sqrtf(warp_sum(ss) * inv_d + kNormEps);
        if (lane == 0) { rinv_out[r] = rinv; if (LAYER) mean_out[r] = mean; }
        T* yr = y + static_cast<size_t>(r) * D;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            float gm[VN], bt[VN];
            ld_f32x_generic<VN>(norm_params + (v * 32 + lane) * VN, gm);
            if (LAYER) ld_f32x_generic<VN>(norm_params + D + (v * 32 + lane) * VN, bt);
            Vec16<T> o;
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                float n = (xv[v][k] - mean) * rinv * gm[k];
                if (LAYER) n += bt[k];
                o.v[k] = from_f32<T>(n);
            }
            st16(yr + (v * 32 + lane) * VN, o);
        }
    }
}

template <typename T, bool LAYER, int NV>
__global__ void __launch_bounds__(256)
norm_bwd_dx_reg_kernel(const T* __restrict__ g, const T* __restrict__ x, const float* __restrict__ gamma,
                       const float* __restrict__ rinv_in, const float* __restrict__ mean_in, const T* __restrict__ add,
                       T* __restrict__ dx, int rows)
{
    constexpr int VN = Vec16<T>::N, D = 32 * NV * VN;
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    float gm[NV][VN];
#pragma unroll
    for (int v = 0; v < NV; ++v) ld_f32x<VN>(gamma + (v * 32 + lane) * VN, gm[v]);
    const float inv_d = 1.0f / static_cast<float>(D);
    for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
        const size_t off = static_cast<size_t>(r) * D;
        const float rinv = rinv_in[r], mean = LAYER ? mean_in[r] : 0.f;
        float gg[NV][VN], nn[NV][VN];
        float s_g = 0.f, s_gn = 0.f;
        Vec16<T> av[NV];
        if (add) {
#pragma unroll
            for (int v = 0; v < NV; ++v) av[v] = ld16(add + off + (v * 32 + lane) * VN);
        }
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const Vec16<T> gv = ld16(g + off + (v * 32 + lane) * VN), xv = ld16(x + off + (v * 32 + lane) * VN);
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                gg[v][k] = to_f32(gv.v[k]) * gm[v][k];
                nn[v][k] = (to_f32(xv.v[k]) - mean) * rinv;
                s_g += gg[v][k]; s_gn += gg[v][k] * nn[v][k];
            }
        }
        const float m_gn = warp_sum(s_gn) * inv_d;
        const float m_g = LAYER ? warp_sum(s_g) * inv_d : 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            Vec16<T> o;
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                float t = (gg[v][k] - m_g - nn[v][k] * m_gn) * rinv;
                if (add) t += to_f32(av[v].v[k]);
                o.v[k] = from_f32<T>(t);
            }
            st16(dx + off + (v * 32 + lane) * VN, o);
        }
    }
}

// The same for wide rows (NV up to 16: 4096 bf16 columns): g and x stay in registers as loaded (packed) and are
// converted once for the two row sums and once for the output; gamma comes from shared memory.  Blocks of four warps,
// two per SM (a row is 16 to 24 KB of loads in flight per warp).
template <typename T, bool LAYER, int NV>
__global__ void __launch_bounds__(128, 2)
norm_bwd_dx_wide_kernel(const T* __restrict__ g, const T* __restrict__ x, const float* __restrict__ gamma,
                        const float* __restrict__ rinv_in, const float* __restrict__ mean_in, const T* __restrict__ add,
                        T* __restrict__ dx, int rows)
{
    constexpr int VN = Vec16<T>::N, D = 32 * NV * VN;
    extern __shared__ __align__(16) float norm_params[];
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    for (int i = threadIdx.x; i < D; i += blockDim.x) norm_params[i] = gamma[i];
    __syncthreads();
    const float inv_d = 1.0f / static_cast<float>(D);
    for (int r = blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += gridDim.x * wpb) {
        const size_t off = static_cast<size_t>(r) * D;
        const float rinv = rinv_in[r], mean = LAYER ? mean_in[r] : 0.f;
        Vec16<T> gv[NV], xv[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) { gv[v] = ld16(g + off + (v * 32 + lane) * VN); xv[v] = ld16(x + off + (v * 32 + lane) * VN); }
        float s_g = 0.f, s_gn = 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            float gm[VN];
            ld_f32x_generic<VN>(norm_params + (v * 32 + lane) * VN, gm);
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                const float gg = to_f32(gv[v].v[k]) * gm[k], nn = (to_f32(xv[v].v[k]) - mean) * rinv;
                s_g += gg; s_gn += gg * nn;
            }
        }
        const float m_gn = warp_sum(s_gn) * inv_d;
        const float m_g = LAYER ? warp_sum(s_g) * inv_d : 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) { forget_derived(gv[v]); forget_derived(xv[v]); }
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            float gm[VN];
            ld_f32x_generic<VN>(norm_params + (v * 32 + lane) * VN, gm);
            Vec16<T> av;
            if (add) av = ld16(add + off + (v * 32 + lane) * VN);
            Vec16<T> o;
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                const float gg = to_f32(gv[v].v[k]) * gm[k], nn = (to_f32(xv[v].v[k]) - mean) * rinv;
                float t = (gg - m_g - nn * m_gn) * rinv;
                if (add) t += to_f32(av.v[k]);
                o.v[k] = from_f32<T>(t);
            }
            st16(dx + off + (v * 32 + lane) * VN, o);
        }
    }
}

// Norm backward for wide rows with its parameter gradients fused in (d = 256 * NVT * elements per 16 bytes: 2048 and
// 4096 bf16 columns).  A block works on two rows at a time (four at the narrower width), every thread on the same NVT 16-byte vectors of each row, so
// dgamma += sum g*gamma*n, dbeta += sum g and the column sums of the produced dx accumulate in registers; the two row
// sums go through shared memory (one barrier per row group, buffers used in turn).  Every activation is read once.  Each
// block leaves its partial sums in partial[quantity][block][d] (quantities: dgamma, dbeta for LayerNorm, the column sums
// if asked for); colsum_final_kernel adds them up in block order.
template <typename T, bool LAYER, int NVT>
__global__ void __launch_bounds__(256, 2)
norm_bwd_wide_fused_kernel(const T* __restrict__ g, const T* __restrict__ x, const float* __restrict__ gamma,
                           const float* __restrict__ rinv_in, const float* __restrict__ mean_in, const T* __restrict__ add,
                           T* __restrict__ dx, float* __restrict__ partial, int rows, int want_colsum)
{
    constexpr int VN = Vec16<T>::N, D = 256 * NVT * VN, RG = NVT == 1 ? 4 : 2;     // rows per step: 32 KB of g and x in flight
    __shared__ float red[2][8][RG][2];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float gm[NVT][VN], a_dg[NVT][VN], a_db[NVT][VN], a_cs[NVT][VN];
#pragma unroll
    for (int j = 0; j < NVT; ++j) {
        ld_f32x<VN>(gamma + (j * 256 + tid) * VN, gm[j]);
#pragma unroll
        for (int k = 0; k < VN; ++k) { a_dg[j][k] = 0.f; a_db[j][k] = 0.f; a_cs[j][k] = 0.f; }
    }
    const float inv_d = 1.0f / static_cast<float>(D);
    int it = 0;
    for (int r0 = blockIdx.x * RG; r0 < rows; r0 += gridDim.x * RG, ++it) {
        Vec16<T> gv[RG][NVT], xv[RG][NVT];
        float rinv[RG], mean[RG];
#pragma unroll
        for (int rr = 0; rr < RG; ++rr) {
            const int r = r0 + rr;
            const bool live = r < rows;
            rinv[rr] = live ? rinv_in[r] : 0.f;
            mean[rr] = (LAYER && live) ? mean_in[r] : 0.f;
#pragma unroll
            for (int j = 0; j < NVT; ++j) {
                if (live) {
                    gv[rr][j] = ld16(g + static_cast<size_t>(r) * D + (j * 256 + tid) * VN);
                    xv[rr][j] = ld16(x + static_cast<size_t>(r) * D + (j * 256 + tid) * VN);
                } else {
#pragma unroll
                    for (int k = 0; k < VN; ++k) { gv[rr][j].v[k] = from_f32<T>(0.f); xv[rr][j].v[k] = from_f32<T>(0.f); }
                }
            }
        }
#pragma unroll
        for (int rr = 0; rr < RG; ++rr) {
            float s_g = 0.f, s_gn = 0.f;
#pragma unroll
            for (int j = 0; j < NVT; ++j)
#pragma unroll
                for (int k = 0; k < VN; ++k) {
                    const float gg = to_f32(gv[rr][j].v[k]) * gm[j][k], nn = (to_f32(xv[rr][j].v[k]) - mean[rr]) * rinv[rr];
                    s_g += gg; s_gn += gg * nn;
                }
            s_gn = warp_sum(s_gn);
            if (LAYER) s_g = warp_sum(s_g);
            if (lane == 0) { red[it & 1][warp][rr][0] = s_gn; red[it & 1][warp][rr][1] = s_g; }
        }
        __syncthreads();
#pragma unroll
        for (int rr = 0; rr < RG; ++rr) {
            const int r = r0 + rr;
            if (r >= rows) break;
            float m_gn = 0.f, m_g = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) { m_gn += red[it & 1][w][rr][0]; if (LAYER) m_g += red[it & 1][w][rr][1]; }
            m_gn *= inv_d; m_g *= inv_d;
#pragma unroll
            for (int j = 0; j < NVT; ++j) {
                const size_t off = static_cast<size_t>(r) * D + (j * 256 + tid) * VN;
                Vec16<T> av;
                if (add) av = ld16(add + off);
                Vec16<T> o;
#pragma unroll
                for (int k = 0; k < VN; ++k) {
                    const float gr = to_f32(gv[rr][j].v[k]);
                    const float gg = gr * gm[j][k], nn = (to_f32(xv[rr][j].v[k]) - mean[rr]) * rinv[rr];
                    float t = (gg - m_g - nn * m_gn) * rinv[rr];
                    if (add) t += to_f32(av.v[k]);
                    o.v[k] = from_f32<T>(t);
                    a_dg[j][k] += gg * nn;
                    if (LAYER) a_db[j][k] += gr;
                    if (want_colsum) a_cs[j][k] += to_f32(o.v[k]);
                }
                st16(dx + off, o);
            }
        }
    }
    const size_t per = static_cast<size_t>(gridDim.x) * D;
#pragma unroll
    for (int j = 0; j < NVT; ++j)
#pragma unroll
        for (int k = 0; k < VN; ++k) {
            const size_t at = static_cast<size_t>(blockIdx.x) * D + (j * 256 + tid) * VN + k;
            partial[at] = a_dg[j][k];
            if (LAYER) partial[per + at] = a_db[j][k];
            if (want_colsum) partial[(LAYER ? 2 : 1) * per + at] = a_cs[j][k];
        }
}

// norm backward with its parameter gradients fused in.  A lane owns the same columns for every row
// its warp visits, so  dgamma += sum g*gamma*n,  dbeta += sum g  and (optionally) the column sums
// of the produced dx — the bias gradient of the Linear layer that fed this point — accumulate in
// registers.  Warps fold through shared memory, blocks write partials, and the block that finishes
// last adds the partials up in fixed order: deterministic, no extra pass over the activations.
// The rows reach the warps through shared memory: each warp owns a ring of two row slots ([g | x | residual-gradient]
// row, 3 * D * sizeof(T) bytes each) that its lane 0 fills with bulk copies counted on an mbarrier, two rows ahead of
// the one being worked on (the fold buffer of the kernel's end lies over the rings: every copy has landed by then).
// Three slots were measured slower (25.9 against 22.4 us at 16384 x 768): they cost the second block per SM.  Loading a row into registers only when its turn came left the memory system idle while a
// warp reduced and stored (the kernel ran at 0.57 of the copy bandwidth), and prefetching into registers does not fit
// beside the three per-column accumulators.
__device__ int g_fused_error = 0;        // 0 ok; otherwise (code << 16 | block) of the first wait that gave up
constexpr int kNormFusedBlocks = 296;   // two per SM
constexpr int kNormFoldGroup = 17;      // blocks per first-level fold group: about the square root of the block count, so both levels read as many rows
constexpr int kNormFoldCounters = 64;   // ints at the end of the counter array: one per group, the last for the groups

template <typename T, bool LAYER, int NV>
__global__ void __launch_bounds__(256, 2)
norm_bwd_fused_kernel(const T* __restrict__ g, const T* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ rinv_in, const float* __restrict__ mean_in, const T* __restrict__ add,
                      T* __restrict__ dx, float* __restrict__ partial, int* __restrict__ counter,
                      float* __restrict__ dgamma, float* __restrict__ dbeta, float* __restrict__ osum, int rows, int defer)
{
    constexpr int VN = Vec16<T>::N, D = 32 * NV * VN, NQ = 3;
    constexpr int ROW_BYTES = D * static_cast<int>(sizeof(T)), SLOT = 3 * ROW_BYTES;
    extern __shared__ __align__(128) uint8_t nb_smem[];
    constexpr int RING = 2;
    static_assert(8 * RING * SLOT >= 8 * D * static_cast<int>(sizeof(float)), "the fold buffer lies over the rings");
    float (*red)[D] = reinterpret_cast<float (*)[D]>(nb_smem);                      // [8][D], used after the row loop
    uint8_t* ring = nb_smem;                                                        // [warp][RING][SLOT]
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + 8 * RING * SLOT);           // [warp][RING]
    __shared__ int is_last;
    __shared__ int abort_word;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    volatile int* abort_flag = &abort_word;
    if (threadIdx.x == 0) abort_word = 0;
    if (lane == 0) {
        for (int k = 0; k < RING; ++k) mbar_init(smem_u32(bars + RING * warp + k), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    float gm[NV][VN], a_dg[NV][VN], a_db[NV][VN], a_os[NV][VN];
#pragma unroll
    for (int v = 0; v < NV; ++v)
#pragma unroll
        for (int k = 0; k < VN; ++k) { a_dg[v][k] = 0.f; a_db[v][k] = 0.f; a_os[v][k] = 0.f; }
#pragma unroll
    for (int v = 0; v < NV; ++v) ld_f32x<VN>(gamma + (v * 32 + lane) * VN, gm[v]);
    const float inv_d = 1.0f / static_cast<float>(D);
    const int r0 = blockIdx.x * wpb + warp, rstep = gridDim.x * wpb;
    uint8_t* my_ring = ring + warp * RING * SLOT;
    auto request = [&](int r, int slot) {                      // lane 0: the three rows of row r into a slot
        const uint32_t bar = smem_u32(bars + RING * warp + slot), dst = smem_u32(my_ring + slot * SLOT);
        const size_t off = static_cast<size_t>(r) * D;
        mbar_expect_tx(bar, add ? 3 * ROW_BYTES : 2 * ROW_BYTES);
        bulk_load_1d(dst, g + off, ROW_BYTES, bar);
        bulk_load_1d(dst + ROW_BYTES, x + off, ROW_BYTES, bar);
        if (add) bulk_load_1d(dst + 2 * ROW_BYTES, add + off, ROW_BYTES, bar);
    };
    if (lane == 0)
        for (int k = 0; k < RING; ++k)
            if (r0 + k * rstep < rows) request(r0 + k * rstep, k);
    float rinv_next = r0 < rows ? rinv_in[r0] : 0.f, mean_next = (LAYER && r0 < rows) ? mean_in[r0] : 0.f;
    int it = 0;
    for (int r = r0; r < rows; r += rstep, ++it) {
        const size_t off = static_cast<size_t>(r) * D;
        const int slot = it % RING;
        const float rinv = rinv_next, mean = mean_next;
        if (r + rstep < rows) { rinv_next = rinv_in[r + rstep]; if (LAYER) mean_next = mean_in[r + rstep]; }
        const bool got = mbar_wait(smem_u32(bars + RING * warp + slot), (it / RING) & 1, abort_flag, 1, &g_fused_error);
        if (!__all_sync(0xffffffffu, got)) break;
        const uint8_t* sl = my_ring + slot * SLOT;
        // two passes over the slot (it is shared memory: cheaper than holding g * gamma and the normalised row in
        // registers beside the three per-column accumulators)
        float s_g = 0.f, s_gn = 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const Vec16<T> gv = *reinterpret_cast<const Vec16<T>*>(sl + (v * 32 + lane) * 16);
            const Vec16<T> xv = *reinterpret_cast<const Vec16<T>*>(sl + ROW_BYTES + (v * 32 + lane) * 16);
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                const float graw = to_f32(gv.v[k]);
                const float ggk = graw * gm[v][k], nnk = (to_f32(xv.v[k]) - mean) * rinv;
                s_g += ggk; s_gn += ggk * nnk;
                a_dg[v][k] += ggk * nnk;
                if (LAYER) a_db[v][k] += graw;
            }
        }
        const float m_gn = warp_sum(s_gn) * inv_d;
        const float m_g = LAYER ? warp_sum(s_g) * inv_d : 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const Vec16<T> gv = *reinterpret_cast<const Vec16<T>*>(sl + (v * 32 + lane) * 16);
            const Vec16<T> xv = *reinterpret_cast<const Vec16<T>*>(sl + ROW_BYTES + (v * 32 + lane) * 16);
            Vec16<T> av;
            if (add) av = *reinterpret_cast<const Vec16<T>*>(sl + 2 * ROW_BYTES + (v * 32 + lane) * 16);
            Vec16<T> o;
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                const float ggk = to_f32(gv.v[k]) * gm[v][k], nnk = (to_f32(xv.v[k]) - mean) * rinv;
                float t = (ggk - m_g - nnk * m_gn) * rinv;
                if (add) t += to_f32(av.v[k]);
                o.v[k] = from_f32<T>(t);
                a_os[v][k] += to_f32(o.v[k]);             // the rounded value: what the next kernel reads
            }
            st16(dx + off + (v * 32 + lane) * VN, o);
        }
        __syncwarp();                                           // every lane is done with the slot
        if (lane == 0 && r + RING * rstep < rows) request(r + RING * rstep, slot);
    }
    // block fold, one quantity at a time, then this block's partial row
    const size_t pstride = static_cast<size_t>(gridDim.x) * D;
#pragma unroll 1
    for (int qn = 0; qn < NQ; ++qn) {
        if ((qn == 1 && !LAYER) || (qn == 2 && !osum)) continue;
        __syncthreads();
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
            for (int k = 0; k < VN; ++k)
                red[warp][(v * 32 + lane) * VN + k] = qn == 0 ? a_dg[v][k] : (qn == 1 ? a_db[v][k] : a_os[v][k]);
        __syncthreads();
        for (int c = threadIdx.x; c < D; c += 256) {
            float sacc = red[0][c];
#pragma unroll
            for (int w = 1; w < 8; ++w) sacc += red[w][c];
            partial[qn * pstride + static_cast<size_t>(blockIdx.x) * D + c] = sacc;
        }
    }
    if (defer) return;          // the partial rows are folded later, by norm_fold_deferred_kernel
    // Two-level fold in fixed order (deterministic, whatever order the blocks finish in): the last block of each
    // group of kNormFoldGroup consecutive blocks adds that group's rows into one group row; the last group to
    // finish adds the group rows into the gradients.  One block folding all 296 rows alone took longer than
    // the pass over the activations.
    const int nb = gridDim.x, ngroups = (nb + kNormFoldGroup - 1) / kNormFoldGroup;
    const int grp_id = blockIdx.x / kNormFoldGroup, grp_first = grp_id * kNormFoldGroup;
    const int grp_size = min(kNormFoldGroup, nb - grp_first);
    float* gpartial = partial + NQ * pstride;                                // [NQ][ngroups][D]
    const size_t gstride = static_cast<size_t>(ngroups) * D;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = (atomicAdd(counter + grp_id, 1) == grp_size - 1);
    __syncthreads();
    if (!is_last) return;
    __threadfence();
#pragma unroll 1
    for (int qn = 0; qn < NQ; ++qn) {
        if ((qn == 1 && !LAYER) || (qn == 2 && !osum)) continue;
        const float* src = partial + qn * pstride + static_cast<size_t>(grp_first) * D;
        for (int c4 = threadIdx.x; c4 < D / 4; c4 += 256) {
            float4 v[kNormFoldGroup];
#pragma unroll
            for (int k = 0; k < kNormFoldGroup; ++k)
                if (k < grp_size) v[k] = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(k) * D) + c4);
            float4 t = v[0];
#pragma unroll
            for (int k = 1; k < kNormFoldGroup; ++k)
                if (k < grp_size) { t.x += v[k].x; t.y += v[k].y; t.z += v[k].z; t.w += v[k].w; }
            reinterpret_cast<float4*>(gpartial + qn * gstride + static_cast<size_t>(grp_id) * D)[c4] = t;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        counter[grp_id] = 0;
        is_last = (atomicAdd(counter + kNormFoldCounters - 1, 1) == ngroups - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
#pragma unroll 1
    for (int qn = 0; qn < NQ; ++qn) {
        if ((qn == 1 && !LAYER) || (qn == 2 && !osum)) continue;
        float* dst = qn == 0 ? dgamma : (qn == 1 ? dbeta : osum);
        const float* src = gpartial + qn * gstride;
        for (int c4 = threadIdx.x; c4 < D / 4; c4 += 256) {
            // all group rows are requested before the first is used: one round trip to L2 instead of one per row
            constexpr int MAXG = (kNormFusedBlocks + kNormFoldGroup - 1) / kNormFoldGroup;
            float4 v[MAXG];
#pragma unroll
            for (int k = 0; k < MAXG; ++k)
                if (k < ngroups) v[k] = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(k) * D) + c4);
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < MAXG; ++k)
                if (k < ngroups) { t.x += v[k].x; t.y += v[k].y; t.z += v[k].z; t.w += v[k].w; }
            float4 o = reinterpret_cast<float4*>(dst)[c4];
            o.x += t.x; o.y += t.y; o.z += t.z; o.w += t.w;
            reinterpret_cast<float4*>(dst)[c4] = o;
        }
    }
    if (threadIdx.x == 0) counter[kNormFoldCounters - 1] = 0;
}

// The cross-block fold of norm_bwd_fused_kernel, deferred: a training step runs that kernel dozens of times per
// micro-batch, and the two fold levels at its end (two fences, two atomics, two round trips to L2 on one block) are a
// third of each launch although nothing needs the parameter gradients before the optimizer.  In deferred mode each
// launch leaves its kNormFusedBlocks partial rows in a slot of its own and this kernel folds all slots at once: block
// (column group, quantity, slot).
__global__ void __launch_bounds__(256)
norm_fold_deferred_kernel(const float* __restrict__ partials, size_t slot_stride, NormFoldSlots slots, float* __restrict__ G,
                          int nblocks, int d)
{
    // 64 float4 columns x 4 row segments per block: segment q sums rows [q*seg, (q+1)*seg) in order, 16 loads in
    // flight; the four segment sums are then added in segment order (fixed order: deterministic)
    __shared__ float4 seg_sum[4][64];
    const int slot = blockIdx.z, qn = blockIdx.y;
    const long long dst_off = qn == 0 ? slots.dgamma[slot] : (qn == 1 ? slots.dbeta[slot] : slots.osum[slot]);
    if (dst_off < 0) return;                                      // uniform over the block
    const int lane = threadIdx.x & 63, q = threadIdx.x >> 6;
    const int c4 = blockIdx.x * 64 + lane;
    const bool live = c4 < d / 4;
    const int seg = (nblocks + 3) / 4;
    const int k0 = q * seg, k1 = min(nblocks, k0 + seg);
    const float* src = partials + slot * slot_stride + static_cast<size_t>(qn) * nblocks * d;
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        int k = k0;
        for (; k + 16 <= k1; k += 16) {
            float4 v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(k + j) * d) + c4);
#pragma unroll
            for (int j = 0; j < 16; ++j) { t.x += v[j].x; t.y += v[j].y; t.z += v[j].z; t.w += v[j].w; }
        }
        for (; k < k1; ++k) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(k) * d) + c4);
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
    }
    seg_sum[q][lane] = t;
    __syncthreads();
    if (q == 0 && live) {
        float4 r = seg_sum[0][lane];
#pragma unroll
        for (int j = 1; j < 4; ++j) { const float4 v = seg_sum[j][lane]; r.x += v.x; r.y += v.y; r.z += v.z; r.w += v.w; }
        float4* dst = reinterpret_cast<float4*>(G + dst_off) + c4;
        float4 o = *dst;
        o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
        *dst = o;
    }
}

// ======================================================================================
// column sums over tokens (parameter gradients that reduce over the token dimension)
//   MODE 0: sum_r g[r][c]                       (bias and LayerNorm-beta gradients)
//   MODE 1: sum_r g[r][c]*gamma[c]*n[r][c]      (norm scale gradient; the reference multiplies by
//                                                gamma — compute_layer.hpp:789-797, 636-644 — kept)
// Stage 1 writes per-chunk partials, stage 2 folds them in fixed order and adds into the gradient.
// ======================================================================================
constexpr int CS_COLS = 64, CS_ROWLANES = 4, CS_CHUNK_ROWS = 128;

template <typename T, int MODE>
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const T* __restrict__ g, long long ldg, const T* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ rinv, const float* __restrict__ mean, float* __restrict__ partial,
                      int rows, int cols)
{
    __shared__ float red[CS_ROWLANES][CS_COLS];
    const int tx = threadIdx.x % CS_COLS, ty = threadIdx.x / CS_COLS;
    const int c = blockIdx.x * CS_COLS + tx;
    const int r0 = blockIdx.y * CS_CHUNK_ROWS, r1 = min(rows, r0 + CS_CHUNK_ROWS);
    float acc = 0.f;
    if (c < cols) {
        const float gm = (MODE == 1) ? gamma[c] : 0.f;
        for (int r = r0 + ty; r < r1; r += CS_ROWLANES) {
            const float gv = to_f32(g[static_cast<size_t>(r) * ldg + c]);
            if (MODE == 0) acc += gv;
            else {
                const float mu = mean ? mean[r] : 0.f;
                acc += gv * gm * ((to_f32(x[static_cast<size_t>(r) * cols + c]) - mu) * rinv[r]);
            }
        }
    }
    red[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && c < cols)
        partial[static_cast<size_t>(blockIdx.y) * cols + c] = (red[0][tx] + red[1][tx]) + (red[2][tx] + red[3][tx]);
}

// Vectorised variant (16-byte loads; needs cols, ldg multiples of the vector width and aligned
// pointers): a block owns 32 vectors of columns x 8 row lanes over one 128-row chunk.  With
// `counters` (one zero-initialised int per column block, reset by the kernel after use) the block
// that finishes last folds all chunk partials in fixed order and adds them into `out`, so the
// second launch disappears while the summation order stays deterministic.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
colsum_vec_kernel(const T* __restrict__ g, long long ldg, const T* __restrict__ x, const float* __restrict__ gamma,
                  const float* __restrict__ rinv, const float* __restrict__ mean, float* __restrict__ partial,
                  int* __restrict__ counters, float* __restrict__ out, int rows, int cols, int chunks, int chunk_rows)
{
    constexpr int VN = Vec16<T>::N;
    constexpr int BW = 32 * VN;                                   // columns per block
    __shared__ float red[8][BW];
    __shared__ int is_last;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c0 = (blockIdx.x * 32 + tx) * VN;
    const int r0 = blockIdx.y * chunk_rows, r1 = min(rows, r0 + chunk_rows);
    float acc[VN];
#pragma unroll
    for (int k = 0; k < VN; ++k) acc[k] = 0.f;
    if (c0 < cols) {
        float gm[VN];
#pragma unroll
        for (int k = 0; k < VN; ++k) gm[k] = (MODE == 1) ? gamma[c0 + k] : 0.f;
#pragma unroll 8
        for (int r = r0 + ty; r < r1; r += 8) {
            const Vec16<T> gv = ld16(g + static_cast<size_t>(r) * ldg + c0);
            if (MODE == 0) {
#pragma unroll
                for (int k = 0; k < VN; ++k) acc[k] += to_f32(gv.v[k]);
            } else {
                const Vec16<T> xv = ld16(x + static_cast<size_t>(r) * cols + c0);
                const float mu = mean ? mean[r] : 0.f, ri = rinv[r];
#pragma unroll
                for (int k = 0; k < VN; ++k) acc[k] += to_f32(gv.v[k]) * gm[k] * ((to_f32(xv.v[k]) - mu) * ri);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < VN; ++k) red[ty][tx * VN + k] = acc[k];
    __syncthreads();
    for (int j = threadIdx.x; j < BW; j += 256) {
        const int c = blockIdx.x * BW + j;
        if (c < cols) {
            float s = red[0][j];
#pragma unroll
            for (int k = 1; k < 8; ++k) s += red[k][j];
            partial[static_cast<size_t>(blockIdx.y) * cols + c] = s;
        }
    }
    if (!counters) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = (atomicAdd(&counters[blockIdx.x], 1) == chunks - 1);
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // final fold by the last block: 4 chunk groups x (BW/4) float4 columns, 8 loads in flight per
    // thread; group g sums chunks g, g+4, ... in order and the groups are combined in fixed order
    constexpr int QW = BW / 4;                                    // float4 columns per block
    float4* red4 = reinterpret_cast<float4*>(&red[0][0]);        // reuse: 8*BW floats >= 4*QW float4
    for (int j0 = 0; j0 < QW; j0 += 64) {
        const int jq = j0 + (threadIdx.x & 63), grp = threadIdx.x >> 6;
        const int c = blockIdx.x * BW + jq * 4;
        float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (jq < QW && c < cols) {
#pragma unroll 8
            for (int k = grp; k < chunks; k += 4) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(partial + static_cast<size_t>(k) * cols + c));
                s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
            }
        }
        __syncthreads();
        red4[grp * 64 + (threadIdx.x & 63)] = s4;
        __syncthreads();
        if (grp == 0 && jq < QW && c < cols) {
            float4 t = red4[threadIdx.x & 63];
#pragma unroll
            for (int gq = 1; gq < 4; ++gq) { const float4 v = red4[gq * 64 + (threadIdx.x & 63)]; t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w; }
            float4 o = *reinterpret_cast<float4*>(out + c);
            o.x += t.x; o.y += t.y; o.z += t.z; o.w += t.w;
            *reinterpret_cast<float4*>(out + c) = o;
        }
    }
    if (threadIdx.x == 0) counters[blockIdx.x] = 0;
}

__global__ void colsum_final_kernel(const float* __restrict__ partial, float* __restrict__ out, int chunks, int cols)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float acc = 0.f;
    for (int k = 0; k < chunks; ++k) acc += partial[static_cast<size_t>(k) * cols + c];
    out[c] += acc;
}

// ======================================================================================
// activations
// ======================================================================================
template <typename T>
__global__ void gelu_fwd_kernel(const T* __restrict__ h1, T* __restrict__ h2, size_t n)
{
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float x = to_f32(h1[i]);
        h2[i] = from_f32<T>(x * sigmoid_t<T>(kGeluBeta * x));
    }
}
template <typename T>
__global__ void gelu_bwd_kernel(const T* __restrict__ g, const T* __restrict__ h1, T* __restrict__ out, size_t n)
{
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float x = to_f32(h1[i]);
        const float s = sigmoid_t<T>(kGeluBeta * x);
        out[i] = from_f32<T>(to_f32(g[i]) * (s * (1.0f + (kGeluBeta * x) * (1.0f - s))));
    }
}

// h1 (rows, 2*ff): columns [0,ff) gate, [ff,2ff) up  ->  h2 (rows, ff) = gate*sigmoid(gate)*up
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ h1, T* __restrict__ h2, int rows, int ff)
{
    constexpr int VN = Vec16<T>::N;
    if ((ff % VN) == 0) {
        const size_t nv = static_cast<size_t>(rows) * (ff / VN);
        for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv;
             i += static_cast<size_t>(gridDim.x) * blockDim.x) {
            const size_t r = i / (ff / VN);
            const int c = static_cast<int>(i % (ff / VN)) * VN;
            auto gv = ld16(h1 + r * 2 * ff + c); auto uv = ld16(h1 + r * 2 * ff + ff + c); Vec16<T> o;
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                const float gt = to_f32(gv.v[k]);
                o.v[k] = from_f32<T>(gt * sigmoid_t<T>(gt) * to_f32(uv.v[k]));
            }
            st16(h2 + r * ff + c, o);
        }
    } else {
        const size_t n = static_cast<size_t>(rows) * ff;
        for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
             i += static_cast<size_t>(gridDim.x) * blockDim.x) {
            const size_t r = i / ff; const int c = static_cast<int>(i % ff);
            const float gt = to_f32(h1[r * 2 * ff + c]);
            h2[i] = from_f32<T>(gt * sigmoid_t<T>(gt) * to_f32(h1[r * 2 * ff + ff + c]));
        }
    }
}
// dh1 (rows, 2*ff) from g (rows, ff) and h1: compute_layer.hpp:436-445
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ g, const T* __restrict__ h1, T* __restrict__ dh1, int rows, int ff)
{
    constexpr int VN = Vec16<T>::N;
    if ((ff % VN) == 0) {
        const size_t nv = static_cast<size_t>(rows) * (ff / VN);
        for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv;
             i += static_cast<size_t>(gridDim.x) * blockDim.x) {
            const size_t r = i / (ff / VN);
            const int c = static_cast<int>(i % (ff / VN)) * VN;
            auto gv = ld16(g + r * ff + c);
            auto gtv = ld16(h1 + r * 2 * ff + c); auto uv = ld16(h1 + r * 2 * ff + ff + c);
            Vec16<T> og, ou;
#pragma unroll
            for (int k = 0; k < VN; ++k) {
                const float go = to_f32(gv.v[k]), gt = to_f32(gtv.v[k]), up = to_f32(uv.v[k]);
                const float s = sigmoid_t<T>(gt);
                og.v[k] = from_f32<T>(go * up * (s * (1.0f + gt * (1.0f - s))));
                ou.v[k] = from_f32<T>(go * gt * s);
            }
            st16(dh1 + r * 2 * ff + c, og);
            st16(dh1 + r * 2 * ff + ff + c, ou);
        }
    } else {
        const size_t n = static_cast<size_t>(rows) * ff;
        for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
             i += static_cast<size_t>(gridDim.x) * blockDim.x) {
            const size_t r = i / ff; const int c = static_cast<int>(i % ff);
            const float go = to_f32(g[i]), gt = to_f32(h1[r * 2 * ff + c]), up = to_f32(h1[r * 2 * ff + ff + c]);
            const float s = sigmoid_t<T>(gt);
            dh1[r * 2 * ff + c] = from_f32<T>(go * up * (s * (1.0f + gt * (1.0f - s))));
            dh1[r * 2 * ff + ff + c] = from_f32<T>(go * gt * s);
        }
    }
}

// ======================================================================================
// fused softmax cross-entropy over token rows: logits (rows, V) are overwritten by their gradient
// ======================================================================================
// stats[0] = number of valid rows, stats[1] = 1/num_valid (0 when none)
__global__ void ce_count_kernel(const int* __restrict__ labels, const float* __restrict__ mask, int rows, int vocab,
                                float* __restrict__ stats)
{
    __shared__ float red[32];
    float c = 0.f;
    for (int i = threadIdx.x; i < rows; i += blockDim.x) {
        const bool ok = (!mask || mask[i] >= 0.5f) && labels[i] >= 0 && labels[i] < vocab;
        c += ok ? 1.f : 0.f;
    }
    c = block_sum(c, red);
    if (threadIdx.x == 0) { stats[0] = c; stats[1] = c > 0.f ? 1.0f / c : 0.f; }
}

// NV 16-byte vectors of the row cached per thread (0 = re-read from memory).  Up to 4 vectors the exponentials are
// kept in registers too (computed once, used for the sum and the gradient); beyond that they are recomputed in the
// last pass, so that a block stays at 64 registers per thread and two blocks share an SM: with one block per SM the
// load, reduce and store phases of a 64 KB row do not overlap with anything.
template <typename T, int NV>
__global__ void __launch_bounds__(512, NV > 4 ? 2 : 0)
ce_fwd_bwd_kernel(T* __restrict__ logits, const int* __restrict__ labels, const float* __restrict__ mask,
                  const float* __restrict__ stats, float grad_scale, float* __restrict__ loss_vec, int rows, int V,
                  int vocab)
{
    constexpr int VN = Vec16<T>::N;
    constexpr bool KEEP_EX = NV > 0 && NV <= 4;
    __shared__ float red[32];
    const int r = blockIdx.x;
    T* row = logits + static_cast<size_t>(r) * V;
    const int lbl = labels[r];
    const bool valid = (!mask || mask[r] >= 0.5f) && lbl >= 0 && lbl < vocab;
    const int nvec = V / VN;          // the launcher guarantees V % VN == 0 when NV > 0
    if (!valid) {
        if (NV > 0) { Vec16<T> z; for (int k = 0; k < VN; ++k) z.v[k] = from_f32<T>(0.f);
            for (int i = threadIdx.x; i < nvec; i += blockDim.x) st16(row + i * VN, z); }
        else for (int i = threadIdx.x; i < V; i += blockDim.x) row[i] = from_f32<T>(0.f);
        if (threadIdx.x == 0) loss_vec[r] = 0.f;
        return;
    }
    const float inv = stats[1] * grad_scale;   // inv_num_valid, times the accumulation scale (text_train.cpp:1253-1258)
    Vec16<T> cache[NV > 0 ? NV : 1];
    float mx = -INFINITY;
    if (NV > 0) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < nvec) { cache[j] = ld16(row + i * VN);
#pragma unroll
                for (int k = 0; k < VN; ++k) mx = fmaxf(mx, to_f32(cache[j].v[k])); }
        }
    } else for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, to_f32(row[i]));
    mx = block_max(mx, red);
    float den = 0.f;
    float ex[KEEP_EX ? NV : 1][VN];
    if (NV > 0) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < nvec) {
#pragma unroll
                for (int k = 0; k < VN; ++k) {
                    const float e = exp_t<T>(to_f32(cache[j].v[k]) - mx);
                    if (KEEP_EX) ex[j][k] = e;
                    den += e;
                } }
        }
    } else for (int i = threadIdx.x; i < V; i += blockDim.x) den += exp_t<T>(to_f32(row[i]) - mx);
    den = block_sum(den, red);
    const float ll = to_f32(row[lbl]);
    __syncthreads();                                  // everyone has read row[lbl] before it is overwritten
    if (threadIdx.x == 0) loss_vec[r] = ll - mx - logf(den);
    const float inv_den = inv / den;
    if (NV > 0) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < nvec) { Vec16<T> o;
#pragma unroll
                for (int k = 0; k < VN; ++k) {
                    float gv = (KEEP_EX ? ex[j][k] : exp_t<T>(to_f32(cache[j].v[k]) - mx)) * inv_den;
                    if (i * VN + k == lbl) gv -= inv;
                    o.v[k] = from_f32<T>(gv);
                }
                st16(row + i * VN, o); }
        }
    } else for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float gv = inv * exp_t<T>(to_f32(row[i]) - mx) / den;
        if (i == lbl) gv -= inv;
        row[i] = from_f32<T>(gv);
    }
}

// loss = -(sum loss_vec) / num_valid (compute_loss.hpp:300-307); single block, fixed order
// The same computation with the rows staged in shared memory: persistent blocks, each with a ring of row slots that
// thread 0 fills with bulk copies (counted on an mbarrier) ahead of the row being worked on; the two passes (maximum with
// sum of exponentials, gradient) read and overwrite the slot, and the finished row leaves as one bulk store while the
// next is computed.  The register-cached kernel above does load -> reduce -> reduce -> store per row with nothing
// overlapping inside a block (0.39 of the copy bandwidth at 16384 x 32768; this kernel: 0.50 with three slots and one
// block per SM, 0.60 with one slot and three blocks per SM, which is how it is launched; the two exponentials per
// element are the next limit: 4096 XU clocks per 64 KB row).  Maximum and sum of exponentials are taken in one pass
// (a running maximum per thread), so the sums differ from the register-cached kernel's in the last bits.  Used for rows
// of 32 KB and more.
template <typename T>
__global__ void __launch_bounds__(512)
ce_staged_kernel(T* __restrict__ logits, const int* __restrict__ labels, const float* __restrict__ mask,
                 const float* __restrict__ stats, float grad_scale, float* __restrict__ loss_vec, int rows, int V, int vocab,
                 int slots)
{
    constexpr int VN = Vec16<T>::N;
    extern __shared__ __align__(128) uint8_t ce_smem[];
    __shared__ float red[32];
    __shared__ int abort_word;
    const uint32_t row_bytes = static_cast<uint32_t>(V) * sizeof(T);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ce_smem + static_cast<size_t>(slots) * row_bytes);
    volatile int* abort_flag = &abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0;
        for (int k = 0; k < slots; ++k) mbar_init(smem_u32(bars + k), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int nvec = V / VN;
    const int first = blockIdx.x, step = gridDim.x;
    auto request = [&](int r, int slot) {
        mbar_expect_tx(smem_u32(bars + slot), row_bytes);
        bulk_load_1d(smem_u32(ce_smem + static_cast<size_t>(slot) * row_bytes), logits + static_cast<size_t>(r) * V, row_bytes, smem_u32(bars + slot));
    };
    if (threadIdx.x == 0)
        for (int k = 0; k < slots; ++k)
            if (first + k * step < rows) request(first + k * step, k);
    const float inv_nv = stats[1] * grad_scale;   // inv_num_valid, times the accumulation scale (text_train.cpp:1253-1258)
    int it = 0;
    for (int r = first; r < rows; r += step, ++it) {
        const int slot = it % slots;
        T* row = reinterpret_cast<T*>(ce_smem + static_cast<size_t>(slot) * row_bytes);
        const int lbl = labels[r];
        const bool valid = (!mask || mask[r] >= 0.5f) && lbl >= 0 && lbl < vocab;
        const bool got = mbar_wait(smem_u32(bars + slot), (it / slots) & 1, abort_flag, 2, &g_fused_error);
        if (__syncthreads_or(!got)) break;
        if (!valid) {
            Vec16<T> z;
#pragma unroll
            for (int k = 0; k < VN; ++k) z.v[k] = from_f32<T>(0.f);
            for (int i = threadIdx.x; i < nvec; i += blockDim.x) *reinterpret_cast<Vec16<T>*>(row + i * VN) = z;
            if (threadIdx.x == 0) loss_vec[r] = 0.f;
        } else {
            // maximum and sum of exponentials in one pass over the slot: a thread's sum is kept relative to its own
            // running maximum (rescaled when a vector raises it) and brought to the row maximum at the end
            float tm = -INFINITY, ts = 0.f;
            for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
                const Vec16<T> v = *reinterpret_cast<const Vec16<T>*>(row + i * VN);
                float vm = to_f32(v.v[0]);
#pragma unroll
                for (int k = 1; k < VN; ++k) vm = fmaxf(vm, to_f32(v.v[k]));
                if (vm > tm) { ts *= exp_t<T>(tm - vm); tm = vm; }      // exp(-inf) = 0 the first time
#pragma unroll
                for (int k = 0; k < VN; ++k) ts += exp_t<T>(to_f32(v.v[k]) - tm);
            }
            const float mx = block_max(tm, red);
            float den = block_sum(tm == -INFINITY ? 0.f : ts * exp_t<T>(tm - mx), red);
            const float ll = to_f32(row[lbl]);
            __syncthreads();                              // everyone has read row[lbl] before it is overwritten
            if (threadIdx.x == 0) loss_vec[r] = ll - mx - logf(den);
            const float inv_den = inv_nv / den;
            for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
                const Vec16<T> v = *reinterpret_cast<const Vec16<T>*>(row + i * VN);
                Vec16<T> o;
#pragma unroll
                for (int k = 0; k < VN; ++k) {
                    float gv = exp_t<T>(to_f32(v.v[k]) - mx) * inv_den;
                    if (i * VN + k == lbl) gv -= inv_nv;
                    o.v[k] = from_f32<T>(gv);
                }
                *reinterpret_cast<Vec16<T>*>(row + i * VN) = o;
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the slot as the bulk store will read it
        __syncthreads();
        if (threadIdx.x == 0) {
            bulk_store_1d(logits + static_cast<size_t>(r) * V, smem_u32(row), row_bytes);
            tma_commit();
            if (r + slots * step < rows) {                // the slot is loaded again once the store has read it
                tma_wait_read0();
                request(r + slots * step, slot);
            }
        }
    }
    if (threadIdx.x == 0) tma_wait_all();                 // shared memory outlives the stores in flight
}

__global__ void ce_loss_kernel(const float* __restrict__ loss_vec, const float* __restrict__ stats, int rows,
                               float* __restrict__ loss_out)
{
    __shared__ float red[32];
    float s = 0.f;
    for (int i = threadIdx.x; i < rows; i += blockDim.x) s += loss_vec[i];
    s = block_sum(s, red);
    if (threadIdx.x == 0) loss_out[0] = stats[0] > 0.f ? -s / stats[0] : 0.f;
}

// ======================================================================================
// optimizers over flat parameter ranges
// ======================================================================================
// hyper[0] = gradient scale (clip * 1/world), read from device memory so no host sync is needed
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, bf16* __restrict__ shadow, size_t n, float lr, float beta1,
                             float beta2, float eps, float decay, float inv_bc1, float inv_bc2,
                             const float* __restrict__ gscale_ptr)
{
    const float gs = gscale_ptr ? gscale_ptr[0] : 1.0f;
    const float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float gr = g[i] * gs;
        float pv = p[i] * decay;                               // AdamW::step decay (compute_optimizer.hpp:397-404)
        const float mv = m[i] * beta1 + omb1 * gr;             // adam_update_ (:262-265)
        const float vv = v[i] * beta2 + (gr * gr) * omb2;      // (:267-274)
        const float ratio = (mv * inv_bc1) / (sqrtf(vv * inv_bc2) + eps);
        pv += ratio * (-lr);
        p[i] = pv; m[i] = mv; v[i] = vv;
        if (shadow) shadow[i] = __float2bfloat16_rn(pv);
    }
}

// sum of squares, two stages, fixed order: partial[block] then one block folds
__global__ void sumsq_partial_kernel(const float* __restrict__ g, size_t n, float* __restrict__ partial)
{
    __shared__ float red[32];
    float s = 0.f;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) { const float x = g[i]; s += x * x; }
    s = block_sum(s, red);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// out[0] = total; when max_norm > 0 also out[1] = norm and out[2] = (norm > max_norm ? max_norm/norm : 1) * post_scale
// (Optimizer::clip_grad_norm, compute_optimizer.hpp:128-138: no epsilon, applied only above the bound)
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int n, float pre_scale, float max_norm,
                                   float post_scale, float* __restrict__ out)
{
    __shared__ float red[32];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
    s = block_sum(s, red);
    if (threadIdx.x == 0) {
        s *= pre_scale * pre_scale;
        out[0] = s;
        const float norm = sqrtf(s);
        out[1] = norm;
        out[2] = ((max_norm > 0.f && norm > max_norm) ? max_norm / norm : 1.0f) * post_scale;
    }
}

// Muon momentum (compute_optimizer.hpp:546-566): v = mu*v + g; u = g + mu*v (Nesterov)
__global__ void muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ vel, float* __restrict__ u,
                                     size_t n, float mu, const float* __restrict__ gscale_ptr)
{
    const float gs = gscale_ptr ? gscale_ptr[0] : 1.0f;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float gr = g[i] * gs;
        const float vv = vel[i] * mu + gr;
        vel[i] = vv;
        u[i] = gr + mu * vv;
    }
}
// X = u * 1/sqrt(|u|^2 + eps^2) (compute_optimizer.hpp:449-456), written as T for the NS GEMMs
template <typename T>
__global__ void muon_normalize_kernel(const float* __restrict__ u, const float* __restrict__ sumsq, float eps,
                                      T* __restrict__ X, size_t n)
{
    const float inv = 1.0f / sqrtf(sumsq[0] + eps * eps);
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) X[i] = from_f32<T>(u[i] * inv);
}
// out = T(alpha*a + beta*b)
template <typename T>
__global__ void axpby_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, float alpha,
                             float beta, size_t n)
{
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        out[i] = from_f32<T>(alpha * to_f32(a[i]) + beta * to_f32(b[i]));
}
// p -= lr * X ; refresh the bf16 shadow
template <typename T>
__global__ void muon_apply_kernel(float* __restrict__ p, const T* __restrict__ X, bf16* __restrict__ shadow, float lr,
                                  size_t n)
{
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float pv = p[i] + (-lr) * to_f32(X[i]);
        p[i] = pv;
        if (shadow) shadow[i] = __float2bfloat16_rn(pv);
    }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, bf16* __restrict__ out, size_t n)
{
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void bf16_to_f32_kernel(const bf16* __restrict__ in, float* __restrict__ out, size_t n)
{
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) out[i] = __bfloat162float(in[i]);
}

// ======================================================================================
// host launchers
// ======================================================================================
#define LAUNCH_CHECK() NNB_LAUNCH_CHECK()

int fused_device_error(int* code)
{
    NNB_CUDA_CHECK(cudaMemcpyFromSymbol(code, g_fused_error, sizeof(int)));
    if (*code) { const int z = 0; NNB_CUDA_CHECK(cudaMemcpyToSymbol(g_fused_error, &z, sizeof(int))); }
    return 0;
}

template <typename T>
int norm_fwd(const T* x, const float* gamma, const float* beta, T* y, float* rinv, float* mean, int rows, int d,
             bool layer, cudaStream_t s)
{
    if (rows == 0) return 0;
    const int grid = grid_for(rows, 8);
    const int grid_reg = grid_for(rows, 8, 3);          // the register-resident kernel: one wave of three blocks per SM, rows prefetched
    constexpr int VN = Vec16<T>::N;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(gamma) |
                           reinterpret_cast<uintptr_t>(beta)) & 15) == 0;
#define NNB_NORM_FWD_REG(nv)                                                                                          \
    if (aligned && d == 32 * VN * nv) {                                                                               \
        if (layer) norm_fwd_reg_kernel<T, true, nv><<<grid_reg, 256, 0, s>>>(x, gamma, beta, y, rinv, mean, rows);     \
        else norm_fwd_reg_kernel<T, false, nv><<<grid_reg, 256, 0, s>>>(x, gamma, beta, y, rinv, mean, rows);          \
        LAUNCH_CHECK();                                                                                               \
        return 0;                                                                                                     \
    }
    NNB_NORM_FWD_REG(1) NNB_NORM_FWD_REG(2) NNB_NORM_FWD_REG(3) NNB_NORM_FWD_REG(4)
#undef NNB_NORM_FWD_REG
    // wider rows (up to 4096 bf16 columns): the row in registers as loaded, the parameters in shared memory
    const int grid_wide = grid_for(rows, 4, 3);
#define NNB_NORM_FWD_WIDE(nv)                                                                                         \
    if (aligned && d == 32 * VN * nv) {                                                                               \
        const size_t smem = static_cast<size_t>(layer ? 2 : 1) * d * sizeof(float);                                   \
        if (layer) norm_fwd_wide_kernel<T, true, nv><<<grid_wide, 128, smem, s>>>(x, gamma, beta, y, rinv, mean, rows); \
        else norm_fwd_wide_kernel<T, false, nv><<<grid_wide, 128, smem, s>>>(x, gamma, beta, y, rinv, mean, rows);     \
        LAUNCH_CHECK();                                                                                               \
        return 0;                                                                                                     \
    }
    NNB_NORM_FWD_WIDE(6) NNB_NORM_FWD_WIDE(8) NNB_NORM_FWD_WIDE(12) NNB_NORM_FWD_WIDE(16)
#undef NNB_NORM_FWD_WIDE
    if (layer) norm_fwd_kernel<T, true><<<grid, 256, 0, s>>>(x, gamma, beta, y, rinv, mean, rows, d);
    else norm_fwd_kernel<T, false><<<grid, 256, 0, s>>>(x, gamma, beta, y, rinv, mean, rows, d);
    LAUNCH_CHECK();
    return 0;
}

// Fold of deferred column-sum slots: block (64 float4 columns, slot) with 4 row segments, like norm_fold_deferred_kernel.
__global__ void __launch_bounds__(256)
colsum_fold_deferred_kernel(const float* __restrict__ base, ColsumFoldSlots slots, float* __restrict__ G)
{
    __shared__ float4 seg_sum[4][64];
    const int slot = blockIdx.y;
    const int cols = slots.cols[slot], chunks = slots.chunks[slot];
    if (blockIdx.x * 64 >= cols / 4) return;                      // uniform over the block
    const int lane = threadIdx.x & 63, q = threadIdx.x >> 6;
    const int c4 = blockIdx.x * 64 + lane;
    const bool live = c4 < cols / 4;
    const int seg = (chunks + 3) / 4;
    const int k0 = q * seg, k1 = min(chunks, k0 + seg);
    const float* src = base + slots.part[slot];
    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        int k = k0;
        for (; k + 8 <= k1; k += 8) {
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(k + j) * cols) + c4);
#pragma unroll
            for (int j = 0; j < 8; ++j) { t.x += v[j].x; t.y += v[j].y; t.z += v[j].z; t.w += v[j].w; }
        }
        for (; k < k1; ++k) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(k) * cols) + c4);
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
    }
    seg_sum[q][lane] = t;
    __syncthreads();
    if (q == 0 && live) {
        float4 r = seg_sum[0][lane];
#pragma unroll
        for (int j = 1; j < 4; ++j) { const float4 v = seg_sum[j][lane]; r.x += v.x; r.y += v.y; r.z += v.z; r.w += v.w; }
        float4* dst = reinterpret_cast<float4*>(G + slots.dst[slot]) + c4;
        float4 o = *dst;
        o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
        *dst = o;
    }
}

int colsum_fold_deferred(const float* partial_base, const ColsumFoldSlots& slots, int n, float* G, cudaStream_t s)
{
    if (n == 0) return 0;
    NNB_ARG_CHECK(n <= kColsumFoldMaxSlots, "too many deferred slots");
    int widest = 0;
    for (int i = 0; i < n; ++i) widest = slots.cols[i] > widest ? slots.cols[i] : widest;
    dim3 grid(static_cast<unsigned>(ceil_div(widest / 4, 64)), static_cast<unsigned>(n));
    colsum_fold_deferred_kernel<<<grid, 256, 0, s>>>(partial_base, slots, G);
    LAUNCH_CHECK();
    return 0;
}

template <typename T>
int colsum_accumulate(const T* g, long long ldg, const T* x, const float* gamma, const float* rinv, const float* mean,
                      int mode, float* out, float* scratch, int rows, int cols, cudaStream_t s, int* counters, ColsumDefer* defer)
{
    if (defer) defer->deferred = false;
    if (rows == 0 || cols == 0) return 0;
    constexpr int VN = Vec16<T>::N;
    int chunks = static_cast<int>(ceil_div(rows, CS_CHUNK_ROWS));
    const bool vec = (cols % VN) == 0 && (ldg % VN) == 0 && (reinterpret_cast<uintptr_t>(g) & 15) == 0 &&
                     (mode == 0 || (reinterpret_cast<uintptr_t>(x) & 15) == 0);
    if (vec) {
        // row chunks sized so that the grid is about four blocks per SM: wide matrices get long chunks (more loads
        // in flight per thread, fewer partial rows for the last block to fold), narrow ones keep 128 rows
        const long long col_blocks = ceil_div(cols, 32 * VN);
        int chunk_rows = static_cast<int>(ceil_div(static_cast<long long>(rows) * col_blocks, 4 * kSmCount));
        chunk_rows = static_cast<int>(ceil_div(chunk_rows < CS_CHUNK_ROWS ? CS_CHUNK_ROWS : chunk_rows, 8) * 8);
        chunks = static_cast<int>(ceil_div(rows, chunk_rows));
        dim3 grid(static_cast<unsigned>(col_blocks), chunks);
        if (counters && grid.x > static_cast<unsigned>(kColsumCounters - kNormFoldCounters)) counters = nullptr;   // the last 64 of the 1024 counters are the norm kernel's
        const bool deferring = defer && defer->partial && (cols % 4) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
        float* part = deferring ? defer->partial : scratch;
        int* cnt = deferring ? nullptr : counters;                // without counters the kernel stops after its chunk partials
        if (mode == 0) colsum_vec_kernel<T, 0><<<grid, 256, 0, s>>>(g, ldg, x, gamma, rinv, mean, part, cnt, out, rows, cols, chunks, chunk_rows);
        else colsum_vec_kernel<T, 1><<<grid, 256, 0, s>>>(g, ldg, x, gamma, rinv, mean, part, cnt, out, rows, cols, chunks, chunk_rows);
        LAUNCH_CHECK();
        if (deferring) { defer->chunks = chunks; defer->deferred = true; return 0; }
        if (counters) return 0;
    } else {
        dim3 grid(static_cast<unsigned>(ceil_div(cols, CS_COLS)), chunks);
        if (mode == 0) colsum_partial_kernel<T, 0><<<grid, 256, 0, s>>>(g, ldg, x, gamma, rinv, mean, scratch, rows, cols);
        else colsum_partial_kernel<T, 1><<<grid, 256, 0, s>>>(g, ldg, x, gamma, rinv, mean, scratch, rows, cols);
        LAUNCH_CHECK();
    }
    colsum_final_kernel<<<static_cast<unsigned>(ceil_div(cols, 128)), 128, 0, s>>>(scratch, out, chunks, cols);
    LAUNCH_CHECK();
    return 0;
}
size_t colsum_scratch_floats(int rows, int cols) { return static_cast<size_t>(ceil_div(rows, CS_CHUNK_ROWS)) * cols; }

size_t norm_bwd_scratch_floats(int rows, int d)
{
    const size_t a = colsum_scratch_floats(rows, d);
    const size_t b = static_cast<size_t>(3) * (kNormFusedBlocks + (kNormFusedBlocks + kNormFoldGroup - 1) / kNormFoldGroup) * d;
    return a > b ? a : b;
}

// floats one deferred slot of norm_bwd holds: three quantities x kNormFusedBlocks partial rows
size_t norm_bwd_defer_slot_floats(int d) { return static_cast<size_t>(3) * kNormFusedBlocks * d; }

// folds `n` deferred slots (destinations are offsets into G, -1 = absent) and adds them into the gradients
int norm_bwd_fold_deferred(const float* partials, const NormFoldSlots& slots, int n, float* G, int d, cudaStream_t s)
{
    if (n == 0) return 0;
    NNB_ARG_CHECK(n <= kNormFoldMaxSlots && (d % 4) == 0, "too many deferred slots or unaligned width");
    dim3 grid(static_cast<unsigned>(ceil_div(d / 4, 64)), 3, static_cast<unsigned>(n));
    norm_fold_deferred_kernel<<<grid, 256, 0, s>>>(partials, norm_bwd_defer_slot_floats(d), slots, G, kNormFusedBlocks, d);
    LAUNCH_CHECK();
    return 0;
}

template <typename T>
int norm_bwd(const T* g, const T* x, const float* gamma, const float* rinv, const float* mean, const T* add, T* dx,
             float* dgamma, float* dbeta, float* scratch, int rows, int d, bool layer, cudaStream_t s, int* counters,
             float* out_colsum, float* defer_partial, bool* deferred)
{
    if (deferred) *deferred = false;
    if (rows == 0) return 0;
    const int grid = grid_for(rows, 8);
    constexpr int VN = Vec16<T>::N;
    const bool aligned = ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx) |
                           reinterpret_cast<uintptr_t>(add) | reinterpret_cast<uintptr_t>(gamma)) & 15) == 0;
    const bool out_ok = ((reinterpret_cast<uintptr_t>(dgamma) | reinterpret_cast<uintptr_t>(dbeta) |
                          reinterpret_cast<uintptr_t>(out_colsum)) & 15) == 0;
    // fused path: needs the caller's zero-initialised completion counter and norm_bwd_scratch_floats of scratch
#define NNB_NORM_BWD_FUSED(nv)                                                                                        \
    if (counters && aligned && out_ok && d == 32 * VN * nv) {                                                         \
        const bool defer = defer_partial != nullptr && deferred != nullptr;                                           \
        float* part = defer ? defer_partial : scratch;                                                                \
        constexpr int smem = 8 * 2 * 3 * 32 * VN * nv * static_cast<int>(sizeof(T)) + 8 * 2 * 8;                                       \
        static PerDeviceOnce once_layer, once_rms;                                                                    \
        if (layer) {                                                                                                  \
            NNB_TRY(once_layer.run([] { return cudaFuncSetAttribute(norm_bwd_fused_kernel<T, true, nv>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); })); \
            norm_bwd_fused_kernel<T, true, nv><<<kNormFusedBlocks, 256, smem, s>>>(                                   \
                g, x, gamma, rinv, mean, add, dx, part, counters + kColsumCounters - kNormFoldCounters, dgamma, dbeta, out_colsum, rows, defer ? 1 : 0); \
        } else {                                                                                                      \
            NNB_TRY(once_rms.run([] { return cudaFuncSetAttribute(norm_bwd_fused_kernel<T, false, nv>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); })); \
            norm_bwd_fused_kernel<T, false, nv><<<kNormFusedBlocks, 256, smem, s>>>(                                  \
                g, x, gamma, rinv, mean, add, dx, part, counters + kColsumCounters - kNormFoldCounters, dgamma, dbeta, out_colsum, rows, defer ? 1 : 0); \
        }                                                                                                             \
        LAUNCH_CHECK();                                                                                               \
        if (defer) *deferred = true;                                                                                  \
        return 0;                                                                                                     \
    }
    NNB_NORM_BWD_FUSED(1) NNB_NORM_BWD_FUSED(2) NNB_NORM_BWD_FUSED(3) NNB_NORM_BWD_FUSED(4)
#undef NNB_NORM_BWD_FUSED
    // wide rows (2048 / 4096 bf16 columns): one pass with the parameter gradients accumulated per block, then their fold.
    // The caller's scratch holds colsum_scratch_floats(rows, d) floats, one row of d per 128 matrix rows: that bounds the
    // number of blocks (each leaves one row per quantity); below one block the passes that follow take over.
    const long long wide_rows_of_scratch = static_cast<long long>(colsum_scratch_floats(rows, d) / static_cast<size_t>(d));
    const int wide_blocks = static_cast<int>(std::min<long long>(std::min<long long>(kNormFusedBlocks, ceil_div(rows, d == 256 * VN ? 4 : 2)),
                                                                 wide_rows_of_scratch / (1 + (layer ? 1 : 0) + (out_colsum ? 1 : 0))));
#define NNB_NORM_BWD_WIDE_FUSED(nvt)                                                                                  \
    if (aligned && scratch && d == 256 * VN * nvt && wide_blocks >= 1) {                                              \
        const int blocks = wide_blocks;                                                                               \
        if (layer) norm_bwd_wide_fused_kernel<T, true, nvt><<<blocks, 256, 0, s>>>(g, x, gamma, rinv, mean, add, dx, scratch, rows, out_colsum ? 1 : 0); \
        else norm_bwd_wide_fused_kernel<T, false, nvt><<<blocks, 256, 0, s>>>(g, x, gamma, rinv, mean, add, dx, scratch, rows, out_colsum ? 1 : 0);      \
        LAUNCH_CHECK();                                                                                               \
        const unsigned fold_grid = static_cast<unsigned>(ceil_div(d, 128));                                           \
        const size_t per = static_cast<size_t>(blocks) * d;                                                           \
        colsum_final_kernel<<<fold_grid, 128, 0, s>>>(scratch, dgamma, blocks, d);                                    \
        LAUNCH_CHECK();                                                                                               \
        if (layer) { colsum_final_kernel<<<fold_grid, 128, 0, s>>>(scratch + per, dbeta, blocks, d); LAUNCH_CHECK(); } \
        if (out_colsum) { colsum_final_kernel<<<fold_grid, 128, 0, s>>>(scratch + (layer ? 2 : 1) * per, out_colsum, blocks, d); LAUNCH_CHECK(); } \
        return 0;                                                                                                     \
    }
    NNB_NORM_BWD_WIDE_FUSED(1) NNB_NORM_BWD_WIDE_FUSED(2)
#undef NNB_NORM_BWD_WIDE_FUSED
    // parameter gradients first: dx may alias g
    NNB_TRY(colsum_accumulate<T>(g, d, x, gamma, rinv, layer ? mean : nullptr, 1, dgamma, scratch, rows, d, s, counters));
    if (layer) NNB_TRY(colsum_accumulate<T>(g, d, nullptr, nullptr, nullptr, nullptr, 0, dbeta, scratch, rows, d, s, counters));
    bool done = false;
#define NNB_NORM_BWD_REG(nv)                                                                                          \
    if (!done && aligned && d == 32 * VN * nv) {                                                                      \
        if (layer) norm_bwd_dx_reg_kernel<T, true, nv><<<grid, 256, 0, s>>>(g, x, gamma, rinv, mean, add, dx, rows);   \
        else norm_bwd_dx_reg_kernel<T, false, nv><<<grid, 256, 0, s>>>(g, x, gamma, rinv, mean, add, dx, rows);        \
        LAUNCH_CHECK();                                                                                               \
        done = true;                                                                                                  \
    }
    NNB_NORM_BWD_REG(1) NNB_NORM_BWD_REG(2) NNB_NORM_BWD_REG(3) NNB_NORM_BWD_REG(4)
#undef NNB_NORM_BWD_REG
#define NNB_NORM_BWD_WIDE(nv)                                                                                         \
    if (!done && aligned && d == 32 * VN * nv) {                                                                      \
        const int grid_wide = grid_for(rows, 4, 2);                                                                   \
        const size_t smem = static_cast<size_t>(d) * sizeof(float);                                                   \
        if (layer) norm_bwd_dx_wide_kernel<T, true, nv><<<grid_wide, 128, smem, s>>>(g, x, gamma, rinv, mean, add, dx, rows);  \
        else norm_bwd_dx_wide_kernel<T, false, nv><<<grid_wide, 128, smem, s>>>(g, x, gamma, rinv, mean, add, dx, rows);       \
        LAUNCH_CHECK();                                                                                               \
        done = true;                                                                                                  \
    }
    NNB_NORM_BWD_WIDE(6) NNB_NORM_BWD_WIDE(8) NNB_NORM_BWD_WIDE(12) NNB_NORM_BWD_WIDE(16)
#undef NNB_NORM_BWD_WIDE
    if (!done) {
        if (layer) norm_bwd_dx_kernel<T, true><<<grid, 256, 0, s>>>(g, x, gamma, rinv, mean, add, dx, rows, d);
        else norm_bwd_dx_kernel<T, false><<<grid, 256, 0, s>>>(g, x, gamma, rinv, mean, add, dx, rows, d);
        LAUNCH_CHECK();
    }
    if (out_colsum) NNB_TRY(colsum_accumulate<T>(dx, d, nullptr, nullptr, nullptr, nullptr, 0, out_colsum, scratch, rows, d, s, counters));
    return 0;
}

template <typename T>
int act_fwd(const T* h1, T* h2, int rows, int ff, bool swiglu, cudaStream_t s)
{
    const size_t n = static_cast<size_t>(rows) * ff;
    if (n == 0) return 0;
    if (swiglu) swiglu_fwd_kernel<T><<<grid_for(static_cast<long long>(n / Vec16<T>::N + 1), 256), 256, 0, s>>>(h1, h2, rows, ff);
    else gelu_fwd_kernel<T><<<grid_for(static_cast<long long>(n), 256), 256, 0, s>>>(h1, h2, n);
    LAUNCH_CHECK();
    return 0;
}
template <typename T>
int act_bwd(const T* g, const T* h1, T* dh1, int rows, int ff, bool swiglu, cudaStream_t s, float* dbias, float* scratch,
            int* counters, ColsumDefer* defer)
{
    if (defer) defer->deferred = false;
    const size_t n = static_cast<size_t>(rows) * ff;
    if (n == 0) return 0;
    constexpr int VN = Vec16<T>::N;
    const int width = swiglu ? 2 * ff : ff;
    if (swiglu) swiglu_bwd_kernel<T><<<grid_for(static_cast<long long>(n / VN + 1), 256), 256, 0, s>>>(g, h1, dh1, rows, ff);
    else gelu_bwd_kernel<T><<<grid_for(static_cast<long long>(n), 256), 256, 0, s>>>(g, h1, dh1, n);
    LAUNCH_CHECK();
    if (dbias) NNB_TRY(colsum_accumulate<T>(dh1, width, nullptr, nullptr, nullptr, nullptr, 0, dbias, scratch, rows, width, s, counters, defer));
    return 0;
}
template <typename T>
int cross_entropy(T* logits, const int* labels, const float* mask, float grad_scale, float* loss_vec, float* stats,
                  float* loss_out, int rows, int V, int vocab, cudaStream_t s)
{
    NNB_ARG_CHECK(rows > 0 && V > 0, "empty input");            // compute_loss.hpp:243-244
    NNB_ARG_CHECK(vocab <= V, "vocab_size > classes");          // cpu_engine.hpp:966-967
    ce_count_kernel<<<1, 1024, 0, s>>>(labels, mask, rows, vocab, stats);
    LAUNCH_CHECK();
    constexpr int VN = Vec16<T>::N;
    const bool vec_ok = (V % VN) == 0;
    const int nvec = V / VN;
    // Rows of 32 to 72 KB go through the staged kernel with one slot per block, so that three blocks (64 KB rows) or four
    // share an SM and one block's reductions and stores hide behind the others' passes (16384 x 32768: 532 us, against
    // 662 us with three slots in one block per SM and 843 us register-cached; 16384 x 16384: 300 against 348 us
    // register-cached).  Shorter rows stay with the register-cached kernel (16384 x 8192: 148 us against 185-193 staged).
    const size_t row_bytes = static_cast<size_t>(V) * sizeof(T);
    if (vec_ok && (row_bytes % 16) == 0 && row_bytes >= 32 * 1024 && row_bytes <= 72 * 1024 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        const int slots = 1;
        const int smem = static_cast<int>(slots * row_bytes) + 64;
        static PerDeviceOnce once;
        NNB_TRY(once.run([] { return cudaFuncSetAttribute(ce_staged_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 512); }));
        int per_sm = 0;
        NNB_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ce_staged_kernel<T>, 512, smem));
        if (per_sm > 0) {
            const long long cap = static_cast<long long>(device_sm_count()) * per_sm;
            const int grid = static_cast<int>(rows < cap ? rows : cap);
            ce_staged_kernel<T><<<grid, 512, smem, s>>>(logits, labels, mask, stats, grad_scale, loss_vec, rows, V, vocab, slots);
            LAUNCH_CHECK();
            ce_loss_kernel<<<1, 1024, 0, s>>>(loss_vec, stats, rows, loss_out);
            LAUNCH_CHECK();
            return 0;
        }
    }
    if (vec_ok && nvec <= 512 * 2) ce_fwd_bwd_kernel<T, 2><<<rows, 512, 0, s>>>(logits, labels, mask, stats, grad_scale, loss_vec, rows, V, vocab);
    else if (vec_ok && nvec <= 512 * 4) ce_fwd_bwd_kernel<T, 4><<<rows, 512, 0, s>>>(logits, labels, mask, stats, grad_scale, loss_vec, rows, V, vocab);
    else if (vec_ok && nvec <= 512 * 8) ce_fwd_bwd_kernel<T, 8><<<rows, 512, 0, s>>>(logits, labels, mask, stats, grad_scale, loss_vec, rows, V, vocab);
    else ce_fwd_bwd_kernel<T, 0><<<rows, 512, 0, s>>>(logits, labels, mask, stats, grad_scale, loss_vec, rows, V, vocab);
    LAUNCH_CHECK();
    ce_loss_kernel<<<1, 1024, 0, s>>>(loss_vec, stats, rows, loss_out);
    LAUNCH_CHECK();
    return 0;
}

int adamw_update(float* p, const float* g, float* m, float* v, bf16* shadow, size_t n, float lr, float beta1,
                 float beta2, float eps, float wd, int t_next, const float* gscale, cudaStream_t s)
{
    if (n == 0) return 0;
    // bias_correction_ (compute_optimizer.hpp:312-317): float pow on the host
    const float bc1 = 1.0f - powf(beta1, static_cast<float>(t_next));
    const float bc2 = 1.0f - powf(beta2, static_cast<float>(t_next));
    const float decay = (wd != 0.f) ? 1.0f - lr * wd : 1.0f;
    adamw_kernel<<<grid_for(static_cast<long long>(n), 256), 256, 0, s>>>(p, g, m, v, shadow, n, lr, beta1, beta2, eps,
                                                                         decay, 1.0f / bc1, 1.0f / bc2, gscale);
    LAUNCH_CHECK();
    return 0;
}

constexpr int SUMSQ_BLOCKS = kSmCount * 4;
size_t sumsq_scratch_floats() { return SUMSQ_BLOCKS; }

int sum_squares(const float* g, size_t n, float pre_scale, float max_norm, float post_scale, float* scratch, float* out,
                cudaStream_t s)
{
    const int blocks = n == 0 ? 1 : grid_for(static_cast<long long>(n), 256, 4);
    sumsq_partial_kernel<<<blocks, 256, 0, s>>>(g, n, scratch);
    LAUNCH_CHECK();
    sumsq_final_kernel<<<1, 1024, 0, s>>>(scratch, blocks, pre_scale, max_norm, post_scale, out);
    LAUNCH_CHECK();
    return 0;
}

int muon_momentum(const float* g, float* vel, float* u, size_t n, float mu, const float* gscale, cudaStream_t s)
{
    if (n == 0) return 0;
    muon_momentum_kernel<<<grid_for(static_cast<long long>(n), 256), 256, 0, s>>>(g, vel, u, n, mu, gscale);
    LAUNCH_CHECK();
    return 0;
}
template <typename T>
int muon_normalize(const float* u, const float* sumsq, float eps, T* X, size_t n, cudaStream_t s)
{
    muon_normalize_kernel<T><<<grid_for(static_cast<long long>(n), 256), 256, 0, s>>>(u, sumsq, eps, X, n);
    LAUNCH_CHECK();
    return 0;
}
template <typename T>
int axpby(const T* a, const T* b, T* out, float alpha, float beta, size_t n, cudaStream_t s)
{
    axpby_kernel<T><<<grid_for(static_cast<long long>(n), 256), 256, 0, s>>>(a, b, out, alpha, beta, n);
    LAUNCH_CHECK();
    return 0;
}
template <typename T>
int muon_apply(float* p, const T* X, bf16* shadow, float lr, size_t n, cudaStream_t s)
{
    muon_apply_kernel<T><<<grid_for(static_cast<long long>(n), 256), 256, 0, s>>>(p, X, shadow, lr, n);
    LAUNCH_CHECK();
    return 0;
}
int f32_to_bf16(const float* in, bf16* out, size_t n, cudaStream_t s)
{
    if (n == 0) return 0;
    f32_to_bf16_kernel<<<grid_for(static_cast<long long>(n), 256), 256, 0, s>>>(in, out, n);
    LAUNCH_CHECK();
    return 0;
}
int bf16_to_f32(const bf16* in, float* out, size_t n, cudaStream_t s)
{
    if (n == 0) return 0;
    bf16_to_f32_kernel<<<grid_for(static_cast<long long>(n), 256), 256, 0, s>>>(in, out, n);
    LAUNCH_CHECK();
    return 0;
}

#define INSTANTIATE(T)                                                                                                 \
    template int norm_fwd<T>(const T*, const float*, const float*, T*, float*, float*, int, int, bool, cudaStream_t);  \
    template int norm_bwd<T>(const T*, const T*, const float*, const float*, const float*, const T*, T*, float*,       \
                             float*, float*, int, int, bool, cudaStream_t, int*, float*, float*, bool*);                \
    template int colsum_accumulate<T>(const T*, long long, const T*, const float*, const float*, const float*, int,    \
                                      float*, float*, int, int, cudaStream_t, int*, ColsumDefer*);                     \
    template int act_fwd<T>(const T*, T*, int, int, bool, cudaStream_t);                                               \
    template int act_bwd<T>(const T*, const T*, T*, int, int, bool, cudaStream_t, float*, float*, int*, ColsumDefer*); \
    template int cross_entropy<T>(T*, const int*, const float*, float, float*, float*, float*, int, int, int,          \
                                  cudaStream_t);                                                                       \
    template int muon_normalize<T>(const float*, const float*, float, T*, size_t, cudaStream_t);                       \
    template int axpby<T>(const T*, const T*, T*, float, float, size_t, cudaStream_t);                                 \
    template int muon_apply<T>(float*, const T*, bf16*, float, size_t, cudaStream_t);
INSTANTIATE(float)
INSTANTIATE(bf16)

}  // namespace nnb
