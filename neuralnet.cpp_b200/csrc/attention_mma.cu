// Fused causal / document-masked / ALiBi attention on bf16 tensor cores (mma.sync m16n8k16, fp32
// accumulate), flash style: scores, mask and probabilities live in registers only.
// Replaces the reference's five two-pass primitives and its materialised (B*H*S, S) path
// (compute_layer.hpp:1193-1252, 1296-1360; cpu_engine.hpp:426-915).
//
// Layout as in attention_simt.cu: qkv (tokens, 3d) = q | k | v, head h at columns h*dk; out/dout
// (tokens, d); lse/dvec (B*H*S).  A CTA is 4 warps x 16 rows = 64 queries (or 64 keys in the dK/dV
// kernel) and walks 64-row tiles of the other operand through swizzled shared memory.
//   forward : S = Q K^T, online softmax, O += P V
//   dQ      : S, dP = dO V^T, dS = P o (dP - D), dQ += dS K          (CTA per query tile)
//   dK, dV  : S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q (CTA per key tile)
// dQ and dK/dV are separate kernels so that no gradient needs atomics: results are deterministic.
#include "kernels.h"

namespace nnb {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// 64 x DK bf16 tile, rows of DK*2 bytes, 16-byte chunks XOR-swizzled so ldmatrix is conflict free
template <int DK> __device__ __forceinline__ uint32_t tile_off(int row, int chunk)
{
    const int sw = (DK == 32) ? ((row >> 1) & 3) : (row & 7);
    return static_cast<uint32_t>(row * (DK * 2) + ((chunk ^ sw) << 4));
}

// copy rows [row0, row0+64) x DK columns of a (rows, ld) matrix into a tile; rows >= limit become zero
template <int DK>
__device__ __forceinline__ void load_tile(uint32_t smem_base, const bf16* __restrict__ src, long long ld, int row0, int limit)
{
    constexpr int CH = DK / 8;
    for (int idx = threadIdx.x; idx < 64 * CH; idx += 128) {
        const int r = idx / CH, c = idx % CH;
        const uint32_t dst = smem_base + tile_off<DK>(r, c);
        if (row0 + r < limit) cp_async16(dst, src + static_cast<long long>(row0 + r) * ld + c * 8);
        else asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0) : "memory");
    }
}

template <int DK> __device__ __forceinline__ void load_a_frags(uint32_t tile, int row0, uint32_t (&f)[DK / 16][4])
{
    const int l = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < DK / 16; ++kk)
        ldsm_x4(tile + tile_off<DK>(row0 + (l & 7) + 8 * ((l >> 3) & 1), kk * 2 + (l >> 4)), f[kk][0], f[kk][1], f[kk][2], f[kk][3]);
}

// acc[nt] += A(16 x DK) * Tile(64 rows as n, DK as k)^T
template <int DK>
__device__ __forceinline__ void mma_a_tileT(float (&acc)[8][4], const uint32_t (&a)[DK / 16][4], uint32_t tile)
{
    const int l = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < DK / 16; ++kk)
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(tile + tile_off<DK>(np * 16 + (l & 7) + 8 * (l >> 4), kk * 2 + ((l >> 3) & 1)), b0, b1, b2, b3);
            mma16816(acc[np * 2], a[kk], b0, b1);
            mma16816(acc[np * 2 + 1], a[kk], b2, b3);
        }
}
// out[nt over DK/8] += P(16 x 64, packed from accumulators) * Tile(64 rows as k, DK as n)
template <int DK>
__device__ __forceinline__ void mma_p_tile(float (&out)[DK / 8][4], const uint32_t (&pa)[4][4], uint32_t tile)
{
    const int l = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
#pragma unroll
        for (int np = 0; np < DK / 16; ++np) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(tile + tile_off<DK>(kk * 16 + (l & 7) + 8 * ((l >> 3) & 1), np * 2 + (l >> 4)), b0, b1, b2, b3);
            mma16816(out[np * 2], pa[kk], b0, b1);
            mma16816(out[np * 2 + 1], pa[kk], b2, b3);
        }
}
__device__ __forceinline__ void pack_p(const float (&s)[8][4], uint32_t (&pa)[4][4])
{
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        pa[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    }
}

struct AttnArgs {
    const bf16* qkv; const bf16* out; const bf16* dout; bf16* o_out; bf16* dqkv;
    float* lse; const float* dvec; const int* doc;
    int B, S, H, alibi;
    float scale;
};

__device__ __forceinline__ float head_slope2(const AttnArgs& a, int h)
{
    return a.alibi ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(a.H)) * kLog2e : 0.f;
}

// ---------------------------------------------------------------- forward
template <int DK>
__global__ void __launch_bounds__(128)
attn_fwd_mma_kernel(const AttnArgs a)
{
    __shared__ __align__(128) uint8_t smem[3 * 64 * DK * 2];
    __shared__ int sdoc_k[64];
    const uint32_t sQ = smem_u32(smem), sK = sQ + 64 * DK * 2, sV = sK + 64 * DK * 2;
    const int qb = gridDim.x - 1 - blockIdx.x;            // heavy (late) query tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int d = a.H * DK;
    const long long ld = 3LL * d;
    const bf16* qbase = a.qkv + static_cast<long long>(b) * a.S * ld + h * DK;
    const bf16* kbase = qbase + d;
    const bf16* vbase = kbase + d;
    const int q0 = qb * 64;

    load_tile<DK>(sQ, qbase, ld, q0, a.S);
    cp_async_wait_all();
    __syncthreads();
    uint32_t qf[DK / 16][4];
    load_a_frags<DK>(sQ, warp * 16, qf);

    const float scale2 = a.scale * kLog2e, slope2 = head_slope2(a, h);
    const int i0 = q0 + warp * 16 + g, i1 = i0 + 8;
    const int doc0 = (a.doc && i0 < a.S) ? a.doc[b * a.S + i0] : 0, doc1 = (a.doc && i1 < a.S) ? a.doc[b * a.S + i1] : 0;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[DK / 8][4];
#pragma unroll
    for (int n = 0; n < DK / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }

    for (int kb = 0; kb <= qb; ++kb) {
        const int k0 = kb * 64;
        __syncthreads();                                   // previous tile fully consumed
        load_tile<DK>(sK, kbase, ld, k0, a.S);
        load_tile<DK>(sV, vbase, ld, k0, a.S);
        if (a.doc && threadIdx.x < 64) sdoc_k[threadIdx.x] = (k0 + threadIdx.x < a.S) ? a.doc[b * a.S + k0 + threadIdx.x] : -1;
        cp_async_wait_all();
        __syncthreads();

        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        mma_a_tileT<DK>(s, qf, sK);

        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = k0 + n * 8 + 2 * t + (e & 1);
                const int i = (e < 2) ? i0 : i1;
                bool ok = j <= i && j < a.S;
                if (a.doc) ok = ok && sdoc_k[j - k0] == ((e < 2) ? doc0 : doc1);
                const float v = ok ? s[n][e] * scale2 - slope2 * static_cast<float>(i - j) : -INFINITY;
                s[n][e] = v;
                if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0, ms1 = (mn1 == -INFINITY) ? 0.f : mn1;
        const float c0 = exp2f(m0 - ms0), c1 = exp2f(m1 - ms1);
        m0 = mn0; m1 = mn1;
        float r0 = 0.f, r1 = 0.f;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            s[n][0] = exp2f(s[n][0] - ms0); s[n][1] = exp2f(s[n][1] - ms0);
            s[n][2] = exp2f(s[n][2] - ms1); s[n][3] = exp2f(s[n][3] - ms1);
            r0 += s[n][0] + s[n][1]; r1 += s[n][2] + s[n][3];
        }
        l0 = l0 * c0 + r0; l1 = l1 * c1 + r1;
#pragma unroll
        for (int n = 0; n < DK / 8; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
        uint32_t pa[4][4];
        pack_p(s, pa);
        mma_p_tile<DK>(o, pa, sV);
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
    bf16* ob = a.o_out + static_cast<long long>(b) * a.S * d + h * DK;
#pragma unroll
    for (int n = 0; n < DK / 8; ++n) {
        const int c = n * 8 + 2 * t;
        if (i0 < a.S) *reinterpret_cast<uint32_t*>(ob + static_cast<long long>(i0) * d + c) = pack_bf16(o[n][0] * inv0, o[n][1] * inv0);
        if (i1 < a.S) *reinterpret_cast<uint32_t*>(ob + static_cast<long long>(i1) * d + c) = pack_bf16(o[n][2] * inv1, o[n][3] * inv1);
    }
    if (t == 0) {
        const long long r = (static_cast<long long>(b) * a.H + h) * a.S;
        if (i0 < a.S) a.lse[r + i0] = (m0 + log2f(l0)) * kLn2;
        if (i1 < a.S) a.lse[r + i1] = (m1 + log2f(l1)) * kLn2;
    }
}

// ---------------------------------------------------------------- backward: dQ
template <int DK>
__global__ void __launch_bounds__(128)
attn_bwd_dq_mma_kernel(const AttnArgs a)
{
    __shared__ __align__(128) uint8_t smem[3 * 64 * DK * 2];
    __shared__ int sdoc_k[64];
    const uint32_t sQ = smem_u32(smem), sK = sQ + 64 * DK * 2, sV = sK + 64 * DK * 2;
    const int qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int d = a.H * DK;
    const long long ld = 3LL * d;
    const bf16* qbase = a.qkv + static_cast<long long>(b) * a.S * ld + h * DK;
    const bf16* kbase = qbase + d;
    const bf16* vbase = kbase + d;
    const bf16* gbase = a.dout + static_cast<long long>(b) * a.S * d + h * DK;
    const int q0 = qb * 64;

    uint32_t qf[DK / 16][4], gf[DK / 16][4];
    load_tile<DK>(sQ, qbase, ld, q0, a.S);
    load_tile<DK>(sK, gbase, d, q0, a.S);                  // dO staged through the K buffer
    cp_async_wait_all();
    __syncthreads();
    load_a_frags<DK>(sQ, warp * 16, qf);
    load_a_frags<DK>(sK, warp * 16, gf);

    const float scale2 = a.scale * kLog2e, slope2 = head_slope2(a, h);
    const int i0 = q0 + warp * 16 + g, i1 = i0 + 8;
    const long long r = (static_cast<long long>(b) * a.H + h) * a.S;
    const float L0 = (i0 < a.S) ? a.lse[r + i0] * kLog2e : 0.f, L1 = (i1 < a.S) ? a.lse[r + i1] * kLog2e : 0.f;
    const float D0 = (i0 < a.S) ? a.dvec[r + i0] : 0.f, D1 = (i1 < a.S) ? a.dvec[r + i1] : 0.f;
    const int doc0 = (a.doc && i0 < a.S) ? a.doc[b * a.S + i0] : 0, doc1 = (a.doc && i1 < a.S) ? a.doc[b * a.S + i1] : 0;
    float dq[DK / 8][4];
#pragma unroll
    for (int n = 0; n < DK / 8; ++n) { dq[n][0] = dq[n][1] = dq[n][2] = dq[n][3] = 0.f; }

    for (int kb = 0; kb <= qb; ++kb) {
        const int k0 = kb * 64;
        __syncthreads();
        load_tile<DK>(sK, kbase, ld, k0, a.S);
        load_tile<DK>(sV, vbase, ld, k0, a.S);
        if (a.doc && threadIdx.x < 64) sdoc_k[threadIdx.x] = (k0 + threadIdx.x < a.S) ? a.doc[b * a.S + k0 + threadIdx.x] : -1;
        cp_async_wait_all();
        __syncthreads();
        float s[8][4], dp[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; dp[n][0] = dp[n][1] = dp[n][2] = dp[n][3] = 0.f; }
        mma_a_tileT<DK>(s, qf, sK);
        mma_a_tileT<DK>(dp, gf, sV);
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = k0 + n * 8 + 2 * t + (e & 1);
                const int i = (e < 2) ? i0 : i1;
                bool ok = j <= i && j < a.S && i < a.S;
                if (a.doc) ok = ok && sdoc_k[j - k0] == ((e < 2) ? doc0 : doc1);
                const float p = ok ? exp2f(s[n][e] * scale2 - slope2 * static_cast<float>(i - j) - ((e < 2) ? L0 : L1)) : 0.f;
                s[n][e] = p * (dp[n][e] - ((e < 2) ? D0 : D1));
            }
        uint32_t pa[4][4];
        pack_p(s, pa);
        mma_p_tile<DK>(dq, pa, sK);
    }
    bf16* ob = a.dqkv + static_cast<long long>(b) * a.S * ld + h * DK;
#pragma unroll
    for (int n = 0; n < DK / 8; ++n) {
        const int c = n * 8 + 2 * t;
        if (i0 < a.S) *reinterpret_cast<uint32_t*>(ob + static_cast<long long>(i0) * ld + c) = pack_bf16(dq[n][0] * a.scale, dq[n][1] * a.scale);
        if (i1 < a.S) *reinterpret_cast<uint32_t*>(ob + static_cast<long long>(i1) * ld + c) = pack_bf16(dq[n][2] * a.scale, dq[n][3] * a.scale);
    }
}

// ---------------------------------------------------------------- backward: dK, dV
template <int DK>
__global__ void __launch_bounds__(128)
attn_bwd_dkv_mma_kernel(const AttnArgs a)
{
    __shared__ __align__(128) uint8_t smem[3 * 64 * DK * 2];
    __shared__ int sdoc_q[64];
    __shared__ float slse[64], sdv[64];
    const uint32_t sK = smem_u32(smem), sQ = sK + 64 * DK * 2, sG = sQ + 64 * DK * 2;
    const int kb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int d = a.H * DK;
    const long long ld = 3LL * d;
    const bf16* qbase = a.qkv + static_cast<long long>(b) * a.S * ld + h * DK;
    const bf16* kbase = qbase + d;
    const bf16* vbase = kbase + d;
    const bf16* gbase = a.dout + static_cast<long long>(b) * a.S * d + h * DK;
    const int k0 = kb * 64;
    const int nqb = static_cast<int>(ceil_div(a.S, 64));

    uint32_t kf[DK / 16][4], vf[DK / 16][4];
    load_tile<DK>(sK, kbase, ld, k0, a.S);
    load_tile<DK>(sQ, vbase, ld, k0, a.S);                 // V staged through the Q buffer
    cp_async_wait_all();
    __syncthreads();
    load_a_frags<DK>(sK, warp * 16, kf);
    load_a_frags<DK>(sQ, warp * 16, vf);

    const float scale2 = a.scale * kLog2e, slope2 = head_slope2(a, h);
    const int j0 = k0 + warp * 16 + g, j1 = j0 + 8;
    const int doc0 = (a.doc && j0 < a.S) ? a.doc[b * a.S + j0] : 0, doc1 = (a.doc && j1 < a.S) ? a.doc[b * a.S + j1] : 0;
    const long long r = (static_cast<long long>(b) * a.H + h) * a.S;
    float dk[DK / 8][4], dv[DK / 8][4];
#pragma unroll
    for (int n = 0; n < DK / 8; ++n) { dk[n][0] = dk[n][1] = dk[n][2] = dk[n][3] = 0.f; dv[n][0] = dv[n][1] = dv[n][2] = dv[n][3] = 0.f; }

    for (int qb = kb; qb < nqb; ++qb) {
        const int q0 = qb * 64;
        __syncthreads();
        load_tile<DK>(sQ, qbase, ld, q0, a.S);
        load_tile<DK>(sG, gbase, d, q0, a.S);
        if (threadIdx.x < 64) {
            const int i = q0 + threadIdx.x;
            slse[threadIdx.x] = (i < a.S) ? a.lse[r + i] * kLog2e : 0.f;
            sdv[threadIdx.x] = (i < a.S) ? a.dvec[r + i] : 0.f;
            if (a.doc) sdoc_q[threadIdx.x] = (i < a.S) ? a.doc[b * a.S + i] : -1;
        }
        cp_async_wait_all();
        __syncthreads();
        float st[8][4], dpt[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) { st[n][0] = st[n][1] = st[n][2] = st[n][3] = 0.f; dpt[n][0] = dpt[n][1] = dpt[n][2] = dpt[n][3] = 0.f; }
        mma_a_tileT<DK>(st, kf, sQ);                       // S^T  = K Q^T   (rows keys, cols queries)
        mma_a_tileT<DK>(dpt, vf, sG);                      // dP^T = V dO^T
        uint32_t pa[4][4];
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int il = n * 8 + 2 * t + (e & 1);
                const int i = q0 + il;
                const int j = (e < 2) ? j0 : j1;
                bool ok = j <= i && i < a.S && j < a.S;
                if (a.doc) ok = ok && sdoc_q[il] == ((e < 2) ? doc0 : doc1);
                const float p = ok ? exp2f(st[n][e] * scale2 - slope2 * static_cast<float>(i - j) - slse[il]) : 0.f;
                st[n][e] = p;
                dpt[n][e] = p * (dpt[n][e] - sdv[il]);
            }
        pack_p(st, pa);
        mma_p_tile<DK>(dv, pa, sG);                        // dV += P^T dO
        pack_p(dpt, pa);
        mma_p_tile<DK>(dk, pa, sQ);                        // dK += dS^T Q
    }
    bf16* ob = a.dqkv + static_cast<long long>(b) * a.S * ld + d + h * DK;
#pragma unroll
    for (int n = 0; n < DK / 8; ++n) {
        const int c = n * 8 + 2 * t;
        if (j0 < a.S) {
            *reinterpret_cast<uint32_t*>(ob + static_cast<long long>(j0) * ld + c) = pack_bf16(dk[n][0] * a.scale, dk[n][1] * a.scale);
            *reinterpret_cast<uint32_t*>(ob + static_cast<long long>(j0) * ld + d + c) = pack_bf16(dv[n][0], dv[n][1]);
        }
        if (j1 < a.S) {
            *reinterpret_cast<uint32_t*>(ob + static_cast<long long>(j1) * ld + c) = pack_bf16(dk[n][2] * a.scale, dk[n][3] * a.scale);
            *reinterpret_cast<uint32_t*>(ob + static_cast<long long>(j1) * ld + d + c) = pack_bf16(dv[n][2], dv[n][3]);
        }
    }
}

template <int DK>
static int run_fwd(const AttnArgs& a, cudaStream_t s)
{
    dim3 grid(static_cast<unsigned>(ceil_div(a.S, 64)), a.H, a.B);
    attn_fwd_mma_kernel<DK><<<grid, 128, 0, s>>>(a);
    NNB_LAUNCH_CHECK();
    return 0;
}
template <int DK>
static int run_bwd(const AttnArgs& a, cudaStream_t s)
{
    dim3 grid(static_cast<unsigned>(ceil_div(a.S, 64)), a.H, a.B);
    attn_bwd_dq_mma_kernel<DK><<<grid, 128, 0, s>>>(a);
    NNB_LAUNCH_CHECK();
    attn_bwd_dkv_mma_kernel<DK><<<grid, 128, 0, s>>>(a);
    NNB_LAUNCH_CHECK();
    return 0;
}

bool attention_mma_supported(int dk, int d) { return (dk == 32 || dk == 64) && (d % 8) == 0; }

int attention_fwd_mma(const bf16* qkv, bf16* out, float* lse, const int* doc, int B, int S, int H, int dk, int alibi,
                      cudaStream_t s)
{
    if (static_cast<long long>(B) * S * H == 0) return 0;
    NNB_ARG_CHECK(B <= 65535 && H <= 65535, "batch / heads exceed the grid limits");
    AttnArgs a{};
    a.qkv = qkv; a.o_out = out; a.lse = lse; a.doc = doc; a.B = B; a.S = S; a.H = H; a.alibi = alibi;
    a.scale = 1.0f / sqrtf(static_cast<float>(dk));
    if (dk == 64) return run_fwd<64>(a, s);
    if (dk == 32) return run_fwd<32>(a, s);
    return -1;
}

int attention_bwd_mma(const bf16* qkv, const bf16* out, const bf16* dout, const float* lse, float* dvec, bf16* dqkv,
                      const int* doc, int B, int S, int H, int dk, int alibi, cudaStream_t s)
{
    if (static_cast<long long>(B) * S * H == 0) return 0;
    NNB_ARG_CHECK(B <= 65535 && H <= 65535, "batch / heads exceed the grid limits");
    NNB_TRY(attention_dvec_bf16(out, dout, dvec, B, S, H, dk, s));
    AttnArgs a{};
    a.qkv = qkv; a.out = out; a.dout = dout; a.dqkv = dqkv; a.lse = const_cast<float*>(lse); a.dvec = dvec; a.doc = doc;
    a.B = B; a.S = S; a.H = H; a.alibi = alibi;
    a.scale = 1.0f / sqrtf(static_cast<float>(dk));
    if (dk == 64) return run_bwd<64>(a, s);
    if (dk == 32) return run_bwd<32>(a, s);
    return -1;
}

}  // namespace nnb
