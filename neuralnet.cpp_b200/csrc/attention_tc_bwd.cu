// Attention backward on the 5th-generation tensor cores: two kernels, no atomics.
//
//   dQ kernel   tile = 128 queries, loop over 64-key blocks up to the diagonal:
//                 S = Q K^T, dP = dO V^T (TMEM, double-buffered) -> workers: P = exp2(S*scale+bias-lse),
//                 dS = P o (dP - D) as bf16 into a K-major shared tile -> dQ += dS K (TMEM accumulator)
//   dK/dV kernel tile = 128 keys, loop over 64-query blocks from the diagonal to the end:
//                 S^T = K Q^T, dP^T = V dO^T -> workers: P^T, dS^T as bf16 tiles ->
//                 dV += P^T dO, dK += dS^T Q (TMEM accumulators)
// Ten warps per CTA: warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 workers; worker (row, half)
// owns one TMEM lane (query resp. key) and 32 of the 64 columns of each block, so workers never
// synchronise with each other.  K/V resp. Q/dO tiles are consumed both K-major (first MMAs) and
// MN-major (second MMAs) from the same shared-memory tile.  Recomputing S in both kernels keeps the
// gradients deterministic (the reference's backward_q / backward_kv split, cpu_engine.hpp:702-915).
#include <type_traits>

#include "kernels.h"
#include "tc_ptx.cuh"

namespace nnb {

__device__ int g_attn_bwd_error = 0;

constexpr int BT = 128 * 128;          // bytes of a 128-row x 64-bf16 tile
constexpr int HT = 64 * 128;           // bytes of a 64-row tile
constexpr float kL2e = 1.4426950408889634f;

struct AttnBwdArgs {
    bf16* dqkv; const float* lse; const float* dvec; const int* doc;
    int B, S, H;
    float scale;
};

__device__ __forceinline__ float ex2a(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// fp32 accumulate, bf16 operands, M = 128, N = 64; B operand K-major or MN-major
constexpr uint32_t IDESC_KK = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(64 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
constexpr uint32_t IDESC_KM = IDESC_KK | (1u << 16);

// Both kernels are persistent: the CTAs resident on an SM walk a list of (tile, head, batch) work items, heaviest
// tiles first, in snake order.  The rings, score buffers and barrier phases run on across tiles, so the loads and
// first MMAs of the next tile overlap the tail and the write-out of the current one.  Two builds of each kernel:
//   NB = 1 (default)  two CTAs per SM, every resource single-buffered (K/V ring of 2, 256 TMEM columns, 80 / 97 KB of
//                     shared memory, 96 registers): while the workers of one CTA are in their dependency chain
//                     (scores ready -> tcgen05.ld -> exp -> dS tile -> next MMA) the other CTA's MMAs run.
//                     Measured 219 us against 255 us per layer at batch 16 x 12 heads x 1024.
//   NB = 2            one CTA per SM with the resident tile, the score buffers and the TMEM gradient accumulators
//                     double-buffered inside the CTA (environment NNB200_ATTN_BWD_CTAS=1, for comparison).
struct BwdTile { int t, h, b; };
__device__ __forceinline__ BwdTile bwd_tile(int w, int H, int HB)
{
    BwdTile r;
    const int hb = w % HB;
    r.t = w / HB;
    r.h = hb % H;
    r.b = hb / H;
    return r;
}

// ======================================================================================
// dQ
// ======================================================================================
// shared memory: Q (2) | dO (2) | ring of (K, V) 64-key tiles | dS (2 buffers) | barriers
// NB = buffers per resource: 2 (one CTA per SM, everything double-buffered inside the CTA) or 1 (two CTAs per SM, each
// single-buffered, so that one CTA's MMAs run while the other's workers are in their dependency chain)
template <int NB> struct DqLayout {
    static constexpr int ST = NB + 1;                               // (K, V) ring stages
    static constexpr int OFF_DO = NB * BT, OFF_RING = 2 * NB * BT, OFF_DS = OFF_RING + ST * 2 * HT, OFF_BAR = OFF_DS + NB * BT,
                         SMEM = OFF_BAR + 256;
    static constexpr uint32_t TMEM_COLS = NB == 2 ? 512u : 256u;    // S | dP | dQ, 64 columns per buffer
};

template <bool DOC, bool ALIBI, int NB>
__global__ void __launch_bounds__(320, 3 - NB)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ128, const __grid_constant__ CUtensorMap tmKV64,
                      const __grid_constant__ CUtensorMap tmDO128, const AttnBwdArgs a)
{
    using LY = DqLayout<NB>;
    constexpr int ST = LY::ST;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;                            // tile buffer q at +q*BT
    uint8_t* sDO = smem + LY::OFF_DO;
    uint8_t* sRing = smem + LY::OFF_RING;           // stage s: K at +s*2*HT, V right after
    uint8_t* sDS = smem + LY::OFF_DS;               // buffer b at +b*BT
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + LY::OFF_BAR);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full0 = bar0, q_empty0 = bar0 + 16, kv_full0 = bar0 + 32, kv_empty0 = bar0 + 56, sp_full0 = bar0 + 80,
                   sp_empty0 = bar0 + 96, ds_full0 = bar0 + 112, ds_empty0 = bar0 + 128, done0 = bar0 + 144, acc_empty0 = bar0 + 160;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = a.H * 64;
    const int nt = a.S / 128, HB = a.H * a.B, total = nt * HB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(q_full0 + 8 * s, 1); mbar_init(q_empty0 + 8 * s, 1); }
        for (int s = 0; s < ST; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(sp_full0 + 8 * s, 1); mbar_init(sp_empty0 + 8 * s, 8);
            mbar_init(ds_full0 + 8 * s, 8); mbar_init(ds_empty0 + 8 * s, 1);
            mbar_init(done0 + 8 * s, 1); mbar_init(acc_empty0 + 8 * s, 8);
        }
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;
        if (*abort_flag) atomicCAS(&g_attn_bwd_error, 0, (9 << 16));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(DqLayout<NB>::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // TMEM columns, 64 per buffer: S buffers first, then the dP buffers, then the dQ accumulators

    if (warp == 0) {
        if (lane == 0 && !*abort_flag) {
            int kv = 0, tn = 0;
            bool ok = true;
            for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
                const BwdTile t = bwd_tile(w, a.H, HB);
                const int qb = nt - 1 - t.t, q0 = qb * 128, nkb = 2 * (qb + 1), row_base = t.b * a.S, qs = tn % NB;
                if (!mbar_wait(q_empty0 + 8 * qs, ((tn / NB) & 1) ^ 1, abort_flag, 11, &g_attn_bwd_error)) break;
                mbar_expect_tx(q_full0 + 8 * qs, 2 * BT);
                tma_load_2d(smem_u32(sQ + qs * BT), &tmQ128, q_full0 + 8 * qs, t.h * 64, row_base + q0);
                tma_load_2d(smem_u32(sDO + qs * BT), &tmDO128, q_full0 + 8 * qs, t.h * 64, row_base + q0);
                for (int kb = 0; kb < nkb; ++kb, ++kv) {
                    const int st = kv % ST;
                    if (!mbar_wait(kv_empty0 + 8 * st, ((kv / ST) & 1) ^ 1, abort_flag, 1, &g_attn_bwd_error)) { ok = false; break; }
                    mbar_expect_tx(kv_full0 + 8 * st, 2 * HT);
                    const uint32_t dst = smem_u32(sRing + st * 2 * HT);
                    tma_load_2d(dst, &tmKV64, kv_full0 + 8 * st, d + t.h * 64, row_base + kb * 64);
                    tma_load_2d(dst + HT, &tmKV64, kv_full0 + 8 * st, 2 * d + t.h * 64, row_base + kb * 64);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && !*abort_flag) {
            int kv0 = 0, tn = 0;
            bool ok = true;
            for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
                const BwdTile t = bwd_tile(w, a.H, HB);
                const int nkb = 2 * (nt - t.t), qs = tn % NB, use = tn / NB;
                ok = mbar_wait(q_full0 + 8 * qs, use & 1, abort_flag, 2, &g_attn_bwd_error);
                // the accumulator this tile writes was read out two tiles ago
                if (ok && use >= 1) ok = mbar_wait(acc_empty0 + 8 * qs, (use - 1) & 1, abort_flag, 12, &g_attn_bwd_error);
                const uint32_t q_addr = smem_u32(sQ + qs * BT), do_addr = smem_u32(sDO + qs * BT);
                const uint32_t tmem_dQ = tmem_base + 2 * NB * 64 + qs * 64;
                auto issue_sdp = [&](int gj) -> bool {
                    const int st = gj % ST, sb = gj % NB, u = gj / NB;
                    if (!mbar_wait(kv_full0 + 8 * st, (gj / ST) & 1, abort_flag, 3, &g_attn_bwd_error)) return false;
                    if (u >= 1 && !mbar_wait(sp_empty0 + 8 * sb, (u - 1) & 1, abort_flag, 4, &g_attn_bwd_error)) return false;
                    tc_fence_after();
                    const uint32_t k_addr = smem_u32(sRing + st * 2 * HT), v_addr = k_addr + HT;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base + sb * 64, smem_desc(q_addr + k * 32, 16, 1024), smem_desc(k_addr + k * 32, 16, 1024), IDESC_KK, k > 0);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base + NB * 64 + sb * 64, smem_desc(do_addr + k * 32, 16, 1024), smem_desc(v_addr + k * 32, 16, 1024), IDESC_KK, k > 0);
                    umma_commit(sp_full0 + 8 * sb);
                    return true;
                };
                auto issue_dq = [&](int gj, bool first) -> bool {
                    const int st = gj % ST, sb = gj % NB;
                    if (!mbar_wait(ds_full0 + 8 * sb, (gj / NB) & 1, abort_flag, 5, &g_attn_bwd_error)) return false;
                    tc_fence_after();
                    const uint32_t ds_addr = smem_u32(sDS + sb * BT), k_addr = smem_u32(sRing + st * 2 * HT);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_dQ, smem_desc(ds_addr + k * 32, 16, 1024), smem_desc(k_addr + k * 2048, HT, 1024), IDESC_KM, (!first || k > 0));
                    umma_commit(ds_empty0 + 8 * sb);
                    umma_commit(kv_empty0 + 8 * st);
                    return true;
                };
                if (ok) ok = issue_sdp(kv0);
                for (int kb = 0; ok && kb < nkb; ++kb) {
                    if (kb + 1 < nkb) ok = issue_sdp(kv0 + kb + 1);
                    if (ok) ok = issue_dq(kv0 + kb, kb == 0);
                }
                if (ok) { umma_commit(done0 + 8 * qs); umma_commit(q_empty0 + 8 * qs); }
                kv0 += nkb;
            }
        }
    } else {
        const int q = warp & 3, hf = (warp - 2) >> 2;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
        const float scale2 = a.scale * kL2e;
        const int sw = row & 7;
        bool ok = !*abort_flag;
        int kv0 = 0, tn = 0;

        for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
            const BwdTile t = bwd_tile(w, a.H, HB);
            const int h = t.h, b = t.b, qb = nt - 1 - t.t, q0 = qb * 128, nkb = 2 * (qb + 1), row_base = b * a.S;
            const int i = q0 + row;
            const float slope2 = ALIBI ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(a.H)) * kL2e : 0.f;
            const int my_doc = DOC ? a.doc[row_base + i] : 0;
            const size_t stat = (static_cast<size_t>(b) * a.H + h) * a.S + i;
            const float lse2 = a.lse[stat] * kL2e, Dv = a.dvec[stat];

            auto block = [&](auto diag_tag, int kb) -> bool {
                constexpr bool DIAG = decltype(diag_tag)::value;
                const int gj = kv0 + kb, sb = gj % NB, u = gj / NB;
                if (!mbar_wait(sp_full0 + 8 * sb, u & 1, abort_flag, 6, &g_attn_bwd_error)) return false;
                tc_fence_after();
                const int k0 = kb * 64 + hf * 32;                     // first key of this thread's 32 columns
                uint32_t rs[32], rp[32];
                tmem_ld32(tmem_base + sb * 64 + lane_addr + hf * 32, rs);
                tmem_ld32(tmem_base + NB * 64 + sb * 64 + lane_addr + hf * 32, rp);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sp_empty0 + 8 * sb);
                const int* dk_ptr = DOC ? a.doc + row_base + k0 : nullptr;
                const float base = (ALIBI ? -slope2 * static_cast<float>(i - k0) : 0.f) - lse2;
                uint32_t pk[16];
#pragma unroll
                for (int cj = 0; cj < 32; cj += 2) {
                    float dsv[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int c = cj + e;
                        const float tt = ALIBI ? fmaf(slope2, static_cast<float>(c), base) : base;
                        float p = ex2a(fmaf(__uint_as_float(rs[c]), scale2, tt));
                        if (DIAG && k0 + c > i) p = 0.f;
                        if (DOC && dk_ptr[c] != my_doc) p = 0.f;
                        dsv[e] = p * (__uint_as_float(rp[c]) - Dv);
                    }
                    __nv_bfloat162 t2 = __floats2bfloat162_rn(dsv[0], dsv[1]);
                    pk[cj >> 1] = *reinterpret_cast<uint32_t*>(&t2);
                }
                if (u >= 1 && !mbar_wait(ds_empty0 + 8 * sb, (u - 1) & 1, abort_flag, 7, &g_attn_bwd_error)) return false;
                uint8_t* drow = sDS + sb * BT + row * 128;
#pragma unroll
                for (int g = 0; g < 4; ++g)
                    *reinterpret_cast<uint4*>(drow + (((hf * 4 + g) ^ sw) << 4)) = make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(ds_full0 + 8 * sb);
                return true;
            };
            for (int kb = 0; ok && kb < nkb - 2; ++kb) ok = block(std::false_type{}, kb);
            for (int kb = nkb - 2; ok && kb < nkb; ++kb) ok = block(std::true_type{}, kb);
            const int acc = tn % NB;
            if (ok) ok = mbar_wait(done0 + 8 * acc, (tn / NB) & 1, abort_flag, 8, &g_attn_bwd_error);
            if (ok) {
                tc_fence_after();
                uint32_t r[32];
                tmem_ld32(tmem_base + 2 * NB * 64 + acc * 64 + lane_addr + hf * 32, r);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);       // the accumulator may be overwritten
                bf16* op = a.dqkv + (static_cast<size_t>(row_base) + i) * (3 * d) + h * 64 + hf * 32;
#pragma unroll
                for (int c = 0; c < 32; c += 8) {
                    Vec16<bf16> o;
#pragma unroll
                    for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(__uint_as_float(r[c + k]) * a.scale);
                    st16(op + c, o);
                }
            }
            kv0 += nkb;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(DqLayout<NB>::TMEM_COLS) : "memory");
    }
}

// ======================================================================================
// dK, dV
// ======================================================================================
// shared memory: K (2) | V (2) | ring of (Q, dO) 64-query tiles | P^T (2) | dS^T (2) | lse, D per stage | barriers
template <int NB> struct KvLayout {
    static constexpr int ST = NB + 1;                               // (Q, dO) ring stages
    static constexpr int OFF_V = NB * BT, OFF_RING = 2 * NB * BT, OFF_PT = OFF_RING + ST * 2 * HT, OFF_DST = OFF_PT + NB * BT,
                         OFF_STAT = OFF_DST + NB * BT, OFF_BAR = OFF_STAT + ST * 512, SMEM = OFF_BAR + 256;
    static constexpr uint32_t TMEM_COLS = NB == 2 ? 512u : 256u;    // S^T | dP^T | (dV, dK) per accumulator pair
};

template <bool DOC, bool ALIBI, int NB>
__global__ void __launch_bounds__(320, 3 - NB)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tmKV128, const __grid_constant__ CUtensorMap tmQ64,
                       const __grid_constant__ CUtensorMap tmDO64, const AttnBwdArgs a)
{
    using LY = KvLayout<NB>;
    constexpr int ST = LY::ST;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem;                            // tile buffer k at +k*BT
    uint8_t* sV = smem + LY::OFF_V;
    uint8_t* sRing = smem + LY::OFF_RING;           // stage s: Q at +s*2*HT, dO right after
    uint8_t* sPT = smem + LY::OFF_PT;
    uint8_t* sDST = smem + LY::OFF_DST;
    float* sStat = reinterpret_cast<float*>(smem + LY::OFF_STAT);   // [stage][lse(64) | D(64)]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + LY::OFF_BAR);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t kv_full0 = bar0, kv_empty0 = bar0 + 16, q_full0 = bar0 + 32, q_empty0 = bar0 + 56, sp_full0 = bar0 + 80,
                   sp_empty0 = bar0 + 96, pd_full0 = bar0 + 112, pd_empty0 = bar0 + 128, done0 = bar0 + 144, acc_empty0 = bar0 + 160;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = a.H * 64;
    const int nt = a.S / 128, HB = a.H * a.B, total = nt * HB;   // key tile 0 has the most query blocks: heavy first

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
        for (int s = 0; s < ST; ++s) { mbar_init(q_full0 + 8 * s, 1); mbar_init(q_empty0 + 8 * s, 1); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(sp_full0 + 8 * s, 1); mbar_init(sp_empty0 + 8 * s, 8);
            mbar_init(pd_full0 + 8 * s, 8); mbar_init(pd_empty0 + 8 * s, 1);
            mbar_init(done0 + 8 * s, 1); mbar_init(acc_empty0 + 8 * s, 8);
        }
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;
        if (*abort_flag) atomicCAS(&g_attn_bwd_error, 0, (9 << 16));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(KvLayout<NB>::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // TMEM columns, 64 per buffer: S^T buffers, dP^T buffers, then per accumulator pair dV and dK

    if (warp == 0) {
        if (lane == 0 && !*abort_flag) {
            int qc = 0, tn = 0;                                    // query-block counter across tiles, tile counter
            bool ok = true;
            for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
                const BwdTile t = bwd_tile(w, a.H, HB);
                const int kt = t.t, k0 = kt * 128, qi0 = kt * 2, nit = a.S / 64 - qi0, row_base = t.b * a.S, ks = tn % NB;
                const size_t stat_base = (static_cast<size_t>(t.b) * a.H + t.h) * a.S;
                if (!mbar_wait(kv_empty0 + 8 * ks, ((tn / NB) & 1) ^ 1, abort_flag, 11, &g_attn_bwd_error)) break;
                mbar_expect_tx(kv_full0 + 8 * ks, 2 * BT);
                tma_load_2d(smem_u32(sK + ks * BT), &tmKV128, kv_full0 + 8 * ks, d + t.h * 64, row_base + k0);
                tma_load_2d(smem_u32(sV + ks * BT), &tmKV128, kv_full0 + 8 * ks, 2 * d + t.h * 64, row_base + k0);
                for (int it = 0; it < nit; ++it, ++qc) {
                    const int st = qc % ST, qs = (qi0 + it) * 64;
                    if (!mbar_wait(q_empty0 + 8 * st, ((qc / ST) & 1) ^ 1, abort_flag, 1, &g_attn_bwd_error)) { ok = false; break; }
                    mbar_expect_tx(q_full0 + 8 * st, 2 * HT + 512);
                    const uint32_t dst = smem_u32(sRing + st * 2 * HT);
                    tma_load_2d(dst, &tmQ64, q_full0 + 8 * st, t.h * 64, row_base + qs);
                    tma_load_2d(dst + HT, &tmDO64, q_full0 + 8 * st, t.h * 64, row_base + qs);
                    bulk_load_1d(smem_u32(sStat + st * 128), a.lse + stat_base + qs, 256, q_full0 + 8 * st);
                    bulk_load_1d(smem_u32(sStat + st * 128 + 64), a.dvec + stat_base + qs, 256, q_full0 + 8 * st);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && !*abort_flag) {
            int qc0 = 0, tn = 0;
            bool ok = true;
            for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
                const BwdTile t = bwd_tile(w, a.H, HB);
                const int nit = a.S / 64 - t.t * 2, ks = tn % NB, use = tn / NB;
                ok = mbar_wait(kv_full0 + 8 * ks, use & 1, abort_flag, 2, &g_attn_bwd_error);
                if (ok && use >= 1) ok = mbar_wait(acc_empty0 + 8 * ks, (use - 1) & 1, abort_flag, 12, &g_attn_bwd_error);
                const uint32_t k_addr = smem_u32(sK + ks * BT), v_addr = smem_u32(sV + ks * BT);
                const uint32_t tmem_dV = tmem_base + 2 * NB * 64 + ks * 128, tmem_dK = tmem_dV + 64;
                auto issue_st = [&](int gi) -> bool {
                    const int st = gi % ST, sb = gi % NB, u = gi / NB;
                    if (!mbar_wait(q_full0 + 8 * st, (gi / ST) & 1, abort_flag, 3, &g_attn_bwd_error)) return false;
                    if (u >= 1 && !mbar_wait(sp_empty0 + 8 * sb, (u - 1) & 1, abort_flag, 4, &g_attn_bwd_error)) return false;
                    tc_fence_after();
                    const uint32_t q_addr = smem_u32(sRing + st * 2 * HT), do_addr = q_addr + HT;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base + sb * 64, smem_desc(k_addr + k * 32, 16, 1024), smem_desc(q_addr + k * 32, 16, 1024), IDESC_KK, k > 0);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base + NB * 64 + sb * 64, smem_desc(v_addr + k * 32, 16, 1024), smem_desc(do_addr + k * 32, 16, 1024), IDESC_KK, k > 0);
                    umma_commit(sp_full0 + 8 * sb);
                    return true;
                };
                auto issue_dkv = [&](int gi, bool first) -> bool {
                    const int st = gi % ST, sb = gi % NB;
                    if (!mbar_wait(pd_full0 + 8 * sb, (gi / NB) & 1, abort_flag, 5, &g_attn_bwd_error)) return false;
                    tc_fence_after();
                    const uint32_t pt_addr = smem_u32(sPT + sb * BT), dst_addr = smem_u32(sDST + sb * BT);
                    const uint32_t q_addr = smem_u32(sRing + st * 2 * HT), do_addr = q_addr + HT;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_dV, smem_desc(pt_addr + k * 32, 16, 1024), smem_desc(do_addr + k * 2048, HT, 1024), IDESC_KM, (!first || k > 0));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_dK, smem_desc(dst_addr + k * 32, 16, 1024), smem_desc(q_addr + k * 2048, HT, 1024), IDESC_KM, (!first || k > 0));
                    umma_commit(pd_empty0 + 8 * sb);
                    umma_commit(q_empty0 + 8 * st);
                    return true;
                };
                if (ok) ok = issue_st(qc0);
                for (int it = 0; ok && it < nit; ++it) {
                    if (it + 1 < nit) ok = issue_st(qc0 + it + 1);
                    if (ok) ok = issue_dkv(qc0 + it, it == 0);
                }
                if (ok) { umma_commit(done0 + 8 * ks); umma_commit(kv_empty0 + 8 * ks); }
                qc0 += nit;
            }
        }
    } else {
        const int q = warp & 3, hf = (warp - 2) >> 2;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
        const float scale2 = a.scale * kL2e;
        const int sw = row & 7;
        bool ok = !*abort_flag;
        int qc0 = 0, tn = 0;

        for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
            const BwdTile t = bwd_tile(w, a.H, HB);
            const int h = t.h, b = t.b, kt = t.t, k0 = kt * 128, qi0 = kt * 2, nit = a.S / 64 - qi0, row_base = b * a.S;
            const int j = k0 + row;                                   // key position
            const float slope2 = ALIBI ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(a.H)) * kL2e : 0.f;
            const int my_doc = DOC ? a.doc[row_base + j] : 0;

            auto block = [&](auto diag_tag, int it) -> bool {
                constexpr bool DIAG = decltype(diag_tag)::value;
                const int gi = qc0 + it, st = gi % ST, sb = gi % NB, u = gi / NB;
                if (!mbar_wait(sp_full0 + 8 * sb, u & 1, abort_flag, 6, &g_attn_bwd_error)) return false;
                tc_fence_after();
                const int qs = (qi0 + it) * 64 + hf * 32;              // first query of this thread's 32 columns
                uint32_t rs[32], rp[32];
                tmem_ld32(tmem_base + sb * 64 + lane_addr + hf * 32, rs);
                tmem_ld32(tmem_base + NB * 64 + sb * 64 + lane_addr + hf * 32, rp);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sp_empty0 + 8 * sb);
                const float4* lse4 = reinterpret_cast<const float4*>(sStat + st * 128 + hf * 32);
                const float4* dv4 = reinterpret_cast<const float4*>(sStat + st * 128 + 64 + hf * 32);
                const int* dq_ptr = DOC ? a.doc + row_base + qs : nullptr;
                const float base = ALIBI ? -slope2 * static_cast<float>(qs - j) : 0.f;
                uint32_t pk[16], dk[16];
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const float4 l4 = lse4[c4], d4 = dv4[c4];
                    const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
                    float pv[4], dsv[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = c4 * 4 + e;
                        const float tt = (ALIBI ? fmaf(-slope2, static_cast<float>(c), base) : 0.f) - ls[e] * kL2e;
                        float p = ex2a(fmaf(__uint_as_float(rs[c]), scale2, tt));
                        if (DIAG && j > qs + c) p = 0.f;
                        if (DOC && dq_ptr[c] != my_doc) p = 0.f;
                        pv[e] = p;
                        dsv[e] = p * (__uint_as_float(rp[c]) - dd[e]);
                    }
                    __nv_bfloat162 t0 = __floats2bfloat162_rn(pv[0], pv[1]), t1 = __floats2bfloat162_rn(pv[2], pv[3]);
                    __nv_bfloat162 u0 = __floats2bfloat162_rn(dsv[0], dsv[1]), u1 = __floats2bfloat162_rn(dsv[2], dsv[3]);
                    pk[c4 * 2] = *reinterpret_cast<uint32_t*>(&t0); pk[c4 * 2 + 1] = *reinterpret_cast<uint32_t*>(&t1);
                    dk[c4 * 2] = *reinterpret_cast<uint32_t*>(&u0); dk[c4 * 2 + 1] = *reinterpret_cast<uint32_t*>(&u1);
                }
                if (u >= 1 && !mbar_wait(pd_empty0 + 8 * sb, (u - 1) & 1, abort_flag, 7, &g_attn_bwd_error)) return false;
                uint8_t* prow = sPT + sb * BT + row * 128;
                uint8_t* drow = sDST + sb * BT + row * 128;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int off = ((hf * 4 + g) ^ sw) << 4;
                    *reinterpret_cast<uint4*>(prow + off) = make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
                    *reinterpret_cast<uint4*>(drow + off) = make_uint4(dk[g * 4], dk[g * 4 + 1], dk[g * 4 + 2], dk[g * 4 + 3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(pd_full0 + 8 * sb);
                return true;
            };
            for (int it = 0; ok && it < 2; ++it) ok = block(std::true_type{}, it);
            for (int it = 2; ok && it < nit; ++it) ok = block(std::false_type{}, it);
            const int acc = tn % NB;
            if (ok) ok = mbar_wait(done0 + 8 * acc, (tn / NB) & 1, abort_flag, 8, &g_attn_bwd_error);
            if (ok) {
                tc_fence_after();
                uint32_t rv[32], rk[32];
                tmem_ld32(tmem_base + 2 * NB * 64 + acc * 128 + lane_addr + hf * 32, rv);
                tmem_ld32(tmem_base + 2 * NB * 64 + 64 + acc * 128 + lane_addr + hf * 32, rk);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);       // the accumulators may be overwritten
                bf16* kp = a.dqkv + (static_cast<size_t>(row_base) + j) * (3 * d) + d + h * 64 + hf * 32;
#pragma unroll
                for (int c = 0; c < 32; c += 8) {
                    Vec16<bf16> ok8, ov8;
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        ok8.v[k] = __float2bfloat16_rn(__uint_as_float(rk[c + k]) * a.scale);
                        ov8.v[k] = __float2bfloat16_rn(__uint_as_float(rv[c + k]));
                    }
                    st16(kp + c, ok8);
                    st16(kp + d + c, ov8);
                }
            }
            qc0 += nit;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(KvLayout<NB>::TMEM_COLS) : "memory");
    }
}

// ======================================================================================
// host
// ======================================================================================
// CTAs per SM of the backward kernels: 2 by default, 1 with NNB200_ATTN_BWD_CTAS=1 (read once; for A/B timing)
static int bwd_ctas_per_sm()
{
    static const int n = [] { const char* e = getenv("NNB200_ATTN_BWD_CTAS"); return (e && e[0] == '1') ? 1 : 2; }();
    return n;
}

template <bool DOC, bool ALIBI, int NB>
static int launch_bwd_tc_nb(const CUtensorMap& q128, const CUtensorMap& q64, const CUtensorMap& do128, const CUtensorMap& do64,
                            const AttnBwdArgs& a, long long tiles, cudaStream_t s)
{
    static bool attr_set = false;
    if (!attr_set) {
        NNB_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dq_tc_kernel<DOC, ALIBI, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, DqLayout<NB>::SMEM));
        NNB_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel<DOC, ALIBI, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, KvLayout<NB>::SMEM));
        attr_set = true;
    }
    const long long cap = static_cast<long long>(kSmCount) * (3 - NB);          // persistent: NB = 1 runs two CTAs per SM
    const dim3 grid(static_cast<unsigned>(tiles < cap ? tiles : cap));
    attn_bwd_dq_tc_kernel<DOC, ALIBI, NB><<<grid, 320, DqLayout<NB>::SMEM, s>>>(q128, q64, do128, a);
    NNB_LAUNCH_CHECK();
    attn_bwd_dkv_tc_kernel<DOC, ALIBI, NB><<<grid, 320, KvLayout<NB>::SMEM, s>>>(q128, q64, do64, a);
    NNB_LAUNCH_CHECK();
    return 0;
}
template <bool DOC, bool ALIBI>
static int launch_bwd_tc(const CUtensorMap& q128, const CUtensorMap& q64, const CUtensorMap& do128, const CUtensorMap& do64,
                         const AttnBwdArgs& a, long long tiles, cudaStream_t s)
{
    if (bwd_ctas_per_sm() == 2) return launch_bwd_tc_nb<DOC, ALIBI, 1>(q128, q64, do128, do64, a, tiles, s);
    return launch_bwd_tc_nb<DOC, ALIBI, 2>(q128, q64, do128, do64, a, tiles, s);
}

int attention_bwd_tc(const bf16* qkv, const bf16* out, const bf16* dout, const float* lse, float* dvec, bf16* dqkv,
                     const int* doc, int B, int S, int H, int dk, int alibi, cudaStream_t s)
{
    if (static_cast<long long>(B) * S * H == 0) return 0;
    NNB_ARG_CHECK(attention_tc_supported(dk, S, H * dk), "shape not supported by the tcgen05 attention kernels");
    NNB_ARG_CHECK(B <= 65535 && H <= 65535, "batch / heads exceed the grid limits");
    NNB_TRY(attention_dvec_bf16(out, dout, dvec, B, S, H, dk, s));
    const int d = H * dk;
    const long long rows = static_cast<long long>(B) * S;
    CUtensorMap q128, q64, do128, do64;
    NNB_TRY(tensor_map_2d(qkv, 3LL * d, rows, 3LL * d, 64, 128, &q128, 2));
    NNB_TRY(tensor_map_2d(qkv, 3LL * d, rows, 3LL * d, 64, 64, &q64, 2));
    NNB_TRY(tensor_map_2d(dout, d, rows, d, 64, 128, &do128, 2));
    NNB_TRY(tensor_map_2d(dout, d, rows, d, 64, 64, &do64, 2));
    AttnBwdArgs a{dqkv, lse, dvec, doc, B, S, H, 1.0f / sqrtf(static_cast<float>(dk))};
    const long long tiles = static_cast<long long>(S / 128) * H * B;
    NNB_ARG_CHECK(tiles < (1ll << 31), "too many attention tiles");
    if (doc && alibi) return launch_bwd_tc<true, true>(q128, q64, do128, do64, a, tiles, s);
    if (doc) return launch_bwd_tc<true, false>(q128, q64, do128, do64, a, tiles, s);
    if (alibi) return launch_bwd_tc<false, true>(q128, q64, do128, do64, a, tiles, s);
    return launch_bwd_tc<false, false>(q128, q64, do128, do64, a, tiles, s);
}

int attention_bwd_device_error(int* code)
{
    NNB_CUDA_CHECK(cudaMemcpyFromSymbol(code, g_attn_bwd_error, sizeof(int)));
    if (*code) { const int z = 0; NNB_CUDA_CHECK(cudaMemcpyToSymbol(g_attn_bwd_error, &z, sizeof(int))); }
    return 0;
}

}  // namespace nnb
