// Attention backward on the 5th-generation tensor cores, head sizes 64 and 128: two kernels, no atomics.
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
// K-major operands wider than 64 values are kept as sub-tiles of 64 columns (one 128-byte swizzle atom per row).
// ALiBi: the bias -slope_h (i - j) is linear in both positions.  In the dQ kernel the tensor core adds its in-block
// part: one more MMA step per score block multiplies a 16-deep tile holding slope_h / scale (three bf16 terms) in
// every row by a constant tile holding the key's position inside the block; the workers add one constant per row.
// The dK/dV kernel spends that shared memory on the third ring stage and steps the bias in registers instead.
// With a table of per-64-row document-id ranges (attention_doc_ranges) every role skips the blocks a document mask
// leaves nothing of; a skipped block would have contributed exact zeros, so no result bit changes.
#include <type_traits>

#include "attention_tc.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace nnb {

__device__ int g_attn_bwd_error = 0;

constexpr int BT = 128 * 128;          // bytes of a 128-row x 64-bf16 tile
constexpr int HT = 64 * 128;           // bytes of a 64-row tile
constexpr int XT = 128 * 32;           // bytes of a 128-row x 16-bf16 tile without swizzle (the ALiBi operand tiles)
constexpr float kL2e = 1.4426950408889634f;

struct AttnBwdArgs {
    bf16* dqkv; const float* lse; const float* dvec; const int* doc; const int2* ranges;
    float* colsum_part;      // null, or [rows / 32][3 d]: column sums of dqkv over each 32 token rows (the QKV bias gradient's partials)
    int B, S, H;
    float scale;
};

__device__ __forceinline__ float ex2a(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// fp32 accumulate, bf16 operands, M = 128; score MMAs: N = 64, both operands K-major; gradient MMAs: N = head size,
// B operand MN-major
constexpr uint32_t IDESC_KK = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(64 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
template <int DK> __host__ __device__ constexpr uint32_t idesc_km() { return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (uint32_t(DK >> 3) << 17) | (uint32_t(128 >> 4) << 24); }

// Unswizzled K-major tiles, 16 values deep: row r, values [8c, 8c + 8) at (r / 8) * 256 + c * 128 + (r % 8) * 16.
// slope_h / scale as three bf16 terms (24 bits) in values 0..2 of every one of the 128 rows; called by a whole warp.
__device__ __forceinline__ void write_slope_tile(uint8_t* tile, int h, int H, float scale, int lane)
{
    const float sv = exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(H)) / scale;
    const bf16 s0 = __float2bfloat16_rn(sv);
    const float r1 = sv - __bfloat162float(s0);
    const bf16 s1 = __float2bfloat16_rn(r1);
    const bf16 s2 = __float2bfloat16_rn(r1 - __bfloat162float(s1));
    const uint32_t w0 = static_cast<uint32_t>(__bfloat16_as_ushort(s0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(s1)) << 16);
    const uint32_t w1 = static_cast<uint32_t>(__bfloat16_as_ushort(s2));
    for (int r = lane; r < 128; r += 32) *reinterpret_cast<uint4*>(tile + (r >> 3) * 256 + (r & 7) * 16) = make_uint4(w0, w1, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
}
// value `sign * r` three times in row r (r < rows), zeros elsewhere; called by the whole block before its first barrier
__device__ __forceinline__ void init_position_tiles(uint8_t* pos_tile, uint8_t* slope_tile, int rows, float sign)
{
    for (int r = threadIdx.x; r < 128; r += blockDim.x) {
        const uint32_t off = (r >> 3) * 256 + (r & 7) * 16;
        const __nv_bfloat162 jj = __floats2bfloat162_rn(sign * static_cast<float>(r), sign * static_cast<float>(r));
        const uint32_t j2 = r < rows ? *reinterpret_cast<const uint32_t*>(&jj) : 0u;
        *reinterpret_cast<uint4*>(pos_tile + off) = make_uint4(j2, j2 & 0xffffu, 0u, 0u);
        *reinterpret_cast<uint4*>(pos_tile + off + 128) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(slope_tile + off) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(slope_tile + off + 128) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Both kernels are persistent: the CTAs resident on an SM draw (tile, head, batch) work items, heaviest tiles first,
// from a counter in global memory (work_counter.cu; the producer warp draws and passes the item on to the other
// roles through a two-slot ring in shared memory), so that a CTA whose tiles ran slowly takes fewer of them.  The
// rings, score buffers and barrier phases run on across tiles, and the tile that stays resident (Q and dO, resp. K
// and V) is handed back with the last score MMA that reads it, so the loads and first MMAs of the next tile overlap
// the tail and the write-out of the current one.  The block ring is three deep: a stage is free only when the
// gradient MMAs of its block are complete, and with two stages the load of block j + 2 (issued when block j retires)
// arrived after the workers had finished block j + 1, a third of every block period.  Score and gradient-tile
// buffers are single; at head size 64 two CTAs share an SM (256 TMEM columns, 102 / 111 KB of shared memory, 96
// registers each), so that while the workers of one CTA are in their dependency chain (scores ready -> tcgen05.ld
// -> exp -> dS tile -> next MMA) the other CTA's MMAs run; at head size 128 one CTA fills the SM.
// Producer side of the work list (whole warp): lane 0 draws the next item and publishes it (or -1 when the list is
// exhausted) in slot n & 3; everybody gets the value.  An item is drawn when the producer is ready to load it, not
// earlier (an item drawn is an item no other CTA can take; drawing one tile ahead, with an L2 prefetch of its first
// operands, was measured slower: the prefetch bought nothing and the balance at the list's end got worse).  When item
// n is published the producer has issued the loads of item n - 1 and the other roles may still be in item n - 2: a
// ring of four slots keeps everything that may still be read.
__device__ __forceinline__ int draw_tile(unsigned int* work, int total, volatile int* slots, uint32_t t_full0, int n, int lane)
{
    int w = 0;
    if (lane == 0) {
        const unsigned int v = atomicAdd(work, 1u);
        w = v < static_cast<unsigned int>(total) ? static_cast<int>(v) : -1;
        slots[n & 3] = w;
        mbar_arrive(t_full0 + 8 * (n & 3));
    }
    return __shfl_sync(0xffffffffu, w, 0);
}
// The producer's last act: the CTA that leaves last puts the counter pair back to zero for the next launch.
__device__ __forceinline__ void leave_work_list(unsigned int* work, int lane)
{
    if (lane == 0 && atomicAdd(work + 1, 1u) == gridDim.x - 1u) { work[0] = 0u; work[1] = 0u; }
}
// Consumer side (whole warp): the item of round n, -1 at the end or when the wait gave up.
__device__ __forceinline__ int read_tile(volatile int* slots, uint32_t t_full0, int n, volatile int* abort_flag, int* error_word)
{
    const bool got = mbar_wait(t_full0 + 8 * (n & 3), (n >> 2) & 1, abort_flag, 14, error_word);
    if (!__all_sync(0xffffffffu, got)) return -1;
    return slots[n & 3];
}

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
// shared memory: Q | dO | ring of three (K, V) 64-key tiles | dS | ALiBi operand tiles | barriers
template <int DK> struct DqLayout {
    static constexpr int NS = DK / 64;                              // 64-column sub-tiles per operand tile
    static constexpr int ST = 3;                                    // (K, V) ring stages: a stage is free only when its dQ MMA is complete
    static constexpr int OFF_DO = NS * BT, OFF_RING = 2 * NS * BT, OFF_DS = OFF_RING + ST * 2 * NS * HT, OFF_U = OFF_DS + BT,
                         OFF_W = OFF_U + XT, OFF_BAR = OFF_W + XT, SMEM = OFF_BAR + 256;
    static constexpr uint32_t TMEM_COLS = 256u;                     // S [0, 64) | dP [64, 128) | dQ [128, 128 + DK)
    static constexpr int CTAS_PER_SM = DK == 64 ? 2 : 1;
};

template <int DK, bool DOC, bool ALIBI>
__global__ void __launch_bounds__(320, DqLayout<DK>::CTAS_PER_SM)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ128, const __grid_constant__ CUtensorMap tmKV64,
                      const __grid_constant__ CUtensorMap tmDO128, const AttnBwdArgs a, unsigned int* __restrict__ work)
{
    using LY = DqLayout<DK>;
    constexpr int ST = LY::ST, NS = LY::NS, STAGE = 2 * NS * HT;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sDO = smem + LY::OFF_DO;
    uint8_t* sRing = smem + LY::OFF_RING;           // stage s: K at +s*STAGE, V right after
    uint8_t* sDS = smem + LY::OFF_DS;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + LY::OFF_BAR);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, q_empty = bar0 + 8, kv_full0 = bar0 + 16, kv_empty0 = kv_full0 + 8 * ST, sp_full = kv_empty0 + 8 * ST,
                   sp_empty = sp_full + 8, ds_full = sp_full + 16, ds_empty = sp_full + 24, done = sp_full + 32, acc_empty = sp_full + 40,
                   t_full0 = sp_full + 48;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12 + 2 * ST);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* tile_slots = reinterpret_cast<volatile int*>(tmem_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = a.H * DK;
    const int nt = a.S / 128, HB = a.H * a.B, total = nt * HB;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1); mbar_init(q_empty, 1);
        for (int s = 0; s < ST; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
        mbar_init(sp_full, 1); mbar_init(sp_empty, 8);
        mbar_init(ds_full, 8); mbar_init(ds_empty, 1);
        mbar_init(done, 1); mbar_init(acc_empty, 8);
        for (int k = 0; k < 4; ++k) mbar_init(t_full0 + 8 * k, 1);
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;
        if (*abort_flag) atomicCAS(&g_attn_bwd_error, 0, (9 << 16));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(LY::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 64, tmem_dQ = tmem_base + 128;
    uint8_t* sU = smem + LY::OFF_U;                 // slope_h / scale in every query row (rewritten per tile by warp 0)
    uint8_t* sW = smem + LY::OFF_W;                 // key position inside the 64-key block, constant
    if (ALIBI) {
        init_position_tiles(sW, sU, 64, 1.0f);
        __syncthreads();
    }

    // key blocks (64 keys each) of a query tile that the document mask leaves anything of; whole-warp call
    auto tile_mask = [&](int b, int qb, int nkb) -> BlockMask {
        if (!DOC || a.ranges == nullptr) return block_mask_all();
        const int2* rng = a.ranges + static_cast<size_t>(b) * (a.S / 64);
        return doc_block_mask(rng, 0, nkb, 1, rng[2 * qb], rng[2 * qb + 1], nkb - 2, nkb, lane);
    };

    if (warp == 0) {
        int kv = 0, tn = 0;
        bool ok = !*abort_flag;
        for (int w; ok && (w = draw_tile(work, total, tile_slots, t_full0, tn, lane)) >= 0; ++tn) {
            const BwdTile t = bwd_tile(w, a.H, HB);
            const int qb = nt - 1 - t.t, q0 = qb * 128, nkb = 2 * (qb + 1), row_base = t.b * a.S;
            const BlockMask bm = tile_mask(t.b, qb, nkb);
            if (lane == 0) ok = mbar_wait(q_empty, (tn & 1) ^ 1, abort_flag, 11, &g_attn_bwd_error);   // the previous tile's MMAs are done
            ok = __shfl_sync(0xffffffffu, static_cast<int>(ok), 0) != 0;
            if (ALIBI && ok) write_slope_tile(sU, t.h, a.H, a.scale, lane);
            if (lane == 0) {
                if (ok) {
                    mbar_expect_tx(q_full, 2 * NS * BT);
#pragma unroll
                    for (int j = 0; j < NS; ++j) {
                        tma_load_2d(smem_u32(sQ + j * BT), &tmQ128, q_full, t.h * DK + j * 64, row_base + q0);
                        tma_load_2d(smem_u32(sDO + j * BT), &tmDO128, q_full, t.h * DK + j * 64, row_base + q0);
                    }
                }
                for (int kb = 0; ok && kb < nkb; ++kb) {
                    if (!block_active(bm, kb)) continue;
                    const int st = kv % ST;
                    if (!mbar_wait(kv_empty0 + 8 * st, ((kv / ST) & 1) ^ 1, abort_flag, 1, &g_attn_bwd_error)) { ok = false; break; }
                    mbar_expect_tx(kv_full0 + 8 * st, STAGE);
                    const uint32_t dst = smem_u32(sRing + st * STAGE);
#pragma unroll
                    for (int j = 0; j < NS; ++j) {
                        tma_load_2d(dst + j * HT, &tmKV64, kv_full0 + 8 * st, d + t.h * DK + j * 64, row_base + kb * 64);
                        tma_load_2d(dst + NS * HT + j * HT, &tmKV64, kv_full0 + 8 * st, 2 * d + t.h * DK + j * 64, row_base + kb * 64);
                    }
                    ++kv;
                }
            }
            kv = __shfl_sync(0xffffffffu, kv, 0);
            ok = __shfl_sync(0xffffffffu, static_cast<int>(ok), 0) != 0;
        }
        leave_work_list(work, lane);
    } else if (warp == 1) {
        int kv0 = 0, tn = 0;
        bool ok = !*abort_flag;
        for (int w; ok && (w = read_tile(tile_slots, t_full0, tn, abort_flag, &g_attn_bwd_error)) >= 0; ++tn) {
            const BwdTile t = bwd_tile(w, a.H, HB);
            const int qb = nt - 1 - t.t, nkb = 2 * (qb + 1);
            const BlockMask bm = tile_mask(t.b, qb, nkb);
            if (lane == 0) {
                const int nact = block_count(bm, nkb);
                ok = mbar_wait(q_full, tn & 1, abort_flag, 2, &g_attn_bwd_error);
                const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDO);
                auto issue_sdp = [&](int gj) -> bool {
                    const int st = gj % ST;
                    if (!mbar_wait(kv_full0 + 8 * st, (gj / ST) & 1, abort_flag, 3, &g_attn_bwd_error)) return false;
                    if (gj >= 1 && !mbar_wait(sp_empty, (gj - 1) & 1, abort_flag, 4, &g_attn_bwd_error)) return false;
                    tc_fence_after();
                    const uint32_t k_addr = smem_u32(sRing + st * STAGE), v_addr = k_addr + NS * HT;
#pragma unroll
                    for (int k = 0; k < DK / 16; ++k)
                        umma_bf16(tmem_S, smem_desc(q_addr + (k >> 2) * BT + (k & 3) * 32, 16, 1024),
                                  smem_desc(k_addr + (k >> 2) * HT + (k & 3) * 32, 16, 1024), IDESC_KK, k > 0);
                    if (ALIBI)       // + (slope / scale) * (key position inside the block)
                        umma_bf16(tmem_S, smem_desc_noswizzle(smem_u32(sU), 128, 256), smem_desc_noswizzle(smem_u32(sW), 128, 256), IDESC_KK, 1u);
#pragma unroll
                    for (int k = 0; k < DK / 16; ++k)
                        umma_bf16(tmem_dP, smem_desc(do_addr + (k >> 2) * BT + (k & 3) * 32, 16, 1024),
                                  smem_desc(v_addr + (k >> 2) * HT + (k & 3) * 32, 16, 1024), IDESC_KK, k > 0);
                    umma_commit(sp_full);
                    return true;
                };
                auto issue_dq = [&](int gj, bool first) -> bool {
                    const int st = gj % ST;
                    if (!mbar_wait(ds_full, gj & 1, abort_flag, 5, &g_attn_bwd_error)) return false;
                    // the accumulator this tile writes was read out by the workers at the end of the previous tile
                    if (first && tn >= 1 && !mbar_wait(acc_empty, (tn - 1) & 1, abort_flag, 12, &g_attn_bwd_error)) return false;
                    tc_fence_after();
                    const uint32_t ds_addr = smem_u32(sDS), k_addr = smem_u32(sRing + st * STAGE);
#pragma unroll
                    for (int k = 0; k < 4; ++k)          // K as an MN-major B operand: the next 64 head columns are one sub-tile on
                        umma_bf16(tmem_dQ, smem_desc(ds_addr + k * 32, 16, 1024), smem_desc(k_addr + k * 2048, HT, 1024), idesc_km<DK>(), (!first || k > 0));
                    umma_commit(ds_empty);
                    umma_commit(kv_empty0 + 8 * st);
                    return true;
                };
                // Q and dO are read by the score MMAs only: they are handed back with the last of those, so that the next
                // tile's loads overlap the last block's worker pass, its dQ MMA and the write-out
                if (ok) ok = issue_sdp(kv0);
                if (ok && nact == 1) umma_commit(q_empty);
                for (int j = 0; ok && j < nact; ++j) {
                    if (j + 1 < nact) {
                        ok = issue_sdp(kv0 + j + 1);
                        if (ok && j + 2 == nact) umma_commit(q_empty);
                    }
                    if (ok) ok = issue_dq(kv0 + j, j == 0);
                }
                if (ok) umma_commit(done);
                kv0 += nact;
            }
            kv0 = __shfl_sync(0xffffffffu, kv0, 0);
            ok = __shfl_sync(0xffffffffu, static_cast<int>(ok), 0) != 0;
        }
    } else {
        const int q = warp & 3, hf = (warp - 2) >> 2;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
        const float scale2 = a.scale * kL2e;
        const int sw = row & 7;
        constexpr int OC = DK / 2;                              // dQ columns this thread writes
        bool ok = !*abort_flag;
        int kv0 = 0, tn = 0;

        for (int w; ok && (w = read_tile(tile_slots, t_full0, tn, abort_flag, &g_attn_bwd_error)) >= 0; ++tn) {
            const BwdTile t = bwd_tile(w, a.H, HB);
            const int h = t.h, b = t.b, qb = nt - 1 - t.t, q0 = qb * 128, nkb = 2 * (qb + 1), row_base = b * a.S;
            const BlockMask bm = tile_mask(b, qb, nkb);
            const int i = q0 + row;
            const float slope2 = ALIBI ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(a.H)) * kL2e : 0.f;
            const int my_doc = DOC ? a.doc[row_base + i] : 0;
            const size_t stat = (static_cast<size_t>(b) * a.H + h) * a.S + i;
            const float lse2 = a.lse[stat] * kL2e, Dv = a.dvec[stat];

            auto block = [&](auto diag_tag, int kb, int cnt) -> bool {
                constexpr bool DIAG = decltype(diag_tag)::value;
                const int gj = kv0 + cnt;
                if (!mbar_wait(sp_full, gj & 1, abort_flag, 6, &g_attn_bwd_error)) return false;
                tc_fence_after();
                const int k0 = kb * 64 + hf * 32;                     // first key of this thread's 32 columns
                uint32_t rs[32], rp[32];
                tmem_ld32(tmem_S + lane_addr + hf * 32, rs);
                tmem_ld32(tmem_dP + lane_addr + hf * 32, rp);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sp_empty);
                const int* dk_ptr = DOC ? a.doc + row_base + k0 : nullptr;
                // base-2 exponent of P: raw * scale2 + cc, the in-block part of the ALiBi bias being in raw already
                const float cc = (ALIBI ? -slope2 * static_cast<float>(i - kb * 64) : 0.f) - lse2;
                const uint64_t cc2 = pack2(cc, cc), scale2x2 = pack2(scale2, scale2), negD2 = pack2(-Dv, -Dv);
                uint32_t pk[16];
#pragma unroll
                for (int cj = 0; cj < 32; cj += 2) {
                    float x0, x1;
                    unpack2(fma2(pack2(__uint_as_float(rs[cj]), __uint_as_float(rs[cj + 1])), scale2x2, cc2), x0, x1);
                    float p0 = ex2a(x0), p1 = ex2a(x1);
                    if (DIAG && k0 + cj > i) p0 = 0.f;
                    if (DIAG && k0 + cj + 1 > i) p1 = 0.f;
                    if (DOC && dk_ptr[cj] != my_doc) p0 = 0.f;
                    if (DOC && dk_ptr[cj + 1] != my_doc) p1 = 0.f;
                    float d0, d1;
                    unpack2(mul2(pack2(p0, p1), add2(pack2(__uint_as_float(rp[cj]), __uint_as_float(rp[cj + 1])), negD2)), d0, d1);
                    __nv_bfloat162 t2 = __floats2bfloat162_rn(d0, d1);
                    pk[cj >> 1] = *reinterpret_cast<uint32_t*>(&t2);
                }
                if (gj >= 1 && !mbar_wait(ds_empty, (gj - 1) & 1, abort_flag, 7, &g_attn_bwd_error)) return false;
                uint8_t* drow = sDS + row * 128;
#pragma unroll
                for (int g = 0; g < 4; ++g)
                    *reinterpret_cast<uint4*>(drow + (((hf * 4 + g) ^ sw) << 4)) = make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(ds_full);
                return true;
            };
            int cnt = 0;
            for (int kb = 0; ok && kb < nkb - 2; ++kb) {
                if (!block_active(bm, kb)) continue;
                ok = block(std::false_type{}, kb, cnt);
                ++cnt;
            }
            for (int kb = nkb - 2; ok && kb < nkb; ++kb, ++cnt) ok = block(std::true_type{}, kb, cnt);
            if (ok) ok = mbar_wait(done, tn & 1, abort_flag, 8, &g_attn_bwd_error);
            if (ok) {
                tc_fence_after();
                bf16* op = a.dqkv + (static_cast<size_t>(row_base) + i) * (3 * d) + h * DK + hf * OC;
#pragma unroll
                for (int c0 = 0; c0 < OC; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_dQ + lane_addr + hf * OC + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        Vec16<bf16> o;
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            o.v[k] = __float2bfloat16_rn(__uint_as_float(r[c + k]) * a.scale);
                            r[c + k] = __float_as_uint(__bfloat162float(o.v[k]));        // what is stored, for the column sums
                        }
                        st16(op + c0 + c, o);
                    }
                    if (a.colsum_part) {                                // this warp's 32 rows of 32 columns
                        float v[32];
#pragma unroll
                        for (int c = 0; c < 32; ++c) v[c] = __uint_as_float(r[c]);
                        const float sum = lane_sums32(v, lane);
                        a.colsum_part[(static_cast<size_t>(row_base + q0) / 32 + q) * (3 * d) + h * DK + hf * OC + c0 + lane] = sum;
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty);                  // the accumulator may be overwritten
            }
            kv0 += cnt;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(LY::TMEM_COLS) : "memory");
    }
}

// ======================================================================================
// dK, dV
// ======================================================================================
// shared memory: K | V | ring of three Q tiles (64 queries) | ring of two dO tiles | P^T | dS^T | lse per Q stage, D per
// dO stage | barriers.  A stage is free only when the dK / dV MMAs of its block are complete, so with two stages the
// load of block i + 2 would arrive after the workers have finished block i + 1.  Shared memory has room for one more
// 8 KB tile per CTA, not two: Q, which the first MMA of a block needs (and with it the exponentials), gets it, and
// S^T and dP^T are handed to the workers separately so that dP^T of a block may come half a block later.
template <int DK> struct KvLayout {
    static constexpr int NS = DK / 64;
    static constexpr int QST = 3, DST = 2;                          // Q and dO ring stages
    static constexpr int OFF_V = NS * BT, OFF_QR = 2 * NS * BT, OFF_DOR = OFF_QR + QST * NS * HT, OFF_PT = OFF_DOR + DST * NS * HT,
                         OFF_DST = OFF_PT + BT, OFF_STAT = OFF_DST + BT, OFF_BAR = OFF_STAT + (QST + DST) * 256, SMEM = OFF_BAR + 256;
    static constexpr uint32_t TMEM_COLS = DK == 64 ? 256u : 512u;   // S^T [0, 64) | dP^T [64, 128) | dV [128, 128 + DK) | dK after it
    static constexpr int CTAS_PER_SM = DK == 64 ? 2 : 1;
};

template <int DK, bool DOC, bool ALIBI>
__global__ void __launch_bounds__(320, KvLayout<DK>::CTAS_PER_SM)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tmKV128, const __grid_constant__ CUtensorMap tmQ64,
                       const __grid_constant__ CUtensorMap tmDO64, const AttnBwdArgs a, unsigned int* __restrict__ work)
{
    using LY = KvLayout<DK>;
    constexpr int QST = LY::QST, DST = LY::DST, NS = LY::NS, QSTAGE = NS * HT;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem;
    uint8_t* sV = smem + LY::OFF_V;
    uint8_t* sQR = smem + LY::OFF_QR;               // Q ring
    uint8_t* sDOR = smem + LY::OFF_DOR;             // dO ring
    uint8_t* sPT = smem + LY::OFF_PT;
    uint8_t* sDST = smem + LY::OFF_DST;
    float* sLse = reinterpret_cast<float*>(smem + LY::OFF_STAT);    // [Q stage][64]
    float* sD = sLse + QST * 64;                                    // [dO stage][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + LY::OFF_BAR);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t kv_full = bar0, kv_empty = bar0 + 8, q_full0 = bar0 + 16, q_empty0 = q_full0 + 8 * QST, do_full0 = q_empty0 + 8 * QST,
                   do_empty0 = do_full0 + 8 * DST, s_full = do_empty0 + 8 * DST, s_empty = s_full + 8, dp_full = s_full + 16,
                   dp_empty = s_full + 24, pd_full = s_full + 32, pd_empty = s_full + 40, done = s_full + 48, acc_empty = s_full + 56,
                   t_full0 = s_full + 64;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14 + 2 * QST + 2 * DST);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* tile_slots = reinterpret_cast<volatile int*>(tmem_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = a.H * DK;
    const int nt = a.S / 128, HB = a.H * a.B, total = nt * HB;   // key tile 0 has the most query blocks: heavy first

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1); mbar_init(kv_empty, 1);
        for (int s = 0; s < QST; ++s) { mbar_init(q_full0 + 8 * s, 1); mbar_init(q_empty0 + 8 * s, 1); }
        for (int s = 0; s < DST; ++s) { mbar_init(do_full0 + 8 * s, 1); mbar_init(do_empty0 + 8 * s, 1); }
        mbar_init(s_full, 1); mbar_init(s_empty, 8); mbar_init(dp_full, 1); mbar_init(dp_empty, 8);
        mbar_init(pd_full, 8); mbar_init(pd_empty, 1);
        mbar_init(done, 1); mbar_init(acc_empty, 8);
        for (int k = 0; k < 4; ++k) mbar_init(t_full0 + 8 * k, 1);
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;
        if (*abort_flag) atomicCAS(&g_attn_bwd_error, 0, (9 << 16));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(LY::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_ST = tmem_base, tmem_dPT = tmem_base + 64, tmem_dV = tmem_base + 128, tmem_dK = tmem_base + 128 + DK;

    // query blocks (64 queries each, from the diagonal on) of a key tile that the document mask leaves anything of
    auto tile_mask = [&](int b, int kt, int nit) -> BlockMask {
        if (!DOC || a.ranges == nullptr) return block_mask_all();
        const int2* rng = a.ranges + static_cast<size_t>(b) * (a.S / 64);
        return doc_block_mask(rng, 2 * kt, nit, 1, rng[2 * kt], rng[2 * kt + 1], 0, 2, lane);
    };

    if (warp == 0) {
        int qc = 0, tn = 0;                                    // query-block counter across tiles, tile counter
        bool ok = !*abort_flag;
        for (int w; ok && (w = draw_tile(work, total, tile_slots, t_full0, tn, lane)) >= 0; ++tn) {
            const BwdTile t = bwd_tile(w, a.H, HB);
            const int kt = t.t, k0 = kt * 128, qi0 = kt * 2, nit = a.S / 64 - qi0, row_base = t.b * a.S;
            const BlockMask bm = tile_mask(t.b, kt, nit);
            if (lane == 0) ok = mbar_wait(kv_empty, (tn & 1) ^ 1, abort_flag, 11, &g_attn_bwd_error);   // the previous tile's MMAs are done
            ok = __shfl_sync(0xffffffffu, static_cast<int>(ok), 0) != 0;
            if (lane == 0) {
                const size_t stat_base = (static_cast<size_t>(t.b) * a.H + t.h) * a.S;
                if (ok) {
                    mbar_expect_tx(kv_full, 2 * NS * BT);
#pragma unroll
                    for (int j = 0; j < NS; ++j) {
                        tma_load_2d(smem_u32(sK + j * BT), &tmKV128, kv_full, d + t.h * DK + j * 64, row_base + k0);
                        tma_load_2d(smem_u32(sV + j * BT), &tmKV128, kv_full, 2 * d + t.h * DK + j * 64, row_base + k0);
                    }
                }
                for (int it = 0; ok && it < nit; ++it) {
                    if (!block_active(bm, it)) continue;
                    // Both rings are released by the gradient MMAs of a block; the Q ring is one stage deeper, so when
                    // block qc - 2 retires this thread loads dO of block qc and, at once, Q of block qc + 1.
                    const int qst = qc % QST, dst = qc % DST, qs = (qi0 + it) * 64;
                    if (!mbar_wait(q_empty0 + 8 * qst, ((qc / QST) & 1) ^ 1, abort_flag, 1, &g_attn_bwd_error)) { ok = false; break; }
                    mbar_expect_tx(q_full0 + 8 * qst, QSTAGE + 256);
#pragma unroll
                    for (int j = 0; j < NS; ++j)
                        tma_load_2d(smem_u32(sQR + qst * QSTAGE + j * HT), &tmQ64, q_full0 + 8 * qst, t.h * DK + j * 64, row_base + qs);
                    bulk_load_1d(smem_u32(sLse + qst * 64), a.lse + stat_base + qs, 256, q_full0 + 8 * qst);
                    if (!mbar_wait(do_empty0 + 8 * dst, ((qc / DST) & 1) ^ 1, abort_flag, 15, &g_attn_bwd_error)) { ok = false; break; }
                    mbar_expect_tx(do_full0 + 8 * dst, QSTAGE + 256);
#pragma unroll
                    for (int j = 0; j < NS; ++j)
                        tma_load_2d(smem_u32(sDOR + dst * QSTAGE + j * HT), &tmDO64, do_full0 + 8 * dst, t.h * DK + j * 64, row_base + qs);
                    bulk_load_1d(smem_u32(sD + dst * 64), a.dvec + stat_base + qs, 256, do_full0 + 8 * dst);
                    ++qc;
                }
            }
            qc = __shfl_sync(0xffffffffu, qc, 0);
            ok = __shfl_sync(0xffffffffu, static_cast<int>(ok), 0) != 0;
        }
        leave_work_list(work, lane);
    } else if (warp == 1) {
        int qc0 = 0, tn = 0;
        bool ok = !*abort_flag;
        for (int w; ok && (w = read_tile(tile_slots, t_full0, tn, abort_flag, &g_attn_bwd_error)) >= 0; ++tn) {
            const BwdTile t = bwd_tile(w, a.H, HB);
            const int nit = a.S / 64 - t.t * 2;
            const BlockMask bm = tile_mask(t.b, t.t, nit);
            if (lane == 0) {
                const int nact = block_count(bm, nit);
                ok = mbar_wait(kv_full, tn & 1, abort_flag, 2, &g_attn_bwd_error);
                const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
                auto issue_s = [&](int gi) -> bool {               // S^T = K Q^T: needs Q of the block and the score columns
                    const int st = gi % QST;
                    if (!mbar_wait(q_full0 + 8 * st, (gi / QST) & 1, abort_flag, 3, &g_attn_bwd_error)) return false;
                    if (gi >= 1 && !mbar_wait(s_empty, (gi - 1) & 1, abort_flag, 4, &g_attn_bwd_error)) return false;
                    tc_fence_after();
                    const uint32_t q_addr = smem_u32(sQR + st * QSTAGE);
#pragma unroll
                    for (int k = 0; k < DK / 16; ++k)
                        umma_bf16(tmem_ST, smem_desc(k_addr + (k >> 2) * BT + (k & 3) * 32, 16, 1024),
                                  smem_desc(q_addr + (k >> 2) * HT + (k & 3) * 32, 16, 1024), IDESC_KK, k > 0);
                    umma_commit(s_full);
                    return true;
                };
                auto issue_dp = [&](int gi) -> bool {              // dP^T = V dO^T: needs dO of the block and the dP columns
                    const int st = gi % DST;
                    if (!mbar_wait(do_full0 + 8 * st, (gi / DST) & 1, abort_flag, 16, &g_attn_bwd_error)) return false;
                    if (gi >= 1 && !mbar_wait(dp_empty, (gi - 1) & 1, abort_flag, 17, &g_attn_bwd_error)) return false;
                    tc_fence_after();
                    const uint32_t do_addr = smem_u32(sDOR + st * QSTAGE);
#pragma unroll
                    for (int k = 0; k < DK / 16; ++k)
                        umma_bf16(tmem_dPT, smem_desc(v_addr + (k >> 2) * BT + (k & 3) * 32, 16, 1024),
                                  smem_desc(do_addr + (k >> 2) * HT + (k & 3) * 32, 16, 1024), IDESC_KK, k > 0);
                    umma_commit(dp_full);
                    return true;
                };
                auto issue_dkv = [&](int gi, bool first) -> bool {
                    const int qst = gi % QST, dst = gi % DST;
                    if (!mbar_wait(pd_full, gi & 1, abort_flag, 5, &g_attn_bwd_error)) return false;
                    // the accumulators this tile writes were read out by the workers at the end of the previous tile
                    if (first && tn >= 1 && !mbar_wait(acc_empty, (tn - 1) & 1, abort_flag, 12, &g_attn_bwd_error)) return false;
                    tc_fence_after();
                    const uint32_t pt_addr = smem_u32(sPT), dst_addr = smem_u32(sDST);
                    const uint32_t q_addr = smem_u32(sQR + qst * QSTAGE), do_addr = smem_u32(sDOR + dst * QSTAGE);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_dV, smem_desc(pt_addr + k * 32, 16, 1024), smem_desc(do_addr + k * 2048, HT, 1024), idesc_km<DK>(), (!first || k > 0));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_dK, smem_desc(dst_addr + k * 32, 16, 1024), smem_desc(q_addr + k * 2048, HT, 1024), idesc_km<DK>(), (!first || k > 0));
                    umma_commit(pd_empty);
                    umma_commit(q_empty0 + 8 * qst);
                    umma_commit(do_empty0 + 8 * dst);
                    return true;
                };
                // K and V are read by the score MMAs only: handed back with the last of those (see the dQ kernel)
                if (ok) ok = issue_s(qc0) && issue_dp(qc0);
                if (ok && nact == 1) umma_commit(kv_empty);
                for (int j = 0; ok && j < nact; ++j) {
                    if (j + 1 < nact) {
                        ok = issue_s(qc0 + j + 1) && issue_dp(qc0 + j + 1);
                        if (ok && j + 2 == nact) umma_commit(kv_empty);
                    }
                    if (ok) ok = issue_dkv(qc0 + j, j == 0);
                }
                if (ok) umma_commit(done);
                qc0 += nact;
            }
            qc0 = __shfl_sync(0xffffffffu, qc0, 0);
            ok = __shfl_sync(0xffffffffu, static_cast<int>(ok), 0) != 0;
        }
    } else {
        const int q = warp & 3, hf = (warp - 2) >> 2;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
        const float scale2 = a.scale * kL2e;
        const int sw = row & 7;
        constexpr int OC = DK / 2;                              // dK / dV columns this thread writes
        bool ok = !*abort_flag;
        int qc0 = 0, tn = 0;

        for (int w; ok && (w = read_tile(tile_slots, t_full0, tn, abort_flag, &g_attn_bwd_error)) >= 0; ++tn) {
            const BwdTile t = bwd_tile(w, a.H, HB);
            const int h = t.h, b = t.b, kt = t.t, k0 = kt * 128, qi0 = kt * 2, nit = a.S / 64 - qi0, row_base = b * a.S;
            const BlockMask bm = tile_mask(b, kt, nit);
            const int j = k0 + row;                                   // key position
            const float slope2 = ALIBI ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(a.H)) * kL2e : 0.f;
            const int my_doc = DOC ? a.doc[row_base + j] : 0;

            auto block = [&](auto diag_tag, int it, int cnt) -> bool {
                constexpr bool DIAG = decltype(diag_tag)::value;
                const int gi = qc0 + cnt;
                if (!mbar_wait(s_full, gi & 1, abort_flag, 6, &g_attn_bwd_error)) return false;
                tc_fence_after();
                const int qs = (qi0 + it) * 64 + hf * 32;              // first query of this thread's 32 columns
                uint32_t rs[32], rp[32];
                tmem_ld32(tmem_ST + lane_addr + hf * 32, rs);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_empty);
                const float4* lse4 = reinterpret_cast<const float4*>(sLse + (gi % QST) * 64 + hf * 32);
                const float4* dv4 = reinterpret_cast<const float4*>(sD + (gi % DST) * 64 + hf * 32);
                const int* dq_ptr = DOC ? a.doc + row_base + qs : nullptr;
                // base-2 exponent of P^T: raw * scale2 - slope2 * (query - key) - lse2 of the column's query; the bias of a
                // pair of columns is carried along and stepped by -2 slope2 (this kernel has no shared memory left for the
                // operand tiles with which the other kernels let the tensor core add the bias)
                const float base = ALIBI ? -slope2 * static_cast<float>(qs - j) : 0.f;
                uint64_t base2 = pack2(base, base - slope2);
                const uint64_t step2 = pack2(-2.f * slope2, -2.f * slope2), scale2x2 = pack2(scale2, scale2), negl2e = pack2(-kL2e, -kL2e),
                               neg1 = pack2(-1.f, -1.f);
                // first the exponentials (they need S^T and the log-sum-exp only); P stays in rs as fp32 for the second half
                uint32_t pk[16], dk[16];
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const float4 l4 = lse4[c4];
                    const uint64_t lsp[2] = {pack2(l4.x, l4.y), pack2(l4.z, l4.w)};
#pragma unroll
                    for (int e2 = 0; e2 < 2; ++e2) {
                        const int c = c4 * 4 + e2 * 2;
                        float x0, x1;
                        unpack2(fma2(lsp[e2], negl2e, fma2(pack2(__uint_as_float(rs[c]), __uint_as_float(rs[c + 1])), scale2x2, base2)), x0, x1);
                        if (ALIBI) base2 = add2(base2, step2);
                        float p0 = ex2a(x0), p1 = ex2a(x1);
                        if (DIAG && j > qs + c) p0 = 0.f;
                        if (DIAG && j > qs + c + 1) p1 = 0.f;
                        if (DOC && dq_ptr[c] != my_doc) p0 = 0.f;
                        if (DOC && dq_ptr[c + 1] != my_doc) p1 = 0.f;
                        rs[c] = __float_as_uint(p0);
                        rs[c + 1] = __float_as_uint(p1);
                        __nv_bfloat162 tp = __floats2bfloat162_rn(p0, p1);
                        pk[c4 * 2 + e2] = *reinterpret_cast<uint32_t*>(&tp);
                    }
                }
                // then dS^T = P^T o (dP^T - D): dP^T of this block may arrive later than S^T (its ring is one stage shorter)
                if (!mbar_wait(dp_full, gi & 1, abort_flag, 18, &g_attn_bwd_error)) return false;
                tc_fence_after();
                tmem_ld32(tmem_dPT + lane_addr + hf * 32, rp);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(dp_empty);
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const float4 d4 = dv4[c4];
                    const uint64_t ddp[2] = {pack2(d4.x, d4.y), pack2(d4.z, d4.w)};
#pragma unroll
                    for (int e2 = 0; e2 < 2; ++e2) {
                        const int c = c4 * 4 + e2 * 2;
                        float d0, d1;
                        unpack2(mul2(pack2(__uint_as_float(rs[c]), __uint_as_float(rs[c + 1])),
                                     fma2(ddp[e2], neg1, pack2(__uint_as_float(rp[c]), __uint_as_float(rp[c + 1])))), d0, d1);
                        __nv_bfloat162 td = __floats2bfloat162_rn(d0, d1);
                        dk[c4 * 2 + e2] = *reinterpret_cast<uint32_t*>(&td);
                    }
                }
                if (gi >= 1 && !mbar_wait(pd_empty, (gi - 1) & 1, abort_flag, 7, &g_attn_bwd_error)) return false;
                uint8_t* prow = sPT + row * 128;
                uint8_t* drow = sDST + row * 128;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int off = ((hf * 4 + g) ^ sw) << 4;
                    *reinterpret_cast<uint4*>(prow + off) = make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
                    *reinterpret_cast<uint4*>(drow + off) = make_uint4(dk[g * 4], dk[g * 4 + 1], dk[g * 4 + 2], dk[g * 4 + 3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(pd_full);
                return true;
            };
            int cnt = 0;
            for (int it = 0; ok && it < 2; ++it, ++cnt) ok = block(std::true_type{}, it, cnt);
            for (int it = 2; ok && it < nit; ++it) {
                if (!block_active(bm, it)) continue;
                ok = block(std::false_type{}, it, cnt);
                ++cnt;
            }
            if (ok) ok = mbar_wait(done, tn & 1, abort_flag, 8, &g_attn_bwd_error);
            if (ok) {
                tc_fence_after();
                bf16* kp = a.dqkv + (static_cast<size_t>(row_base) + j) * (3 * d) + d + h * DK + hf * OC;
#pragma unroll
                for (int c0 = 0; c0 < OC; c0 += 32) {
                    uint32_t rv[32], rk[32];
                    tmem_ld32(tmem_dV + lane_addr + hf * OC + c0, rv);
                    tmem_ld32(tmem_dK + lane_addr + hf * OC + c0, rk);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        Vec16<bf16> ok8, ov8;
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            ok8.v[k] = __float2bfloat16_rn(__uint_as_float(rk[c + k]) * a.scale);
                            ov8.v[k] = __float2bfloat16_rn(__uint_as_float(rv[c + k]));
                            rk[c + k] = __float_as_uint(__bfloat162float(ok8.v[k]));     // what is stored, for the column sums
                            rv[c + k] = __float_as_uint(__bfloat162float(ov8.v[k]));
                        }
                        st16(kp + c0 + c, ok8);
                        st16(kp + d + c0 + c, ov8);
                    }
                    if (a.colsum_part) {
                        float v[32];
                        float* dst = a.colsum_part + (static_cast<size_t>(row_base + k0) / 32 + q) * (3 * d) + d + h * DK + hf * OC + c0 + lane;
#pragma unroll
                        for (int c = 0; c < 32; ++c) v[c] = __uint_as_float(rk[c]);
                        dst[0] = lane_sums32(v, lane);
#pragma unroll
                        for (int c = 0; c < 32; ++c) v[c] = __uint_as_float(rv[c]);
                        dst[d] = lane_sums32(v, lane);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty);                  // the accumulators may be overwritten
            }
            qc0 += cnt;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(LY::TMEM_COLS) : "memory");
    }
}

// ======================================================================================
// host
// ======================================================================================
template <int DK, bool DOC, bool ALIBI>
static int launch_bwd_tc(const CUtensorMap& q128, const CUtensorMap& q64, const CUtensorMap& do128, const CUtensorMap& do64,
                         const AttnBwdArgs& a, long long tiles, cudaStream_t s)
{
    static PerDeviceOnce once;
    NNB_TRY(once.run([] {
        const cudaError_t e = cudaFuncSetAttribute(attn_bwd_dq_tc_kernel<DK, DOC, ALIBI>, cudaFuncAttributeMaxDynamicSharedMemorySize, DqLayout<DK>::SMEM);
        if (e != cudaSuccess) return e;
        return cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel<DK, DOC, ALIBI>, cudaFuncAttributeMaxDynamicSharedMemorySize, KvLayout<DK>::SMEM);
    }));
    const long long cap = static_cast<long long>(device_sm_count()) * DqLayout<DK>::CTAS_PER_SM;   // persistent kernels
    const dim3 grid(static_cast<unsigned>(tiles < cap ? tiles : cap));
    unsigned int* work = nullptr;                   // both kernels find the pair at zero and leave it at zero
    NNB_TRY(work_counter_pair(s, &work));
    attn_bwd_dq_tc_kernel<DK, DOC, ALIBI><<<grid, 320, DqLayout<DK>::SMEM, s>>>(q128, q64, do128, a, work);
    NNB_LAUNCH_CHECK();
    attn_bwd_dkv_tc_kernel<DK, DOC, ALIBI><<<grid, 320, KvLayout<DK>::SMEM, s>>>(q128, q64, do64, a, work);
    NNB_LAUNCH_CHECK();
    return 0;
}

int attention_bwd_tc(const bf16* qkv, const bf16* out, const bf16* dout, const float* lse, float* dvec, bf16* dqkv,
                     const int* doc, const int* doc_ranges, int B, int S, int H, int dk, int alibi, cudaStream_t s, bool have_dvec,
                     float* colsum_part)
{
    if (static_cast<long long>(B) * S * H == 0) return 0;
    NNB_ARG_CHECK(attention_tc_supported(dk, S, H * dk), "shape not supported by the tcgen05 attention kernels");
    if (!have_dvec) NNB_TRY(attention_dvec_bf16(out, dout, dvec, B, S, H, dk, s));
    const int d = H * dk;
    const long long rows = static_cast<long long>(B) * S;
    CUtensorMap q128, q64, do128, do64;
    NNB_TRY(tensor_map_2d(qkv, 3LL * d, rows, 3LL * d, 64, 128, &q128, 2));
    NNB_TRY(tensor_map_2d(qkv, 3LL * d, rows, 3LL * d, 64, 64, &q64, 2));
    NNB_TRY(tensor_map_2d(dout, d, rows, d, 64, 128, &do128, 2));
    NNB_TRY(tensor_map_2d(dout, d, rows, d, 64, 64, &do64, 2));
    AttnBwdArgs a{dqkv, lse, dvec, doc, doc ? reinterpret_cast<const int2*>(doc_ranges) : nullptr, colsum_part, B, S, H, 1.0f / sqrtf(static_cast<float>(dk))};
    const long long tiles = static_cast<long long>(S / 128) * H * B;
    NNB_ARG_CHECK(tiles < (1ll << 31), "too many attention tiles");
#define NNB_BWD(DKV)                                                                                      \
    do {                                                                                                  \
        if (doc && alibi) return launch_bwd_tc<DKV, true, true>(q128, q64, do128, do64, a, tiles, s);     \
        if (doc) return launch_bwd_tc<DKV, true, false>(q128, q64, do128, do64, a, tiles, s);             \
        if (alibi) return launch_bwd_tc<DKV, false, true>(q128, q64, do128, do64, a, tiles, s);           \
        return launch_bwd_tc<DKV, false, false>(q128, q64, do128, do64, a, tiles, s);                     \
    } while (0)
    if (dk == 64) NNB_BWD(64);
    NNB_BWD(128);
#undef NNB_BWD
}

int attention_bwd_device_error(int* code)
{
    NNB_CUDA_CHECK(cudaMemcpyFromSymbol(code, g_attn_bwd_error, sizeof(int)));
    if (*code) { const int z = 0; NNB_CUDA_CHECK(cudaMemcpyToSymbol(g_attn_bwd_error, &z, sizeof(int))); }
    return 0;
}

}  // namespace nnb
