// Fused causal / document-masked / ALiBi attention forward on the 5th-generation tensor cores.  Head size 64 runs the
// kernel of attention_tc_fwd64.cuh (four one-chain CTAs per SM); this file holds the kernel for head size 128, the
// per-64-row document ranges, and the host entry point for both.
//
// Head size 128.  Persistent: one CTA per SM walks the list of (128-query tile, head, batch) work items, longest tiles
// first, in snake order (snake_tile in tc_ptx.cuh).  Ten warps:
//   warp 0      TMA producer: the tile's Q, then per 128-key block one K tile and one V tile (ring of two)
//   warp 1      MMA issuer:   S = Q K^T   (128 x 128 x head)  into TMEM columns [0, 128)
//                             O' = P V    (128 x head x 128)  into TMEM columns [128, 128 + head)
//   warps 2..9  softmax: thread (row, half) owns 64 of the 128 score columns of one query row (two warps share each
//               32-lane TMEM quadrant).  It reads its scores from TMEM twice, 32 columns at a time (row maximum, then
//               P), so that it never holds more than 32 of them; applies scale, causal / document mask and ALiBi bias;
//               exchanges the row maximum with its partner through shared memory; writes P as bf16 into a K-major
//               128B-swizzled shared tile (the A operand of the second MMA) and folds its half of the columns of O'
//               into registers; at the end of a tile it normalises and stores its output row.
// Q, K, S and P are single-buffered (the key tile is released as soon as Q K^T has read it).  All ring positions and
// barrier phases are counted across tiles, so the first loads and MMAs of the next tile overlap the write-out of this one.
// K-major operands wider than 64 values are kept as sub-tiles of 64 columns (one 128-byte swizzle atom per row);
// V is consumed as an MN-major B operand straight from its (key, head) tile.  Nothing of size (S, S) reaches memory.
// (The kernel is a template over the head size; only 128 is instantiated.)
//
// ALiBi: the bias -slope_h (i - j) is linear in the key position, so the tensor core adds it: one more MMA step per
// block multiplies a (128 x 16) tile that holds slope_h / scale, split into three bf16 terms (24 bits), in every query
// row by a constant tile that holds the key's position inside the block (exact in bf16) three times.  What is left
// per block is one constant per row (slope_h * first key of the block; the -slope_h * i term cannot change a row's
// softmax and is put back into the log-sum-exp at the end), so a score costs one packed multiply-add and one ex2.
//
// Document masks: with a table of per-64-row (min, max) document ids (attention_doc_ranges) every role skips the key
// blocks whose id range cannot meet the query tile's range.  A skipped block would have contributed P = 0 everywhere,
// so the result is bit-identical with and without the table.
//
// Replaces batched_matmul_reduce / _softmax_denom / _softmax_apply and the materialised score path of the reference
// (compute_layer.hpp:1193-1252; cpu_engine.hpp:426-699) and the per-step host mask build (:2081-2128, 2226-2246).
// Every wait is bounded; a wait that gives up raises a status word, the softmax warps learn of it together at their
// next exchange barrier, and the CTA drains.
#include <type_traits>

#include "attention_tc.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace nnb {

__device__ int g_attn_error = 0;

constexpr int AQ = 128, AK = 128;
constexpr int A_TILE = 128 * 128;                  // bytes of a 128-row x 64-bf16 sub-tile
constexpr float kLog2eF = 1.4426950408889634f, kLn2F = 0.6931471805599453f;

// shared memory: Q | K | V ring of two | P (two 64-key halves) | row-max exchange | ALiBi operand tiles | barriers
constexpr int A_BIAS_TILE = 128 * 32;              // bytes of a 128-row x 16-bf16 tile without swizzle
template <int DK> struct FwdLayout {
    static constexpr int NS = DK / 64;                                  // 64-column sub-tiles per operand tile
    static constexpr int OFF_K = NS * A_TILE, OFF_V = 2 * NS * A_TILE, OFF_P = 4 * NS * A_TILE, OFF_X = OFF_P + 2 * A_TILE,
                         OFF_U = OFF_X + 2 * 2 * 128 * 4, OFF_W = OFF_U + A_BIAS_TILE, OFF_BAR = OFF_W + A_BIAS_TILE,
                         SMEM = OFF_BAR + 256;
    static constexpr uint32_t TMEM_COLS = 256;                          // scores [0, 128), O' [128, 128 + DK)
    static constexpr int CTAS_PER_SM = DK == 64 ? 2 : 1;
};

struct AttnTcArgs {
    bf16* out; float* lse; const int* doc; const int2* ranges;
    int B, S, H, alibi;
    float scale;
};

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Barrier of the 256 softmax threads that also ORs a flag over them.  Every wait a softmax thread gives up on is
// carried to the next of these barriers, where all eight warps leave together; nobody is left alone at one.
__device__ __forceinline__ bool softmax_any(bool pred)
{
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 2, 256, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"(static_cast<uint32_t>(pred)) : "memory");
    return r != 0;
}

// work item w of a persistent CTA: query tiles in descending length, heads and batches inside
struct AttnTile { int qb, h, b; };
__device__ __forceinline__ AttnTile attn_tile(int w, int nq, int H, int HB)
{
    AttnTile t;
    const int hb = w % HB;
    t.qb = nq - 1 - w / HB;
    t.h = hb % H;
    t.b = hb / H;
    return t;
}

template <int DK, bool DOC, bool ALIBI>
__global__ void __launch_bounds__(320, FwdLayout<DK>::CTAS_PER_SM)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQKV, const AttnTcArgs a)
{
    using LY = FwdLayout<DK>;
    constexpr int NS = LY::NS, TILE = NS * A_TILE;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;                            // one query tile
    uint8_t* sK = smem + LY::OFF_K;                // one key tile: free again as soon as Q K^T of its block has run
    uint8_t* sV = smem + LY::OFF_V;                // two value tiles
    uint8_t* sP = smem + LY::OFF_P;                // one P tile (two 64-key halves)
    float* sX = reinterpret_cast<float*>(smem + LY::OFF_X);   // [buffer][half][row]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + LY::OFF_BAR);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, q_empty = bar0 + 8, k_full = bar0 + 16, k_empty = bar0 + 24, v_full0 = bar0 + 32, v_empty0 = bar0 + 48,
                   s_full = bar0 + 64, s_empty = bar0 + 72, p_full = bar0 + 80, p_empty = bar0 + 88, o_full = bar0 + 96, o_empty = bar0 + 104;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = a.H * DK;
    const int nq = a.S / AQ;
    const int total = nq * a.H * a.B;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1); mbar_init(q_empty, 1); mbar_init(k_full, 1); mbar_init(k_empty, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 1); }
        mbar_init(s_full, 1); mbar_init(s_empty, 8); mbar_init(p_full, 8); mbar_init(p_empty, 1);
        mbar_init(o_full, 1); mbar_init(o_empty, 8);
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;        // the swizzled tiles need a 1024-byte aligned base
        if (*abort_flag) atomicCAS(&g_attn_error, 0, (9 << 16));
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
    const uint32_t tmem_O = tmem_base + 128;
    uint8_t* sU = smem + LY::OFF_U;                // slope_h / scale in every query row (rewritten per tile by warp 0)
    uint8_t* sW = smem + LY::OFF_W;                // key position inside the block, constant
    if (ALIBI) {
        // unswizzled K-major tiles, 16 values deep: row r, values [8c, 8c + 8) at (r / 8) * 256 + c * 128 + (r % 8) * 16
        for (int r = threadIdx.x; r < 128; r += blockDim.x) {
            const uint32_t off = (r >> 3) * 256 + (r & 7) * 16;
            const __nv_bfloat162 jj = __floats2bfloat162_rn(static_cast<float>(r), static_cast<float>(r));
            const uint32_t j2 = *reinterpret_cast<const uint32_t*>(&jj);
            *reinterpret_cast<uint4*>(sW + off) = make_uint4(j2, j2 & 0xffffu, 0u, 0u);      // [r, r, r, 0, 0, 0, 0, 0]
            *reinterpret_cast<uint4*>(sW + off + 128) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(sU + off) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(sU + off + 128) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
    }

    // instruction descriptors: fp32 accumulate, bf16 operands; S: N=128, both K-major; PV: N=DK, B MN-major
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(AK >> 3) << 17) | (uint32_t(AQ >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (uint32_t(DK >> 3) << 17) | (uint32_t(AQ >> 4) << 24);

    // Every role walks the same list of tiles and, inside a tile, the same list of active key blocks; the ring / buffer
    // positions and barrier phases run on across tiles (kv: count of key blocks processed; tn: tile counter).
    // A whole warp evaluates the block mask (one ballot per 32 blocks); lane 0 of warps 0 and 1 then does the work.
    auto tile_mask = [&](const AttnTile& t, int nkb) -> BlockMask {
        if (!DOC || a.ranges == nullptr) return block_mask_all();
        const int2* rng = a.ranges + static_cast<size_t>(t.b) * (a.S / 64);
        return doc_block_mask(rng, 0, nkb, 2, rng[2 * t.qb], rng[2 * t.qb + 1], nkb - 1, nkb, lane);
    };

    if (warp == 0) {
        int kv = 0, tn = 0;
        bool ok = !*abort_flag;
        for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
            const AttnTile t = attn_tile(w, nq, a.H, a.H * a.B);
            const int nkb = t.qb + 1, row_base = t.b * a.S;
            const BlockMask bm = tile_mask(t, nkb);
            if (lane == 0) ok = mbar_wait(q_empty, (tn & 1) ^ 1, abort_flag, 11, &g_attn_error);   // the previous tile's MMAs are done
            ok = __shfl_sync(0xffffffffu, static_cast<int>(ok), 0) != 0;
            if (ALIBI && ok) {
                // this head's slope / scale as three bf16 terms, in every query row of the U tile
                const float sv = exp2f(-8.0f * static_cast<float>(t.h) / static_cast<float>(a.H)) / a.scale;
                const bf16 s0 = __float2bfloat16_rn(sv);
                const float r1 = sv - __bfloat162float(s0);
                const bf16 s1 = __float2bfloat16_rn(r1);
                const bf16 s2 = __float2bfloat16_rn(r1 - __bfloat162float(s1));
                const uint32_t w0 = static_cast<uint32_t>(__bfloat16_as_ushort(s0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(s1)) << 16);
                const uint32_t w1 = static_cast<uint32_t>(__bfloat16_as_ushort(s2));
                for (int r = lane; r < 128; r += 32)
                    *reinterpret_cast<uint4*>(sU + (r >> 3) * 256 + (r & 7) * 16) = make_uint4(w0, w1, 0u, 0u);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
            }
            if (lane == 0) {
                if (ok) {
                    mbar_expect_tx(q_full, TILE);
#pragma unroll
                    for (int j = 0; j < NS; ++j) tma_load_2d(smem_u32(sQ + j * A_TILE), &tmQKV, q_full, t.h * DK + j * 64, row_base + t.qb * AQ);
                }
                for (int kb = 0; ok && kb < nkb; ++kb) {
                    if (!block_active(bm, kb)) continue;
                    if (!mbar_wait(k_empty, (kv & 1) ^ 1, abort_flag, 1, &g_attn_error)) { ok = false; break; }
                    mbar_expect_tx(k_full, TILE);
#pragma unroll
                    for (int j = 0; j < NS; ++j) tma_load_2d(smem_u32(sK + j * A_TILE), &tmQKV, k_full, d + t.h * DK + j * 64, row_base + kb * AK);
                    const int vs = kv & 1;
                    if (!mbar_wait(v_empty0 + 8 * vs, ((kv >> 1) & 1) ^ 1, abort_flag, 12, &g_attn_error)) { ok = false; break; }
                    mbar_expect_tx(v_full0 + 8 * vs, TILE);
#pragma unroll
                    for (int j = 0; j < NS; ++j)
                        tma_load_2d(smem_u32(sV + vs * TILE + j * A_TILE), &tmQKV, v_full0 + 8 * vs, 2 * d + t.h * DK + j * 64, row_base + kb * AK);
                    ++kv;
                }
            }
            kv = __shfl_sync(0xffffffffu, kv, 0);
            ok = __shfl_sync(0xffffffffu, static_cast<int>(ok), 0) != 0;
        }
    } else if (warp == 1) {
        int kv = 0, tn = 0;
        bool ok = !*abort_flag;
        for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
            const AttnTile t = attn_tile(w, nq, a.H, a.H * a.B);
            const int nkb = t.qb + 1;
            const BlockMask bm = tile_mask(t, nkb);
            if (lane == 0) {
                ok = mbar_wait(q_full, tn & 1, abort_flag, 2, &g_attn_error);
                const uint32_t q_addr = smem_u32(sQ);
                auto issue_s = [&](int gj) -> bool {
                    if (!mbar_wait(k_full, gj & 1, abort_flag, 5, &g_attn_error)) return false;
                    if (gj >= 1 && !mbar_wait(s_empty, (gj - 1) & 1, abort_flag, 6, &g_attn_error)) return false;
                    tc_fence_after();
                    const uint32_t k_addr = smem_u32(sK);
#pragma unroll
                    for (int k = 0; k < DK / 16; ++k) {
                        const uint32_t o = (k >> 2) * A_TILE + (k & 3) * 32;
                        umma_bf16(tmem_base, smem_desc(q_addr + o, 16, 1024), smem_desc(k_addr + o, 16, 1024), IDESC_S, k > 0 ? 1u : 0u);
                    }
                    if (ALIBI)       // + (slope / scale) * (key position inside the block)
                        umma_bf16(tmem_base, smem_desc_noswizzle(smem_u32(sU), 128, 256), smem_desc_noswizzle(smem_u32(sW), 128, 256), IDESC_S, 1u);
                    umma_commit(s_full);
                    umma_commit(k_empty);                           // the key tile is free once these MMAs have read it
                    return true;
                };
                auto issue_pv = [&](int gj) -> bool {
                    const int vs = gj & 1;
                    if (!mbar_wait(p_full, gj & 1, abort_flag, 3, &g_attn_error)) return false;
                    if (gj >= 1 && !mbar_wait(o_empty, (gj - 1) & 1, abort_flag, 4, &g_attn_error)) return false;
                    if (!mbar_wait(v_full0 + 8 * vs, (gj >> 1) & 1, abort_flag, 13, &g_attn_error)) return false;
                    tc_fence_after();
                    const uint32_t p_addr = smem_u32(sP);
                    const uint32_t v_addr = smem_u32(sV + vs * TILE);
#pragma unroll
                    for (int k = 0; k < AK / 16; ++k) {
                        const uint64_t da = smem_desc(p_addr + (k >> 2) * A_TILE + (k & 3) * 32, 16, 1024);
                        const uint64_t db = smem_desc(v_addr + k * 2048, A_TILE, 1024);   // the next 64 head columns: one sub-tile on
                        umma_bf16(tmem_O, da, db, IDESC_PV, k > 0 ? 1u : 0u);
                    }
                    umma_commit(o_full);
                    umma_commit(p_empty);
                    umma_commit(v_empty0 + 8 * vs);
                    return true;
                };
                // the scores of the next active block are issued before P V of the current one
                const int nact = block_count(bm, nkb);
                if (ok) ok = issue_s(kv);
                for (int j = 0; ok && j < nact; ++j) {
                    if (j + 1 < nact) ok = issue_s(kv + j + 1);
                    if (ok) ok = issue_pv(kv + j);
                }
                if (ok) umma_commit(q_empty);                   // the query tile is free once this tile's MMAs are done
                kv += nact;
            }
            kv = __shfl_sync(0xffffffffu, kv, 0);
            ok = __shfl_sync(0xffffffffu, static_cast<int>(ok), 0) != 0;
        }
    } else {
        const int q = warp & 3, hf = (warp - 2) >> 2;          // TMEM lane quadrant, column half
        const int row = q * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
        const float scale2 = a.scale * kLog2eF;
        const int sw = row & 7;
        constexpr int OC = DK / 2;                              // output columns this thread keeps
        bool ok = true, bad = *abort_flag != 0;                 // bad: a wait of this thread gave up (reported at the next barrier)
        int kv0 = 0, xc = 0;                                    // key-block counter; exchange counter (alternates the sX buffer)

        for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps) {
            const AttnTile t = attn_tile(w, nq, a.H, a.H * a.B);
            const int h = t.h, b = t.b, q0 = t.qb * AQ, nkb = t.qb + 1, row_base = b * a.S;
            const BlockMask bm = tile_mask(t, nkb);
            const int i = q0 + row;                            // query position inside the sequence
            const float slope2 = ALIBI ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(a.H)) * kLog2eF : 0.f;
            const int my_doc = DOC ? a.doc[row_base + i] : 0;
            // Running maximum and sum in the base-2 domain.  With ALiBi the -slope2 * i term of the bias is left out
            // here (it is the same for every key of the row) and goes back into the log-sum-exp at the end.
            float m_run = -INFINITY, l_run = 0.f;
            uint64_t o_acc[OC / 2];                            // packed pairs of output columns
#pragma unroll
            for (int c = 0; c < OC / 2; ++c) o_acc[c] = 0ull;
            const uint64_t scale2x2 = pack2(scale2, scale2);

            auto fold_o = [&](int gj) -> bool {                 // o_acc += O'(gj), this thread's columns
                if (!mbar_wait(o_full, gj & 1, abort_flag, 7, &g_attn_error)) return false;
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < OC; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_O + lane_addr + hf * OC + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 16; ++c)
                        o_acc[c0 / 2 + c] = add2(o_acc[c0 / 2 + c], pack2(__uint_as_float(r[2 * c]), __uint_as_float(r[2 * c + 1])));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(o_empty);
                return true;
            };

            // One 128-key block, the cnt-th active one of the tile.  DIAG: the block on the diagonal (causal mask
            // inside it).  The tensor core left raw = q.k (+ slope / scale * position inside the block) in TMEM, so
            // the base-2 score of column cj is raw * scale2 + okb with okb = slope2 * (first key of the block).
            auto block = [&](auto diag_tag, int kb, int cnt) -> bool {
                constexpr bool DIAG = decltype(diag_tag)::value;
                const int gj = kv0 + cnt;
                bad |= !mbar_wait(s_full, gj & 1, abort_flag, 8, &g_attn_error);
                tc_fence_after();
                const int k0 = kb * AK;
                const int* dk_ptr = DOC ? a.doc + row_base + k0 + hf * 64 : nullptr;
                const float okb = ALIBI ? slope2 * static_cast<float>(k0) : 0.f;
                auto masked = [&](int cj) -> bool {             // cj is a literal once unrolled
                    bool m = false;
                    if (DIAG) m = hf * 64 + cj > row;
                    if (DOC) m = m || dk_ptr[cj] != my_doc;
                    return m;
                };
                // Two passes over the scores in TMEM, 32 columns at a time, so that the thread never holds more than
                // 32 of them: the first finds the row maximum (of the raw values: the scale is positive), the second
                // makes P.  The score buffer is released after the second pass.
                float mxr = -INFINITY;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + lane_addr + hf * 64 + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) {
                        float v = __uint_as_float(r[jj]);
                        if ((DIAG || DOC) && masked(c * 32 + jj)) v = -INFINITY;
                        mxr = fmaxf(mxr, v);
                    }
                }
                const float mx = fmaf(mxr, scale2, okb);         // -inf stays -inf
                float* xs = sX + (xc & 1) * 256;
                ++xc;
                xs[hf * 128 + row] = mx;
                if (softmax_any(bad)) return false;             // the same answer in all eight warps
                const float m_new = fmaxf(m_run, fmaxf(mx, xs[(hf ^ 1) * 128 + row]));
                const float ms = (m_new == -INFINITY) ? 0.f : m_new;
                const float corr = ex2_approx(m_run - ms);
                if (cnt >= 1) bad |= !fold_o(gj - 1);
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
                    const uint64_t corr2 = pack2(corr, corr);
#pragma unroll
                    for (int c = 0; c < OC / 2; ++c) o_acc[c] = mul2(o_acc[c], corr2);
                }
                if (gj >= 1) bad |= !mbar_wait(p_empty, (gj - 1) & 1, abort_flag, 10, &g_attn_error);
                uint8_t* prow = sP + hf * A_TILE + row * 128;
                const uint64_t shift2 = pack2(okb - ms, okb - ms);
                uint64_t rs2 = 0ull;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + lane_addr + hf * 64 + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int jj = g * 8 + e * 2;
                            float x0, x1;
                            unpack2(fma2(pack2(__uint_as_float(r[jj]), __uint_as_float(r[jj + 1])), scale2x2, shift2), x0, x1);
                            float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                            if ((DIAG || DOC) && masked(c * 32 + jj)) p0 = 0.f;
                            if ((DIAG || DOC) && masked(c * 32 + jj + 1)) p1 = 0.f;
                            rs2 = add2(rs2, pack2(p0, p1));
                            __nv_bfloat162 tt = __floats2bfloat162_rn(p0, p1);
                            pk[e] = *reinterpret_cast<uint32_t*>(&tt);
                        }
                        *reinterpret_cast<uint4*>(prow + (((c * 4 + g) ^ sw) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_empty);            // both passes have read the scores
                float rs_lo, rs_hi;
                unpack2(rs2, rs_lo, rs_hi);
                l_run = l_run * corr + (rs_lo + rs_hi);
                m_run = m_new;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
                return true;
            };
            int cnt = 0;
            for (int kb = 0; ok && kb < nkb - 1; ++kb) {
                if (!block_active(bm, kb)) continue;
                ok = block(std::false_type{}, kb, cnt);
                ++cnt;
            }
            if (ok) { ok = block(std::true_type{}, nkb - 1, cnt); ++cnt; }
            if (!ok) break;                                     // decided at a barrier: uniform over the softmax warps
            bad |= !fold_o(kv0 + cnt - 1);
            // the row sum is split over the two halves: exchange once more
            float* xs = sX + (xc & 1) * 256;
            ++xc;
            xs[hf * 128 + row] = l_run;
            if (softmax_any(bad)) break;
            {
                const float l_tot = l_run + xs[(hf ^ 1) * 128 + row];
                const float inv = 1.0f / l_tot;
                bf16* op = a.out + (static_cast<size_t>(row_base) + i) * d + h * DK + hf * OC;
                const uint64_t inv2 = pack2(inv, inv);
#pragma unroll
                for (int c = 0; c < OC; c += 8) {
                    uint32_t pk[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float v0, v1;
                        unpack2(mul2(o_acc[c / 2 + k], inv2), v0, v1);
                        __nv_bfloat162 tt = __floats2bfloat162_rn(v0, v1);
                        pk[k] = *reinterpret_cast<uint32_t*>(&tt);
                    }
                    *reinterpret_cast<uint4*>(op + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
                // log-sum-exp in natural units; the ALiBi term left out of the running maximum comes back here
                if (hf == 0)
                    a.lse[(static_cast<size_t>(b) * a.H + h) * a.S + i] = (m_run + log2f(l_tot) - slope2 * static_cast<float>(i)) * kLn2F;
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

}  // namespace nnb

#include "attention_tc_fwd64.cuh"

namespace nnb {

// ---------------------------------------------------------------- document ranges
// ranges[b * S/64 + blk] = (min, max) of the document ids of rows [64 blk, 64 blk + 64) of sequence b: one warp per block
__global__ void doc_ranges_kernel(const int* __restrict__ doc, int2* __restrict__ ranges, int nblocks)
{
    const int blk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (blk >= nblocks) return;
    const int a0 = doc[static_cast<size_t>(blk) * 64 + lane], a1 = doc[static_cast<size_t>(blk) * 64 + 32 + lane];
    int lo = min(a0, a1), hi = max(a0, a1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if (lane == 0) ranges[blk] = make_int2(lo, hi);
}

int attention_doc_ranges(const int* doc, int B, int S, int* ranges, cudaStream_t s)
{
    NNB_ARG_CHECK(doc && ranges, "document ids and the range table are required");
    NNB_ARG_CHECK(S % 64 == 0, "the sequence length must be a multiple of 64");
    const int nblocks = B * (S / 64);
    if (nblocks == 0) return 0;
    doc_ranges_kernel<<<static_cast<unsigned>(ceil_div(nblocks, 8)), 256, 0, s>>>(doc, reinterpret_cast<int2*>(ranges), nblocks);
    NNB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- host
template <int DK, bool DOC, bool ALIBI>
static int launch_fwd_tc(const CUtensorMap& tm, const AttnTcArgs& a, long long tiles, cudaStream_t s)
{
    using LY = FwdLayout<DK>;
    static PerDeviceOnce once;
    NNB_TRY(once.run([] { return cudaFuncSetAttribute(attn_fwd_tc_kernel<DK, DOC, ALIBI>, cudaFuncAttributeMaxDynamicSharedMemorySize, LY::SMEM); }));
    const long long slots = static_cast<long long>(device_sm_count()) * LY::CTAS_PER_SM;
    const dim3 grid(static_cast<unsigned>(tiles < slots ? tiles : slots));     // persistent: each CTA walks the tile list
    attn_fwd_tc_kernel<DK, DOC, ALIBI><<<grid, 320, LY::SMEM, s>>>(tm, a);
    NNB_LAUNCH_CHECK();
    return 0;
}

bool attention_tc_supported(int dk, int S, int d) { return (dk == 64 || dk == 128) && (S % AQ) == 0 && (d % 8) == 0; }

int attention_fwd_tc(const bf16* qkv, bf16* out, float* lse, const int* doc, const int* doc_ranges, int B, int S, int H, int dk,
                     int alibi, cudaStream_t s)
{
    if (static_cast<long long>(B) * S * H == 0) return 0;
    NNB_ARG_CHECK(attention_tc_supported(dk, S, H * dk), "shape not supported by the tcgen05 attention kernel");
    CUtensorMap tm;
    const int d = H * dk;
    NNB_TRY(tensor_map_2d(qkv, 3LL * d, static_cast<long long>(B) * S, 3LL * d, 64, 128, &tm, 2));
    AttnTcArgs a{out, lse, doc, doc ? reinterpret_cast<const int2*>(doc_ranges) : nullptr, B, S, H, alibi, 1.0f / sqrtf(static_cast<float>(dk))};
    const long long tiles = static_cast<long long>(S / AQ) * H * B;
    NNB_ARG_CHECK(tiles < (1ll << 31), "too many attention tiles");
#define NNB_FWD(DKV)                                                                          \
    do {                                                                                      \
        if (doc && alibi) return launch_fwd_tc<DKV, true, true>(tm, a, tiles, s);             \
        if (doc) return launch_fwd_tc<DKV, true, false>(tm, a, tiles, s);                     \
        if (alibi) return launch_fwd_tc<DKV, false, true>(tm, a, tiles, s);                   \
        return launch_fwd_tc<DKV, false, false>(tm, a, tiles, s);                             \
    } while (0)
    if (dk == 64) {
        CUtensorMap tkv;
        NNB_TRY(tensor_map_2d(qkv, 3LL * d, static_cast<long long>(B) * S, 3LL * d, 64, Fwd64::KB, &tkv, 2));
        if (doc && alibi) return launch_fwd_tc64<true, true>(tm, tkv, a, tiles, s);
        if (doc) return launch_fwd_tc64<true, false>(tm, tkv, a, tiles, s);
        if (alibi) return launch_fwd_tc64<false, true>(tm, tkv, a, tiles, s);
        return launch_fwd_tc64<false, false>(tm, tkv, a, tiles, s);
    }
    NNB_FWD(128);
#undef NNB_FWD
}

int attention_device_error(int* code)
{
    NNB_CUDA_CHECK(cudaMemcpyFromSymbol(code, g_attn_error, sizeof(int)));
    if (*code) { const int z = 0; NNB_CUDA_CHECK(cudaMemcpyToSymbol(g_attn_error, &z, sizeof(int))); }
    return 0;
}

}  // namespace nnb
