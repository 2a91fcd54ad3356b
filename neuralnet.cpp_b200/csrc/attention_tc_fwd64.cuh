// Attention forward for head size 64 (included by attention_tc.cu): four small CTAs per SM instead of two large ones.
//
// The kernel for the general case couples eight softmax warps of a CTA at two barriers per key block, and an SM runs
// two such chains; its issue slots are idle three quarters of the time, waiting on TMEM loads, barriers and the tensor
// core in turn.  Here a CTA is one short chain and an SM runs four of them:
//   * 64-key blocks: scores take 64 TMEM columns, the output 64, so a CTA needs 128 columns and four CTAs fit an SM;
//   * one thread per query row (four softmax warps, one per TMEM lane quadrant): the row maximum and the row sum need no
//     exchange between threads, and the softmax warps meet nowhere but at the mbarrier that hands P to the MMA warp;
//   * the output accumulates in TMEM across key blocks (the P V MMAs add into it); a thread touches its output row only
//     when the reference point of its exponentials has to move: the running maximum may run ahead of the reference by up
//     to 2^8 before the row (sum and output) is rescaled, so after the first blocks of a tile that is rare;
//   * Q, K, V, S and P are single-buffered: 55 KB of shared memory per CTA.
// Five warps: a control warp whose lane 0 issues every TMA load and every MMA in the order the data dependencies give,
// and four softmax warps.  The CTAs draw their (128-query tile, head, batch) items, longest first, from a counter in
// global memory (work_counter.cu); the control thread passes each item on through a two-slot ring in shared memory.
// The control thread treats the key blocks of successive tiles as one stream: while the softmax warps finish the last
// block of a tile and write its output rows, the next tile's Q and first K / V tiles are loaded and its first score
// MMA is issued.  The score columns are handed back (s_free) as soon as the second pass has read them, before the
// exponentials are done, so the next score MMA overlaps the rest of the block.
// ALiBi-by-MMA, document block skipping, bounded waits and the status word are those of the general kernel.
#pragma once

namespace nnb {

struct Fwd64 {
    static constexpr int KB = 64;                                       // keys per block
    static constexpr int K_TILE = KB * 128;                             // bytes of a 64-row x 64-bf16 tile
    static constexpr int OFF_K = A_TILE, OFF_V = OFF_K + K_TILE, OFF_P = OFF_V + K_TILE, OFF_U = OFF_P + A_TILE,
                         OFF_W = OFF_U + A_BIAS_TILE, OFF_BAR = OFF_W + A_BIAS_TILE / 2, SMEM = 55 * 1024;
    static constexpr uint32_t TMEM_COLS = 128;                          // scores [0, 64), output [64, 128)
    static constexpr int CTAS_PER_SM = 4, THREADS = 160;
    static constexpr float LAZY = 8.0f;                                 // log2 of the head-room of the exponentials
};
static_assert(Fwd64::OFF_BAR + 128 <= Fwd64::SMEM, "barriers do not fit");

template <bool DOC, bool ALIBI>
__global__ void __launch_bounds__(Fwd64::THREADS, Fwd64::CTAS_PER_SM)
attn_fwd_tc64_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV, const AttnTcArgs a,
                     unsigned int* __restrict__ work)
{
    using LY = Fwd64;
    constexpr int DK = 64, KB = LY::KB;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = smem + LY::OFF_K;
    uint8_t* sV = smem + LY::OFF_V;
    uint8_t* sP = smem + LY::OFF_P;
    uint8_t* sU = smem + LY::OFF_U;                // slope_h / scale in every query row (rewritten per tile by warp 0)
    uint8_t* sW = smem + LY::OFF_W;                // key position inside the block, constant
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + LY::OFF_BAR);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, k_full = bar0 + 8, v_full = bar0 + 16, s_full = bar0 + 24, p_full = bar0 + 32, pv_done = bar0 + 40, o_empty = bar0 + 48,
                   s_free = bar0 + 56, t_full0 = bar0 + 64;     // t_full: two barriers
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* tile_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);      // two entries

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = a.H * DK;
    const int nq = a.S / AQ;
    const int total = nq * a.H * a.B;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1); mbar_init(k_full, 1); mbar_init(v_full, 1);
        mbar_init(s_full, 1); mbar_init(p_full, 4); mbar_init(pv_done, 1); mbar_init(o_empty, 4);
        mbar_init(s_free, 4); mbar_init(t_full0, 1); mbar_init(t_full0 + 8, 1);
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;        // the swizzled tiles need a 1024-byte aligned base
        if (*abort_flag) atomicCAS(&g_attn_error, 0, (9 << 16));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(LY::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (ALIBI) {
        // unswizzled K-major tiles, 16 values deep: row r, values [8c, 8c + 8) at (r / 8) * 256 + c * 128 + (r % 8) * 16
        for (int r = threadIdx.x; r < 128; r += blockDim.x) {
            const uint32_t off = (r >> 3) * 256 + (r & 7) * 16;
            if (r < KB) {
                const __nv_bfloat162 jj = __floats2bfloat162_rn(static_cast<float>(r), static_cast<float>(r));
                const uint32_t j2 = *reinterpret_cast<const uint32_t*>(&jj);
                *reinterpret_cast<uint4*>(sW + off) = make_uint4(j2, j2 & 0xffffu, 0u, 0u);      // [r, r, r, 0, 0, 0, 0, 0]
                *reinterpret_cast<uint4*>(sW + off + 128) = make_uint4(0u, 0u, 0u, 0u);
            }
            *reinterpret_cast<uint4*>(sU + off) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(sU + off + 128) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_O = tmem_base + 64;

    // instruction descriptors: fp32 accumulate, bf16 operands, M = 128, N = 64; S: both K-major; PV: B MN-major
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(KB >> 3) << 17) | (uint32_t(AQ >> 4) << 24);
    constexpr uint32_t IDESC_PV = IDESC_S | (1u << 16);

    // Every role walks the same list of tiles and, inside a tile, the same list of active 64-key blocks (the two blocks
    // on the diagonal are always active); kv counts the key blocks processed, tn the tiles, and give the barrier phases.
    auto tile_mask = [&](const AttnTile& t, int nkb) -> BlockMask {
        if (!DOC || a.ranges == nullptr) return block_mask_all();
        const int2* rng = a.ranges + static_cast<size_t>(t.b) * (a.S / 64);
        return doc_block_mask(rng, 0, nkb, 1, rng[2 * t.qb], rng[2 * t.qb + 1], nkb - 2, nkb, lane);
    };

    if (warp == 0) {
        if (lane == 0) {
            // Control thread.  s_full doubles as "the key tile, the query tile and the slope tile have been read", pv_done
            // as "the value tile and P have been read".  kv counts key blocks, tn tiles: they give the barrier phases.
            int kv = 0, tn = 0;
            bool ok = !*abort_flag;
            const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), p_addr = smem_u32(sP), v_addr = smem_u32(sV);
            auto wait1 = [&](uint32_t bar, uint32_t parity, int code) -> bool { return mbar_wait(bar, parity, abort_flag, code, &g_attn_error); };
            auto issue_s = [&]() {
#pragma unroll
                for (int k = 0; k < DK / 16; ++k)
                    umma_bf16(tmem_base, smem_desc(q_addr + k * 32, 16, 1024), smem_desc(k_addr + k * 32, 16, 1024), IDESC_S, k > 0 ? 1u : 0u);
                if (ALIBI)       // + (slope / scale) * (key position inside the block)
                    umma_bf16(tmem_base, smem_desc_noswizzle(smem_u32(sU), 128, 256), smem_desc_noswizzle(smem_u32(sW), 128, 256), IDESC_S, 1u);
                umma_commit(s_full);
            };
            auto issue_pv = [&](bool first) {                  // first block of a tile: the output columns start from zero
#pragma unroll
                for (int k = 0; k < KB / 16; ++k)
                    umma_bf16(tmem_O, smem_desc(p_addr + k * 32, 16, 1024), smem_desc(v_addr + k * 2048, A_TILE, 1024), IDESC_PV,
                              (first && k == 0) ? 0u : 1u);
                umma_commit(pv_done);
            };
            // position in the stream of key blocks: tile (w < 0: the list is exhausted), block, document range of the tile
            struct Pos { int w, h, row_base, q0, nkb, kb, tmin, tmax; const int2* rng; };
            // The next item is drawn when two blocks of the current tile are left (about the latency of the draw), not
            // earlier: an item drawn is an item no other CTA can take.
            unsigned int drawn = atomicAdd(work, 1u);
            bool have_draw = true;
            int tiles_out = 0;                                  // tiles handed to the softmax warps so far
            auto active = [&](const Pos& p, int kb) -> bool {   // the same rule as doc_block_mask
                if (!DOC || p.rng == nullptr || p.nkb > 128 || kb >= p.nkb - 2) return true;
                const int2 r = p.rng[kb];
                return !(r.y < p.tmin || r.x > p.tmax);
            };
            auto open_tile = [&](Pos& p) {                      // the next item of the list, handed to the softmax warps as well
                if (!have_draw) drawn = atomicAdd(work, 1u);
                have_draw = false;
                p.w = drawn < static_cast<unsigned int>(total) ? static_cast<int>(drawn) : -1;
                tile_slot[tiles_out & 1] = p.w;
                mbar_arrive(t_full0 + 8 * (tiles_out & 1));
                ++tiles_out;
                if (p.w < 0) return;
                const AttnTile t = attn_tile(p.w, nq, a.H, a.H * a.B);
                p.h = t.h; p.row_base = t.b * a.S; p.q0 = t.qb * AQ; p.nkb = 2 * (t.qb + 1); p.kb = 0;
                p.rng = nullptr;
                if (DOC && a.ranges != nullptr) {
                    p.rng = a.ranges + static_cast<size_t>(t.b) * (a.S / 64);
                    const int2 ta = p.rng[2 * t.qb], tb = p.rng[2 * t.qb + 1];
                    p.tmin = min(ta.x, tb.x); p.tmax = max(ta.y, tb.y);
                }
                while (!active(p, p.kb)) ++p.kb;                // the diagonal blocks are always active
            };
            auto load_q = [&](const Pos& p) {
                if (ALIBI) {
                    // this head's slope / scale as three bf16 terms, in every query row of the slope tile
                    const float sv = exp2f(-8.0f * static_cast<float>(p.h) / static_cast<float>(a.H)) / a.scale;
                    const bf16 s0 = __float2bfloat16_rn(sv);
                    const float r1 = sv - __bfloat162float(s0);
                    const bf16 s1 = __float2bfloat16_rn(r1);
                    const bf16 s2 = __float2bfloat16_rn(r1 - __bfloat162float(s1));
                    const uint32_t w0 = static_cast<uint32_t>(__bfloat16_as_ushort(s0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(s1)) << 16);
                    const uint32_t w1 = static_cast<uint32_t>(__bfloat16_as_ushort(s2));
#pragma unroll 4
                    for (int r = 0; r < 128; ++r)
                        *reinterpret_cast<uint4*>(sU + (r >> 3) * 256 + (r & 7) * 16) = make_uint4(w0, w1, 0u, 0u);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                mbar_expect_tx(q_full, A_TILE);
                tma_load_2d(q_addr, &tmQ, q_full, p.h * DK, p.row_base + p.q0);
            };
            auto load_k = [&](const Pos& p) {
                mbar_expect_tx(k_full, LY::K_TILE);
                tma_load_2d(k_addr, &tmKV, k_full, d + p.h * DK, p.row_base + p.kb * KB);
            };
            auto load_v = [&](const Pos& p) {
                mbar_expect_tx(v_full, LY::K_TILE);
                tma_load_2d(v_addr, &tmKV, v_full, 2 * d + p.h * DK, p.row_base + p.kb * KB);
            };

            Pos cur;
            open_tile(cur);
            if (ok && cur.w >= 0) {
                load_q(cur); load_k(cur); load_v(cur);
                ok = wait1(q_full, 0, 2) && wait1(k_full, 0, 5);
                if (ok) { tc_fence_after(); issue_s(); }
            }
            bool first = true;                                  // cur is the first block of its tile
            while (ok && cur.w >= 0) {
                // the block after cur in the stream: the next active block of the tile, or the first of the next tile
                Pos nxt = cur;
                bool new_tile = false;
                if (!have_draw && cur.kb >= cur.nkb - 3) { drawn = atomicAdd(work, 1u); have_draw = true; }
                ++nxt.kb;
                while (nxt.kb < nxt.nkb && !active(nxt, nxt.kb)) ++nxt.kb;
                if (nxt.kb >= nxt.nkb) { open_tile(nxt); new_tile = true; }
                const bool more = nxt.w >= 0;
                if (more) {
                    // the score MMA of cur is complete: K (and, at a tile's end, Q and the slope tile) may be overwritten
                    if (!(ok = wait1(s_full, kv & 1, 1))) break;
                    if (new_tile) load_q(nxt);
                    load_k(nxt);
                    // the softmax warps have read the scores of cur: the next score MMA may overwrite them
                    if (!(ok = wait1(s_free, kv & 1, 6))) break;
                    if (new_tile && !(ok = wait1(q_full, (tn + 1) & 1, 2))) break;
                    if (!(ok = wait1(k_full, (kv + 1) & 1, 5))) break;
                    tc_fence_after();
                    issue_s();
                }
                if (!(ok = wait1(p_full, kv & 1, 3))) break;    // P of cur is written
                if (first && tn >= 1 && !(ok = wait1(o_empty, (tn - 1) & 1, 4))) break;   // the output rows of the tile before are read out
                if (!(ok = wait1(v_full, kv & 1, 13))) break;
                tc_fence_after();
                issue_pv(first);
                ++kv;
                if (!more) break;
                if (!(ok = wait1(pv_done, (kv - 1) & 1, 12))) break;     // the value tile is free
                load_v(nxt);
                first = new_tile;
                if (new_tile) ++tn;
                cur = nxt;
            }
            // every CTA ends with one failed draw; the CTA that leaves last puts the counter pair back to zero
            if (atomicAdd(work + 1, 1u) == gridDim.x - 1u) { work[0] = 0u; work[1] = 0u; }
        }
    } else {
        const int q = warp & 3;                                // TMEM lane quadrant
        const int row = q * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
        const float scale2 = a.scale * kLog2eF;
        const uint64_t scale2x2 = pack2(scale2, scale2);
        const int sw = row & 7;
        uint8_t* prow = sP + row * 128;
        bool ok = !*abort_flag;
        int kv0 = 0, tn = 0;
        // a wait by the whole warp; the warp goes on only if every lane saw the barrier
        auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {
            const bool got = mbar_wait(bar, parity, abort_flag, code, &g_attn_error);
            return __all_sync(0xffffffffu, got);
        };

        for (; ok; ++tn) {
            if (!wait_all(t_full0 + 8 * (tn & 1), (tn >> 1) & 1, 14)) break;
            const int w = tile_slot[tn & 1];
            if (w < 0) break;
            const AttnTile t = attn_tile(w, nq, a.H, a.H * a.B);
            const int h = t.h, b = t.b, q0 = t.qb * AQ, nkb = 2 * (t.qb + 1), row_base = b * a.S;
            const BlockMask bm = tile_mask(t, nkb);
            const int i = q0 + row;                            // query position inside the sequence
            const float slope2 = ALIBI ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(a.H)) * kLog2eF : 0.f;
            const int my_doc = DOC ? a.doc[row_base + i] : 0;
            // Base-2 domain.  m_run: maximum of the row so far; m_ref: the value the exponentials are taken against
            // (m_ref <= m_run <= m_ref + LAZY); l_run: sum of 2^(score - m_ref).  With ALiBi the -slope2 * i term of the bias
            // is left out here (the same for every key of the row) and goes back into the log-sum-exp at the end.
            float m_run = -INFINITY, m_ref = -INFINITY, l_run = 0.f;

            // One 64-key block, the cnt-th active one of the tile.  The tensor core left raw = q.k (+ slope / scale *
            // position inside the block) in TMEM, so the base-2 score of column cj is raw * scale2 + okb with okb = slope2 *
            // (first key of the block).  A 32-column chunk is handled without any mask when no row of the warp needs one
            // (no document ids, and the chunk lies before the diagonal for all 32 rows).  This lambda has one call site on
            // purpose: inlined twice, the register allocator spilled inside the chunk loops.
            auto block = [&](int kb, int cnt) -> bool {
                const int gj = kv0 + cnt;
                if (!wait_all(s_full, gj & 1, 8)) return false;
                tc_fence_after();
                const int k0 = kb * KB;
                const float okb = ALIBI ? slope2 * static_cast<float>(k0) : 0.f;
                // bit cj of vis: this row may attend to key cj of the block (columns 0..lim are at or before the query)
                const int lim = row - (k0 - q0);
                const int lim0 = q * 32 - (k0 - q0);            // the smallest lim of the warp
                uint32_t vis_lo = lim >= 31 ? 0xffffffffu : (lim < 0 ? 0u : (2u << lim) - 1u);
                uint32_t vis_hi = lim >= 63 ? 0xffffffffu : (lim < 32 ? 0u : (2u << (lim - 32)) - 1u);
                if (DOC) {
                    const int4* dk4 = reinterpret_cast<const int4*>(a.doc + row_base + k0);
                    uint32_t same_lo = 0u, same_hi = 0u;
#pragma unroll 2
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const int4 da = dk4[c4], db = dk4[c4 + 8];
                        same_lo |= (static_cast<uint32_t>(da.x == my_doc) | (static_cast<uint32_t>(da.y == my_doc) << 1) |
                                    (static_cast<uint32_t>(da.z == my_doc) << 2) | (static_cast<uint32_t>(da.w == my_doc) << 3)) << (4 * c4);
                        same_hi |= (static_cast<uint32_t>(db.x == my_doc) | (static_cast<uint32_t>(db.y == my_doc) << 1) |
                                    (static_cast<uint32_t>(db.z == my_doc) << 2) | (static_cast<uint32_t>(db.w == my_doc) << 3)) << (4 * c4);
                    }
                    vis_lo &= same_lo;
                    vis_hi &= same_hi;
                }
                float mxr = -INFINITY;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    // nothing of the chunk is visible to any row of the warp: past the diagonal, or other documents only
                    if (lim0 + 31 < 32 * c || (DOC && __all_sync(0xffffffffu, (c == 0 ? vis_lo : vis_hi) == 0u))) continue;
                    uint32_t r[32];
                    tmem_ld32(tmem_base + lane_addr + c * 32, r);
                    tmem_ld_wait();
                    if (!DOC && lim0 >= 32 * c + 31) {          // uniform over the warp
#pragma unroll
                        for (int jj = 0; jj < 32; ++jj) mxr = fmaxf(mxr, __uint_as_float(r[jj]));
                    } else {
                        const uint32_t vis = c == 0 ? vis_lo : vis_hi;
#pragma unroll
                        for (int jj = 0; jj < 32; ++jj) mxr = fmaxf(mxr, ((vis >> jj) & 1u) ? __uint_as_float(r[jj]) : -INFINITY);
                    }
                }
                m_run = fmaxf(m_run, fmaf(mxr, scale2, okb));   // -inf stays -inf
                // P of the block before has been multiplied (its buffer is free) and the output columns are at rest
                if (cnt >= 1 && !wait_all(pv_done, (gj - 1) & 1, 10)) return false;
                const bool move = m_run > m_ref + LY::LAZY;     // also the first finite maximum of the row (m_ref = -inf)
                if (__any_sync(0xffffffffu, move)) {
                    const float corr = move ? ex2_approx(m_ref - m_run) : 1.0f;      // 0 when m_ref = -inf
                    if (move) m_ref = m_run;
                    l_run *= corr;
                    if (cnt >= 1) {
                        tc_fence_after();
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            uint32_t r[32];
                            tmem_ld32(tmem_O + lane_addr + c * 32, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj) r[jj] = __float_as_uint(__uint_as_float(r[jj]) * corr);
                            tmem_st32(tmem_O + lane_addr + c * 32, r);
                        }
                        tmem_st_wait();
                    }
                }
                const float ms = (m_ref == -INFINITY) ? 0.f : m_ref;
                const uint64_t shift2 = pack2(okb - ms, okb - ms);
                uint64_t rs2 = 0ull;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    // nothing of the chunk is visible to any row of the warp (uniform): P = 0
                    const bool none = lim0 + 31 < 32 * c || (DOC && __all_sync(0xffffffffu, (c == 0 ? vis_lo : vis_hi) == 0u));
                    uint32_t r[32];
                    if (!none) {
                        tmem_ld32(tmem_base + lane_addr + c * 32, r);
                        tmem_ld_wait();
                    }
                    if (c == 1) {                               // the scores are in registers: the columns go back to the tensor core
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(s_free);
                    }
                    if (none) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) *reinterpret_cast<uint4*>(prow + (((c * 4 + g) ^ sw) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                        continue;
                    }
                    const bool plain = !DOC && lim0 >= 32 * c + 31;   // uniform over the warp
                    const uint32_t vis = plain ? 0xffffffffu : (c == 0 ? vis_lo : vis_hi);
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int jj = g * 8 + e * 2;
                            float x0, x1;
                            unpack2(fma2(pack2(__uint_as_float(r[jj]), __uint_as_float(r[jj + 1])), scale2x2, shift2), x0, x1);
                            float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
                            if (!plain) {
                                if (!((vis >> jj) & 1u)) p0 = 0.f;
                                if (!((vis >> (jj + 1)) & 1u)) p1 = 0.f;
                            }
                            rs2 = add2(rs2, pack2(p0, p1));
                            __nv_bfloat162 tt = __floats2bfloat162_rn(p0, p1);
                            pk[e] = *reinterpret_cast<uint32_t*>(&tt);
                        }
                        *reinterpret_cast<uint4*>(prow + (((c * 4 + g) ^ sw) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
                float rs_lo, rs_hi;
                unpack2(rs2, rs_lo, rs_hi);
                l_run += rs_lo + rs_hi;
                tc_fence_before();                              // the score columns are read, the output columns written
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
                return true;
            };
            int cnt = 0;
            for (int kb = 0; ok && kb < nkb; ++kb) {
                if (!block_active(bm, kb)) continue;
                ok = block(kb, cnt);
                ++cnt;
            }
            if (!ok) break;
            if (!wait_all(pv_done, (kv0 + cnt - 1) & 1, 7)) break;
            tc_fence_after();
            {
                const float inv = 1.0f / l_run;
                bf16* op = a.out + (static_cast<size_t>(row_base) + i) * d + h * DK;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_O + lane_addr + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 tt = __floats2bfloat162_rn(__uint_as_float(r[g * 8 + 2 * e]) * inv, __uint_as_float(r[g * 8 + 2 * e + 1]) * inv);
                            pk[e] = *reinterpret_cast<uint32_t*>(&tt);
                        }
                        *reinterpret_cast<uint4*>(op + c * 32 + g * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
                // log-sum-exp in natural units; the ALiBi term left out of the maximum comes back here
                a.lse[(static_cast<size_t>(b) * a.H + h) * a.S + i] = (m_ref + log2f(l_run) - slope2 * static_cast<float>(i)) * kLn2F;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_empty);                // the next tile's first P V may overwrite the output columns
            kv0 += cnt;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(LY::TMEM_COLS) : "memory");
    }
}

template <bool DOC, bool ALIBI>
static int launch_fwd_tc64(const CUtensorMap& tq, const CUtensorMap& tkv, const AttnTcArgs& a, long long tiles, cudaStream_t s)
{
    static PerDeviceOnce once;
    NNB_TRY(once.run([] { return cudaFuncSetAttribute(attn_fwd_tc64_kernel<DOC, ALIBI>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd64::SMEM); }));
    const long long slots = static_cast<long long>(device_sm_count()) * Fwd64::CTAS_PER_SM;
    const dim3 grid(static_cast<unsigned>(tiles < slots ? tiles : slots));     // persistent: each CTA draws tiles until none is left
    unsigned int* work = nullptr;
    NNB_TRY(work_counter_pair(s, &work));
    attn_fwd_tc64_kernel<DOC, ALIBI><<<grid, Fwd64::THREADS, Fwd64::SMEM, s>>>(tq, tkv, a, work);
    NNB_LAUNCH_CHECK();
    return 0;
}

}  // namespace nnb
