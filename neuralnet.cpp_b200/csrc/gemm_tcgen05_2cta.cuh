// CTA-pair variant of the bf16 GEMM (included by gemm_tcgen05.cu): a cluster of two CTAs on two SMs works
// on one 256 x 256 output tile with tcgen05.mma.cta_group::2.  Each CTA loads 128 rows of A and 128 rows of
// B per k-block (32 KB instead of the 48 KB a lone CTA needs for its 128 x 256 tile), which is what lifts
// the shared-memory bandwidth ceiling of the one-CTA kernel; each keeps the 128 accumulator rows it will
// store in its own TMEM.
//
//   rank 0 (leader)  warp 0: TMA producer for its halves      warp 1: issues every MMA of the pair
//   rank 1           warp 0: TMA producer for its halves      warp 1: idle after the TMEM allocation
//   both             warps 2..9: epilogue of the CTA's own 128 rows (TMEM -> registers -> swizzled shared
//                    memory -> TMA store / reduce-add) in two independent groups of four warps that take
//                    alternate 128-byte column blocks, so the drain of a tile keeps pace with a main loop
//                    that is as short as 12 k-blocks (K = 768)
//   both             warps 10, 11: in the GLUB form with column sums, each sums the columns of one of the two
//                    gradient tiles of a block; otherwise they go straight to the barrier at the end
// Barriers: full[s] lives in the leader and counts the bytes of all four loads of a stage (the peer's loads
// name it through its shared::cluster address); empty[s] and tfull[a] exist in both CTAs and are signalled
// together by a multicast tcgen05.commit; tempty[a] lives in the leader and takes one arrival from each of
// the sixteen epilogue warps of the pair.  All TMA loads are plain (no cluster multicast).  Every wait is
// bounded as in the one-CTA kernel; a CTA that gives up still joins the cluster barrier at the end, so its
// shared memory and TMEM outlive anything the peer may still send to them.
//
// RES: a bf16 residual (same shape and leading dimension as the output) is added in the epilogue.  Read straight from
// global memory by the thread that owns the row it is a round trip to L2 or HBM per column block inside the drain (the
// out-projection of the benchmark model took 40 us against 24 us for the same product without residual), and fetched
// ahead into registers it cost the kernel its register budget.  In this form each epilogue group has a second staging
// tile into which its elected thread TMA-loads the residual tile of the group's next column block (of this unit or
// the next) as soon as the group has consumed the previous one, a whole block period ahead; the threads read it with
// the swizzle they write the output with.  The 32 KB come out of the operand ring (five stages instead of six).
//
// DOT: the tile in the residual slot is not added but multiplied in: every thread sums, over the 64 columns of a
// block, the product of the bf16 value it stores and the element of the other matrix at the same place, and writes the
// sum to dot_out[(m / dot_S * dot_H + block) * dot_S + m % dot_S].  With the output gradient of the attention
// out-projection as the product and the attention output as the other matrix this is the row term
// D = rowsum(dO * O) of the attention backward pass (64 columns = one head), which then needs no pass of its own.
//
// GLUB: the product is the gradient of a SwiGLU block's activation (the input gradient of its second projection) and
// is not stored: all eight epilogue warps work on one 64-column block at a time; the elected thread TMA-loads the gate
// and up tiles of the first projection's output (the map in the residual slot, up columns glu_ff further right) into
// one of two sets of two tiles, a block ahead; the warps turn them in place into the gradients of gate and up
// (compute_layer.hpp:436-445; each thread rewrites the chunks of its own row) from the product as rounded to bf16,
// and both are stored through the output map, bit for bit what the activation's backward kernel gives on the stored
// product.  With colsum_part, warps 10 and 11 then read the two tiles back and leave their column sums over the CTA's
// 128 rows (the bias gradient of the first projection, one partial row per 128 matrix rows); the set is loaded into
// again only when they are done with it.
//
// DB: each epilogue group has two staging tiles and uses them in turn, so a block's conversion does not wait for the
// previous block's store to have read its tile; the 32 KB come out of the operand ring as in the RES form.
//
// GLU: the product is the first projection of a SwiGLU feed-forward block (compute_layer.hpp:395-445): B holds the
// gate rows [0, ff) and then the up rows [ff, 2 ff).  The leader stages 128 gate rows and its peer the 128 up rows of
// the same columns, so every CTA's accumulator has gate in columns [0, 128) and up in [128, 256) of one 128-column
// slice, and an epilogue group owns a matching pair of 64-column blocks.  It stores both (the backward pass reads
// them) and, through the map in the residual slot, gate * sigmoid(gate) * up computed from the values as rounded to
// bf16, which is bit for bit what a separate pass over the stored projection gives.  Each group has two staging tiles.
#pragma once

namespace nnb {

constexpr int PAIR_BN_HALF = 128;                                // rows of B each CTA stages per k-block
constexpr int PAIR_STAGE_BYTES = A_STAGE_BYTES + PAIR_BN_HALF * BK * 2;

template <bool A_MN, bool B_MN, int STAGES, bool RES, bool GLU = false, bool DB = false, bool DOT = false, bool GLUB = false>
__global__ void __launch_bounds__(384, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmR, const GemmParams p)
{
    constexpr int BN = 256;                                      // accumulator columns per CTA
    constexpr int B_STAGE_BYTES = PAIR_BN_HALF * BK * 2;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    // instruction descriptor of the pair MMA: fp32 accumulate, bf16 x bf16, operand majors, N = 256, M = 256
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(A_MN) << 15) | (uint32_t(B_MN) << 16) |
                               (uint32_t(256 >> 3) << 17) | (uint32_t(256 >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    // the same offsets in both CTAs: the dynamic shared window starts at the same address in every CTA of a kernel
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint8_t* sC = sB + STAGES * B_STAGE_BYTES;
    uint8_t* sR = sC + 2 * C_STAGE_BYTES;                                 // RES: one residual tile per epilogue group
    constexpr bool RT = RES || DOT;                                       // a second tile comes in through the residual slot
    float* sBias = reinterpret_cast<float*>(sR + ((RT || GLU || DB || GLUB) ? 2 * C_STAGE_BYTES : 0));
    uint64_t* bars = reinterpret_cast<uint64_t*>(sBias + BN);             // each epilogue group keeps the bias of its own 128 columns
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
    const uint32_t tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16, drain_bar = tempty0 + 16, res_full0 = drain_bar + 8;
    const uint32_t tile_ready0 = res_full0 + 16, sums_done0 = tile_ready0 + 16;   // GLUB with column sums: hand-offs with warp 10
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 11);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                     // 0 = leader
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 16); }
        mbar_init(drain_bar, 1);
        mbar_init(res_full0, 1); mbar_init(res_full0 + 8, 1);
        for (int k = 0; k < 2; ++k) { mbar_init(tile_ready0 + 8 * k, 1); mbar_init(sums_done0 + 8 * k, 2); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                          // the peer's barriers exist before anything is sent to them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles = p.tiles_m * p.tiles_n;
    const int units = tiles * p.splits;

    // GLUB: the 64-column blocks of this CTA in the order its epilogue takes them; false at the end of the list
    struct BlockCursor { int u, cb; };
    auto glub_next = [&](BlockCursor& c, int& n0, int& m0) -> bool {
        for (;;) {
            if (++c.cb * 64 >= BN) { c.u += pairs; c.cb = 0; }
            if (c.u >= units) return false;
            const int t = c.u % tiles;
            const int tile_n = t / p.tiles_m, tile_m = t - tile_n * p.tiles_m;
            n0 = tile_n * BN + c.cb * 64; m0 = tile_m * 256 + static_cast<int>(rank) * 128;
            if (n0 < p.N && m0 < p.M) return true;
        }
    };

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t leader_full0 = mapa_shared(full0, 0);
            int it = 0;
            for (int u = pair; u < units && !*abort_flag; u += pairs) {
                const int split = u / tiles, t = u - split * tiles;
                const int tile_n = t / p.tiles_m, tile_m = t - tile_n * p.tiles_m;
                const int kb0 = split * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                const int row_a = tile_m * 256 + static_cast<int>(rank) * 128;      // this CTA's rows of A (and of D)
                const int row_b = GLU ? static_cast<int>(rank) * p.glu_ff + tile_n * 128  // gate rows in the leader, up rows in the peer
                                       : tile_n * 256 + static_cast<int>(rank) * 128;     // this CTA's rows of B (columns of D)
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, 1, &g_gemm_error)) break;
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * PAIR_STAGE_BYTES);
                    const uint32_t fb = leader_full0 + 8 * s;
                    const uint32_t a_dst = smem_u32(sA + s * A_STAGE_BYTES), b_dst = smem_u32(sB + s * B_STAGE_BYTES);
                    if (!A_MN) tma_load_2d_pair(a_dst, &tmA, fb, kb * BK, row_a);
                    else
                        for (int j = 0; j < 2; ++j) tma_load_2d_pair(a_dst + j * (BK * 128), &tmA, fb, row_a + j * 64, kb * BK);
                    if (!B_MN) tma_load_2d_pair(b_dst, &tmB, fb, kb * BK, row_b);
                    else
                        for (int j = 0; j < 2; ++j) tma_load_2d_pair(b_dst + j * (BK * 128), &tmB, fb, row_b + j * 64, kb * BK);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            int it = 0, tc = 0;
            for (int u = pair; u < units && !*abort_flag; u += pairs, ++tc) {
                const int split = u / tiles;
                const int kb0 = split * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                const int acc = tc & 1;
                const uint32_t acc_ph = (tc >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * acc, acc_ph ^ 1, abort_flag, 2, &g_gemm_error)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                bool ok = true;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag, 3, &g_gemm_error)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES), b_addr = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t da = A_MN ? smem_desc(a_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                                 : smem_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
                        const uint64_t db = B_MN ? smem_desc(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                                 : smem_desc(b_addr + k * (UMMA_K * 2), 16, 1024);
                        umma_bf16_pair(d_tmem, da, db, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(empty0 + 8 * s, 3);         // frees the stage in both CTAs
                }
                if (!ok) break;
                umma_commit_pair(tfull0 + 8 * acc, 3);           // accumulators complete in both CTAs
            }
            // nothing issued above may still be reading the peer's shared memory or writing its TMEM when
            // the pair leaves: wait (bounded) for the tensor cores to drain
            umma_commit_pair(drain_bar, 1);
            mbar_wait(drain_bar, 0, abort_flag, 5, &g_gemm_error);
        }
    } else if (warp < 10) {
        // Two epilogue groups of four warps; group g takes the column blocks cb with (cb & 1) == g, has its own
        // staging tile, bias copy, named barrier and bulk-store queue, and never synchronises with the other.
        const int q = warp & 3;                                  // TMEM lane quadrant this warp may read
        const int grp = (warp - 2) >> 2;
        const int bar_id = 1 + grp;
        const int grp_tid = threadIdx.x - 64 - grp * 128;        // 0..127 inside the group
        const bool elected = grp_tid == 0;
        const int r_local = q * 32 + lane;
        const uint32_t leader_tempty0 = mapa_shared(tempty0, 0);
        const int CB = p.c_bf16 ? 64 : 32;                       // columns per 128-byte staging row
        uint8_t* stage = sC + grp * C_STAGE_BYTES;
        uint8_t* srow = stage + r_local * 128;
        float* bias_s = sBias + grp * (BN / 2);
        uint8_t* rstage = sR + grp * C_STAGE_BYTES;
        const uint8_t* rrow = rstage + r_local * 128;
        const uint32_t res_full = res_full0 + 8 * grp;
        int res_uses = 0;                                            // residual tiles of this group consumed so far (barrier phase)
        // The elected thread requests the residual tiles in the order the group drains column blocks, always one ahead:
        // (ru, rcb) is the block requested last.  A block the drain loop skips (beyond N or M) is skipped here too.
        int ru = pair, rcb = grp - 2;
        auto request_next_residual = [&]() {
            for (;;) {
                rcb += 2;
                if (rcb * 64 >= BN) { ru += pairs; rcb = grp; }
                if (ru >= units) return;
                const int t = ru % tiles;
                const int tile_n = t / p.tiles_m, tile_m = t - tile_n * p.tiles_m;
                const int n0 = tile_n * BN + rcb * 64, m0 = tile_m * 256 + static_cast<int>(rank) * 128;
                if (n0 >= p.N || m0 >= p.M) continue;
                mbar_expect_tx(res_full, C_STAGE_BYTES);
                tma_load_2d(smem_u32(rstage), &tmR, res_full, n0, m0);
                return;
            }
        };
        if (RT && elected) request_next_residual();
        // GLUB: blocks in the order all eight warps take them; the elected thread keeps the loads one block ahead
        const bool glub_elected = GLUB && threadIdx.x == 64;
        int glub_blocks = 0, glub_requested = 0;
        BlockCursor g_req{pair, -1};
        // loads of the next block into the set it will be turned in (an L2 prefetch of the tiles two blocks further on
        // was measured slower: 93.8 against 86.5 us at 16384 x 2048 x 768)
        auto glub_request = [&]() {
            int n0, m0;
            if (!glub_next(g_req, n0, m0)) return;
            const int set = glub_requested & 1;
            ++glub_requested;
            mbar_expect_tx(res_full0 + 8 * set, 2 * C_STAGE_BYTES);
            tma_load_2d(smem_u32(sC + set * C_STAGE_BYTES), &tmR, res_full0 + 8 * set, n0, m0);
            tma_load_2d(smem_u32(sR + set * C_STAGE_BYTES), &tmR, res_full0 + 8 * set, p.glu_ff + n0, m0);
        };
        if (glub_elected) glub_request();
        int tc = 0, blk = 0;
        for (int u = pair; u < units; u += pairs, ++tc) {
            const int split = u / tiles, t = u - split * tiles;
            const int tile_n = t / p.tiles_m, tile_m = t - tile_n * p.tiles_m;
            const int acc = tc & 1;
            const uint32_t acc_ph = (tc >> 1) & 1;
            const bool add_extra = (split == 0);
            const bool use_bias = p.bias_n && add_extra;
            float bias_reg = 0.f;                                // fetched while the accumulators are still being computed
            if (GLU) {                                           // slots [0, 64): gate columns of the group, [64, 128): up columns
                if (use_bias) bias_reg = p.bias_n[(grp_tid >> 6) * p.glu_ff + tile_n * 128 + grp * 64 + (grp_tid & 63)];
            } else if (use_bias) {                               // slot j of the group: column block 2*(j/CB)+grp, column j%CB of it
                const int col = tile_n * BN + (2 * (grp_tid / CB) + grp) * CB + grp_tid % CB;
                if (col < p.N) bias_reg = p.bias_n[col];
            }
            const bool arrived = mbar_wait(tfull0 + 8 * acc, acc_ph, abort_flag, 4, &g_gemm_error);
            if (group_any(bar_id, !arrived || *abort_flag)) break;
            tc_fence_after();
            if (use_bias) bias_s[grp_tid] = bias_reg;            // the previous tile's readers are past their last group_bar
            const int m0 = tile_m * 256 + static_cast<int>(rank) * 128;
            const int m = m0 + r_local;
            const bool row_ok = m < p.M;
            const int dot_b = DOT ? m / p.dot_S : 0;
            const long long row_off = static_cast<long long>(m) * p.ldc;
            if (GLU) {
                if (m0 < p.M) {
                    const uint32_t tg = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + grp * 64;   // gate; up is 128 columns on
                    const int n0 = tile_n * 128 + grp * 64;
                    uint8_t* xrow = srow;                            // staging tile X: gate, then up
                    uint8_t* yrow = rstage + r_local * 128;          // staging tile Y: the activation
                    uint32_t ra[32], rb[32];
                    uint32_t upk[32];                                // the up block as packed bf16 pairs, stored in pass 2
                    // 32 accumulator columns + bias, rounded to bf16: packed pairs (what is stored) and the rounded values
                    auto round_bias = [&](const uint32_t (&r)[32], const float* b, uint32_t* pk, float (&v)[32]) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                        if (use_bias) {
                            const float4* b4 = reinterpret_cast<const float4*>(b);
#pragma unroll
                            for (int j = 0; j < 8; ++j) { const float4 t4 = b4[j]; v[4 * j] += t4.x; v[4 * j + 1] += t4.y; v[4 * j + 2] += t4.z; v[4 * j + 3] += t4.w; }
                        }
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const uint32_t w = pack_bf16x2(v[j], v[j + 1]);
                            pk[j >> 1] = w;
                            v[j] = __uint_as_float(w << 16);
                            v[j + 1] = __uint_as_float(w & 0xffff0000u);
                        }
                    };
                    auto put = [&](uint8_t* row, const uint32_t* pk, int half) {     // 16 packed pairs = 32 columns
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            *reinterpret_cast<uint4*>(row + (((half * 4 + j) ^ (r_local & 7)) << 4)) =
                                make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
                    };
                    // pass 1: gate into X, the activation into Y.  Both tiles were handed to the store queue a pass or more ago.
                    tmem_ld32(tg, ra);
                    tmem_ld32(tg + 128, rb);
                    tmem_ld_wait();
                    if (elected) tma_wait_read0();
                    group_bar(bar_id);                               // also orders the bias slots written above
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (half == 1) {
                            tmem_ld32(tg + 32, ra);
                            tmem_ld32(tg + 128 + 32, rb);
                            tmem_ld_wait();
                        }
                        float g[32], u[32];
                        uint32_t pk[16];
                        round_bias(ra, bias_s + half * 32, pk, g);
                        put(xrow, pk, half);
                        round_bias(rb, bias_s + 64 + half * 32, upk + half * 16, u);
#pragma unroll
                        for (int j = 0; j < 32; j += 2)
                            pk[j >> 1] = pack_bf16x2(g[j] * sigmoid_fast(g[j]) * u[j], g[j + 1] * sigmoid_fast(g[j + 1]) * u[j + 1]);
                        put(yrow, pk, half);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    group_bar(bar_id);
                    if (elected) {
                        tma_store_2d(&tmC, smem_u32(stage), n0, m0);
                        tma_commit();
                        tma_store_2d(&tmR, smem_u32(rstage), n0, m0);
                        tma_commit();
                        tma_wait_read1();                            // pass 2: up into X once the gate store has read it
                    }
                    group_bar(bar_id);
                    put(xrow, upk, 0);
                    put(xrow, upk + 16, 1);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    group_bar(bar_id);
                    if (elected) {
                        tma_store_2d(&tmC, smem_u32(stage), p.glu_ff + n0, m0);
                        tma_commit();
                    }
                }
            } else if (GLUB) {
                // All eight warps work on one 64-column block at a time, the two warps of a TMEM lane quadrant on 32
                // columns each, so that two sets of (gate, up) tiles can be used in turn: while a block is turned in
                // place in one set, the loads of the next block arrive in the other.
                if (m0 < p.M) {
                    const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + grp * 32;
                    uint32_t ra[32];
#pragma unroll 1
                    for (int cb = 0; cb * 64 < BN; ++cb) {
                        const int n0 = tile_n * BN + cb * 64;
                        if (n0 >= p.N) break;
                        const int set = glub_blocks & 1;
                        uint8_t* gtile = sC + set * C_STAGE_BYTES;
                        uint8_t* utile = sR + set * C_STAGE_BYTES;
                        if (glub_elected) {
                            tma_wait_read0();                        // the other set's stores (the block before this one) have read it
                            // ... and so has the warp that sums its columns
                            if (p.colsum_part && glub_blocks >= 1)
                                mbar_wait(sums_done0 + 8 * (set ^ 1), ((glub_blocks - 1) >> 1) & 1, abort_flag, 13, &g_gemm_error);
                            glub_request();
                        }
                        tmem_ld32(tbase + cb * 64, ra);
                        tmem_ld_wait();
                        const bool got = mbar_wait(res_full0 + 8 * set, (glub_blocks >> 1) & 1, abort_flag, 11, &g_gemm_error);
                        ++glub_blocks;
                        // a wait that gave up has raised the abort flag: this thread goes on (on stale tiles, inside its own
                        // rows) so that nobody is left alone at the barrier below, and all leave together at the next tile
                        (void)got;
                        uint8_t* grow = gtile + r_local * 128;
                        uint8_t* urow = utile + r_local * 128;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            const int chunk = ((grp * 4 + (j >> 3)) ^ (r_local & 7)) << 4;
                            const Vec16<bf16> gv = *reinterpret_cast<const Vec16<bf16>*>(grow + chunk);
                            const Vec16<bf16> uv = *reinterpret_cast<const Vec16<bf16>*>(urow + chunk);
                            Vec16<bf16> og, ou;
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                const float go = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ra[j + k])));
                                const float gt = __bfloat162float(gv.v[k]), up = __bfloat162float(uv.v[k]);
                                const float sg = sigmoid_fast(gt);
                                og.v[k] = __float2bfloat16_rn(go * up * (sg * (1.0f + gt * (1.0f - sg))));
                                ou.v[k] = __float2bfloat16_rn(go * gt * sg);
                            }
                            *reinterpret_cast<uint4*>(grow + chunk) = *reinterpret_cast<const uint4*>(&og);
                            *reinterpret_cast<uint4*>(urow + chunk) = *reinterpret_cast<const uint4*>(&ou);
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        all_epilogue_bar();
                        if (glub_elected) {
                            tma_store_2d(&tmC, smem_u32(gtile), n0, m0);
                            tma_store_2d(&tmC, smem_u32(utile), p.glu_ff + n0, m0);
                            tma_commit();
                            if (p.colsum_part) mbar_arrive(tile_ready0 + 8 * set);   // warp 10 may sum the set's columns
                        }
                    }
                }
            } else if (m0 < p.M) {
            // In the bf16 case (two 32-column halves per block) the second half is fetched from TMEM while the first
            // is converted.  Nothing is fetched across loop iterations: a register written by tcgen05.ld must not be
            // touched, not even moved by the compiler at a loop edge, before the wait that follows it.
            uint32_t ra[32], rb[32];
            const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
            const bool piped = CB == 64;
#pragma unroll 1
            for (int cb = grp; cb * CB < BN; cb += 2) {
                const int n0 = tile_n * BN + cb * CB;
                if (n0 >= p.N) break;
                if (DB) {                                        // two staging tiles per group, used in turn
                    stage = ((blk & 1) ? sR : sC) + grp * C_STAGE_BYTES;
                    srow = stage + r_local * 128;
                    ++blk;
                    if (elected) tma_wait_read1();               // the store before the group's previous one has read this tile
                } else if (elected) tma_wait_read0();            // the group's previous store has read the staging tile
                group_bar(bar_id);
                if (piped) {
                    tmem_ld32(tbase + cb * CB, ra);
                    tmem_ld_wait();
                    tmem_ld32(tbase + cb * CB + 32, rb);         // in flight while the first half is converted
                } else {
                    tmem_ld32(tbase + cb * CB, ra);
                    tmem_ld_wait();
                }
                float dot = 0.f;
                auto emit = [&](const uint32_t (&r)[32], int half) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = p.alpha * __uint_as_float(r[j]);
                    if (use_bias) {
                        const float4* b4 = reinterpret_cast<const float4*>(bias_s + (cb >> 1) * CB + half * 32);
#pragma unroll
                        for (int j = 0; j < 8; ++j) { const float4 b = b4[j]; v[4 * j] += b.x; v[4 * j + 1] += b.y; v[4 * j + 2] += b.z; v[4 * j + 3] += b.w; }
                    }
                    const int nh = n0 + half * 32;
                    if (p.c_bf16) {
                        const bf16* rp = (!RES && p.residual && add_extra && row_ok) ? static_cast<const bf16*>(p.residual) + row_off + nh : nullptr;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            if (RES) {                            // rows and columns beyond the matrix were filled with zeros by the load
                                const Vec16<bf16> rr = *reinterpret_cast<const Vec16<bf16>*>(rrow + (((half * 4 + (j >> 3)) ^ (r_local & 7)) << 4));
#pragma unroll
                                for (int k = 0; k < 8; ++k) v[j + k] += __bfloat162float(rr.v[k]);
                            } else if (rp && nh + j + 8 <= p.N) { const Vec16<bf16> rr = ld16(rp + j);
#pragma unroll
                                for (int k = 0; k < 8; ++k) v[j + k] += __bfloat162float(rr.v[k]); }
                            else if (rp) { for (int k = 0; k < 8; ++k) if (nh + j + k < p.N) v[j + k] += __bfloat162float(rp[j + k]); }
                            Vec16<bf16> o;
#pragma unroll
                            for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(v[j + k]);
                            if (DOT) {                            // zeros beyond the matrix, as above
                                const Vec16<bf16> rr = *reinterpret_cast<const Vec16<bf16>*>(rrow + (((half * 4 + (j >> 3)) ^ (r_local & 7)) << 4));
#pragma unroll
                                for (int k = 0; k < 8; ++k) dot = fmaf(__bfloat162float(o.v[k]), __bfloat162float(rr.v[k]), dot);
                            }
                            const int chunk = half * 4 + (j >> 3);
                            *reinterpret_cast<uint4*>(srow + ((chunk ^ (r_local & 7)) << 4)) = *reinterpret_cast<const uint4*>(&o);
                        }
                    } else {
                        const float* rp = (p.residual && add_extra && row_ok) ? static_cast<const float*>(p.residual) + row_off + nh : nullptr;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                            if (rp && nh + j + 4 <= p.N) { const float4 rr = *reinterpret_cast<const float4*>(rp + j); o.x += rr.x; o.y += rr.y; o.z += rr.z; o.w += rr.w; }
                            else if (rp) { if (nh + j < p.N) o.x += rp[j]; if (nh + j + 1 < p.N) o.y += rp[j + 1]; if (nh + j + 2 < p.N) o.z += rp[j + 2]; }
                            const int chunk = j >> 2;
                            *reinterpret_cast<float4*>(srow + ((chunk ^ (r_local & 7)) << 4)) = o;
                        }
                    }
                };
                if (RT) {                                        // this block's residual tile, requested a block period ago
                    const bool got = mbar_wait(res_full, res_uses & 1, abort_flag, 11, &g_gemm_error);
                    ++res_uses;
                    if (group_any(bar_id, !got)) break;
                }
                emit(ra, 0);
                if (piped) tmem_ld_wait();                       // second half
                if (CB == 64) emit(rb, 1);
                if (DOT && row_ok)
                    p.dot_out[(static_cast<size_t>(dot_b) * p.dot_H + (n0 >> 6)) * p.dot_S + (m - dot_b * p.dot_S)] = dot;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                group_bar(bar_id);
                if (elected) {
                    if (p.accumulate) tma_reduce_add_2d(&tmC, smem_u32(stage), n0, m0);
                    else tma_store_2d(&tmC, smem_u32(stage), n0, m0);
                    tma_commit();
                    if (RT) request_next_residual();             // the group is past its reads of the residual tile
                }
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_tempty0 + 8 * acc);
        }
        if (elected) tma_wait_all();
    } else if (GLUB && p.colsum_part != nullptr) {
        // Warps 10 and 11 of the GLUB form: column sums of the gate-gradient tile (warp 10) and of the up-gradient tile
        // (warp 11) of every block over the CTA's 128 rows (rows beyond the matrix hold zeros), read from the staging
        // tiles while the eight epilogue warps are on the next block: fc1's bias gradient as one partial row per 128
        // matrix rows, in a fixed order.  Lane (c, rs) takes 16-byte chunk c of rows [32 rs, 32 rs + 32).
        BlockCursor cur{pair, -1};
        int n0, m0;
        const int c = lane & 7, rs = lane >> 3, which = warp - 10;
        for (int k = 0; glub_next(cur, n0, m0); ++k) {
            const int set = k & 1;
            if (!mbar_wait(tile_ready0 + 8 * set, (k >> 1) & 1, abort_flag, 14, &g_gemm_error)) break;
            const uint8_t* tile = (which ? sR : sC) + set * C_STAGE_BYTES;
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll 8
            for (int i = 0; i < 32; ++i) {
                const int r = rs * 32 + i;
                const uint4 v4 = *reinterpret_cast<const uint4*>(tile + r * 128 + ((c ^ (r & 7)) << 4));
                const uint32_t w[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[2 * j] += __uint_as_float(w[j] << 16);
                    acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(sums_done0 + 8 * set);        // (with the other warp's arrival) the set may be loaded into again
#pragma unroll
            for (int st = 8; st <= 16; st <<= 1)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], st);
            if (rs == 0) {
                float* dst = p.colsum_part + static_cast<size_t>(m0 >> 7) * (2 * p.glu_ff) + which * p.glu_ff + n0 + c * 8;
                *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                          // nobody leaves while the peer may still address this CTA
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace nnb
