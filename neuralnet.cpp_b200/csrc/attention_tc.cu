// Fused causal / document-masked / ALiBi attention forward on the 5th-generation tensor cores.
//
// Persistent: one CTA per SM walks the list of (128-query tile, head, batch) work items, longest tiles first,
// in snake order (snake_tile in tc_ptx.cuh).  Ten warps:
//   warp 0      TMA producer: the tile's Q (two tile buffers, so the next tile's Q is fetched early), then K/V
//               tiles of 128 keys through a 3-stage ring that runs on across tiles
//   warp 1      MMA issuer:   S = Q K^T   (128x128x64)  into one of two TMEM score buffers
//                             O' = P V    (128x64x128)  into TMEM columns [256,320)
//   warps 2..9  softmax: thread (row, half) owns 64 of the 128 score columns of one query row
//               (two warps share each 32-lane TMEM quadrant; four per quadrant with 32 columns each
//               measured slower: 104 against 98 us at batch 16 x 12 heads x 1024).  It reads its scores
//               once with tcgen05.ld, applies scale, causal / document mask and ALiBi bias, exchanges the
//               row maximum with its partner through shared memory, writes P as bf16 into a K-major
//               128B-swizzled shared tile (the A operand of the second MMA) and folds its 32 columns
//               of O' into registers; at the end of a tile it normalises and stores its output row.
// The score buffer and the P tile are double-buffered, so Q K^T of block k+1 and P V of block k run
// on the tensor core while the softmax warps work on block k / k+1; all buffer positions and barrier
// phases are counted across tiles, so the first MMAs of the next tile overlap the write-out of this one.
// V is consumed as an MN-major B operand straight from its (key, head_dim) tile.  Nothing of size (S, S)
// ever reaches memory.
// Replaces batched_matmul_reduce / _softmax_denom / _softmax_apply and the materialised score path
// of the reference (compute_layer.hpp:1193-1252; cpu_engine.hpp:426-699).
// Every wait is bounded; a wait that gives up raises a status word, the softmax warps learn of it together
// at their next exchange barrier, and the CTA drains.
#include <type_traits>

#include "kernels.h"
#include "tc_ptx.cuh"

namespace nnb {

__device__ int g_attn_error = 0;

constexpr int AQ = 128, AK = 128, ADK = 64;
constexpr int A_TILE = 128 * 128;                  // bytes of a 128-row x 64-bf16 tile
constexpr int A_KV_STAGES = 3;
// Q (2 tiles) | K,V ring | P (2 buffers x two 64-key halves) | row-max exchange | barriers
constexpr int A_OFF_KV = 2 * A_TILE, A_OFF_P = A_OFF_KV + A_KV_STAGES * 2 * A_TILE, A_OFF_X = A_OFF_P + 4 * A_TILE,
              A_OFF_BAR = A_OFF_X + 2 * 2 * 128 * 4, A_SMEM = A_OFF_BAR + 256;
constexpr uint32_t A_TMEM_COLS = 512;
constexpr float kLog2eF = 1.4426950408889634f, kLn2F = 0.6931471805599453f;

struct AttnTcArgs {
    bf16* out; float* lse; const int* doc;
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

template <bool DOC, bool ALIBI>
__global__ void __launch_bounds__(320, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQKV, const AttnTcArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;                            // two query tiles: the next one is fetched while this one is in use
    uint8_t* sKV = smem + A_OFF_KV;                // stage s: K at sKV + s*2*A_TILE, V right after it
    uint8_t* sP = smem + A_OFF_P;                  // buffer b at sP + b*2*A_TILE (two 64-key halves)
    float* sX = reinterpret_cast<float*>(smem + A_OFF_X);   // [buffer][half][row]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A_OFF_BAR);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full0 = bar0, q_empty0 = bar0 + 16, kv_full0 = bar0 + 32, kv_empty0 = bar0 + 56, s_full0 = bar0 + 80,
                   s_empty0 = bar0 + 96, p_full0 = bar0 + 112, p_empty0 = bar0 + 128, o_full = bar0 + 144, o_empty = bar0 + 152;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = a.H * ADK;
    const int nq = a.S / AQ;
    const int total = nq * a.H * a.B;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(q_full0 + 8 * s, 1); mbar_init(q_empty0 + 8 * s, 1); }
        for (int s = 0; s < A_KV_STAGES; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(s_full0 + 8 * s, 1); mbar_init(s_empty0 + 8 * s, 8);
            mbar_init(p_full0 + 8 * s, 8); mbar_init(p_empty0 + 8 * s, 1);
        }
        mbar_init(o_full, 1); mbar_init(o_empty, 8);
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;        // the swizzled tiles need a 1024-byte aligned base
        if (*abort_flag) atomicCAS(&g_attn_error, 0, (9 << 16));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(A_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_O = tmem_base + 256;

    // instruction descriptors: fp32 accumulate, bf16 operands; S: N=128, both K-major; PV: N=64, B MN-major
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(AK >> 3) << 17) | (uint32_t(AQ >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (uint32_t(ADK >> 3) << 17) | (uint32_t(AQ >> 4) << 24);

    // Every role walks the same list of tiles; the ring / buffer positions and barrier phases run on across
    // tiles (kv: key-block counter; gj: the same counter as seen by the score / P / O' buffers; tn: tile counter).
    if (warp == 0) {
        if (lane == 0 && !*abort_flag) {
            int kv = 0, tn = 0;
            bool ok = true;
            for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
                const AttnTile t = attn_tile(w, nq, a.H, a.H * a.B);
                const int nkb = t.qb + 1, row_base = t.b * a.S, qs = tn & 1;
                if (!mbar_wait(q_empty0 + 8 * qs, ((tn >> 1) & 1) ^ 1, abort_flag, 11, &g_attn_error)) break;
                mbar_expect_tx(q_full0 + 8 * qs, A_TILE);
                tma_load_2d(smem_u32(sQ + qs * A_TILE), &tmQKV, q_full0 + 8 * qs, t.h * ADK, row_base + t.qb * AQ);
                for (int kb = 0; kb < nkb; ++kb, ++kv) {
                    const int s = kv % A_KV_STAGES;
                    const uint32_t ph = (kv / A_KV_STAGES) & 1;
                    if (!mbar_wait(kv_empty0 + 8 * s, ph ^ 1, abort_flag, 1, &g_attn_error)) { ok = false; break; }
                    mbar_expect_tx(kv_full0 + 8 * s, 2 * A_TILE);
                    const uint32_t kdst = smem_u32(sKV + s * 2 * A_TILE);
                    tma_load_2d(kdst, &tmQKV, kv_full0 + 8 * s, d + t.h * ADK, row_base + kb * AK);
                    tma_load_2d(kdst + A_TILE, &tmQKV, kv_full0 + 8 * s, 2 * d + t.h * ADK, row_base + kb * AK);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && !*abort_flag) {
            int kv0 = 0, tn = 0;                                // kv0: key-block counter at the start of the tile
            bool ok = true;
            for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
                const AttnTile t = attn_tile(w, nq, a.H, a.H * a.B);
                const int nkb = t.qb + 1, qs = tn & 1;
                ok = mbar_wait(q_full0 + 8 * qs, (tn >> 1) & 1, abort_flag, 2, &g_attn_error);
                const uint32_t q_addr = smem_u32(sQ + qs * A_TILE);
                auto issue_s = [&](int gj) -> bool {
                    const int st = gj % A_KV_STAGES, sb = gj & 1, u = gj >> 1;
                    if (!mbar_wait(kv_full0 + 8 * st, (gj / A_KV_STAGES) & 1, abort_flag, 5, &g_attn_error)) return false;
                    if (u >= 1 && !mbar_wait(s_empty0 + 8 * sb, (u - 1) & 1, abort_flag, 6, &g_attn_error)) return false;
                    tc_fence_after();
                    const uint32_t k_addr = smem_u32(sKV + st * 2 * A_TILE);
#pragma unroll
                    for (int k = 0; k < ADK / 16; ++k)
                        umma_bf16(tmem_base + sb * 128, smem_desc(q_addr + k * 32, 16, 1024), smem_desc(k_addr + k * 32, 16, 1024),
                                  IDESC_S, k > 0 ? 1u : 0u);
                    umma_commit(s_full0 + 8 * sb);
                    return true;
                };
                auto issue_pv = [&](int gj) -> bool {
                    const int st = gj % A_KV_STAGES, pb = gj & 1;
                    if (!mbar_wait(p_full0 + 8 * pb, (gj >> 1) & 1, abort_flag, 3, &g_attn_error)) return false;
                    if (gj >= 1 && !mbar_wait(o_empty, (gj - 1) & 1, abort_flag, 4, &g_attn_error)) return false;
                    tc_fence_after();
                    const uint32_t p_addr = smem_u32(sP + pb * 2 * A_TILE);
                    const uint32_t v_addr = smem_u32(sKV + st * 2 * A_TILE + A_TILE);
#pragma unroll
                    for (int k = 0; k < AK / 16; ++k) {
                        const uint64_t da = smem_desc(p_addr + (k >> 2) * A_TILE + (k & 3) * 32, 16, 1024);
                        const uint64_t db = smem_desc(v_addr + k * 2048, A_TILE, 1024);
                        umma_bf16(tmem_O, da, db, IDESC_PV, k > 0 ? 1u : 0u);
                    }
                    umma_commit(o_full);
                    umma_commit(p_empty0 + 8 * pb);
                    umma_commit(kv_empty0 + 8 * st);
                    return true;
                };
                if (ok) ok = issue_s(kv0);
                for (int kb = 0; ok && kb < nkb; ++kb) {
                    if (kb + 1 < nkb) ok = issue_s(kv0 + kb + 1);
                    if (ok) ok = issue_pv(kv0 + kb);
                }
                if (ok) umma_commit(q_empty0 + 8 * qs);         // the query tile is free once this tile's MMAs are done
                kv0 += nkb;
            }
        }
    } else {
        const int q = warp & 3, hf = (warp - 2) >> 2;          // TMEM lane quadrant, column half
        const int row = q * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
        const float scale2 = a.scale * kLog2eF;
        const int sw = row & 7;
        bool ok = true, bad = *abort_flag != 0;                 // bad: a wait of this thread gave up (reported at the next barrier)
        int kv0 = 0, xc = 0;                                    // key-block counter; exchange counter (alternates the sX buffer)

        for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps) {
            const AttnTile t = attn_tile(w, nq, a.H, a.H * a.B);
            const int h = t.h, b = t.b, q0 = t.qb * AQ, nkb = t.qb + 1, row_base = b * a.S;
            const int i = q0 + row;                            // query position inside the sequence
            const float slope2 = ALIBI ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(a.H)) * kLog2eF : 0.f;
            const int my_doc = DOC ? a.doc[row_base + i] : 0;
            float m_run = -INFINITY, l_run = 0.f;
            float o_acc[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) o_acc[c] = 0.f;

            auto fold_o = [&](int gj) -> bool {                 // o_acc += O'(gj), this thread's 32 columns
                if (!mbar_wait(o_full, gj & 1, abort_flag, 7, &g_attn_error)) return false;
                tc_fence_after();
                uint32_t r[32];
                tmem_ld32(tmem_O + lane_addr + hf * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) o_acc[c] += __uint_as_float(r[c]);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(o_empty);
                return true;
            };

            // One 128-key block.  DIAG: the block on the diagonal (causal mask inside it).  The score of
            // column cj is r*scale2 + (slope2*cj + abase); with the loops unrolled cj is a literal.
            auto block = [&](auto diag_tag, int kb) -> bool {
                constexpr bool DIAG = decltype(diag_tag)::value;
                const int gj = kv0 + kb, sb = gj & 1, u = gj >> 1;
                bad |= !mbar_wait(s_full0 + 8 * sb, u & 1, abort_flag, 8, &g_attn_error);
                tc_fence_after();
                const int k0 = kb * AK;
                const int* dk_ptr = DOC ? a.doc + row_base + k0 + hf * 64 : nullptr;
                const float abase = ALIBI ? -slope2 * static_cast<float>(i - k0 - hf * 64) : 0.f;
                float s[64];
                {
                    uint32_t r0[32], r1[32];
                    tmem_ld32(tmem_base + sb * 128 + lane_addr + hf * 64, r0);
                    tmem_ld32(tmem_base + sb * 128 + lane_addr + hf * 64 + 32, r1);
                    tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) { s[jj] = __uint_as_float(r0[jj]); s[32 + jj] = __uint_as_float(r1[jj]); }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_empty0 + 8 * sb);  // scores are in registers: the buffer may be overwritten
                float mx = -INFINITY;
#pragma unroll
                for (int cj = 0; cj < 64; ++cj) {
                    float sc = ALIBI ? fmaf(s[cj], scale2, fmaf(slope2, static_cast<float>(cj), abase)) : s[cj] * scale2;
                    if (DIAG && hf * 64 + cj > row) sc = -INFINITY;
                    if (DOC && dk_ptr[cj] != my_doc) sc = -INFINITY;
                    s[cj] = sc;
                    mx = fmaxf(mx, sc);
                }
                float* xs = sX + (xc & 1) * 256;
                ++xc;
                xs[hf * 128 + row] = mx;
                if (softmax_any(bad)) return false;             // the same answer in all eight warps
                const float m_new = fmaxf(m_run, fmaxf(mx, xs[(hf ^ 1) * 128 + row]));
                const float ms = (m_new == -INFINITY) ? 0.f : m_new;
                const float corr = ex2_approx(m_run - ms);
                if (kb >= 1) bad |= !fold_o(gj - 1);
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) o_acc[c] *= corr;
                }
                if (u >= 1) bad |= !mbar_wait(p_empty0 + 8 * sb, (u - 1) & 1, abort_flag, 10, &g_attn_error);
                uint8_t* prow = sP + sb * 2 * A_TILE + hf * A_TILE + row * 128;
                float rs = 0.f;
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    uint32_t pk[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float p0 = ex2_approx(s[g * 8 + e * 2] - ms), p1 = ex2_approx(s[g * 8 + e * 2 + 1] - ms);
                        rs += p0 + p1;
                        __nv_bfloat162 tt = __floats2bfloat162_rn(p0, p1);
                        pk[e] = *reinterpret_cast<uint32_t*>(&tt);
                    }
                    *reinterpret_cast<uint4*>(prow + ((g ^ sw) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
                l_run = l_run * corr + rs;
                m_run = m_new;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full0 + 8 * sb);
                return true;
            };
            for (int kb = 0; ok && kb < nkb - 1; ++kb) ok = block(std::false_type{}, kb);
            if (ok) ok = block(std::true_type{}, nkb - 1);
            if (!ok) break;                                     // decided at a barrier: uniform over the softmax warps
            bad |= !fold_o(kv0 + nkb - 1);
            // the row sum is split over the two halves: exchange once more
            float* xs = sX + (xc & 1) * 256;
            ++xc;
            xs[hf * 128 + row] = l_run;
            if (softmax_any(bad)) break;
            {
                const float l_tot = l_run + xs[(hf ^ 1) * 128 + row];
                const float inv = 1.0f / l_tot;
                bf16* op = a.out + (static_cast<size_t>(row_base) + i) * d + h * ADK + hf * 32;
#pragma unroll
                for (int c = 0; c < 32; c += 8) {
                    Vec16<bf16> o;
#pragma unroll
                    for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(o_acc[c + k] * inv);
                    st16(op + c, o);
                }
                if (hf == 0) a.lse[(static_cast<size_t>(b) * a.H + h) * a.S + i] = (m_run + log2f(l_tot)) * kLn2F;
            }
            kv0 += nkb;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(A_TMEM_COLS) : "memory");
    }
}

// The same kernel with every resource single-buffered, so that two CTAs fit on an SM (98 KB of shared memory, 256 TMEM
// columns each): while the softmax warps of one CTA are in their dependency chain the other CTA's MMAs run.  The key
// tile is freed as soon as Q K^T of its block has run, the value tiles go through a ring of two.
constexpr int A2_OFF_K = A_TILE, A2_OFF_V = 2 * A_TILE, A2_OFF_P = 4 * A_TILE, A2_OFF_X = 6 * A_TILE, A2_OFF_BAR = A2_OFF_X + 2 * 2 * 128 * 4,
              A2_SMEM = A2_OFF_BAR + 256;
constexpr uint32_t A2_TMEM_COLS = 256;

template <bool DOC, bool ALIBI>
__global__ void __launch_bounds__(320, 2)
attn_fwd_tc2_kernel(const __grid_constant__ CUtensorMap tmQKV, const AttnTcArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;                            // one query tile
    uint8_t* sK = smem + A2_OFF_K;                 // one key tile: free again as soon as Q K^T of its block has run
    uint8_t* sV = smem + A2_OFF_V;                 // two value tiles
    uint8_t* sP = smem + A2_OFF_P;                 // one P tile (two 64-key halves)
    float* sX = reinterpret_cast<float*>(smem + A2_OFF_X);   // [buffer][half][row]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A2_OFF_BAR);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, q_empty = bar0 + 8, k_full = bar0 + 16, k_empty = bar0 + 24, v_full0 = bar0 + 32, v_empty0 = bar0 + 48,
                   s_full = bar0 + 64, s_empty = bar0 + 72, p_full = bar0 + 80, p_empty = bar0 + 88, o_full = bar0 + 96, o_empty = bar0 + 104;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = a.H * ADK;
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
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(A2_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_O = tmem_base + 128;           // scores in columns [0,128), O' in [128,192)

    // instruction descriptors: fp32 accumulate, bf16 operands; S: N=128, both K-major; PV: N=64, B MN-major
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(AK >> 3) << 17) | (uint32_t(AQ >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (uint32_t(ADK >> 3) << 17) | (uint32_t(AQ >> 4) << 24);

    // Every role walks the same list of tiles; the ring / buffer positions and barrier phases run on across
    // tiles (kv: key-block counter; gj: the same counter as seen by the score / P / O' buffers; tn: tile counter).
    if (warp == 0) {
        if (lane == 0 && !*abort_flag) {
            int kv = 0, tn = 0;
            bool ok = true;
            for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
                const AttnTile t = attn_tile(w, nq, a.H, a.H * a.B);
                const int nkb = t.qb + 1, row_base = t.b * a.S;
                if (!mbar_wait(q_empty, (tn & 1) ^ 1, abort_flag, 11, &g_attn_error)) break;
                mbar_expect_tx(q_full, A_TILE);
                tma_load_2d(smem_u32(sQ), &tmQKV, q_full, t.h * ADK, row_base + t.qb * AQ);
                for (int kb = 0; kb < nkb; ++kb, ++kv) {
                    if (!mbar_wait(k_empty, (kv & 1) ^ 1, abort_flag, 1, &g_attn_error)) { ok = false; break; }
                    mbar_expect_tx(k_full, A_TILE);
                    tma_load_2d(smem_u32(sK), &tmQKV, k_full, d + t.h * ADK, row_base + kb * AK);
                    const int vs = kv & 1;
                    if (!mbar_wait(v_empty0 + 8 * vs, ((kv >> 1) & 1) ^ 1, abort_flag, 12, &g_attn_error)) { ok = false; break; }
                    mbar_expect_tx(v_full0 + 8 * vs, A_TILE);
                    tma_load_2d(smem_u32(sV + vs * A_TILE), &tmQKV, v_full0 + 8 * vs, 2 * d + t.h * ADK, row_base + kb * AK);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && !*abort_flag) {
            int kv0 = 0, tn = 0;                                // kv0: key-block counter at the start of the tile
            bool ok = true;
            for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps, ++tn) {
                const AttnTile t = attn_tile(w, nq, a.H, a.H * a.B);
                const int nkb = t.qb + 1;
                ok = mbar_wait(q_full, tn & 1, abort_flag, 2, &g_attn_error);
                const uint32_t q_addr = smem_u32(sQ);
                auto issue_s = [&](int gj) -> bool {
                    if (!mbar_wait(k_full, gj & 1, abort_flag, 5, &g_attn_error)) return false;
                    if (gj >= 1 && !mbar_wait(s_empty, (gj - 1) & 1, abort_flag, 6, &g_attn_error)) return false;
                    tc_fence_after();
                    const uint32_t k_addr = smem_u32(sK);
#pragma unroll
                    for (int k = 0; k < ADK / 16; ++k)
                        umma_bf16(tmem_base, smem_desc(q_addr + k * 32, 16, 1024), smem_desc(k_addr + k * 32, 16, 1024),
                                  IDESC_S, k > 0 ? 1u : 0u);
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
                    const uint32_t v_addr = smem_u32(sV + vs * A_TILE);
#pragma unroll
                    for (int k = 0; k < AK / 16; ++k) {
                        const uint64_t da = smem_desc(p_addr + (k >> 2) * A_TILE + (k & 3) * 32, 16, 1024);
                        const uint64_t db = smem_desc(v_addr + k * 2048, A_TILE, 1024);
                        umma_bf16(tmem_O, da, db, IDESC_PV, k > 0 ? 1u : 0u);
                    }
                    umma_commit(o_full);
                    umma_commit(p_empty);
                    umma_commit(v_empty0 + 8 * vs);
                    return true;
                };
                if (ok) ok = issue_s(kv0);
                for (int kb = 0; ok && kb < nkb; ++kb) {
                    if (kb + 1 < nkb) ok = issue_s(kv0 + kb + 1);
                    if (ok) ok = issue_pv(kv0 + kb);
                }
                if (ok) umma_commit(q_empty);                   // the query tile is free once this tile's MMAs are done
                kv0 += nkb;
            }
        }
    } else {
        const int q = warp & 3, hf = (warp - 2) >> 2;          // TMEM lane quadrant, column half
        const int row = q * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
        const float scale2 = a.scale * kLog2eF;
        const int sw = row & 7;
        bool ok = true, bad = *abort_flag != 0;                 // bad: a wait of this thread gave up (reported at the next barrier)
        int kv0 = 0, xc = 0;                                    // key-block counter; exchange counter (alternates the sX buffer)

        for (int ps = 0, w; ok && (w = snake_tile(ps)) < total; ++ps) {
            const AttnTile t = attn_tile(w, nq, a.H, a.H * a.B);
            const int h = t.h, b = t.b, q0 = t.qb * AQ, nkb = t.qb + 1, row_base = b * a.S;
            const int i = q0 + row;                            // query position inside the sequence
            const float slope2 = ALIBI ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(a.H)) * kLog2eF : 0.f;
            const int my_doc = DOC ? a.doc[row_base + i] : 0;
            float m_run = -INFINITY, l_run = 0.f;
            float o_acc[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) o_acc[c] = 0.f;

            auto fold_o = [&](int gj) -> bool {                 // o_acc += O'(gj), this thread's 32 columns
                if (!mbar_wait(o_full, gj & 1, abort_flag, 7, &g_attn_error)) return false;
                tc_fence_after();
                uint32_t r[32];
                tmem_ld32(tmem_O + lane_addr + hf * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) o_acc[c] += __uint_as_float(r[c]);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(o_empty);
                return true;
            };

            // One 128-key block.  DIAG: the block on the diagonal (causal mask inside it).  The score of
            // column cj is r*scale2 + (slope2*cj + abase); with the loops unrolled cj is a literal.
            auto block = [&](auto diag_tag, int kb) -> bool {
                constexpr bool DIAG = decltype(diag_tag)::value;
                const int gj = kv0 + kb;
                bad |= !mbar_wait(s_full, gj & 1, abort_flag, 8, &g_attn_error);
                tc_fence_after();
                const int k0 = kb * AK;
                const int* dk_ptr = DOC ? a.doc + row_base + k0 + hf * 64 : nullptr;
                const float abase = ALIBI ? -slope2 * static_cast<float>(i - k0 - hf * 64) : 0.f;
                // Two passes over the scores in TMEM, 32 columns at a time, so that the thread never holds more than
                // 32 of them: the first finds the row maximum, the second makes P.  The score buffer is released
                // after the second pass.
                auto score = [&](float raw, int cj) -> float {
                    // cj is a literal once unrolled: nothing here is loop-invariant, so nothing is kept live across the passes
                    float sc = ALIBI ? fmaf(slope2, static_cast<float>(cj), fmaf(raw, scale2, abase)) : raw * scale2;
                    if (DIAG && hf * 64 + cj > row) sc = -INFINITY;
                    if (DOC && dk_ptr[cj] != my_doc) sc = -INFINITY;
                    return sc;
                };
                float mx = -INFINITY;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + lane_addr + hf * 64 + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) mx = fmaxf(mx, score(__uint_as_float(r[jj]), c * 32 + jj));
                }
                float* xs = sX + (xc & 1) * 256;
                ++xc;
                xs[hf * 128 + row] = mx;
                if (softmax_any(bad)) return false;             // the same answer in all eight warps
                const float m_new = fmaxf(m_run, fmaxf(mx, xs[(hf ^ 1) * 128 + row]));
                const float ms = (m_new == -INFINITY) ? 0.f : m_new;
                const float corr = ex2_approx(m_run - ms);
                if (kb >= 1) bad |= !fold_o(gj - 1);
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) o_acc[c] *= corr;
                }
                if (gj >= 1) bad |= !mbar_wait(p_empty, (gj - 1) & 1, abort_flag, 10, &g_attn_error);
                uint8_t* prow = sP + hf * A_TILE + row * 128;
                float rs = 0.f;
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
                            const float p0 = ex2_approx(score(__uint_as_float(r[jj]), c * 32 + jj) - ms);
                            const float p1 = ex2_approx(score(__uint_as_float(r[jj + 1]), c * 32 + jj + 1) - ms);
                            rs += p0 + p1;
                            __nv_bfloat162 tt = __floats2bfloat162_rn(p0, p1);
                            pk[e] = *reinterpret_cast<uint32_t*>(&tt);
                        }
                        *reinterpret_cast<uint4*>(prow + (((c * 4 + g) ^ sw) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_empty);            // both passes have read the scores
                l_run = l_run * corr + rs;
                m_run = m_new;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
                return true;
            };
            for (int kb = 0; ok && kb < nkb - 1; ++kb) ok = block(std::false_type{}, kb);
            if (ok) ok = block(std::true_type{}, nkb - 1);
            if (!ok) break;                                     // decided at a barrier: uniform over the softmax warps
            bad |= !fold_o(kv0 + nkb - 1);
            // the row sum is split over the two halves: exchange once more
            float* xs = sX + (xc & 1) * 256;
            ++xc;
            xs[hf * 128 + row] = l_run;
            if (softmax_any(bad)) break;
            {
                const float l_tot = l_run + xs[(hf ^ 1) * 128 + row];
                const float inv = 1.0f / l_tot;
                bf16* op = a.out + (static_cast<size_t>(row_base) + i) * d + h * ADK + hf * 32;
#pragma unroll
                for (int c = 0; c < 32; c += 8) {
                    Vec16<bf16> o;
#pragma unroll
                    for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(o_acc[c + k] * inv);
                    st16(op + c, o);
                }
                if (hf == 0) a.lse[(static_cast<size_t>(b) * a.H + h) * a.S + i] = (m_run + log2f(l_tot)) * kLn2F;
            }
            kv0 += nkb;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(A2_TMEM_COLS) : "memory");
    }
}

template <bool DOC, bool ALIBI>
static int launch_fwd_tc(const CUtensorMap& tm, const AttnTcArgs& a, dim3 grid, cudaStream_t s)
{
    static bool attr_set = false;
    if (!attr_set) {
        NNB_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_tc_kernel<DOC, ALIBI>, cudaFuncAttributeMaxDynamicSharedMemorySize, A_SMEM));
        attr_set = true;
    }
    attn_fwd_tc_kernel<DOC, ALIBI><<<grid, 320, A_SMEM, s>>>(tm, a);
    NNB_LAUNCH_CHECK();
    return 0;
}

template <bool DOC, bool ALIBI>
static int launch_fwd_tc2(const CUtensorMap& tm, const AttnTcArgs& a, dim3 grid, cudaStream_t s)
{
    static bool attr_set = false;
    if (!attr_set) {
        NNB_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_tc2_kernel<DOC, ALIBI>, cudaFuncAttributeMaxDynamicSharedMemorySize, A2_SMEM));
        attr_set = true;
    }
    attn_fwd_tc2_kernel<DOC, ALIBI><<<grid, 320, A2_SMEM, s>>>(tm, a);
    NNB_LAUNCH_CHECK();
    return 0;
}

// CTAs per SM of the forward kernel: 2 (single-buffered) unless NNB200_ATTN_FWD_CTAS=1 asks for the double-buffered one.
static int fwd_ctas_per_sm()
{
    static const int v = [] { const char* e = getenv("NNB200_ATTN_FWD_CTAS"); return (e && e[0] == '1') ? 1 : 2; }();
    return v;
}

bool attention_tc_supported(int dk, int S, int d) { return dk == ADK && (S % AQ) == 0 && (d % 8) == 0; }

int attention_fwd_tc(const bf16* qkv, bf16* out, float* lse, const int* doc, int B, int S, int H, int dk, int alibi,
                     cudaStream_t s)
{
    if (static_cast<long long>(B) * S * H == 0) return 0;
    NNB_ARG_CHECK(attention_tc_supported(dk, S, H * dk), "shape not supported by the tcgen05 attention kernel");
    NNB_ARG_CHECK(B <= 65535 && H <= 65535, "batch / heads exceed the grid limits");
    CUtensorMap tm;
    const int d = H * dk;
    NNB_TRY(tensor_map_2d(qkv, 3LL * d, static_cast<long long>(B) * S, 3LL * d, ADK, 128, &tm, 2));
    AttnTcArgs a{out, lse, doc, B, S, H, alibi, 1.0f / sqrtf(static_cast<float>(dk))};
    const long long tiles = static_cast<long long>(S / AQ) * H * B;
    NNB_ARG_CHECK(tiles < (1ll << 31), "too many attention tiles");
    const int per_sm = fwd_ctas_per_sm();
    const long long slots = static_cast<long long>(kSmCount) * per_sm;
    dim3 grid(static_cast<unsigned>(tiles < slots ? tiles : slots));           // persistent: each CTA walks the tile list
    if (per_sm == 2) {
        if (doc && alibi) return launch_fwd_tc2<true, true>(tm, a, grid, s);
        if (doc) return launch_fwd_tc2<true, false>(tm, a, grid, s);
        if (alibi) return launch_fwd_tc2<false, true>(tm, a, grid, s);
        return launch_fwd_tc2<false, false>(tm, a, grid, s);
    }
    if (doc && alibi) return launch_fwd_tc<true, true>(tm, a, grid, s);
    if (doc) return launch_fwd_tc<true, false>(tm, a, grid, s);
    if (alibi) return launch_fwd_tc<false, true>(tm, a, grid, s);
    return launch_fwd_tc<false, false>(tm, a, grid, s);
}

int attention_device_error(int* code)
{
    NNB_CUDA_CHECK(cudaMemcpyFromSymbol(code, g_attn_error, sizeof(int)));
    if (*code) { const int z = 0; NNB_CUDA_CHECK(cudaMemcpyToSymbol(g_attn_error, &z, sizeof(int))); }
    return 0;
}

}  // namespace nnb
