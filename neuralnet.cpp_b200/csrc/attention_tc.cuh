// Shared by the tcgen05 attention kernels (forward and backward): which key / query blocks of a tile a document mask
// leaves anything of.  The table holds one (min, max) pair of document ids per 64 rows of a sequence
// (attention_doc_ranges); a block is skipped when its id range cannot meet the range of the tile it is paired with.
// A skipped block would have contributed exact zeros, so skipping changes no result bit.
#pragma once
#include "common.cuh"

namespace nnb {

// bit j = block j of the tile's list is active; lists longer than 128 blocks are not filtered
struct BlockMask { uint32_t w[4]; };

__device__ __forceinline__ BlockMask block_mask_all()
{
    BlockMask m;
    m.w[0] = m.w[1] = m.w[2] = m.w[3] = 0xffffffffu;
    return m;
}
__device__ __forceinline__ bool block_active(const BlockMask& m, int j)
{
    if (j >= 128) return true;
    const uint32_t word = j < 32 ? m.w[0] : (j < 64 ? m.w[1] : (j < 96 ? m.w[2] : m.w[3]));
    return (word >> (j & 31)) & 1u;
}
// active blocks among the first n of the list
__device__ __forceinline__ int block_count(const BlockMask& m, int n)
{
    if (n > 128) return n;
    int c = 0;
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
        const int rem = n - wd * 32;
        if (rem <= 0) break;
        c += __popc(rem >= 32 ? m.w[wd] : (m.w[wd] & ((1u << rem) - 1u)));
    }
    return c;
}
// Called by a whole warp.  Block j of the list (0 <= j < nblocks) covers the table entries [(first + j) * per,
// (first + j + 1) * per) of `rng` (the table of this sequence); (ta, tb) are the two entries of the 128-row tile the
// blocks are paired with.  Blocks [force0, force1) — the ones on the diagonal, which hold the tile's own rows — are
// always active, whatever the table says, so every role counts at least those.
__device__ __forceinline__ BlockMask doc_block_mask(const int2* rng, int first, int nblocks, int per, int2 ta, int2 tb,
                                                    int force0, int force1, int lane)
{
    BlockMask m = block_mask_all();
    if (nblocks > 128) return m;
    const int tmin = min(ta.x, tb.x), tmax = max(ta.y, tb.y);
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
        if (wd * 32 >= nblocks) break;                      // uniform over the warp
        const int j = wd * 32 + lane;
        bool act = true;
        if (j < nblocks && !(j >= force0 && j < force1)) {
            int lo = INT_MAX, hi = INT_MIN;
            for (int e = 0; e < per; ++e) {
                const int2 r = rng[(first + j) * per + e];
                lo = min(lo, r.x);
                hi = max(hi, r.y);
            }
            act = !(hi < tmin || lo > tmax);
        }
        m.w[wd] = __ballot_sync(0xffffffffu, act);
    }
    return m;
}

}  // namespace nnb
