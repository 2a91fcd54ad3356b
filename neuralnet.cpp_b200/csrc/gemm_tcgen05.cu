// bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma (fp32 accumulators in
// TMEM) -> tcgen05.ld epilogue.  Persistent, warp-specialised, one CTA per SM:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM owner + MMA issuer (one elected lane)
//   warps 2..5  epilogue: each owns one 32-lane TMEM quadrant of the 128-row accumulator
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
//
//   D[M,N] = alpha * A[M,K] * B[N,K]^T  (+ bias[n]) (+ residual[m,n])          store as bf16 or fp32
//   D[M,N] += alpha * A * B^T                                                   fp32, atomically (split-K)
// Either operand may be K-major (K contiguous) or MN-major (M resp. N contiguous): the forward
// projections are K-major x K-major, the input-gradient GEMMs read the weight MN-major and the
// weight-gradient GEMMs read both operands MN-major (K = tokens), so no transposed copies exist.
//
// This replaces cublasSgemm + the separate bias / add passes of the reference
// (cuda/cuda_kernels.cu:527-563, compute_layer.hpp:151-195).
// All TMA loads are plain (no cluster multicast).  Every mbarrier wait is bounded: after about a
// second it raises an error flag the host can read, and the CTA drains and frees its TMEM.
#include <cuda.h>

#include <mutex>
#include <unordered_map>
#include <vector>

#include "kernels.h"
#include "tc_ptx.cuh"

namespace nnb {

__device__ int g_gemm_error = 0;   // 0 ok; otherwise (code << 16 | blockIdx) of the first wait that gave up

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int C_STAGE_BYTES = BM * 128;

struct GemmParams {
    int M, N, K;
    int tiles_m, tiles_n, splits, kb_per_split, kb_total;
    void* C;
    long long ldc;
    int c_bf16, accumulate, vec_ok, tma_store;
    const float* bias_n;
    const void* residual;
    float alpha;
    int glu_ff;                 // SwiGLU variant of the pair kernel: rows of B per half (gate rows, then up rows); 0 otherwise
    float* colsum_part;         // SwiGLU-backward variant: column sums of the output per 128 rows, [ceil(M / 128)][2 glu_ff]; or null
    float* dot_out;             // row-dot variant: sums per (row, 64-column block), laid out [row / dot_S][block][row % dot_S]
    int dot_S, dot_H;
};

// ---------------------------------------------------------------- kernel
template <int BN, bool A_MN, bool B_MN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p)
{
    constexpr int B_STAGE_BYTES = BN * BK * 2;
    constexpr uint32_t TMEM_COLS = 2 * BN;                      // two accumulator buffers (256 or 512 columns)
    // instruction descriptor: fp32 accumulate, bf16 x bf16, operand majors, N >> 3, M >> 4
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(A_MN) << 15) | (uint32_t(B_MN) << 16) |
                               (uint32_t(BN >> 3) << 17) | (uint32_t(BM >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint8_t* sC = sB + STAGES * B_STAGE_BYTES;                   // 2 staging tiles of 128 rows x 128 bytes
    float* sBias = reinterpret_cast<float*>(sC + 2 * C_STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sBias + BN);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
    const uint32_t tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles = p.tiles_m * p.tiles_n;
    const int units = tiles * p.splits;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int u = blockIdx.x; u < units && !*abort_flag; u += gridDim.x) {
                const int split = u / tiles, t = u - split * tiles;
                const int tile_n = t / p.tiles_m, tile_m = t - tile_n * p.tiles_m;
                const int kb0 = split * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, 1, &g_gemm_error)) break;
                    const uint32_t fb = full0 + 8 * s;
                    mbar_expect_tx(fb, A_STAGE_BYTES + B_STAGE_BYTES);
                    const uint32_t a_dst = smem_u32(sA + s * A_STAGE_BYTES), b_dst = smem_u32(sB + s * B_STAGE_BYTES);
                    if (!A_MN) tma_load_2d(a_dst, &tmA, fb, kb * BK, tile_m * BM);
                    else
                        for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * (BK * 128), &tmA, fb, tile_m * BM + j * 64, kb * BK);
                    if (!B_MN) tma_load_2d(b_dst, &tmB, fb, kb * BK, tile_n * BN);
                    else
                        for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), &tmB, fb, tile_n * BN + j * 64, kb * BK);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, tc = 0;
            for (int u = blockIdx.x; u < units && !*abort_flag; u += gridDim.x, ++tc) {
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
                        umma_bf16(d_tmem, da, db, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty0 + 8 * s);          // frees the stage once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(tfull0 + 8 * acc);            // accumulator complete
            }
        }
    } else {
        const int q = warp & 3;                           // TMEM lane quadrant this warp may read
        const int epi_tid = threadIdx.x - 64;             // 0..127 over the four epilogue warps
        const bool elected = epi_tid == 0;
        const int r_local = q * 32 + lane;                // row of the 128-row tile this thread owns
        int tc = 0, blk = 0;
        if (p.tma_store) {
            // Coalesced epilogue: accumulators -> registers -> swizzled 128-byte rows in shared memory ->
            // one TMA store (or TMA reduce-add for split-K) per 128 x 128-byte block; ragged edges are
            // clipped by the tensor map.  Two staging tiles alternate so a store drains while the next fills.
            const int CB = p.c_bf16 ? 64 : 32;            // columns per 128-byte row
            for (int u = blockIdx.x; u < units; u += gridDim.x, ++tc) {
                const int split = u / tiles, t = u - split * tiles;
                const int tile_n = t / p.tiles_m, tile_m = t - tile_n * p.tiles_m;
                const int acc = tc & 1;
                const uint32_t acc_ph = (tc >> 1) & 1;
                const bool arrived = mbar_wait(tfull0 + 8 * acc, acc_ph, abort_flag, 4, &g_gemm_error);
                if (epi_any(!arrived || *abort_flag)) break;
                tc_fence_after();
                const bool add_extra = (split == 0);      // bias / residual enter once when K is split
                const bool use_bias = p.bias_n && add_extra;
                if (use_bias)
                    for (int j = epi_tid; j < BN; j += 128) sBias[j] = (tile_n * BN + j < p.N) ? p.bias_n[tile_n * BN + j] : 0.f;
                const int m = tile_m * BM + r_local;
                const bool row_ok = m < p.M;
                const long long row_off = static_cast<long long>(m) * p.ldc;
#pragma unroll 1
                for (int cb = 0; cb * CB < BN; ++cb, ++blk) {
                    const int n0 = tile_n * BN + cb * CB;
                    if (n0 >= p.N) break;
                    uint8_t* stage = sC + (blk & 1) * C_STAGE_BYTES;
                    if (elected) tma_wait_read1();        // the store that used this tile two blocks ago has read it
                    epi_bar();
                    uint8_t* srow = stage + r_local * 128;
#pragma unroll 1
                    for (int half = 0; half * 32 < CB; ++half) {
                        uint32_t r[32];
                        tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + cb * CB + half * 32, r);
                        tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = p.alpha * __uint_as_float(r[j]);
                        if (use_bias) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] += sBias[cb * CB + half * 32 + j];
                        }
                        const int nh = n0 + half * 32;
                        if (p.c_bf16) {
                            const bf16* rp = (p.residual && add_extra && row_ok) ? static_cast<const bf16*>(p.residual) + row_off + nh : nullptr;
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                if (rp && nh + j + 8 <= p.N) { const Vec16<bf16> rr = ld16(rp + j);
#pragma unroll
                                    for (int k = 0; k < 8; ++k) v[j + k] += __bfloat162float(rr.v[k]); }
                                else if (rp) { for (int k = 0; k < 8; ++k) if (nh + j + k < p.N) v[j + k] += __bfloat162float(rp[j + k]); }
                                Vec16<bf16> o;
#pragma unroll
                                for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(v[j + k]);
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
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    epi_bar();
                    if (elected) {
                        if (p.accumulate) tma_reduce_add_2d(&tmC, smem_u32(stage), n0, tile_m * BM);
                        else tma_store_2d(&tmC, smem_u32(stage), n0, tile_m * BM);
                        tma_commit();
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
            }
            if (elected) tma_wait_all();                  // shared memory must outlive the stores in flight
        } else
        for (int u = blockIdx.x; u < units; u += gridDim.x, ++tc) {
            if (*abort_flag) break;
            const int split = u / tiles, t = u - split * tiles;
            const int tile_n = t / p.tiles_m, tile_m = t - tile_n * p.tiles_m;
            const int acc = tc & 1;
            const uint32_t acc_ph = (tc >> 1) & 1;
            if (!mbar_wait(tfull0 + 8 * acc, acc_ph, abort_flag, 4, &g_gemm_error)) break;
            tc_fence_after();
            const int m = tile_m * BM + q * 32 + lane;
            const bool row_ok = m < p.M;
            const long long row_off = static_cast<long long>(m) * p.ldc;
            const bool add_extra = (split == 0);          // bias / residual enter once when K is split
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                const int n0 = tile_n * BN + c0;
                if (n0 >= p.N) break;
                uint32_t r[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c0, r);
                tmem_ld_wait();
                if (!row_ok) continue;
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = p.alpha * __uint_as_float(r[j]);
                if (p.bias_n && add_extra) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) if (n0 + j < p.N) v[j] += p.bias_n[n0 + j];
                }
                if (p.accumulate) {
                    float* cp = static_cast<float*>(p.C) + row_off + n0;
                    if (p.vec_ok && n0 + 32 <= p.N) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) atomicAdd(reinterpret_cast<float4*>(cp + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
                    } else {
                        for (int j = 0; j < 32; ++j) if (n0 + j < p.N) atomicAdd(cp + j, v[j]);
                    }
                } else if (p.c_bf16) {
                    bf16* cp = static_cast<bf16*>(p.C) + row_off + n0;
                    const bf16* rp = p.residual ? static_cast<const bf16*>(p.residual) + row_off + n0 : nullptr;
                    if (p.vec_ok && n0 + 32 <= p.N) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            Vec16<bf16> o;
                            if (rp) { const Vec16<bf16> rr = ld16(rp + j);
#pragma unroll
                                for (int k = 0; k < 8; ++k) v[j + k] += __bfloat162float(rr.v[k]); }
#pragma unroll
                            for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(v[j + k]);
                            st16(cp + j, o);
                        }
                    } else {
                        for (int j = 0; j < 32; ++j) if (n0 + j < p.N) {
                            float x = v[j];
                            if (rp) x += __bfloat162float(rp[j]);
                            cp[j] = __float2bfloat16_rn(x);
                        }
                    }
                } else {
                    float* cp = static_cast<float*>(p.C) + row_off + n0;
                    const float* rp = p.residual ? static_cast<const float*>(p.residual) + row_off + n0 : nullptr;
                    if (p.vec_ok && n0 + 32 <= p.N) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                            if (rp) { const float4 rr = *reinterpret_cast<const float4*>(rp + j); o.x += rr.x; o.y += rr.y; o.z += rr.z; o.w += rr.w; }
                            *reinterpret_cast<float4*>(cp + j) = o;
                        }
                    } else {
                        for (int j = 0; j < 32; ++j) if (n0 + j < p.N) cp[j] = v[j] + (rp ? rp[j] : 0.f);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace nnb
#include "gemm_tcgen05_2cta.cuh"
namespace nnb {

// ---------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

struct MapKey {
    const void* ptr; long long inner, outer, ld; int box_inner, box_outer, esz;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && inner == o.inner && outer == o.outer && ld == o.ld && box_inner == o.box_inner && box_outer == o.box_outer && esz == o.esz; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const
    {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        for (long long v : {k.inner, k.outer, k.ld, static_cast<long long>(k.box_inner), static_cast<long long>(k.box_outer), static_cast<long long>(k.esz)})
            h = h * 1000003u ^ static_cast<size_t>(v);
        return h;
    }
};

// 2-D tensor map (bf16 when esz = 2, fp32 when esz = 4): `inner` contiguous elements per row, `outer`
// rows `ld` elements apart; 128-byte swizzle
int tensor_map_2d(const void* ptr, long long inner, long long outer, long long ld, int box_inner, int box_outer,
                  CUtensorMap* out, int esz)
{
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{ptr, inner, outer, ld, box_inner, box_outer, esz};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) { fprintf(stderr, "nnb200: cuTensorMapEncodeTiled not available from the driver\n"); return -2; }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * static_cast<cuuint64_t>(esz)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "nnb200: cuTensorMapEncodeTiled failed (%d)\n", static_cast<int>(r)); return -2; }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return 0;
}

static int sm_count() { return device_sm_count(); }

// Optional per-launch timing: CUDA events recorded on the launching stream around each GEMM kernel,
// so a benchmark can report achieved FLOP/s of this kernel from inside a real training step.
struct GemmProfile {
    bool on = false;
    std::vector<cudaEvent_t> events;     // pairs: start, stop
    size_t used = 0;
    // Two classes: 0 = the product with bias / residual / row-dot epilogues, 1 = launches whose epilogue also runs an
    // activation (SwiGLU forward or backward), which outlasts a short main loop and would blur the GEMM's own figure.
    std::vector<unsigned char> cls;      // per pair
    double flops[2] = {0.0, 0.0};
    // Only the launches of one stream are recorded, that of the first GEMM after enabling: event pairs of launches that
    // overlap on other streams (the Newton-Schulz lanes of Muon) would add up to more than the time that passed.
    bool have_stream = false;
    cudaStream_t stream = nullptr;
};
static GemmProfile g_prof;

static bool prof_takes(cudaStream_t s)
{
    if (!g_prof.on) return false;
    if (!g_prof.have_stream) { g_prof.have_stream = true; g_prof.stream = s; }
    return g_prof.stream == s;
}
static void prof_close(cudaStream_t s, int cls, double flops);
static cudaEvent_t prof_event(cudaStream_t s)
{
    if (g_prof.used == g_prof.events.size()) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
        g_prof.events.push_back(e);
    }
    cudaEvent_t e = g_prof.events[g_prof.used++];
    cudaEventRecord(e, s);
    return e;
}

static void prof_close(cudaStream_t s, int cls, double flops)
{
    prof_event(s);
    g_prof.cls.resize(g_prof.used / 2);
    g_prof.cls[g_prof.used / 2 - 1] = static_cast<unsigned char>(cls);
    g_prof.flops[cls] += flops;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tcm, const GemmParams& p, cudaStream_t s)
{
    constexpr int STAGES = (BN == 256) ? 4 : 6;
    constexpr int SMEM = STAGES * (A_STAGE_BYTES + BN * BK * 2) + 2 * C_STAGE_BYTES + BN * 4 + 1024 + 256;
    static_assert(SMEM <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
    static PerDeviceOnce once;
    NNB_TRY(once.run([] { return cudaFuncSetAttribute(gemm_bf16_kernel<BN, A_MN, B_MN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM); }));
    const int units = p.tiles_m * p.tiles_n * p.splits;
    const int grid = units < sm_count() ? units : sm_count();
    const bool rec = prof_takes(s);
    if (rec) prof_event(s);
    gemm_bf16_kernel<BN, A_MN, B_MN, STAGES><<<grid, 192, SMEM, s>>>(ta, tb, tcm, p);
    if (rec) prof_close(s, 0, 2.0 * p.M * p.N * p.K);
    NNB_LAUNCH_CHECK();
    return 0;
}

constexpr int PAIR_THREADS = 384;     // producer, MMA, eight epilogue warps, and two warps that sum columns in the SwiGLU-backward form
// CTA pairs that can be resident at once (GPCs with an odd SM count strand one SM each)
template <typename Kernel>
static int max_pairs(Kernel kernel, int smem)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * sm_count());
    cfg.blockDim = dim3(PAIR_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 0; }
    return n;
}

constexpr int PAIR_STAGES = 6;
constexpr int PAIR_STAGES_RES = 5;                          // the residual staging tiles take one operand stage's room
constexpr int PAIR_SMEM = PAIR_STAGES * PAIR_STAGE_BYTES + 2 * C_STAGE_BYTES + 256 * 4 + 1024 + 256;
static_assert(PAIR_STAGES_RES * PAIR_STAGE_BYTES + 4 * C_STAGE_BYTES + 256 * 4 + 1024 + 256 <= PAIR_SMEM, "the residual variant must fit the same shared memory");
static_assert(PAIR_SMEM <= 232448, "exceeds the 227 KB of shared memory a CTA may use");

// number of CTA pairs the current device runs at once; 0 = the pair kernel cannot be used there
static int pair_capacity()
{
    static std::atomic<int> cache[64];                      // per device: 0 = not asked yet, -1 = unavailable
    const int dev = current_device_slot();
    int n = cache[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaFuncSetAttribute(gemm_bf16_pair_kernel<false, false, PAIR_STAGES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM) != cudaSuccess) { cudaGetLastError(); n = -1; }
        else n = max_pairs(gemm_bf16_pair_kernel<false, false, PAIR_STAGES, false>, PAIR_SMEM);
        if (n <= 0) n = -1;
        cache[dev].store(n, std::memory_order_relaxed);
    }
    return n > 0 ? n : 0;
}

template <bool A_MN, bool B_MN, bool RES = false, bool GLU = false, bool DB = false, bool DOT = false, bool GLUB = false>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tcm, const CUtensorMap& tr, const GemmParams& p, cudaStream_t s)
{
    constexpr int STAGES = (RES || GLU || DB || DOT || GLUB) ? PAIR_STAGES_RES : PAIR_STAGES;
    static PerDeviceOnce once;
    NNB_TRY(once.run([] { return cudaFuncSetAttribute(gemm_bf16_pair_kernel<A_MN, B_MN, STAGES, RES, GLU, DB, DOT, GLUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM); }));
    const int units = p.tiles_m * p.tiles_n * p.splits;
    const int pairs = units < pair_capacity() ? units : pair_capacity();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(PAIR_THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    const bool rec = prof_takes(s);
    if (rec) prof_event(s);
    NNB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_bf16_pair_kernel<A_MN, B_MN, STAGES, RES, GLU, DB, DOT, GLUB>, ta, tb, tcm, tr, p));
    if (rec) prof_close(s, (GLU || GLUB) ? 1 : 0, (GLU ? 4.0 : 2.0) * p.M * p.N * p.K);     // GLU: p.N is half the product's width
    NNB_LAUNCH_CHECK();
    return 0;
}

int gemm_bf16(const bf16* A, const bf16* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
              int a_mn, int b_mn, int c_bf16, float alpha, const float* bias_n, const void* residual, int accumulate,
              cudaStream_t stream)
{
    if (M <= 0 || N <= 0) return 0;
    NNB_ARG_CHECK(K > 0, "K must be positive");
    NNB_ARG_CHECK((lda % 8) == 0 && (ldb % 8) == 0, "operand leading dimensions must be multiples of 8 elements (16 bytes)");
    NNB_ARG_CHECK(((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0, "operands must be 16-byte aligned");
    NNB_ARG_CHECK(!(accumulate && c_bf16), "accumulate needs an fp32 destination");
    NNB_ARG_CHECK(!(accumulate && residual), "accumulate and residual are exclusive");

    GemmParams p{};
    p.M = M; p.N = N; p.K = K;
    p.C = C; p.ldc = ldc; p.c_bf16 = c_bf16; p.accumulate = accumulate;
    p.bias_n = bias_n; p.residual = residual; p.alpha = alpha;
    const int esz = c_bf16 ? 2 : 4;
    p.vec_ok = ((ldc * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0) &&
               (!residual || (reinterpret_cast<uintptr_t>(residual) & 15) == 0);
    // 256 x 256 tiles on CTA pairs when the output has more than one 128-row and one 128-column block and
    // the coalesced (TMA-store) epilogue applies; a product too small to give half the pairs a tile runs 128 x 128 tiles
    // on single CTAs instead (1024^3: 64 tiles instead of 16)
    const bool few_tiles = !accumulate && 2 * ceil_div(M, 256) * ceil_div(N, 256) <= pair_capacity();
    const int BN = (N > 128 && !few_tiles) ? 256 : 128;
    const bool pair = p.vec_ok && M > 128 && N > 128 && pair_capacity() > 0 && !few_tiles;
    p.tiles_m = static_cast<int>(ceil_div(M, pair ? 256 : BM));
    p.tiles_n = static_cast<int>(ceil_div(N, BN));
    p.kb_total = static_cast<int>(ceil_div(K, BK));
    p.splits = 1;
    if (accumulate) {
        // split K so the work units fill whole waves of the machine: minimise waves/splits
        const int tiles = p.tiles_m * p.tiles_n, sms = pair ? pair_capacity() : sm_count();
        double best = 1e30;
        for (int sp = 1; sp <= 32 && p.kb_total / sp >= 4; ++sp) {
            const double cost = static_cast<double>(ceil_div(static_cast<long long>(tiles) * sp, sms)) / sp + 0.02 * sp;
            if (cost < best - 1e-9) { best = cost; p.splits = sp; }
        }
    }
    p.kb_per_split = static_cast<int>(ceil_div(p.kb_total, p.splits));
    p.splits = static_cast<int>(ceil_div(p.kb_total, p.kb_per_split));

    CUtensorMap ta, tb;
    if (!a_mn) NNB_TRY(tensor_map_2d(A, K, M, lda, BK, BM, &ta, 2));
    else NNB_TRY(tensor_map_2d(A, M, K, lda, 64, BK, &ta, 2));
    if (!b_mn) NNB_TRY(tensor_map_2d(B, K, N, ldb, BK, pair ? PAIR_BN_HALF : BN, &tb, 2));
    else NNB_TRY(tensor_map_2d(B, N, K, ldb, 64, BK, &tb, 2));
    CUtensorMap tcm = ta;                      // unused placeholder when the direct epilogue runs
    p.tma_store = p.vec_ok;
    if (p.tma_store) NNB_TRY(tensor_map_2d(C, N, M, ldc, c_bf16 ? 64 : 32, BM, &tcm, esz));

    if (pair) {
        // a bf16 residual of a forward projection (both operands K-major) goes through its own staging tiles
        if (!a_mn && !b_mn && residual && c_bf16) {
            CUtensorMap tr;
            NNB_TRY(tensor_map_2d(residual, N, M, ldc, 64, BM, &tr, 2));
            return launch_gemm_pair<false, false, true>(ta, tb, tcm, tr, p, stream);
        }
        // Two staging tiles per epilogue group (and five operand stages instead of six) where it was measured faster:
        // short main loops of the forward projections (K <= 1024: 16384 x 2304 x 768 55.3 -> 51.2 us, 16384 x 8192 x 768
        // 170.0 -> 161.6) and the split-K weight gradients (768 x 768 x 16384 23.4 -> 22.0 us); the input-gradient
        // products (B read MN-major) lose 1-2 % with five stages and keep six.
        if (!a_mn && !b_mn && p.kb_per_split <= 16) return launch_gemm_pair<false, false, false, false, true>(ta, tb, tcm, tcm, p, stream);
        if (a_mn && b_mn) return launch_gemm_pair<true, true, false, false, true>(ta, tb, tcm, tcm, p, stream);
        if (!a_mn && !b_mn) return launch_gemm_pair<false, false>(ta, tb, tcm, tcm, p, stream);
        if (!a_mn && b_mn) return launch_gemm_pair<false, true>(ta, tb, tcm, tcm, p, stream);
        return launch_gemm_pair<true, false>(ta, tb, tcm, tcm, p, stream);
    }
#define GO(bn, am, bm) return launch_gemm<bn, am, bm>(ta, tb, tcm, p, stream)
    if (BN == 256) {
        if (!a_mn && !b_mn) GO(256, false, false);
        if (!a_mn && b_mn) GO(256, false, true);
        if (a_mn && !b_mn) GO(256, true, false);
        GO(256, true, true);
    } else {
        if (!a_mn && !b_mn) GO(128, false, false);
        if (!a_mn && b_mn) GO(128, false, true);
        if (a_mn && !b_mn) GO(128, true, false);
        GO(128, true, true);
    }
#undef GO
}

// H1[M, 2 ff] = X[M, K] W[2 ff, K]^T + bias and H2[M, ff] = gate * sigmoid(gate) * up in one launch (the pair kernel's
// SwiGLU epilogue).  gemm_swiglu_supported says whether the shape can take this path; the caller otherwise runs the
// projection and the activation as two kernels, with the same results bit for bit.
bool gemm_swiglu_supported(int M, int ff, int K)
{
    return M > 128 && ff >= 128 && (ff % 128) == 0 && K > 0 && (K % 8) == 0 && pair_capacity() > 0;
}
int gemm_bf16_swiglu(const bf16* X, const bf16* W, const float* bias, bf16* H1, bf16* H2, int M, int ff, int K, cudaStream_t stream)
{
    NNB_ARG_CHECK(gemm_swiglu_supported(M, ff, K), "shape not supported by the fused SwiGLU projection");
    NNB_ARG_CHECK(((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(H1) |
                    reinterpret_cast<uintptr_t>(H2)) & 15) == 0, "operands must be 16-byte aligned");
    GemmParams p{};
    p.M = M; p.N = ff; p.K = K;
    p.C = H1; p.ldc = 2LL * ff; p.c_bf16 = 1; p.accumulate = 0;
    p.bias_n = bias; p.residual = nullptr; p.alpha = 1.0f;
    p.vec_ok = 1; p.tma_store = 1; p.glu_ff = ff;
    p.tiles_m = static_cast<int>(ceil_div(M, 256));
    p.tiles_n = ff / 128;
    p.kb_total = static_cast<int>(ceil_div(K, BK));
    p.splits = 1;
    p.kb_per_split = p.kb_total;
    CUtensorMap ta, tb, t1, t2;
    NNB_TRY(tensor_map_2d(X, K, M, K, BK, BM, &ta, 2));
    NNB_TRY(tensor_map_2d(W, K, 2 * ff, K, BK, PAIR_BN_HALF, &tb, 2));
    NNB_TRY(tensor_map_2d(H1, 2 * ff, M, 2LL * ff, 64, BM, &t1, 2));
    NNB_TRY(tensor_map_2d(H2, ff, M, ff, 64, BM, &t2, 2));
    return launch_gemm_pair<false, false, false, true>(ta, tb, t1, t2, p, stream);
}

// Input gradient of a SwiGLU block's second projection taken through the activation in one launch:
// dH1[M, 2 ff] = (dgate | dup) of (dY[M, K] W[K, ff]) at H1[M, 2 ff] = (gate | up); W stored (K, ff), ff contiguous.
// Bit-identical to gemm_bf16 into a (M, ff) buffer followed by act_bwd.  colsum_partial (may be null; 16-byte aligned):
// ceil(M / 128) rows of 2 ff floats that receive the column sums of dH1 over each 128 rows (what the bias gradient of
// the first projection is folded from), every element written.
bool gemm_swiglu_bwd_supported(int M, int ff, int K)
{
    return M > 128 && ff > 128 && (ff % 64) == 0 && K > 0 && (K % 8) == 0 && pair_capacity() > 0;
}
int gemm_bf16_swiglu_bwd(const bf16* dY, const bf16* W, const bf16* H1, bf16* dH1, int M, int ff, int K, float* colsum_partial,
                         cudaStream_t stream)
{
    NNB_ARG_CHECK(gemm_swiglu_bwd_supported(M, ff, K), "shape not supported by the fused SwiGLU input gradient");
    NNB_ARG_CHECK(((reinterpret_cast<uintptr_t>(dY) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(H1) |
                    reinterpret_cast<uintptr_t>(dH1)) & 15) == 0, "operands must be 16-byte aligned");
    GemmParams p{};
    p.M = M; p.N = ff; p.K = K;
    p.C = dH1; p.ldc = 2LL * ff; p.c_bf16 = 1; p.accumulate = 0;
    p.alpha = 1.0f; p.vec_ok = 1; p.tma_store = 1; p.glu_ff = ff;
    NNB_ARG_CHECK((reinterpret_cast<uintptr_t>(colsum_partial) & 15) == 0, "the partial sums must be 16-byte aligned");
    p.colsum_part = colsum_partial;
    p.tiles_m = static_cast<int>(ceil_div(M, 256));
    p.tiles_n = static_cast<int>(ceil_div(ff, 256));
    p.kb_total = static_cast<int>(ceil_div(K, BK));
    p.splits = 1;
    p.kb_per_split = p.kb_total;
    CUtensorMap ta, tb, tcm, tr;
    NNB_TRY(tensor_map_2d(dY, K, M, K, BK, BM, &ta, 2));
    NNB_TRY(tensor_map_2d(W, ff, K, ff, 64, BK, &tb, 2));
    NNB_TRY(tensor_map_2d(dH1, 2LL * ff, M, 2LL * ff, 64, BM, &tcm, 2));
    NNB_TRY(tensor_map_2d(H1, 2LL * ff, M, 2LL * ff, 64, BM, &tr, 2));
    return launch_gemm_pair<false, true, false, false, false, false, true>(ta, tb, tcm, tr, p, stream);
}

// dX[M, N] = dY[M, K] W[K, N] (W stored (K, N), N contiguous) and, from the same epilogue, the sums over each 64-column
// block of dX (as stored in bf16) times `other` (M, N): dot_out[(m / S * H + block) * S + m % S], H = N / 64 blocks.
bool gemm_rowdot_supported(int M, int N, int K, int S, int H)
{
    return M > 128 && N > 128 && N == 64 * H && S > 0 && (M % S) == 0 && K > 0 && (K % 8) == 0 && pair_capacity() > 0;
}
int gemm_bf16_dx_rowdot(const bf16* dY, const bf16* W, bf16* dX, const bf16* other, float* dot_out, int M, int N, int K, int S, int H,
                        cudaStream_t stream)
{
    NNB_ARG_CHECK(gemm_rowdot_supported(M, N, K, S, H), "shape not supported by the row-dot epilogue");
    NNB_ARG_CHECK(((reinterpret_cast<uintptr_t>(dY) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(dX) |
                    reinterpret_cast<uintptr_t>(other)) & 15) == 0 && dot_out, "operands must be 16-byte aligned");
    GemmParams p{};
    p.M = M; p.N = N; p.K = K;
    p.C = dX; p.ldc = N; p.c_bf16 = 1; p.accumulate = 0;
    p.alpha = 1.0f; p.vec_ok = 1; p.tma_store = 1;
    p.dot_out = dot_out; p.dot_S = S; p.dot_H = H;
    p.tiles_m = static_cast<int>(ceil_div(M, 256));
    p.tiles_n = static_cast<int>(ceil_div(N, 256));
    p.kb_total = static_cast<int>(ceil_div(K, BK));
    p.splits = 1;
    p.kb_per_split = p.kb_total;
    CUtensorMap ta, tb, tcm, tr;
    NNB_TRY(tensor_map_2d(dY, K, M, K, BK, BM, &ta, 2));
    NNB_TRY(tensor_map_2d(W, N, K, N, 64, BK, &tb, 2));
    NNB_TRY(tensor_map_2d(dX, N, M, N, 64, BM, &tcm, 2));
    NNB_TRY(tensor_map_2d(other, N, M, N, 64, BM, &tr, 2));
    return launch_gemm_pair<false, true, false, false, false, true>(ta, tb, tcm, tr, p, stream);
}

int gemm_pair_capacity() { return pair_capacity(); }

int gemm_profile_enable(int enable)
{
    g_prof.on = enable != 0;
    if (g_prof.on) { g_prof.used = 0; g_prof.flops[0] = g_prof.flops[1] = 0.0; g_prof.have_stream = false; }
    return 0;
}
int gemm_profile_read(int cls, double* total_ms, double* total_flops, int* launches)
{
    NNB_ARG_CHECK(cls == 0 || cls == 1, "class must be 0 or 1");
    double ms = 0.0;
    int n = 0;
    for (size_t i = 0; i + 1 < g_prof.used; i += 2) {
        if (g_prof.cls[i / 2] != cls) continue;
        NNB_CUDA_CHECK(cudaEventSynchronize(g_prof.events[i + 1]));
        float t = 0.f;
        NNB_CUDA_CHECK(cudaEventElapsedTime(&t, g_prof.events[i], g_prof.events[i + 1]));
        ms += t;
        ++n;
    }
    *total_ms = ms; *total_flops = g_prof.flops[cls]; *launches = n;
    return 0;
}

int gemm_device_error(int* code)
{
    NNB_CUDA_CHECK(cudaMemcpyFromSymbol(code, g_gemm_error, sizeof(int)));
    return 0;
}
int gemm_clear_device_error()
{
    const int z = 0;
    NNB_CUDA_CHECK(cudaMemcpyToSymbol(g_gemm_error, &z, sizeof(int)));
    return 0;
}

}  // namespace nnb
