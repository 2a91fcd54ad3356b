// Token / position embedding forward and its deterministic backward.
//
// Forward fuses what GPTModel::forward builds from transpose + gather_rows + transpose + add
// (compute_layer.hpp:2792-2809, 2535-2548): x[i] = token_emb[id_i] (+ pos_table[i % seq]); an
// out-of-range id gives a zero embedding row (cpu_engine.hpp:150-158).
//
// Backward is scatter_add_rows (compute_layer.hpp:2882-2891): dst[id_i] += g[i].  The CPU engine
// adds rows in ascending i (cpu_engine.hpp:203-214); atomics cannot reproduce that order, so the
// token positions are sorted by (id, i) and each destination row is accumulated by one block that
// walks its segment in ascending i — the fp32 result is bit-identical to the sequential loop.
#include "kernels.h"

namespace nnb {

template <typename T>
__global__ void embed_fwd_kernel(const float* __restrict__ tok_emb, const float* __restrict__ pos_table,
                                 const int* __restrict__ tokens, T* __restrict__ x, int n_tok, int seq, int d, int vocab)
{
    const int warps = (gridDim.x * blockDim.x) >> 5, lane = threadIdx.x & 31;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n_tok; i += warps) {
        const int id = tokens[i];
        const bool ok = id >= 0 && id < vocab;
        const float* e = tok_emb + static_cast<size_t>(ok ? id : 0) * d;
        const float* p = pos_table ? pos_table + static_cast<size_t>(i % seq) * d : nullptr;
        T* xr = x + static_cast<size_t>(i) * d;
        if ((d & 3) == 0) {
            for (int c = lane * 4; c < d; c += 128) {
                float4 v = ok ? *reinterpret_cast<const float4*>(e + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                if (p) { const float4 q = *reinterpret_cast<const float4*>(p + c); v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w; }
                xr[c] = from_f32<T>(v.x); xr[c + 1] = from_f32<T>(v.y); xr[c + 2] = from_f32<T>(v.z); xr[c + 3] = from_f32<T>(v.w);
            }
        } else {
            for (int c = lane; c < d; c += 32) xr[c] = from_f32<T>((ok ? e[c] : 0.f) + (p ? p[c] : 0.f));
        }
    }
}


// keys[i] = (id << 32 | i) for valid ids, ~0 for padding / out-of-range ids (ignored by scatter-add)
__global__ void make_keys_kernel(const int* __restrict__ tokens, unsigned long long* __restrict__ keys, int n_tok,
                                 int n_pad, int vocab)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pad) return;
    unsigned long long k = ~0ull;
    if (i < n_tok) { const int id = tokens[i]; if (id >= 0 && id < vocab) k = (static_cast<unsigned long long>(id) << 32) | static_cast<unsigned>(i); }
    keys[i] = k;
}

// one compare-exchange stage of a bitonic sorting network over n_pad (power of two) keys
__global__ void bitonic_stage_kernel(unsigned long long* __restrict__ keys, int n_pad, int k, int j)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pad) return;
    const int partner = i ^ j;
    if (partner > i) {
        const unsigned long long a = keys[i], b = keys[partner];
        const bool up = (i & k) == 0;
        if ((a > b) == up) { keys[i] = b; keys[partner] = a; }
    }
}
// all stages with j < 1024 for one k, inside shared memory (2048 keys per block)
__global__ void __launch_bounds__(1024) bitonic_local_kernel(unsigned long long* __restrict__ keys, int n_pad, int k_begin, int k_end)
{
    __shared__ unsigned long long s[2048];
    const int base = blockIdx.x * 2048;
    for (int t = threadIdx.x; t < 2048; t += 1024) s[t] = (base + t < n_pad) ? keys[base + t] : ~0ull;
    __syncthreads();
    for (int k = k_begin; k <= k_end; k <<= 1) {
        for (int j = min(k >> 1, 1024); j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < 2048; t += 1024) {
                const int partner = t ^ j;
                if (partner > t) {
                    const unsigned long long a = s[t], b = s[partner];
                    const bool up = ((base + t) & k) == 0;
                    if ((a > b) == up) { s[t] = b; s[partner] = a; }
                }
            }
            __syncthreads();
        }
    }
    for (int t = threadIdx.x; t < 2048; t += 1024) if (base + t < n_pad) keys[base + t] = s[t];
}

// segment heads: seg_start[s] = first sorted position of the s-th distinct id; count in n_seg[0]
__global__ void segment_heads_kernel(const unsigned long long* __restrict__ keys, int n_pad, int* __restrict__ flags)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pad) return;
    const unsigned long long k = keys[i];
    const bool valid = k != ~0ull;
    flags[i] = (valid && (i == 0 || (keys[i - 1] >> 32) != (k >> 32))) ? 1 : 0;
}

// Work item = (segment head, 128-column slice): a block adds the rows of one token id, in ascending
// position order, into 128 columns of its destination row.  Threads own columns, so every thread
// performs the same sequential fp32 sum as the CPU loop; the segment's positions are staged through
// shared memory and the row loads of 32 positions are issued together, ahead of the ordered adds.
// Long segments (frequent tokens) are spread over d/128 blocks instead of serialising one block.
template <typename T>
__global__ void __launch_bounds__(128)
scatter_segments_kernel(float* __restrict__ dst, const unsigned long long* __restrict__ keys, const int* __restrict__ flags,
                        const T* __restrict__ g, int n_pad, int d)
{
    __shared__ unsigned spos[256];
    const int nchunk = (d + 127) / 128;
    const long long work_total = static_cast<long long>(n_pad) * nchunk;
    for (long long w = blockIdx.x; w < work_total; w += gridDim.x) {
        const int h = static_cast<int>(w / nchunk), cc = static_cast<int>(w % nchunk);
        if (!flags[h]) continue;                                   // block-uniform
        const unsigned id = static_cast<unsigned>(keys[h] >> 32);
        const int c = cc * 128 + threadIdx.x;
        const bool col_ok = c < d;
        float acc = col_ok ? dst[static_cast<size_t>(id) * d + c] : 0.f;
        for (int base = h;; base += 256) {
            __syncthreads();
            for (int t = threadIdx.x; t < 256; t += 128) {
                const int pidx = base + t;
                unsigned v = 0xffffffffu;
                if (pidx < n_pad) { const unsigned long long k = keys[pidx]; if (k != ~0ull && static_cast<unsigned>(k >> 32) == id) v = static_cast<unsigned>(k); }
                spos[t] = v;
            }
            __syncthreads();
            if (col_ok) {
                for (int t = 0; t < 256; t += 32) {
                    if (spos[t] == 0xffffffffu) break;
                    float v[32];
#pragma unroll
                    for (int k = 0; k < 32; ++k) {
                        const unsigned pz = spos[t + k];
                        v[k] = (pz != 0xffffffffu) ? to_f32(g[static_cast<size_t>(pz) * d + c]) : 0.f;
                    }
#pragma unroll
                    for (int k = 0; k < 32; ++k) if (spos[t + k] != 0xffffffffu) acc += v[k];
                }
            }
            if (spos[255] == 0xffffffffu) break;                    // segment ended inside this batch (block-uniform)
        }
        if (col_ok) dst[static_cast<size_t>(id) * d + c] = acc;
    }
}

// learned position gradient: pos_grad[t] += g[b*seq + t] for b ascending (scatter_add_rows with the
// cached position indices, compute_layer.hpp:2573-2580)
template <typename T>
__global__ void pos_bwd_kernel(float* __restrict__ pos_grad, const T* __restrict__ g, int batch, int seq, int d)
{
    const size_t n = static_cast<size_t>(seq) * d;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float acc = pos_grad[i];
        for (int b = 0; b < batch; ++b) acc += to_f32(g[static_cast<size_t>(b) * n + i]);
        pos_grad[i] = acc;
    }
}

static int next_pow2(int n) { int p = 1; while (p < n) p <<= 1; return p; }

size_t embed_bwd_scratch_bytes(int n_tok)
{
    const size_t n_pad = static_cast<size_t>(next_pow2(n_tok < 2048 ? 2048 : n_tok));
    return n_pad * sizeof(unsigned long long) + n_pad * sizeof(int);
}

template <typename T>
int embed_fwd(const float* tok_emb, const float* pos_table, const int* tokens, T* x, int n_tok, int seq, int d, int vocab,
              cudaStream_t s)
{
    if (n_tok == 0) return 0;
    embed_fwd_kernel<T><<<grid_for(n_tok, 8), 256, 0, s>>>(tok_emb, pos_table, tokens, x, n_tok, seq, d, vocab);
    NNB_LAUNCH_CHECK();
    return 0;
}


template <typename T>
int embed_bwd(float* tok_grad, float* pos_grad, const int* tokens, const T* g, void* scratch, int batch, int seq, int d,
              int vocab, cudaStream_t s)
{
    const int n_tok = batch * seq;
    if (n_tok == 0) return 0;
    const int n_pad = next_pow2(n_tok < 2048 ? 2048 : n_tok);
    auto* keys = static_cast<unsigned long long*>(scratch);
    int* flags = reinterpret_cast<int*>(keys + n_pad);
    const unsigned blocks = static_cast<unsigned>(ceil_div(n_pad, 256));
    make_keys_kernel<<<blocks, 256, 0, s>>>(tokens, keys, n_tok, n_pad, vocab);
    NNB_LAUNCH_CHECK();
    // bitonic network: k = 2..2048 entirely in shared memory, then global stages for j >= 2048 and
    // a shared-memory tail for j < 2048 of each larger k
    bitonic_local_kernel<<<n_pad / 2048, 1024, 0, s>>>(keys, n_pad, 2, 2048);
    NNB_LAUNCH_CHECK();
    for (int k = 4096; k <= n_pad; k <<= 1) {
        for (int j = k >> 1; j >= 2048; j >>= 1) {
            bitonic_stage_kernel<<<blocks, 256, 0, s>>>(keys, n_pad, k, j);
            NNB_LAUNCH_CHECK();
        }
        bitonic_local_kernel<<<n_pad / 2048, 1024, 0, s>>>(keys, n_pad, k, k);
        NNB_LAUNCH_CHECK();
    }
    segment_heads_kernel<<<blocks, 256, 0, s>>>(keys, n_pad, flags);
    NNB_LAUNCH_CHECK();
    scatter_segments_kernel<T><<<kSmCount * 16, 128, 0, s>>>(tok_grad, keys, flags, g, n_pad, d);
    NNB_LAUNCH_CHECK();
    if (pos_grad) {
        pos_bwd_kernel<T><<<grid_for(static_cast<long long>(seq) * d, 256), 256, 0, s>>>(pos_grad, g, batch, seq, d);
        NNB_LAUNCH_CHECK();
    }
    return 0;
}

template int embed_fwd<float>(const float*, const float*, const int*, float*, int, int, int, int, cudaStream_t);
template int embed_fwd<bf16>(const float*, const float*, const int*, bf16*, int, int, int, int, cudaStream_t);
template int embed_bwd<float>(float*, float*, const int*, const float*, void*, int, int, int, int, cudaStream_t);
template int embed_bwd<bf16>(float*, float*, const int*, const bf16*, void*, int, int, int, int, cudaStream_t);

}  // namespace nnb
