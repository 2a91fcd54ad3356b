// Incremental inference with a key/value cache: one token per call through every block of the model.
// Follows GPTModel::forward_step / GPTBlock::forward_step / AttentionBase::forward_step of the reference
// (compute_layer.hpp:2906-2950, 1426-1511; ALiBi bias of a step :2267-2290; rotary encoding of a step :964-988), which
// issues about thirty engine primitives, four transposes of the whole cache and two host-built matrices per block and
// token; here a block is five launches (six with rotary positions) and nothing of the cache is copied.
// A single token is all matrix-vector work, bound by reading the weights once: the kernels are warp-per-output-row
// products with 16-byte loads over bf16 weights (the shadow copy, in bf16 mode) or the fp32 master weights (check mode),
// fp32 activations and an fp32 cache in both modes.  The normalisation before a projection and the activation before
// fc2 are applied while the input vector is staged in shared memory (every block does it for itself: the vector is a
// few KB), the attention over the cache is split over chunks of 32 cached rows per head, and the token id, position
// and cache length are read from device memory, so that the launches of a token are the same every time and a caller
// may replay them as a CUDA graph (nnb200_gpt_forward_step_dev).
#include <cmath>
#include <vector>

#include "kernels.h"
#include "nnb200.h"

namespace nnb {

struct DecodeWs { size_t kv, table, x, xn, qkv, att, xmid, h1, h2, logits, step, part, count, total; };
constexpr int kDecodeChunk = 32;                    // cached rows per attention block: a block is one round of loads, bound by their latency
static DecodeWs decode_ws(const nnb200_gpt_config& c)
{
    DecodeWs W;
    const size_t d = c.d_model, S = c.seq, fc1 = c.act == 1 ? 2 * static_cast<size_t>(c.d_ff) : c.d_ff;
    size_t off = 0;
    auto take = [&](size_t floats) { const size_t o = off; off = (off + floats * 4 + 255) / 256 * 256; return o; };
    W.kv = take(static_cast<size_t>(c.layers) * 2 * S * d);
    W.table = take(S * d);
    W.x = take(d); W.xn = take(d); W.qkv = take(3 * d); W.att = take(d); W.xmid = take(d);
    W.h1 = take(fc1); W.h2 = take(c.d_ff); W.logits = take(c.vocab);
    const size_t chunks = (S + kDecodeChunk - 1) / kDecodeChunk;
    W.step = take(4);                                            // token id, position, cache length
    W.part = take(static_cast<size_t>(c.heads) * chunks * (d / c.heads + 2));   // per (head, chunk): maximum, sum, weighted values
    W.count = take(static_cast<size_t>(c.heads));               // chunks of a head that have finished (back to zero after each step)
    W.total = off;
    return W;
}

__global__ void decode_set_step_kernel(int* __restrict__ step, int token, int pos, int cur_len)
{
    step[0] = token; step[1] = pos; step[2] = cur_len;
}

// x = token embedding (+ position row); pos_table: learned or sinusoidal rows, or null
__global__ void decode_embed_kernel(const float* __restrict__ tok_emb, const float* __restrict__ pos_table, const int* __restrict__ step,
                                    int vocab, float* __restrict__ x, int d)
{
    const int id = step[0], pos = step[1];
    const bool ok = id >= 0 && id < vocab;                      // an id out of range looks up a zero row (cpu_engine.hpp:150-158)
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < d; c += gridDim.x * blockDim.x)
        x[c] = (ok ? tok_emb[static_cast<size_t>(id) * d + c] : 0.f) + (pos_table ? pos_table[static_cast<size_t>(pos) * d + c] : 0.f);
}

// y[o] = W[o, :] . f(x) + bias[o] (+ residual[o]); one warp per output row, 16-byte loads along the row.  The input
// vector is staged in shared memory by every block, and f is applied on the way:
//   PRE 0: f = identity;
//   PRE 1: f = norm(x) * gamma (+ beta), eps 1e-5 inside the rsqrt (compute_layer.hpp:495, 687; LayerNorm when `layer`);
//   PRE 2: x holds fc1's output: f = SwiGLU (gate * sigmoid(gate) * up, `in` values out of 2 * in; compute_layer.hpp:
//          375-404) or QuickGeLU (:266-295) when `layer` is 0 / 1.
template <typename WT, int PRE>
__global__ void __launch_bounds__(256) gemv_kernel(const WT* __restrict__ W, const float* __restrict__ x, const float* __restrict__ gamma,
                                                   const float* __restrict__ beta, int layer, const float* __restrict__ bias,
                                                   const float* __restrict__ residual, float* __restrict__ y, int out, int in)
{
    constexpr int VN = Vec16<WT>::N;
    extern __shared__ float xs[];                               // `in` floats
    __shared__ float red[32];
    if (PRE == 1) {
        float mean = 0.f;
        for (int c = threadIdx.x; c < in; c += blockDim.x) xs[c] = x[c];          // one trip to global memory, the passes read the copy
        __syncthreads();
        if (layer) {
            float sacc = 0.f;
            for (int c = threadIdx.x; c < in; c += blockDim.x) sacc += xs[c];
            mean = block_sum(sacc, red) / static_cast<float>(in);
            __syncthreads();
        }
        float q = 0.f;
        for (int c = threadIdx.x; c < in; c += blockDim.x) { const float v = xs[c] - mean; q += v * v; }
        const float rinv = rsqrtf(block_sum(q, red) / static_cast<float>(in) + 1e-5f);
        for (int c = threadIdx.x; c < in; c += blockDim.x) xs[c] = (xs[c] - mean) * rinv * gamma[c] + (beta ? beta[c] : 0.f);
    } else if (PRE == 2) {
        for (int c = threadIdx.x; c < in; c += blockDim.x) {
            if (layer == 0) { const float g = x[c]; xs[c] = g / (1.0f + expf(-g)) * x[in + c]; }
            else { const float v = x[c]; xs[c] = v / (1.0f + expf(-1.702f * v)); }
        }
    } else {
        for (int c = threadIdx.x; c < in; c += blockDim.x) xs[c] = x[c];
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warps = (gridDim.x * blockDim.x) >> 5;
    for (int o = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; o < out; o += warps) {
        const WT* w = W + static_cast<size_t>(o) * in;
        float acc = 0.f;
        if ((in % VN) == 0) {
            for (int c = lane * VN; c < in; c += 32 * VN) {
                const Vec16<WT> v = ld16(w + c);
#pragma unroll
                for (int k = 0; k < VN; ++k) acc = fmaf(to_f32(v.v[k]), xs[c + k], acc);
            }
        } else {
            for (int c = lane; c < in; c += 32) acc = fmaf(to_f32(w[c]), xs[c], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) y[o] = acc + (bias ? bias[o] : 0.f) + (residual ? residual[o] : 0.f);
    }
}

// Rotary encoding of the Q and K thirds of one token's qkv vector at position `pos` (table: cos (seq, dk/2) then sin)
__global__ void decode_rope_kernel(float* __restrict__ qkv, const float* __restrict__ table, const int* __restrict__ step, int seq, int heads,
                                   int dk)
{
    const int pos = step[2];                                    // the rotation of a step is by the cache row it lands in
    const int half = dk / 2, n = 2 * heads * half;
    for (int w = blockIdx.x * blockDim.x + threadIdx.x; w < n; w += gridDim.x * blockDim.x) {
        const int j = w % half, h = (w / half) % heads, which = w / (half * heads);
        float* lo = qkv + which * heads * dk + h * dk + j;
        const float c = table[static_cast<size_t>(pos) * half + j], sn = table[static_cast<size_t>(seq) * half + static_cast<size_t>(pos) * half + j];
        const float a = lo[0], b = lo[half];
        lo[0] = a * c - b * sn;
        lo[half] = b * c + a * sn;
    }
}

// Attention of one token over the cache, split over chunks of kDecodeChunk cached rows: block (head, chunk).  The block
// of chunk cur_len / kDecodeChunk appends this token's key and value to the cache (row cur_len) first.  Every block
// computes the scores of its rows (q_h . k_j / sqrt(dk) - slope_h (cur_len - j)), their maximum, the sum of the
// exponentials against it and the weighted values, and leaves them as a partial; the block of a head that finishes last
// merges the head's partials in chunk order (the same order whatever the finishing order) and writes out_h.
// Chunks beyond the cache length leave at once: the grid is the same for every cache length.
__global__ void __launch_bounds__(128) decode_attn_kernel(const float* __restrict__ qkv, float* __restrict__ kc, float* __restrict__ vc,
                                                          float* __restrict__ out, const int* __restrict__ step, float* __restrict__ part,
                                                          int* __restrict__ count, int d, int dk, int heads, int alibi, float scale)
{
    __shared__ float sc[kDecodeChunk];
    __shared__ float red[32];
    __shared__ float qs[256];
    __shared__ float ov[2][256];
    __shared__ int last;
    const int h = blockIdx.x, chunk = blockIdx.y, nchunks_max = gridDim.y;
    const int cur_len = step[2], n = cur_len + 1;
    const int j0 = chunk * kDecodeChunk;
    if (j0 >= n) return;
    const int nchunks = (n + kDecodeChunk - 1) / kDecodeChunk;
    const int rows = min(kDecodeChunk, n - j0);
    for (int c = threadIdx.x; c < dk; c += blockDim.x) qs[c] = qkv[h * dk + c];
    if (cur_len >= j0 && cur_len < j0 + kDecodeChunk)
        for (int c = threadIdx.x; c < dk; c += blockDim.x) {
            kc[static_cast<size_t>(cur_len) * d + h * dk + c] = qkv[d + h * dk + c];
            vc[static_cast<size_t>(cur_len) * d + h * dk + c] = qkv[2 * d + h * dk + c];
        }
    __syncthreads();
    const float slope = alibi ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(heads)) : 0.f;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float mx = -INFINITY;
#pragma unroll 8
    for (int r = warp; r < rows; r += nwarps) {
        const int j = j0 + r;
        const float* kr = kc + static_cast<size_t>(j) * d + h * dk;
        float acc = 0.f;
        for (int c = lane; c < dk; c += 32) acc = fmaf(qs[c], kr[c], acc);
        acc = warp_sum(acc) * scale - slope * static_cast<float>(cur_len - j);
        if (lane == 0) sc[r] = acc;
        mx = fmaxf(mx, acc);
    }
    mx = block_max(mx, red);
    __syncthreads();
    float den = 0.f;
    for (int r = threadIdx.x; r < rows; r += blockDim.x) { const float e = expf(sc[r] - mx); sc[r] = e; den += e; }
    den = block_sum(den, red);
    __syncthreads();
    // weighted values: thread (column, half of the rows); head sizes up to 256 with 128 threads need one or more rounds
    float* my = part + (static_cast<size_t>(h) * nchunks_max + chunk) * (dk + 2);
    for (int c0 = 0; c0 < dk; c0 += 64) {
        const int c = c0 + (threadIdx.x & 63), half = threadIdx.x >> 6;
        float acc = 0.f;
        if (c < dk) {
#pragma unroll 8
            for (int r = half; r < rows; r += 2) acc = fmaf(sc[r], vc[static_cast<size_t>(j0 + r) * d + h * dk + c], acc);
        }
        ov[half][c0 + (threadIdx.x & 63)] = acc;
        __syncthreads();
        if (half == 0 && c < dk) my[2 + c] = ov[0][c] + ov[1][c];
        __syncthreads();
    }
    if (threadIdx.x == 0) { my[0] = mx; my[1] = den; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = (atomicAdd(count + h, 1) == nchunks - 1);
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x == 0) count[h] = 0;
    const float* hp = part + static_cast<size_t>(h) * nchunks_max * (dk + 2);
    float gm = -INFINITY;
    for (int k = 0; k < nchunks; ++k) gm = fmaxf(gm, __ldcg(hp + static_cast<size_t>(k) * (dk + 2)));
    float gden = 0.f;
    for (int k = 0; k < nchunks; ++k) gden += __ldcg(hp + static_cast<size_t>(k) * (dk + 2) + 1) * expf(__ldcg(hp + static_cast<size_t>(k) * (dk + 2)) - gm);
    const float inv = 1.0f / gden;
    for (int c = threadIdx.x; c < dk; c += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < nchunks; ++k)
            acc = fmaf(__ldcg(hp + static_cast<size_t>(k) * (dk + 2) + 2 + c), expf(__ldcg(hp + static_cast<size_t>(k) * (dk + 2)) - gm), acc);
        out[h * dk + c] = acc * inv;
    }
}

template <typename WT, int PRE>
static int gemv(const WT* W, const float* x, const float* gamma, const float* beta, int layer, const float* bias, const float* residual,
                float* y, int out, int in, cudaStream_t s)
{
    NNB_ARG_CHECK(static_cast<size_t>(in) * sizeof(float) <= 48 * 1024, "input vector too long for the decode matrix-vector kernel");
    gemv_kernel<WT, PRE><<<grid_for(static_cast<long long>(out) * 32, 256), 256, static_cast<size_t>(in) * sizeof(float), s>>>(
        W, x, gamma, beta, layer, bias, residual, y, out, in);
    NNB_LAUNCH_CHECK();
    return 0;
}

// `step` (device): token id, position, cache length
template <typename WT>
static int forward_step_t(const nnb200_gpt_config& c, const float* P, const WT* Wt, uint8_t* ws, const int* step, float* logits_out,
                          cudaStream_t s)
{
    const DecodeLayout L = decode_layout(c);
    const DecodeWs W = decode_ws(c);
    const int d = c.d_model, ff = c.d_ff, fc1 = c.act == 1 ? 2 * ff : ff, dk = d / c.heads;
    const int ln = c.norm == 0 ? 1 : 0;
    NNB_ARG_CHECK(dk <= 256, "head size above 256");
    auto F = [&](size_t off) { return reinterpret_cast<float*>(ws + off); };
    auto PB = [&](long long off) { return off >= 0 ? P + off : nullptr; };
    const float* pos_table = nullptr;
    if (c.pos == 0) pos_table = P + L.pos_emb;
    else if (c.pos == 1) pos_table = F(W.table);
    decode_embed_kernel<<<grid_for(d, 256), 256, 0, s>>>(P + L.tok_emb, pos_table, step, c.vocab, F(W.x), d);
    NNB_LAUNCH_CHECK();
    const size_t layer_kv = static_cast<size_t>(2) * c.seq * d;
    const dim3 attn_grid(static_cast<unsigned>(c.heads), static_cast<unsigned>((c.seq + kDecodeChunk - 1) / kDecodeChunk));
    float* x = F(W.x);
    float* xmid = F(W.xmid);
    for (int l = 0; l < c.layers; ++l) {
        const DecodeLayer& lp = L.layers[l];
        float* kc = F(W.kv) + static_cast<size_t>(l) * layer_kv;
        float* vc = kc + static_cast<size_t>(c.seq) * d;
        NNB_TRY((gemv<WT, 1>(Wt + lp.wqkv, x, P + lp.g1, PB(lp.be1), ln, P + lp.bqkv, nullptr, F(W.qkv), 3 * d, d, s)));
        if (c.pos == 3) {
            decode_rope_kernel<<<grid_for(static_cast<long long>(c.heads) * dk, 256), 256, 0, s>>>(F(W.qkv), F(W.table), step, c.seq, c.heads, dk);
            NNB_LAUNCH_CHECK();
        }
        decode_attn_kernel<<<attn_grid, 128, 0, s>>>(F(W.qkv), kc, vc, F(W.att), step, F(W.part), reinterpret_cast<int*>(F(W.count)), d, dk,
                                                     c.heads, c.pos == 2 ? 1 : 0, 1.0f / sqrtf(static_cast<float>(dk)));
        NNB_LAUNCH_CHECK();
        NNB_TRY((gemv<WT, 0>(Wt + lp.wo, F(W.att), nullptr, nullptr, 0, P + lp.bo, x, xmid, d, d, s)));          // + residual (GPTBlock::forward_step)
        NNB_TRY((gemv<WT, 1>(Wt + lp.w1, xmid, P + lp.g2, PB(lp.be2), ln, P + lp.b1, nullptr, F(W.h1), fc1, d, s)));
        NNB_TRY((gemv<WT, 2>(Wt + lp.w2, F(W.h1), nullptr, nullptr, c.act == 1 ? 0 : 1, P + lp.b2, xmid, x, d, ff, s)));   // + residual
    }
    return gemv<WT, 1>(Wt + L.lm_w, x, P + L.lnf_g, PB(L.lnf_b), ln, P + L.lm_b, nullptr, logits_out ? logits_out : F(W.logits), c.vocab, d, s);
}

}  // namespace nnb

using namespace nnb;

extern "C" {

long long nnb200_gpt_decode_workspace_bytes(const nnb200_gpt_config* cfg)
{
    if (nnb200_gpt_arena_elems(cfg) < 0) return -1;             // validates the configuration
    return static_cast<long long>(decode_ws(*cfg).total);
}

int nnb200_gpt_decode_init(const nnb200_gpt_config* cfg, void* workspace, void* stream)
{
    if (nnb200_gpt_arena_elems(cfg) < 0 || !workspace) { fprintf(stderr, "nnb200_gpt_decode_init: bad arguments\n"); return -1; }
    const DecodeWs W = decode_ws(*cfg);
    const int S = cfg->seq, d = cfg->d_model;
    std::vector<float> tab;
    if (cfg->pos == 3) {
        tab.resize(static_cast<size_t>(S) * (d / cfg->heads));
        rope_table_host(S, d / cfg->heads, tab.data());
    } else if (cfg->pos == 1) {
        // SinusoidalPositionEncoder (compute_layer.hpp:2604-2622), with the reference's float calls
        tab.resize(static_cast<size_t>(S) * d);
        for (int pos = 0; pos < S; ++pos)
            for (int i = 0; i < d; ++i) {
                const float angle = static_cast<float>(pos) / std::pow(10000.0f, static_cast<float>(2 * (i / 2)) / static_cast<float>(d));
                tab[static_cast<size_t>(pos) * d + i] = (i % 2 == 0) ? std::sin(angle) : std::cos(angle);
            }
    }
    NNB_CUDA_CHECK(cudaMemsetAsync(static_cast<uint8_t*>(workspace) + W.count, 0, static_cast<size_t>(cfg->heads) * sizeof(int), to_stream(stream)));
    if (!tab.empty()) {
        NNB_CUDA_CHECK(cudaMemcpyAsync(static_cast<uint8_t*>(workspace) + W.table, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, to_stream(stream)));
        NNB_CUDA_CHECK(cudaStreamSynchronize(to_stream(stream)));          // `tab` is pageable host memory about to go away
    }
    return 0;
}

static int forward_step_any(const nnb200_gpt_config* cfg, const float* params, const void* params_bf16, uint8_t* ws, const int* step,
                            float* logits_out, cudaStream_t s)
{
    if (cfg->precision == 1) {
        NNB_ARG_CHECK(params_bf16 != nullptr, "bf16 mode needs the bf16 parameter shadow");
        return forward_step_t<bf16>(*cfg, params, static_cast<const bf16*>(params_bf16), ws, step, logits_out, s);
    }
    return forward_step_t<float>(*cfg, params, params, ws, step, logits_out, s);
}

int nnb200_gpt_forward_step(const nnb200_gpt_config* cfg, const float* params, const void* params_bf16, void* workspace, int token_id,
                            int pos, int cur_len, float* logits_out, void* stream)
{
    if (nnb200_gpt_arena_elems(cfg) < 0 || !params || !workspace) { fprintf(stderr, "nnb200_gpt_forward_step: bad arguments\n"); return -1; }
    NNB_ARG_CHECK(cur_len >= 0 && cur_len < cfg->seq, "the cache holds seq rows: cur_len must be in [0, seq)");
    NNB_ARG_CHECK(pos >= 0 && pos < cfg->seq, "position out of range");
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int* step = reinterpret_cast<int*>(ws + decode_ws(*cfg).step);
    decode_set_step_kernel<<<1, 1, 0, to_stream(stream)>>>(step, token_id, pos, cur_len);
    NNB_LAUNCH_CHECK();
    return forward_step_any(cfg, params, params_bf16, ws, step, logits_out, to_stream(stream));
}

int nnb200_gpt_decode_set_step(int32_t* step_dev, int token_id, int pos, int cur_len, void* stream)
{
    NNB_ARG_CHECK(step_dev != nullptr, "null step buffer");
    decode_set_step_kernel<<<1, 1, 0, to_stream(stream)>>>(step_dev, token_id, pos, cur_len);
    NNB_LAUNCH_CHECK();
    return 0;
}

int nnb200_gpt_forward_step_dev(const nnb200_gpt_config* cfg, const float* params, const void* params_bf16, void* workspace,
                                const int32_t* step_dev, float* logits_out, void* stream)
{
    if (nnb200_gpt_arena_elems(cfg) < 0 || !params || !workspace || !step_dev) { fprintf(stderr, "nnb200_gpt_forward_step_dev: bad arguments\n"); return -1; }
    return forward_step_any(cfg, params, params_bf16, static_cast<uint8_t*>(workspace), step_dev, logits_out, to_stream(stream));
}

}  // extern "C"
