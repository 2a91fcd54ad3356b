// Incremental inference with a key/value cache: one token per call through every block of the model.
// Follows GPTModel::forward_step / GPTBlock::forward_step / AttentionBase::forward_step of the reference
// (compute_layer.hpp:2906-2950, 1426-1511; ALiBi bias of a step :2267-2290; rotary encoding of a step :964-988), which
// issues about thirty engine primitives, four transposes of the whole cache and two host-built matrices per block and
// token; here a block is eight launches and nothing of the cache is copied.
// A single token is all matrix-vector work, bound by reading the weights once: the kernels are warp-per-output-row
// products with 16-byte loads over bf16 weights (the shadow copy, in bf16 mode) or the fp32 master weights (check mode),
// fp32 activations and an fp32 cache in both modes.
#include <cmath>
#include <vector>

#include "kernels.h"
#include "nnb200.h"

namespace nnb {

struct DecodeWs { size_t kv, table, x, xn, qkv, att, xmid, h1, h2, logits, total; };
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
    W.total = off;
    return W;
}

__global__ void decode_embed_kernel(const float* __restrict__ tok_emb, const float* __restrict__ pos_row, int id, int vocab,
                                    float* __restrict__ x, int d)
{
    const bool ok = id >= 0 && id < vocab;                      // an id out of range looks up a zero row (cpu_engine.hpp:150-158)
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < d; c += gridDim.x * blockDim.x)
        x[c] = (ok ? tok_emb[static_cast<size_t>(id) * d + c] : 0.f) + (pos_row ? pos_row[c] : 0.f);
}

// y = norm(x) * gamma (+ beta) of one vector; eps 1e-5 inside the rsqrt (compute_layer.hpp:495, 687); one block
__global__ void __launch_bounds__(256) decode_norm_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                          const float* __restrict__ beta, float* __restrict__ y, int d, int layer)
{
    __shared__ float red[32];
    float s = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) s += x[c];
    const float mean = layer ? block_sum(s, red) / static_cast<float>(d) : 0.f;
    float q = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) { const float v = x[c] - mean; q += v * v; }
    const float rinv = rsqrtf(block_sum(q, red) / static_cast<float>(d) + 1e-5f);
    for (int c = threadIdx.x; c < d; c += blockDim.x) y[c] = (x[c] - mean) * rinv * gamma[c] + (beta ? beta[c] : 0.f);
}

// y[o] = W[o, :] . x + bias[o] (+ residual[o]); one warp per output row, 16-byte loads along the row
template <typename WT>
__global__ void __launch_bounds__(256) gemv_kernel(const WT* __restrict__ W, const float* __restrict__ x, const float* __restrict__ bias,
                                                   const float* __restrict__ residual, float* __restrict__ y, int out, int in)
{
    constexpr int VN = Vec16<WT>::N;
    const int lane = threadIdx.x & 31, warps = (gridDim.x * blockDim.x) >> 5;
    for (int o = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; o < out; o += warps) {
        const WT* w = W + static_cast<size_t>(o) * in;
        float acc = 0.f;
        if ((in % VN) == 0) {
            for (int c = lane * VN; c < in; c += 32 * VN) {
                const Vec16<WT> v = ld16(w + c);
#pragma unroll
                for (int k = 0; k < VN; ++k) acc = fmaf(to_f32(v.v[k]), x[c + k], acc);
            }
        } else {
            for (int c = lane; c < in; c += 32) acc = fmaf(to_f32(w[c]), x[c], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) y[o] = acc + (bias ? bias[o] : 0.f) + (residual ? residual[o] : 0.f);
    }
}

// Rotary encoding of the Q and K thirds of one token's qkv vector at position `pos` (table: cos (seq, dk/2) then sin)
__global__ void decode_rope_kernel(float* __restrict__ qkv, const float* __restrict__ table, int pos, int seq, int heads, int dk)
{
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

// One head per block.  Appends this token's key and value to the cache (row cur_len), then
// out_h = softmax(q_h . K_h^T / sqrt(dk) - slope_h (cur_len - j)) V_h over the rows [0, cur_len] of the cache.
// A warp per key for the scores (lanes along the head: coalesced), a thread per head column for the output.
__global__ void __launch_bounds__(256) decode_attn_kernel(const float* __restrict__ qkv, float* __restrict__ kc, float* __restrict__ vc,
                                                          float* __restrict__ out, int cur_len, int d, int dk, int heads, int alibi, float scale)
{
    extern __shared__ float sc[];                               // cur_len + 1 scores, then 32 floats for the reductions
    const int h = blockIdx.x, n = cur_len + 1;
    float* red = sc + n;
    const float* q = qkv + h * dk;
    for (int c = threadIdx.x; c < dk; c += blockDim.x) {
        kc[static_cast<size_t>(cur_len) * d + h * dk + c] = qkv[d + h * dk + c];
        vc[static_cast<size_t>(cur_len) * d + h * dk + c] = qkv[2 * d + h * dk + c];
    }
    __syncthreads();
    const float slope = alibi ? exp2f(-8.0f * static_cast<float>(h) / static_cast<float>(heads)) : 0.f;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float mx = -INFINITY;
    for (int j = warp; j < n; j += nwarps) {
        const float* kr = kc + static_cast<size_t>(j) * d + h * dk;
        float acc = 0.f;
        for (int c = lane; c < dk; c += 32) acc = fmaf(q[c], kr[c], acc);
        acc = warp_sum(acc) * scale - slope * static_cast<float>(cur_len - j);
        if (lane == 0) sc[j] = acc;
        mx = fmaxf(mx, acc);
    }
    mx = block_max(mx, red);
    __syncthreads();
    float den = 0.f;
    for (int j = threadIdx.x; j < n; j += blockDim.x) { const float e = expf(sc[j] - mx); sc[j] = e; den += e; }
    den = block_sum(den, red);
    __syncthreads();
    const float inv = 1.0f / den;
    for (int c = threadIdx.x; c < dk; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < n; ++j) acc = fmaf(sc[j], vc[static_cast<size_t>(j) * d + h * dk + c], acc);
        out[h * dk + c] = acc * inv;
    }
}

__global__ void decode_act_kernel(const float* __restrict__ h1, float* __restrict__ h2, int ff, int swiglu)
{
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < ff; c += gridDim.x * blockDim.x) {
        if (swiglu) { const float g = h1[c]; h2[c] = g / (1.0f + expf(-g)) * h1[ff + c]; }          // compute_layer.hpp:375-404
        else { const float v = h1[c]; h2[c] = v / (1.0f + expf(-1.702f * v)); }                    // QuickGeLU, :266-295
    }
}

template <typename WT>
static int gemv(const WT* W, const float* x, const float* bias, const float* residual, float* y, int out, int in, cudaStream_t s)
{
    gemv_kernel<WT><<<grid_for(static_cast<long long>(out) * 32, 256), 256, 0, s>>>(W, x, bias, residual, y, out, in);
    NNB_LAUNCH_CHECK();
    return 0;
}

template <typename WT>
static int forward_step_t(const nnb200_gpt_config& c, const float* P, const WT* Wt, uint8_t* ws, int token, int pos, int cur_len,
                          float* logits_out, cudaStream_t s)
{
    const DecodeLayout L = decode_layout(c);
    const DecodeWs W = decode_ws(c);
    const int d = c.d_model, ff = c.d_ff, fc1 = c.act == 1 ? 2 * ff : ff, dk = d / c.heads;
    const bool ln = c.norm == 0;
    auto F = [&](size_t off) { return reinterpret_cast<float*>(ws + off); };
    auto PB = [&](long long off) { return off >= 0 ? P + off : nullptr; };
    const float* pos_row = nullptr;
    if (c.pos == 0) pos_row = P + L.pos_emb + static_cast<size_t>(pos) * d;
    else if (c.pos == 1) pos_row = F(W.table) + static_cast<size_t>(pos) * d;
    decode_embed_kernel<<<grid_for(d, 256), 256, 0, s>>>(P + L.tok_emb, pos_row, token, c.vocab, F(W.x), d);
    NNB_LAUNCH_CHECK();
    const size_t layer_kv = static_cast<size_t>(2) * c.seq * d;
    float* x = F(W.x);
    float* xmid = F(W.xmid);
    for (int l = 0; l < c.layers; ++l) {
        const DecodeLayer& lp = L.layers[l];
        float* kc = F(W.kv) + static_cast<size_t>(l) * layer_kv;
        float* vc = kc + static_cast<size_t>(c.seq) * d;
        decode_norm_kernel<<<1, 256, 0, s>>>(x, P + lp.g1, PB(lp.be1), F(W.xn), d, ln ? 1 : 0);
        NNB_LAUNCH_CHECK();
        NNB_TRY(gemv<WT>(Wt + lp.wqkv, F(W.xn), P + lp.bqkv, nullptr, F(W.qkv), 3 * d, d, s));
        if (c.pos == 3) {
            decode_rope_kernel<<<grid_for(static_cast<long long>(c.heads) * dk, 256), 256, 0, s>>>(F(W.qkv), F(W.table), cur_len, c.seq, c.heads, dk);
            NNB_LAUNCH_CHECK();
        }
        decode_attn_kernel<<<c.heads, 256, (static_cast<size_t>(cur_len) + 1 + 32) * sizeof(float), s>>>(
            F(W.qkv), kc, vc, F(W.att), cur_len, d, dk, c.heads, c.pos == 2 ? 1 : 0, 1.0f / sqrtf(static_cast<float>(dk)));
        NNB_LAUNCH_CHECK();
        NNB_TRY(gemv<WT>(Wt + lp.wo, F(W.att), P + lp.bo, x, xmid, d, d, s));                    // + residual (GPTBlock::forward_step)
        decode_norm_kernel<<<1, 256, 0, s>>>(xmid, P + lp.g2, PB(lp.be2), F(W.xn), d, ln ? 1 : 0);
        NNB_LAUNCH_CHECK();
        NNB_TRY(gemv<WT>(Wt + lp.w1, F(W.xn), P + lp.b1, nullptr, F(W.h1), fc1, d, s));
        decode_act_kernel<<<grid_for(ff, 256), 256, 0, s>>>(F(W.h1), F(W.h2), ff, c.act == 1 ? 1 : 0);
        NNB_LAUNCH_CHECK();
        NNB_TRY(gemv<WT>(Wt + lp.w2, F(W.h2), P + lp.b2, xmid, x, d, ff, s));                      // + residual
    }
    decode_norm_kernel<<<1, 256, 0, s>>>(x, P + L.lnf_g, PB(L.lnf_b), F(W.xn), d, ln ? 1 : 0);
    NNB_LAUNCH_CHECK();
    return gemv<WT>(Wt + L.lm_w, F(W.xn), P + L.lm_b, nullptr, logits_out ? logits_out : F(W.logits), c.vocab, d, s);
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
    if (!tab.empty()) {
        NNB_CUDA_CHECK(cudaMemcpyAsync(static_cast<uint8_t*>(workspace) + W.table, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, to_stream(stream)));
        NNB_CUDA_CHECK(cudaStreamSynchronize(to_stream(stream)));          // `tab` is pageable host memory about to go away
    }
    return 0;
}

int nnb200_gpt_forward_step(const nnb200_gpt_config* cfg, const float* params, const void* params_bf16, void* workspace, int token_id,
                            int pos, int cur_len, float* logits_out, void* stream)
{
    if (nnb200_gpt_arena_elems(cfg) < 0 || !params || !workspace) { fprintf(stderr, "nnb200_gpt_forward_step: bad arguments\n"); return -1; }
    NNB_ARG_CHECK(cur_len >= 0 && cur_len < cfg->seq, "the cache holds seq rows: cur_len must be in [0, seq)");
    NNB_ARG_CHECK(pos >= 0 && pos < cfg->seq, "position out of range");
    NNB_ARG_CHECK((static_cast<size_t>(cur_len) + 33) * sizeof(float) <= 48 * 1024, "context too long for the decode attention kernel");
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    if (cfg->precision == 1) {
        NNB_ARG_CHECK(params_bf16 != nullptr, "bf16 mode needs the bf16 parameter shadow");
        return forward_step_t<bf16>(*cfg, params, static_cast<const bf16*>(params_bf16), ws, token_id, pos, cur_len, logits_out, to_stream(stream));
    }
    return forward_step_t<float>(*cfg, params, params, ws, token_id, pos, cur_len, logits_out, to_stream(stream));
}

}  // extern "C"
