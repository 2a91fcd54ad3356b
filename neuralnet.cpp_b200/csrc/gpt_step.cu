// Host orchestration of the fused GPT training step: one forward, loss, backward over the
// token-major activations, in fp32 check mode or bf16 tensor-core mode.  The order of operations
// is the one of GPTModel::forward/backward and GPTBlock (compute_layer.hpp:2783-2896, 2366-2405);
// what the reference issues as ~40 primitive calls per block is issued here as 4 GEMMs, one fused
// attention and a handful of fused row kernels.  All buffers come from the caller's workspace.
#include <cmath>
#include <vector>

#include "kernels.h"
#include "nnb200.h"

namespace nnb {

constexpr long long kAlign = 64;    // arena tensors start on 256-byte boundaries (TMA wants 16)

static long long align_up(long long v, long long a) { return (v + a - 1) / a * a; }

struct LayerParams {
    long long bqkv, bo, g1, be1, b1, b2, g2, be2;     // vector region
    long long wqkv, wo, w1, w2;                       // matrix region
};
struct ArenaLayout {
    long long tok_emb, pos_emb, lnf_g, lnf_b, lm_w, lm_b;
    std::vector<LayerParams> layers;
    long long matrix_begin, total;
    std::vector<long long> layer_matrix_begin;       // size layers+1
};

static bool config_ok(const nnb200_gpt_config* c)
{
    return c && c->vocab > 0 && c->d_model > 0 && c->heads > 0 && c->layers > 0 && c->d_ff > 0 && c->seq > 0 &&
           c->batch > 0 && c->d_model % c->heads == 0 && c->act >= 0 && c->act <= 1 && c->norm >= 0 && c->norm <= 1 &&
           c->pos >= 0 && c->pos <= 3 && (c->pos != 3 || (c->d_model / c->heads) % 2 == 0) && c->precision >= 0 &&
           c->precision <= 1;
}

static ArenaLayout make_layout(const nnb200_gpt_config& c)
{
    ArenaLayout L;
    const long long d = c.d_model, ff = c.d_ff, V = c.vocab, S = c.seq;
    const long long fc1 = c.act == 1 ? 2 * ff : ff;
    const bool ln = c.norm == 0;
    long long off = 0;
    auto take = [&](long long n) { const long long o = off; off = align_up(off + n, kAlign); return o; };
    L.tok_emb = take(V * d);
    L.pos_emb = c.pos == 0 ? take(S * d) : -1;
    L.layers.resize(c.layers);
    for (auto& lp : L.layers) {
        lp.bqkv = take(3 * d); lp.bo = take(d);
        lp.g1 = take(d); lp.be1 = ln ? take(d) : -1;
        lp.b1 = take(fc1); lp.b2 = take(d);
        lp.g2 = take(d); lp.be2 = ln ? take(d) : -1;
    }
    L.lnf_g = take(d); L.lnf_b = ln ? take(d) : -1;
    L.lm_w = take(V * d); L.lm_b = take(V);
    L.matrix_begin = off;
    for (auto& lp : L.layers) {
        L.layer_matrix_begin.push_back(off);
        lp.wqkv = take(3 * d * d); lp.wo = take(d * d); lp.w1 = take(fc1 * d); lp.w2 = take(d * ff);
    }
    L.layer_matrix_begin.push_back(off);
    L.total = off;
    return L;
}

DecodeLayout decode_layout(const nnb200_gpt_config& c)
{
    const ArenaLayout L = make_layout(c);
    DecodeLayout D{L.tok_emb, L.pos_emb, L.lnf_g, L.lnf_b, L.lm_w, L.lm_b, {}};
    for (const auto& lp : L.layers) D.layers.push_back(DecodeLayer{lp.wqkv, lp.bqkv, lp.wo, lp.bo, lp.g1, lp.be1, lp.w1, lp.b1, lp.w2, lp.b2, lp.g2, lp.be2});
    return D;
}

// ---------------------------------------------------------------- workspace
struct LayerActs { size_t x_in, xn1, qkv, attn, x_mid, xn2, h1, h2; size_t rinv1, mean1, rinv2, mean2, lse; };
// floats of the deferred column-sum slot of the QKV bias gradient: one partial row per 32 token rows (what the write-outs
// of the attention backward kernels leave), which also holds the coarser partials of the column-sum kernel
static size_t wide_slot_floats(long long rows, long long cols) { return static_cast<size_t>(ceil_div(rows, 32) * cols); }

struct Workspace {
    size_t sin_table, stats, loss, loss_vec;
    std::vector<LayerActs> layers;
    size_t x_final, xnf, rinvf, meanf, logits;
    size_t g_a, g_b, d_xn, d_h2, d_h1, d_attn, d_qkv, dvec, colsum, counters, embed_scratch, norm_partials, colsum_partials, doc_ranges;
    size_t total;
};

static Workspace make_workspace(const nnb200_gpt_config& c)
{
    Workspace W;
    const size_t esz = c.precision == 1 ? 2 : 4;
    const size_t N = static_cast<size_t>(c.batch) * c.seq, d = c.d_model, ff = c.d_ff, V = c.vocab;
    const size_t fc1 = c.act == 1 ? 2 * ff : ff;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off = (off + bytes + 255) / 256 * 256; return o; };
    W.sin_table = take(static_cast<size_t>(c.seq) * d * 4);
    W.stats = take(16); W.loss = take(16); W.loss_vec = take(N * 4);
    W.layers.resize(c.layers);
    for (auto& a : W.layers) {
        a.x_in = take(N * d * esz); a.xn1 = take(N * d * esz); a.qkv = take(N * 3 * d * esz); a.attn = take(N * d * esz);
        a.x_mid = take(N * d * esz); a.xn2 = take(N * d * esz); a.h1 = take(N * fc1 * esz); a.h2 = take(N * ff * esz);
        a.rinv1 = take(N * 4); a.mean1 = take(N * 4); a.rinv2 = take(N * 4); a.mean2 = take(N * 4);
        a.lse = take(static_cast<size_t>(c.batch) * c.heads * c.seq * 4);
    }
    W.x_final = take(N * d * esz); W.xnf = take(N * d * esz); W.rinvf = take(N * 4); W.meanf = take(N * 4);
    W.logits = take(N * V * esz);
    W.g_a = take(N * d * esz); W.g_b = take(N * d * esz); W.d_xn = take(N * d * esz);
    W.d_h2 = take(N * ff * esz); W.d_h1 = take(N * fc1 * esz); W.d_attn = take(N * d * esz); W.d_qkv = take(N * 3 * d * esz);
    W.dvec = take(static_cast<size_t>(c.batch) * c.heads * c.seq * 4);
    const size_t widest = std::max(std::max(fc1, 3 * d), V);
    W.colsum = take(std::max(colsum_scratch_floats(static_cast<int>(N), static_cast<int>(widest)),
                             norm_bwd_scratch_floats(static_cast<int>(N), static_cast<int>(d))) * 4);
    W.counters = take(kColsumCounters * sizeof(int));
    // one slot per norm backward of a micro-batch (2 per layer + the final norm) for the deferred parameter-gradient fold
    const size_t norm_slots = 2 * static_cast<size_t>(c.layers) + 1;
    W.norm_partials = take(norm_slots <= kNormFoldMaxSlots ? norm_slots * norm_bwd_defer_slot_floats(static_cast<int>(d)) * 4 : 0);
    // and one per bias gradient that has a column-sum pass of its own: the LM head, and fc1 and qkv of every layer
    W.colsum_partials = take(2 * static_cast<size_t>(c.layers) + 1 <= kColsumFoldMaxSlots
                                 ? (colsum_scratch_floats(static_cast<int>(N), static_cast<int>(V)) +
                                    c.layers * (colsum_scratch_floats(static_cast<int>(N), static_cast<int>(fc1)) +
                                                wide_slot_floats(static_cast<int>(N), static_cast<int>(3 * d)))) * 4
                                 : 0);
    W.embed_scratch = take(embed_bwd_scratch_bytes(static_cast<int>(N)));
    W.doc_ranges = take((N / 64 + 1) * 2 * sizeof(int));      // (min, max) document id per 64 token rows
    W.total = off;
    return W;
}

// ---------------------------------------------------------------- typed step
template <typename T> struct Mode;
template <> struct Mode<float> { static constexpr bool bf = false; };
template <> struct Mode<bf16> { static constexpr bool bf = true; };

// Y[N_tok, out] = X[N_tok, in] W[out, in]^T + b (+ residual)
template <typename T>
static int linear_fwd(const T* X, const float* Wf, const bf16* Wh, const float* bias, const T* residual, T* Y, int ntok,
                      int in, int out, cudaStream_t s)
{
    if (Mode<T>::bf)
        return gemm_bf16(reinterpret_cast<const bf16*>(X), Wh, Y, ntok, out, in, in, in, out, 0, 0, 1, 1.0f, bias, residual, 0, s);
    return sgemm_strided(reinterpret_cast<const float*>(X), Wf, reinterpret_cast<float*>(Y), ntok, out, in, in, 1, in, 1,
                         out, 1, 0, 0, 0, 1.0f, bias, nullptr, reinterpret_cast<const float*>(residual), 0, s);
}
// dX[N_tok, in] = dY[N_tok, out] W[out, in]
template <typename T>
static int linear_bwd_input(const T* dY, const float* Wf, const bf16* Wh, T* dX, int ntok, int in, int out, cudaStream_t s)
{
    if (Mode<T>::bf)
        return gemm_bf16(reinterpret_cast<const bf16*>(dY), Wh, dX, ntok, in, out, out, in, in, 0, 1, 1, 1.0f, nullptr, nullptr, 0, s);
    return sgemm_strided(reinterpret_cast<const float*>(dY), Wf, reinterpret_cast<float*>(dX), ntok, in, out, out, 1, 1, in,
                         in, 1, 0, 0, 0, 1.0f, nullptr, nullptr, nullptr, 0, s);
}
// dW[out, in] += dY^T X ; db[out] += column sums of dY
template <typename T>
static int linear_bwd_params(const T* dY, const T* X, float* dW, float* db, float* scratch, int* counters, int ntok, int in,
                             int out, cudaStream_t s, ColsumDefer* defer = nullptr)
{
    if (Mode<T>::bf)
        NNB_TRY(gemm_bf16(reinterpret_cast<const bf16*>(dY), reinterpret_cast<const bf16*>(X), dW, out, in, ntok, out, in, in,
                          1, 1, 0, 1.0f, nullptr, nullptr, 1, s));
    else
        NNB_TRY(sgemm_strided(reinterpret_cast<const float*>(dY), reinterpret_cast<const float*>(X), dW, out, in, ntok, 1,
                              out, 1, in, in, 1, 0, 0, 0, 1.0f, nullptr, nullptr, nullptr, 1, s));
    if (defer) defer->deferred = false;
    if (!db) return 0;                       // the bias gradient was already summed by the kernel that produced dY
    return colsum_accumulate<T>(dY, out, nullptr, nullptr, nullptr, nullptr, 0, db, scratch, ntok, out, s, counters, defer);
}

template <typename T>
static int attention_fwd(const T* qkv, T* out, float* lse, const int* doc, const int* ranges, const nnb200_gpt_config& c, cudaStream_t s)
{
    const int dk = c.d_model / c.heads, alibi = c.pos == 2;
    if constexpr (Mode<T>::bf) {
        if (attention_tc_supported(dk, c.seq, c.d_model)) return attention_fwd_tc(qkv, out, lse, doc, ranges, c.batch, c.seq, c.heads, dk, alibi, s);
        if (attention_mma_supported(dk, c.d_model)) return attention_fwd_mma(qkv, out, lse, doc, c.batch, c.seq, c.heads, dk, alibi, s);
    }
    return attention_fwd_simt<T>(qkv, out, lse, doc, c.batch, c.seq, c.heads, dk, alibi, s);
}
template <typename T>
static int attention_bwd(const T* qkv, const T* out, const T* dout, const float* lse, float* dvec, T* dqkv, const int* doc,
                         const int* ranges, const nnb200_gpt_config& c, cudaStream_t s, bool have_dvec = false,
                         float* colsum_part = nullptr)          // the last two: honoured by the tcgen05 kernels only
{
    const int dk = c.d_model / c.heads, alibi = c.pos == 2;
    if constexpr (Mode<T>::bf) {
        if (attention_tc_supported(dk, c.seq, c.d_model))
            return attention_bwd_tc(qkv, out, dout, lse, dvec, dqkv, doc, ranges, c.batch, c.seq, c.heads, dk, alibi, s, have_dvec, colsum_part);
        if (attention_mma_supported(dk, c.d_model))
            return attention_bwd_mma(qkv, out, dout, lse, dvec, dqkv, doc, c.batch, c.seq, c.heads, dk, alibi, s);
    }
    return attention_bwd_simt<T>(qkv, out, dout, lse, dvec, dqkv, doc, c.batch, c.seq, c.heads, dk, alibi, s);
}

template <typename T>
static int forward_t(const nnb200_gpt_config& c, const float* P, const bf16* H, uint8_t* ws, const int* tokens,
                     const int* doc, cudaStream_t s)
{
    const ArenaLayout L = make_layout(c);
    const Workspace W = make_workspace(c);
    const int N = c.batch * c.seq, d = c.d_model, ff = c.d_ff, fc1 = c.act == 1 ? 2 * ff : ff;
    const bool ln = c.norm == 0, swiglu = c.act == 1;
    auto A = [&](size_t off) { return reinterpret_cast<T*>(ws + off); };
    auto F = [&](size_t off) { return reinterpret_cast<float*>(ws + off); };
    auto PB = [&](long long off) { return off >= 0 ? P + off : nullptr; };

    const float* pos_table = c.pos == 0 ? P + L.pos_emb : (c.pos == 1 ? F(W.sin_table) : nullptr);
    // document-id range of every 64 token rows, once per micro-batch: the attention kernels of every layer, forward
    // and backward, skip the blocks it shows to be fully masked (what build_attention_mask leaves as -inf everywhere)
    const int* ranges = nullptr;
    if (Mode<T>::bf && doc && attention_tc_supported(d / c.heads, c.seq, d)) {
        NNB_TRY(attention_doc_ranges(doc, c.batch, c.seq, reinterpret_cast<int*>(ws + W.doc_ranges), s));
        ranges = reinterpret_cast<const int*>(ws + W.doc_ranges);
    }
    T* x = A(W.layers[0].x_in);
    NNB_TRY(embed_fwd<T>(P + L.tok_emb, pos_table, tokens, x, N, c.seq, d, c.vocab, s));
    for (int l = 0; l < c.layers; ++l) {
        const LayerParams& lp = L.layers[l];
        const LayerActs& a = W.layers[l];
        T* x_next = (l + 1 < c.layers) ? A(W.layers[l + 1].x_in) : A(W.x_final);
        NNB_TRY(norm_fwd<T>(A(a.x_in), P + lp.g1, PB(lp.be1), A(a.xn1), F(a.rinv1), F(a.mean1), N, d, ln, s));
        NNB_TRY(linear_fwd<T>(A(a.xn1), P + lp.wqkv, H ? H + lp.wqkv : nullptr, P + lp.bqkv, nullptr, A(a.qkv), N, d, 3 * d, s));
        // rotary positions: Q and K are rotated in place, so the backward pass sees the rotated values (AttentionBase::forward, compute_layer.hpp:1178-1185)
        if (c.pos == 3) NNB_TRY(rope_apply<T>(A(a.qkv), F(W.sin_table), N, c.seq, c.heads, d / c.heads, 3 * d, false, s));
        NNB_TRY(attention_fwd<T>(A(a.qkv), A(a.attn), F(a.lse), doc, ranges, c, s));
        NNB_TRY(linear_fwd<T>(A(a.attn), P + lp.wo, H ? H + lp.wo : nullptr, P + lp.bo, A(a.x_in), A(a.x_mid), N, d, d, s));
        NNB_TRY(norm_fwd<T>(A(a.x_mid), P + lp.g2, PB(lp.be2), A(a.xn2), F(a.rinv2), F(a.mean2), N, d, ln, s));
        if (Mode<T>::bf && swiglu && gemm_swiglu_supported(N, ff, d)) {
            // projection and activation in one launch (the SwiGLU epilogue of the pair GEMM); same values as the two below
            NNB_TRY(gemm_bf16_swiglu(reinterpret_cast<const bf16*>(A(a.xn2)), H + lp.w1, P + lp.b1, reinterpret_cast<bf16*>(A(a.h1)),
                                     reinterpret_cast<bf16*>(A(a.h2)), N, ff, d, s));
        } else {
            NNB_TRY(linear_fwd<T>(A(a.xn2), P + lp.w1, H ? H + lp.w1 : nullptr, P + lp.b1, nullptr, A(a.h1), N, d, fc1, s));
            NNB_TRY(act_fwd<T>(A(a.h1), A(a.h2), N, ff, swiglu, s));
        }
        NNB_TRY(linear_fwd<T>(A(a.h2), P + lp.w2, H ? H + lp.w2 : nullptr, P + lp.b2, A(a.x_mid), x_next, N, ff, d, s));
    }
    NNB_TRY(norm_fwd<T>(A(W.x_final), P + L.lnf_g, PB(L.lnf_b), A(W.xnf), F(W.rinvf), F(W.meanf), N, d, ln, s));
    NNB_TRY(linear_fwd<T>(A(W.xnf), P + L.lm_w, H ? H + L.lm_w : nullptr, P + L.lm_b, nullptr, A(W.logits), N, d, c.vocab, s));
    return 0;
}

template <typename T>
static int backward_t(const nnb200_gpt_config& c, const float* P, const bf16* H, float* G, uint8_t* ws, const int* tokens,
                      const int* doc, void* const* events, cudaStream_t s)
{
    const ArenaLayout L = make_layout(c);
    const Workspace W = make_workspace(c);
    const int N = c.batch * c.seq, d = c.d_model, ff = c.d_ff, fc1 = c.act == 1 ? 2 * ff : ff;
    const bool ln = c.norm == 0, swiglu = c.act == 1;
    auto A = [&](size_t off) { return reinterpret_cast<T*>(ws + off); };
    auto F = [&](size_t off) { return reinterpret_cast<float*>(ws + off); };
    auto PB = [&](long long off) { return off >= 0 ? P + off : nullptr; };
    auto GB = [&](long long off) { return off >= 0 ? G + off : nullptr; };
    auto Hh = [&](long long off) { return H ? H + off : nullptr; };
    float* cs = F(W.colsum);
    int* cn = reinterpret_cast<int*>(ws + W.counters);
    // the table the forward pass of this micro-batch left in the workspace (same tokens, same document ids)
    const int* ranges = (Mode<T>::bf && doc && attention_tc_supported(d / c.heads, c.seq, d)) ? reinterpret_cast<const int*>(ws + W.doc_ranges) : nullptr;
    // the norm backward kernels leave their per-block partial sums of the scale / shift / bias gradients in a slot each;
    // one kernel after the last layer folds all slots into the gradient arena (nothing reads them before the optimizer)
    const bool defer = 2 * c.layers + 1 <= kNormFoldMaxSlots;
    const size_t slot_floats = norm_bwd_defer_slot_floats(d);
    NormFoldSlots slots;
    int nslots = 0;
    auto slot_ptr = [&]() -> float* { return defer ? F(W.norm_partials) + nslots * slot_floats : nullptr; };
    auto slot_done = [&](bool deferred, long long dgamma, long long dbeta, long long osum) {
        if (!deferred) return;
        slots.dgamma[nslots] = dgamma; slots.dbeta[nslots] = dbeta; slots.osum[nslots] = osum;
        ++nslots;
    };
    bool was_deferred = false;
    ColsumFoldSlots csl;
    int ncs = 0;
    size_t cs_off = 0;                                            // floats used of W.colsum_partials
    ColsumDefer cd{nullptr, 0, false};
    auto cs_begin = [&]() -> ColsumDefer* {
        if (!defer) return nullptr;
        cd.partial = F(W.colsum_partials) + cs_off; cd.chunks = 0; cd.deferred = false;
        return &cd;
    };
    auto cs_done = [&](long long dst, int cols, bool wide = false) {
        if (!cd.deferred) return;
        csl.dst[ncs] = dst; csl.part[ncs] = static_cast<long long>(cs_off); csl.chunks[ncs] = cd.chunks; csl.cols[ncs] = cols;
        ++ncs;
        cs_off += wide ? wide_slot_floats(N, cols) : colsum_scratch_floats(N, cols);
        cd.deferred = false;
    };

    // LM head and final norm (GPTModel::backward, compute_layer.hpp:2849-2856)
    T* dlogits = A(W.logits);
    NNB_TRY(linear_bwd_params<T>(dlogits, A(W.xnf), G + L.lm_w, G + L.lm_b, cs, cn, N, d, c.vocab, s, cs_begin()));
    cs_done(L.lm_b, c.vocab);
    // lm_head.W's gradient is final here (its bias gradient only after the deferred fold at the end)
    if (events && events[c.layers + 1]) NNB_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(events[c.layers + 1]), s));
    NNB_TRY(linear_bwd_input<T>(dlogits, P + L.lm_w, Hh(L.lm_w), A(W.d_xn), N, d, c.vocab, s));
    T* g = A(W.g_a);
    T* g_other = A(W.g_b);
    // each norm backward also sums the columns of the gradient it produces: that is the bias gradient
    // of the Linear layer whose output this gradient belongs to (fc2 of the layer below, or wo)
    NNB_TRY(norm_bwd<T>(A(W.d_xn), A(W.x_final), P + L.lnf_g, F(W.rinvf), F(W.meanf), nullptr, g, G + L.lnf_g, GB(L.lnf_b),
                        cs, N, d, ln, s, cn, G + L.layers[c.layers - 1].b2, slot_ptr(), &was_deferred));
    slot_done(was_deferred, L.lnf_g, L.lnf_b, L.layers[c.layers - 1].b2);

    for (int l = c.layers - 1; l >= 0; --l) {
        const LayerParams& lp = L.layers[l];
        const LayerActs& a = W.layers[l];
        // FeedForward::backward (compute_layer.hpp:1674-1688)
        NNB_TRY(linear_bwd_params<T>(g, A(a.h2), G + lp.w2, nullptr, cs, cn, N, ff, d, s));
        bool fused_act = false;
        if constexpr (Mode<T>::bf) {
            if (swiglu && gemm_swiglu_bwd_supported(N, ff, d)) {
                // the activation's backward pass in the epilogue of fc2's input-gradient GEMM; fc1's bias gradient after it
                // (with the deferred fold its epilogue also leaves the column sums per 128 rows: no pass over d_h1 for them)
                ColsumDefer* dfr = cs_begin();
                NNB_TRY(gemm_bf16_swiglu_bwd(reinterpret_cast<const bf16*>(g), Hh(lp.w2), reinterpret_cast<const bf16*>(A(a.h1)),
                                             reinterpret_cast<bf16*>(A(W.d_h1)), N, ff, d, dfr ? dfr->partial : nullptr, s));
                if (dfr) { dfr->chunks = static_cast<int>(ceil_div(N, 128)); dfr->deferred = true; }
                else NNB_TRY(colsum_accumulate<T>(A(W.d_h1), fc1, nullptr, nullptr, nullptr, nullptr, 0, G + lp.b1, cs, N, fc1, s, cn, nullptr));
                fused_act = true;
            }
        }
        if (!fused_act) {
            NNB_TRY(linear_bwd_input<T>(g, P + lp.w2, Hh(lp.w2), A(W.d_h2), N, ff, d, s));
            NNB_TRY(act_bwd<T>(A(W.d_h2), A(a.h1), A(W.d_h1), N, ff, swiglu, s, G + lp.b1, cs, cn, cs_begin()));   // also sums fc1's bias gradient
        }
        cs_done(lp.b1, fc1);
        NNB_TRY(linear_bwd_params<T>(A(W.d_h1), A(a.xn2), G + lp.w1, nullptr, cs, cn, N, d, fc1, s));
        NNB_TRY(linear_bwd_input<T>(A(W.d_h1), P + lp.w1, Hh(lp.w1), A(W.d_xn), N, d, fc1, s));
        // grad_r1 = grad_output + norm2.backward (GPTBlock::backward, compute_layer.hpp:2388-2404)
        NNB_TRY(norm_bwd<T>(A(W.d_xn), A(a.x_mid), P + lp.g2, F(a.rinv2), F(a.mean2), g, g_other, G + lp.g2, GB(lp.be2), cs,
                            N, d, ln, s, cn, G + lp.bo, slot_ptr(), &was_deferred));
        slot_done(was_deferred, lp.g2, lp.be2, lp.bo);
        std::swap(g, g_other);
        // AttentionBase::backward (compute_layer.hpp:1271-1412)
        NNB_TRY(linear_bwd_params<T>(g, A(a.attn), G + lp.wo, nullptr, cs, cn, N, d, d, s));
        // with 64-wide heads on the tcgen05 kernels, the out-projection's input-gradient GEMM also leaves
        // rowsum(dO * O) per head and row, which the attention backward pass would otherwise compute in a pass of its own
        bool have_dvec = false;
        if constexpr (Mode<T>::bf) {
            if (d / c.heads == 64 && attention_tc_supported(64, c.seq, d) && gemm_rowdot_supported(N, d, d, c.seq, c.heads)) {
                NNB_TRY(gemm_bf16_dx_rowdot(reinterpret_cast<const bf16*>(g), Hh(lp.wo), reinterpret_cast<bf16*>(A(W.d_attn)),
                                            reinterpret_cast<const bf16*>(A(a.attn)), F(W.dvec), N, d, d, c.seq, c.heads, s));
                have_dvec = true;
            }
        }
        if (!have_dvec) NNB_TRY(linear_bwd_input<T>(g, P + lp.wo, Hh(lp.wo), A(W.d_attn), N, d, d, s));
        // On the tcgen05 kernels the write-outs of dQ, dK and dV also leave their column sums per 32 rows: the QKV bias
        // gradient without a pass over d_qkv.  Not with rotary positions: there the bias sees the gradient rotated back.
        ColsumDefer* qkv_dfr = nullptr;
        if constexpr (Mode<T>::bf) {
            if (c.pos != 3 && attention_tc_supported(d / c.heads, c.seq, d)) qkv_dfr = cs_begin();
        }
        NNB_TRY(attention_bwd<T>(A(a.qkv), A(a.attn), A(W.d_attn), F(a.lse), F(W.dvec), A(W.d_qkv), doc, ranges, c, s, have_dvec,
                                 qkv_dfr ? qkv_dfr->partial : nullptr));
        if (qkv_dfr) { qkv_dfr->chunks = static_cast<int>(N / 32); qkv_dfr->deferred = true; cs_done(lp.bqkv, 3 * d, true); }
        // the gradients of the rotated Q and K go back through the inverse rotation (compute_layer.hpp:1365-1372)
        if (c.pos == 3) NNB_TRY(rope_apply<T>(A(W.d_qkv), F(W.sin_table), N, c.seq, c.heads, d / c.heads, 3 * d, true, s));
        if (qkv_dfr) {
            NNB_TRY(linear_bwd_params<T>(A(W.d_qkv), A(a.xn1), G + lp.wqkv, nullptr, cs, cn, N, d, 3 * d, s));
        } else {
            NNB_TRY(linear_bwd_params<T>(A(W.d_qkv), A(a.xn1), G + lp.wqkv, G + lp.bqkv, cs, cn, N, d, 3 * d, s, cs_begin()));
            cs_done(lp.bqkv, 3 * d, true);
        }
        NNB_TRY(linear_bwd_input<T>(A(W.d_qkv), P + lp.wqkv, Hh(lp.wqkv), A(W.d_xn), N, d, 3 * d, s));
        NNB_TRY(norm_bwd<T>(A(W.d_xn), A(a.x_in), P + lp.g1, F(a.rinv1), F(a.mean1), g, g_other, G + lp.g1, GB(lp.be1), cs, N,
                            d, ln, s, cn, l >= 1 ? G + L.layers[l - 1].b2 : nullptr, slot_ptr(), &was_deferred));
        slot_done(was_deferred, lp.g1, lp.be1, l >= 1 ? L.layers[l - 1].b2 : -1);
        std::swap(g, g_other);
        if (events && events[l]) NNB_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(events[l]), s));
    }
    NNB_TRY(norm_bwd_fold_deferred(F(W.norm_partials), slots, nslots, G, d, s));
    NNB_TRY(colsum_fold_deferred(F(W.colsum_partials), csl, ncs, G, s));
    // embeddings (compute_layer.hpp:2882-2891): deterministic scatter-add
    NNB_TRY(embed_bwd<T>(G + L.tok_emb, c.pos == 0 ? G + L.pos_emb : nullptr, tokens, g, ws + W.embed_scratch, c.batch, c.seq,
                         d, c.vocab, s));
    if (g != A(W.g_a))   // keep the input gradient at a fixed place for inspection
        NNB_CUDA_CHECK(cudaMemcpyAsync(A(W.g_a), g, static_cast<size_t>(N) * d * sizeof(T), cudaMemcpyDeviceToDevice, s));
    if (events && events[c.layers]) NNB_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(events[c.layers]), s));
    return 0;
}

}  // namespace nnb

using namespace nnb;

extern "C" {

int nnb200_gpt_param_table(const nnb200_gpt_config* cfg, long long* offsets, int32_t* rows, int32_t* cols)
{
    if (!config_ok(cfg)) { fprintf(stderr, "nnb200: invalid GPT configuration\n"); return -1; }
    const nnb200_gpt_config& c = *cfg;
    const ArenaLayout L = make_layout(c);
    const int d = c.d_model, ff = c.d_ff, fc1 = c.act == 1 ? 2 * ff : ff;
    int n = 0;
    auto put = [&](long long off, int r, int cc) {
        if (offsets) { offsets[n] = off; rows[n] = r; cols[n] = cc; }
        ++n;
    };
    put(L.tok_emb, c.vocab, d);
    if (c.pos == 0) put(L.pos_emb, c.seq, d);
    for (const auto& lp : L.layers) {
        for (int k = 0; k < 3; ++k) { put(lp.wqkv + static_cast<long long>(k) * d * d, d, d); put(lp.bqkv + static_cast<long long>(k) * d, d, 1); }
        put(lp.wo, d, d); put(lp.bo, d, 1);
        put(lp.g1, d, 1); if (c.norm == 0) put(lp.be1, d, 1);
        put(lp.w1, fc1, d); put(lp.b1, fc1, 1);
        put(lp.w2, d, ff); put(lp.b2, d, 1);
        put(lp.g2, d, 1); if (c.norm == 0) put(lp.be2, d, 1);
    }
    put(L.lnf_g, d, 1); if (c.norm == 0) put(L.lnf_b, d, 1);
    put(L.lm_w, c.vocab, d); put(L.lm_b, c.vocab, 1);
    return n;
}

long long nnb200_gpt_arena_elems(const nnb200_gpt_config* cfg) { return config_ok(cfg) ? make_layout(*cfg).total : -1; }
long long nnb200_gpt_matrix_region_begin(const nnb200_gpt_config* cfg) { return config_ok(cfg) ? make_layout(*cfg).matrix_begin : -1; }
long long nnb200_gpt_layer_matrix_begin(const nnb200_gpt_config* cfg, int layer)
{
    if (!config_ok(cfg) || layer < 0 || layer > cfg->layers) return -1;
    return make_layout(*cfg).layer_matrix_begin[layer];
}
long long nnb200_gpt_workspace_bytes(const nnb200_gpt_config* cfg)
{
    return config_ok(cfg) ? static_cast<long long>(make_workspace(*cfg).total) : -1;
}
long long nnb200_gpt_workspace_offset(const nnb200_gpt_config* cfg, int which)
{
    if (!config_ok(cfg)) return -1;
    const Workspace W = make_workspace(*cfg);
    switch (which) {
        case 0: return static_cast<long long>(W.logits);
        case 1: return static_cast<long long>(W.loss);
        case 2: return static_cast<long long>(W.g_a);
        case 3: return static_cast<long long>(W.stats);
        default: return -1;
    }
}

int nnb200_gpt_init_workspace(const nnb200_gpt_config* cfg, void* workspace, void* stream)
{
    if (!config_ok(cfg) || !workspace) { fprintf(stderr, "nnb200: invalid GPT configuration or workspace\n"); return -1; }
    // the column-sum kernels expect their completion counters to start at zero (they reset them after use)
    NNB_CUDA_CHECK(cudaMemsetAsync(static_cast<uint8_t*>(workspace) + make_workspace(*cfg).counters, 0,
                                   kColsumCounters * sizeof(int), to_stream(stream)));
    if (cfg->pos == 3) {
        // rotary tables share the slot of the sinusoidal table (seq * d_k floats fit in seq * d_model)
        const Workspace W = make_workspace(*cfg);
        std::vector<float> tab(static_cast<size_t>(cfg->seq) * (cfg->d_model / cfg->heads));
        rope_table_host(cfg->seq, cfg->d_model / cfg->heads, tab.data());
        NNB_CUDA_CHECK(cudaMemcpyAsync(static_cast<uint8_t*>(workspace) + W.sin_table, tab.data(), tab.size() * 4,
                                       cudaMemcpyHostToDevice, to_stream(stream)));
        NNB_CUDA_CHECK(cudaStreamSynchronize(to_stream(stream)));   // `tab` is pageable host memory about to go away
        return 0;
    }
    if (cfg->pos != 1) return 0;
    // SinusoidalPositionEncoder (compute_layer.hpp:2604-2622): built on the host with the same
    // float pow/sin/cos calls as the reference, so the table is bit-identical to the CPU engine's
    const Workspace W = make_workspace(*cfg);
    const int S = cfg->seq, d = cfg->d_model;
    std::vector<float> pe(static_cast<size_t>(S) * d);
    for (int pos = 0; pos < S; ++pos)
        for (int i = 0; i < d; ++i) {
            const float angle = static_cast<float>(pos) / std::pow(10000.0f, static_cast<float>(2 * (i / 2)) / static_cast<float>(d));
            pe[static_cast<size_t>(pos) * d + i] = (i % 2 == 0) ? std::sin(angle) : std::cos(angle);
        }
    NNB_CUDA_CHECK(cudaMemcpyAsync(static_cast<uint8_t*>(workspace) + W.sin_table, pe.data(), pe.size() * 4,
                                   cudaMemcpyHostToDevice, to_stream(stream)));
    NNB_CUDA_CHECK(cudaStreamSynchronize(to_stream(stream)));   // `pe` is pageable host memory about to go away
    return 0;
}

int nnb200_gpt_forward(const nnb200_gpt_config* cfg, const float* params, const void* params_bf16, void* workspace,
                       const int32_t* tokens, const int32_t* doc_ids, void* stream)
{
    if (!config_ok(cfg) || !params || !workspace || !tokens) { fprintf(stderr, "nnb200_gpt_forward: bad arguments\n"); return -1; }
    if (cfg->precision == 1) {
        if (!params_bf16) { fprintf(stderr, "nnb200_gpt_forward: bf16 mode needs the bf16 parameter shadow\n"); return -1; }
        if (cfg->d_model % 8 || cfg->d_ff % 8 || cfg->vocab % 8) { fprintf(stderr, "nnb200_gpt_forward: bf16 mode needs d_model, d_ff, vocab multiples of 8\n"); return -1; }
        return forward_t<bf16>(*cfg, params, static_cast<const bf16*>(params_bf16), static_cast<uint8_t*>(workspace), tokens, doc_ids, to_stream(stream));
    }
    return forward_t<float>(*cfg, params, nullptr, static_cast<uint8_t*>(workspace), tokens, doc_ids, to_stream(stream));
}

int nnb200_gpt_loss(const nnb200_gpt_config* cfg, void* workspace, const int32_t* labels, const float* loss_mask,
                    float grad_scale, void* stream)
{
    if (!config_ok(cfg) || !workspace || !labels) { fprintf(stderr, "nnb200_gpt_loss: bad arguments\n"); return -1; }
    const Workspace W = make_workspace(*cfg);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    const int N = cfg->batch * cfg->seq;
    float* lv = reinterpret_cast<float*>(ws + W.loss_vec);
    float* st = reinterpret_cast<float*>(ws + W.stats);
    float* lo = reinterpret_cast<float*>(ws + W.loss);
    if (cfg->precision == 1)
        return cross_entropy<bf16>(reinterpret_cast<bf16*>(ws + W.logits), labels, loss_mask, grad_scale, lv, st, lo, N, cfg->vocab, cfg->vocab, to_stream(stream));
    return cross_entropy<float>(reinterpret_cast<float*>(ws + W.logits), labels, loss_mask, grad_scale, lv, st, lo, N, cfg->vocab, cfg->vocab, to_stream(stream));
}

int nnb200_gpt_backward(const nnb200_gpt_config* cfg, const float* params, const void* params_bf16, float* grads,
                        void* workspace, const int32_t* tokens, const int32_t* doc_ids, void* const* layer_events,
                        void* stream)
{
    if (!config_ok(cfg) || !params || !grads || !workspace || !tokens) { fprintf(stderr, "nnb200_gpt_backward: bad arguments\n"); return -1; }
    if (cfg->precision == 1) {
        if (!params_bf16) { fprintf(stderr, "nnb200_gpt_backward: bf16 mode needs the bf16 parameter shadow\n"); return -1; }
        return backward_t<bf16>(*cfg, params, static_cast<const bf16*>(params_bf16), grads, static_cast<uint8_t*>(workspace), tokens, doc_ids, layer_events, to_stream(stream));
    }
    return backward_t<float>(*cfg, params, nullptr, grads, static_cast<uint8_t*>(workspace), tokens, doc_ids, layer_events, to_stream(stream));
}

}  // extern "C"
