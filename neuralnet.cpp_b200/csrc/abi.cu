// extern "C" entry points that are thin type dispatchers over the templated launchers, and the
// Muon update (Newton-Schulz iterations as GEMMs).
#include "kernels.h"
#include "nnb200.h"

using namespace nnb;

namespace nnb {

unsigned long long g_launches = 0;

// Bm = b*A + c*A2 + a*I on an (r, r) matrix: the polynomial of one Newton-Schulz step with the
// "+ a*X" term (compute_optimizer.hpp:476-488) folded in as a*I, so X' = Bm X is one GEMM
template <typename T>
__global__ void ns_poly_kernel(const T* __restrict__ A, const T* __restrict__ A2, T* __restrict__ out, int r, float a,
                               float b, float c)
{
    const size_t n = static_cast<size_t>(r) * r;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float v = b * to_f32(A[i]) + c * to_f32(A2[i]);
        if (i / r == i % r) v += a;
        out[i] = from_f32<T>(v);
    }
}

static size_t up256(size_t v) { return (v + 255) / 256 * 256; }

template <typename T>
static int muon_matrix(float* p, const float* u, bf16* shadow, int rows, int cols, float lr, int ns_steps, float eps,
                       uint8_t* scratch, size_t off, cudaStream_t s)
{
    constexpr bool BF = sizeof(T) == 2;
    const size_t n = static_cast<size_t>(rows) * cols;
    const bool transposed = BF && rows > cols;          // bf16 mode iterates on the short side
    const int r = transposed ? cols : rows;
    float* partial = reinterpret_cast<float*>(scratch + off); off += up256(sumsq_scratch_floats() * 4);
    float* out3 = reinterpret_cast<float*>(scratch + off); off += 256;
    T* X = reinterpret_cast<T*>(scratch + off); off += up256(n * sizeof(T));
    T* X2 = reinterpret_cast<T*>(scratch + off); off += up256(n * sizeof(T));
    T* A = reinterpret_cast<T*>(scratch + off); off += up256(static_cast<size_t>(r) * r * sizeof(T));
    T* A2 = reinterpret_cast<T*>(scratch + off); off += up256(static_cast<size_t>(r) * r * sizeof(T));
    T* Bm = reinterpret_cast<T*>(scratch + off);
    constexpr float ka = 3.4445f, kb = -4.7750f, kc = 2.0315f;   // compute_optimizer.hpp:433-435

    NNB_TRY(sum_squares(u, n, 1.0f, 0.f, 1.0f, partial, out3, s));
    NNB_TRY(muon_normalize<T>(u, out3, eps, X, n, s));
    for (int it = 0; it < ns_steps; ++it) {
        if constexpr (BF) {
            const bf16* Xb = reinterpret_cast<const bf16*>(X);
            if (!transposed) NNB_TRY(gemm_bf16(Xb, Xb, A, r, r, cols, cols, cols, r, 0, 0, 1, 1.0f, nullptr, nullptr, 0, s));
            else NNB_TRY(gemm_bf16(Xb, Xb, A, r, r, rows, cols, cols, r, 1, 1, 1, 1.0f, nullptr, nullptr, 0, s));
            NNB_TRY(gemm_bf16(reinterpret_cast<const bf16*>(A), reinterpret_cast<const bf16*>(A), A2, r, r, r, r, r, r, 0, 0, 1,
                              1.0f, nullptr, nullptr, 0, s));
        } else {
            const float* Xf = reinterpret_cast<const float*>(X);
            NNB_TRY(sgemm_strided(Xf, Xf, reinterpret_cast<float*>(A), r, r, cols, cols, 1, cols, 1, r, 1, 0, 0, 0, 1.0f,
                                  nullptr, nullptr, nullptr, 0, s));
            NNB_TRY(sgemm_strided(reinterpret_cast<const float*>(A), reinterpret_cast<const float*>(A),
                                  reinterpret_cast<float*>(A2), r, r, r, r, 1, 1, r, r, 1, 0, 0, 0, 1.0f, nullptr, nullptr,
                                  nullptr, 0, s));
        }
        ns_poly_kernel<T><<<grid_for(static_cast<long long>(r) * r, 256), 256, 0, s>>>(A, A2, Bm, r, ka, kb, kc);
        NNB_LAUNCH_CHECK();
        if constexpr (BF) {
            const bf16* Xb = reinterpret_cast<const bf16*>(X);
            const bf16* Bb = reinterpret_cast<const bf16*>(Bm);
            if (!transposed) NNB_TRY(gemm_bf16(Bb, Xb, X2, rows, cols, rows, rows, cols, cols, 0, 1, 1, 1.0f, nullptr, nullptr, 0, s));
            else NNB_TRY(gemm_bf16(Xb, Bb, X2, rows, cols, cols, cols, cols, cols, 0, 0, 1, 1.0f, nullptr, nullptr, 0, s));
        } else {
            NNB_TRY(sgemm_strided(reinterpret_cast<const float*>(Bm), reinterpret_cast<const float*>(X),
                                  reinterpret_cast<float*>(X2), rows, cols, rows, rows, 1, 1, cols, cols, 1, 0, 0, 0, 1.0f,
                                  nullptr, nullptr, nullptr, 0, s));
        }
        T* t = X; X = X2; X2 = t;
    }
    return muon_apply<T>(p, X, shadow, lr, n, s);
}

}  // namespace nnb

#define DT_CHECK(dtype) NNB_ARG_CHECK((dtype) == 0 || (dtype) == 1, "dtype must be 0 (fp32) or 1 (bf16)")

extern "C" {

int nnb200_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                     long long ldc, int a_mn_major, int b_mn_major, int c_bf16, float alpha, const float* bias_n,
                     const void* residual, int accumulate, void* stream)
{
    return gemm_bf16(static_cast<const bf16*>(A), static_cast<const bf16*>(B), D, M, N, K, lda, ldb, ldc, a_mn_major,
                     b_mn_major, c_bf16, alpha, bias_n, residual, accumulate, to_stream(stream));
}

int nnb200_linear_swiglu_supported(int M, int ff, int K) { return gemm_swiglu_supported(M, ff, K) ? 1 : 0; }
int nnb200_linear_swiglu_forward(const void* x, const void* W, const float* bias, void* h1, void* h2, int M, int ff, int K,
                                 void* stream)
{
    return gemm_bf16_swiglu(static_cast<const bf16*>(x), static_cast<const bf16*>(W), bias, static_cast<bf16*>(h1),
                            static_cast<bf16*>(h2), M, ff, K, to_stream(stream));
}

int nnb200_linear_swiglu_backward_supported(int M, int ff, int K) { return gemm_swiglu_bwd_supported(M, ff, K) ? 1 : 0; }
int nnb200_linear_swiglu_backward(const void* dY, const void* W, const void* h1, void* dh1, int M, int ff, int K,
                                  float* colsum_partial, void* stream)
{
    return gemm_bf16_swiglu_bwd(static_cast<const bf16*>(dY), static_cast<const bf16*>(W), static_cast<const bf16*>(h1),
                                static_cast<bf16*>(dh1), M, ff, K, colsum_partial, to_stream(stream));
}
int nnb200_gemm_bf16_rowdot_supported(int M, int N, int K, int S, int H) { return gemm_rowdot_supported(M, N, K, S, H) ? 1 : 0; }
int nnb200_gemm_bf16_rowdot(const void* dY, const void* W, void* dX, const void* other, float* dot, int M, int N, int K,
                            int S, int H, void* stream)
{
    return gemm_bf16_dx_rowdot(static_cast<const bf16*>(dY), static_cast<const bf16*>(W), static_cast<bf16*>(dX),
                               static_cast<const bf16*>(other), dot, M, N, K, S, H, to_stream(stream));
}

int nnb200_gemm_pair_capacity(void) { return nnb::gemm_pair_capacity(); }
int nnb200_gemm_status(int* host_code)
{
    NNB_ARG_CHECK(host_code != nullptr, "null output");
    NNB_TRY(gemm_device_error(host_code));
    if (*host_code) NNB_TRY(gemm_clear_device_error());
    int attn = 0;
    NNB_TRY(attention_device_error(&attn));                 // reads and clears
    if (!*host_code && attn) *host_code = attn | 0x40000000;  // bit 30 marks the attention forward kernel
    int attn_b = 0;
    NNB_TRY(attention_bwd_device_error(&attn_b));
    if (!*host_code && attn_b) *host_code = attn_b | 0x20000000;   // bit 29: attention backward kernels
    int fused = 0;
    NNB_TRY(fused_device_error(&fused));
    if (!*host_code && fused) *host_code = fused | 0x10000000;    // bit 28: norm backward (bulk-copy waits)
    return 0;
}

int nnb200_attention_doc_ranges(const int32_t* doc_ids, int batch, int seq, int32_t* ranges, void* stream)
{
    return attention_doc_ranges(doc_ids, batch, seq, ranges, to_stream(stream));
}

int nnb200_attention_forward(const void* qkv, void* out, float* lse, const int32_t* doc_ids, const int32_t* doc_ranges,
                             int batch, int seq, int heads, int head_dim, int alibi, int dtype, void* stream)
{
    DT_CHECK(dtype);
    cudaStream_t s = to_stream(stream);
    if (dtype == 1) {
        if (attention_tc_supported(head_dim, seq, heads * head_dim))
            return attention_fwd_tc(static_cast<const bf16*>(qkv), static_cast<bf16*>(out), lse, doc_ids, doc_ranges, batch, seq, heads, head_dim, alibi, s);
        if (attention_mma_supported(head_dim, heads * head_dim))
            return attention_fwd_mma(static_cast<const bf16*>(qkv), static_cast<bf16*>(out), lse, doc_ids, batch, seq, heads, head_dim, alibi, s);
        return attention_fwd_simt<bf16>(static_cast<const bf16*>(qkv), static_cast<bf16*>(out), lse, doc_ids, batch, seq, heads, head_dim, alibi, s);
    }
    return attention_fwd_simt<float>(static_cast<const float*>(qkv), static_cast<float*>(out), lse, doc_ids, batch, seq, heads, head_dim, alibi, s);
}

int nnb200_attention_backward(const void* qkv, const void* out, const void* dout, const float* lse, float* dvec,
                              void* dqkv, const int32_t* doc_ids, const int32_t* doc_ranges, int batch, int seq, int heads,
                              int head_dim, int alibi, int dtype, void* stream)
{
    DT_CHECK(dtype);
    cudaStream_t s = to_stream(stream);
    if (dtype == 1) {
        if (attention_tc_supported(head_dim, seq, heads * head_dim))
            return attention_bwd_tc(static_cast<const bf16*>(qkv), static_cast<const bf16*>(out), static_cast<const bf16*>(dout), lse, dvec, static_cast<bf16*>(dqkv), doc_ids, doc_ranges, batch, seq, heads, head_dim, alibi, s);
        if (attention_mma_supported(head_dim, heads * head_dim))
            return attention_bwd_mma(static_cast<const bf16*>(qkv), static_cast<const bf16*>(out), static_cast<const bf16*>(dout), lse, dvec, static_cast<bf16*>(dqkv), doc_ids, batch, seq, heads, head_dim, alibi, s);
        return attention_bwd_simt<bf16>(static_cast<const bf16*>(qkv), static_cast<const bf16*>(out), static_cast<const bf16*>(dout), lse, dvec, static_cast<bf16*>(dqkv), doc_ids, batch, seq, heads, head_dim, alibi, s);
    }
    return attention_bwd_simt<float>(static_cast<const float*>(qkv), static_cast<const float*>(out), static_cast<const float*>(dout), lse, dvec, static_cast<float*>(dqkv), doc_ids, batch, seq, heads, head_dim, alibi, s);
}

int nnb200_attention_backward_bias_partials(const void* qkv, const void* out, const void* dout, const float* lse, float* dvec,
                                            void* dqkv, const int32_t* doc_ids, const int32_t* doc_ranges,
                                            float* colsum_partial, int batch, int seq, int heads, int head_dim, int alibi,
                                            void* stream)
{
    NNB_ARG_CHECK(colsum_partial != nullptr, "null output");
    return attention_bwd_tc(static_cast<const bf16*>(qkv), static_cast<const bf16*>(out), static_cast<const bf16*>(dout), lse, dvec,
                            static_cast<bf16*>(dqkv), doc_ids, doc_ranges, batch, seq, heads, head_dim, alibi, to_stream(stream),
                            false, colsum_partial);
}

int nnb200_ids_from_float(const float* ids_seq_major, int32_t* out_batch_major, int seq, int batch, void* stream)
{
    NNB_ARG_CHECK(seq >= 0 && batch >= 0 && (static_cast<long long>(seq) * batch == 0 || (ids_seq_major && out_batch_major)), "bad arguments");
    return ids_from_float(ids_seq_major, out_batch_major, seq, batch, to_stream(stream));
}

int nnb200_logits_to_reference(const void* logits_token_major, float* out_vocab_major, int tokens, int vocab, int dtype, void* stream)
{
    DT_CHECK(dtype);
    NNB_ARG_CHECK(tokens >= 0 && vocab >= 0 && (static_cast<long long>(tokens) * vocab == 0 || (logits_token_major && out_vocab_major)), "bad arguments");
    if (dtype == 1) return logits_to_reference<bf16>(static_cast<const bf16*>(logits_token_major), out_vocab_major, tokens, vocab, to_stream(stream));
    return logits_to_reference<float>(static_cast<const float*>(logits_token_major), out_vocab_major, tokens, vocab, to_stream(stream));
}

int nnb200_zero_f32(float* p, size_t n, void* stream) { return zero_f32(p, n, to_stream(stream)); }

int nnb200_norm_forward(const void* x, const float* gamma, const float* beta, void* y, float* rinv, float* mean,
                        int rows, int d, int layer, int dtype, void* stream)
{
    DT_CHECK(dtype);
    if (dtype == 1) return norm_fwd<bf16>(static_cast<const bf16*>(x), gamma, beta, static_cast<bf16*>(y), rinv, mean, rows, d, layer != 0, to_stream(stream));
    return norm_fwd<float>(static_cast<const float*>(x), gamma, beta, static_cast<float*>(y), rinv, mean, rows, d, layer != 0, to_stream(stream));
}

int nnb200_norm_backward(const void* g, const void* x, const float* gamma, const float* rinv, const float* mean,
                         const void* add, void* dx, float* dgamma, float* dbeta, float* scratch, int rows, int d,
                         int layer, int dtype, void* stream)
{
    DT_CHECK(dtype);
    if (dtype == 1)
        return norm_bwd<bf16>(static_cast<const bf16*>(g), static_cast<const bf16*>(x), gamma, rinv, mean, static_cast<const bf16*>(add), static_cast<bf16*>(dx), dgamma, dbeta, scratch, rows, d, layer != 0, to_stream(stream));
    return norm_bwd<float>(static_cast<const float*>(g), static_cast<const float*>(x), gamma, rinv, mean, static_cast<const float*>(add), static_cast<float*>(dx), dgamma, dbeta, scratch, rows, d, layer != 0, to_stream(stream));
}

size_t nnb200_colsum_scratch_floats(int rows, int cols) { return colsum_scratch_floats(rows, cols); }

int nnb200_bias_grad(const void* g, long long ldg, float* out, float* scratch, int rows, int cols, int dtype, void* stream)
{
    DT_CHECK(dtype);
    NNB_ARG_CHECK(rows >= 0 && cols >= 0, "negative shape");
    NNB_ARG_CHECK(rows == 0 || cols == 0 || (g && out && scratch), "null gradient, output or scratch pointer");
    NNB_ARG_CHECK(ldg >= cols, "the row stride is shorter than a row (rows would overlap)");
    if (dtype == 1) return colsum_accumulate<bf16>(static_cast<const bf16*>(g), ldg, nullptr, nullptr, nullptr, nullptr, 0, out, scratch, rows, cols, to_stream(stream));
    return colsum_accumulate<float>(static_cast<const float*>(g), ldg, nullptr, nullptr, nullptr, nullptr, 0, out, scratch, rows, cols, to_stream(stream));
}

int nnb200_activation_forward(const void* h1, void* h2, int rows, int ff, int swiglu, int dtype, void* stream)
{
    DT_CHECK(dtype);
    if (dtype == 1) return act_fwd<bf16>(static_cast<const bf16*>(h1), static_cast<bf16*>(h2), rows, ff, swiglu != 0, to_stream(stream));
    return act_fwd<float>(static_cast<const float*>(h1), static_cast<float*>(h2), rows, ff, swiglu != 0, to_stream(stream));
}
int nnb200_activation_backward(const void* g, const void* h1, void* dh1, int rows, int ff, int swiglu, int dtype,
                               void* stream)
{
    DT_CHECK(dtype);
    if (dtype == 1) return act_bwd<bf16>(static_cast<const bf16*>(g), static_cast<const bf16*>(h1), static_cast<bf16*>(dh1), rows, ff, swiglu != 0, to_stream(stream));
    return act_bwd<float>(static_cast<const float*>(g), static_cast<const float*>(h1), static_cast<float*>(dh1), rows, ff, swiglu != 0, to_stream(stream));
}

int nnb200_cross_entropy(void* logits, const int32_t* labels, const float* mask, float grad_scale, float* loss_vec,
                         float* stats, float* loss_out, int rows, int V, int vocab, int dtype, void* stream)
{
    DT_CHECK(dtype);
    if (dtype == 1) return cross_entropy<bf16>(static_cast<bf16*>(logits), labels, mask, grad_scale, loss_vec, stats, loss_out, rows, V, vocab, to_stream(stream));
    return cross_entropy<float>(static_cast<float*>(logits), labels, mask, grad_scale, loss_vec, stats, loss_out, rows, V, vocab, to_stream(stream));
}

int nnb200_embedding_forward(const float* token_emb, const float* pos_table, const int32_t* tokens, void* x, int tokens_n,
                             int seq, int d, int vocab, int dtype, void* stream)
{
    DT_CHECK(dtype);
    NNB_ARG_CHECK(seq > 0, "seq must be positive");
    if (dtype == 1) return embed_fwd<bf16>(token_emb, pos_table, tokens, static_cast<bf16*>(x), tokens_n, seq, d, vocab, to_stream(stream));
    return embed_fwd<float>(token_emb, pos_table, tokens, static_cast<float*>(x), tokens_n, seq, d, vocab, to_stream(stream));
}
int nnb200_embedding_backward(float* token_grad, float* pos_grad, const int32_t* tokens, const void* g, void* scratch,
                              int batch, int seq, int d, int vocab, int dtype, void* stream)
{
    DT_CHECK(dtype);
    if (dtype == 1) return embed_bwd<bf16>(token_grad, pos_grad, tokens, static_cast<const bf16*>(g), scratch, batch, seq, d, vocab, to_stream(stream));
    return embed_bwd<float>(token_grad, pos_grad, tokens, static_cast<const float*>(g), scratch, batch, seq, d, vocab, to_stream(stream));
}
size_t nnb200_embedding_scratch_bytes(int tokens_n) { return embed_bwd_scratch_bytes(tokens_n); }

int nnb200_rope_table(int seq, int head_dim, float* host_out)
{
    NNB_ARG_CHECK(seq > 0 && head_dim > 0 && head_dim % 2 == 0 && host_out, "rotary table needs seq > 0 and an even head size");
    rope_table_host(seq, head_dim, host_out);
    return 0;
}
int nnb200_rope_apply(void* qkv, const float* table, int tokens_n, int seq, int heads, int head_dim, long long ld, int backward,
                      int dtype, void* stream)
{
    DT_CHECK(dtype);
    NNB_ARG_CHECK(seq > 0 && tokens_n % seq == 0 && ld >= 2LL * heads * head_dim, "tokens must be whole sequences and rows must hold Q and K");
    if (dtype == 1) return rope_apply<bf16>(static_cast<bf16*>(qkv), table, tokens_n, seq, heads, head_dim, ld, backward != 0, to_stream(stream));
    return rope_apply<float>(static_cast<float*>(qkv), table, tokens_n, seq, heads, head_dim, ld, backward != 0, to_stream(stream));
}

int nnb200_adamw_step(float* p, const float* g, float* m, float* v, void* shadow_bf16, size_t n, float lr, float beta1,
                      float beta2, float eps, float weight_decay, int t_next, const float* grad_scale_dev, void* stream)
{
    NNB_ARG_CHECK(t_next >= 1, "t_next is the 1-based step number");
    return adamw_update(p, g, m, v, static_cast<bf16*>(shadow_bf16), n, lr, beta1, beta2, eps, weight_decay, t_next, grad_scale_dev, to_stream(stream));
}

int nnb200_grad_norm_clip(const float* g, size_t n, float pre_scale, float max_norm, float* scratch, float* out3,
                          void* stream)
{
    return sum_squares(g, n, pre_scale, max_norm, pre_scale, scratch, out3, to_stream(stream));
}
size_t nnb200_sumsq_scratch_floats(void) { return sumsq_scratch_floats(); }

size_t nnb200_muon_scratch_bytes(int rows, int cols, int precision)
{
    const size_t n = static_cast<size_t>(rows) * cols, esz = precision == 1 ? 2 : 4;
    const size_t r = (precision == 1 && rows > cols) ? cols : rows;
    return up256(n * 4) + up256(sumsq_scratch_floats() * 4) + 256 + 2 * up256(n * esz) + 3 * up256(r * r * esz);
}

int nnb200_muon_step(float* p, const float* g, float* velocity, void* shadow_bf16, int rows, int cols, float lr,
                     float momentum, int ns_steps, float ns_eps, int precision, void* scratch,
                     const float* grad_scale_dev, void* stream)
{
    NNB_ARG_CHECK(rows > 0 && cols > 0 && scratch != nullptr, "bad shape or scratch");
    NNB_ARG_CHECK(precision == 0 || precision == 1, "precision must be 0 or 1");
    cudaStream_t s = to_stream(stream);
    const size_t n = static_cast<size_t>(rows) * cols;
    uint8_t* sc = static_cast<uint8_t*>(scratch);
    float* u = reinterpret_cast<float*>(sc);
    NNB_TRY(muon_momentum(g, velocity, u, n, momentum, grad_scale_dev, s));
    if (rows > 1 && cols > 1) {
        if (precision == 1) {
            NNB_ARG_CHECK(rows % 8 == 0 && cols % 8 == 0, "bf16 Newton-Schulz needs rows and cols multiples of 8");
            return muon_matrix<bf16>(p, u, static_cast<bf16*>(shadow_bf16), rows, cols, lr, ns_steps, ns_eps, sc, up256(n * 4), s);
        }
        return muon_matrix<float>(p, u, static_cast<bf16*>(shadow_bf16), rows, cols, lr, ns_steps, ns_eps, sc, up256(n * 4), s);
    }
    return muon_apply<float>(p, u, static_cast<bf16*>(shadow_bf16), lr, n, s);     // non-2-D: p -= lr*u
}

// Auxiliary streams ("lanes") of the current device, created on first use, and one event per lane plus one for the fork.
namespace {
constexpr int kMaxLanes = 16;
struct Lanes { cudaStream_t stream[kMaxLanes] = {}; cudaEvent_t done[kMaxLanes] = {}; cudaEvent_t fork = nullptr; int made = 0; };
Lanes g_lanes[64];
int lanes_for_device(int want, Lanes** out)
{
    Lanes& L = g_lanes[nnb::current_device_slot()];
    if (!L.fork) NNB_CUDA_CHECK(cudaEventCreateWithFlags(&L.fork, cudaEventDisableTiming));
    for (; L.made < want; ++L.made) {
        NNB_CUDA_CHECK(cudaStreamCreateWithFlags(&L.stream[L.made], cudaStreamNonBlocking));
        NNB_CUDA_CHECK(cudaEventCreateWithFlags(&L.done[L.made], cudaEventDisableTiming));
    }
    *out = &L;
    return 0;
}
}  // namespace

int nnb200_muon_step_many(int count, float* const* p, const float* const* g, float* const* velocity, void* const* shadow_bf16,
                          const int* rows, const int* cols, float lr, float momentum, int ns_steps, float ns_eps, int precision,
                          void* scratch, size_t scratch_bytes_per_lane, int lanes, const float* grad_scale_dev, void* stream)
{
    NNB_ARG_CHECK(count >= 0 && lanes >= 1 && lanes <= kMaxLanes, "bad count or lane count (1..16)");
    if (count == 0) return 0;
    NNB_ARG_CHECK(p && g && velocity && rows && cols && scratch, "null argument");
    for (int i = 0; i < count; ++i)
        NNB_ARG_CHECK(nnb200_muon_scratch_bytes(rows[i], cols[i], precision) <= scratch_bytes_per_lane, "a lane's scratch is too small for one of the matrices");
    if (lanes > count) lanes = count;
    cudaStream_t s = to_stream(stream);
    Lanes* L = nullptr;
    NNB_TRY(lanes_for_device(lanes, &L));
    // fork: every lane starts behind what is queued on `stream`; join: `stream` continues behind every lane
    NNB_CUDA_CHECK(cudaEventRecord(L->fork, s));
    for (int l = 0; l < lanes; ++l) NNB_CUDA_CHECK(cudaStreamWaitEvent(L->stream[l], L->fork, 0));
    int rc = 0;
    for (int i = 0; i < count && rc == 0; ++i) {
        const int l = i % lanes;
        rc = nnb200_muon_step(p[i], g[i], velocity[i], shadow_bf16 ? shadow_bf16[i] : nullptr, rows[i], cols[i], lr, momentum, ns_steps,
                              ns_eps, precision, static_cast<uint8_t*>(scratch) + static_cast<size_t>(l) * scratch_bytes_per_lane,
                              grad_scale_dev, L->stream[l]);
    }
    for (int l = 0; l < lanes; ++l) {
        NNB_CUDA_CHECK(cudaEventRecord(L->done[l], L->stream[l]));
        NNB_CUDA_CHECK(cudaStreamWaitEvent(s, L->done[l], 0));
    }
    return rc;
}

unsigned long long nnb200_launch_count(int reset)
{
    const unsigned long long v = g_launches;
    if (reset) g_launches = 0;
    return v;
}

int nnb200_gemm_profile(int enable) { return gemm_profile_enable(enable); }
int nnb200_gemm_profile_read(double* host_total_ms, double* host_total_flops, int* host_launches)
{
    NNB_ARG_CHECK(host_total_ms && host_total_flops && host_launches, "null output");
    return gemm_profile_read(0, host_total_ms, host_total_flops, host_launches);
}
int nnb200_gemm_profile_read_fused(double* host_total_ms, double* host_total_flops, int* host_launches)
{
    NNB_ARG_CHECK(host_total_ms && host_total_flops && host_launches, "null output");
    return gemm_profile_read(1, host_total_ms, host_total_flops, host_launches);
}

int nnb200_f32_to_bf16(const float* in, void* out, size_t n, void* stream) { return f32_to_bf16(in, static_cast<bf16*>(out), n, to_stream(stream)); }
int nnb200_bf16_to_f32(const void* in, float* out, size_t n, void* stream) { return bf16_to_f32(static_cast<const bf16*>(in), out, n, to_stream(stream)); }

}  // extern "C"
