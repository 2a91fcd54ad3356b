// Internal C++ interface between the translation units of the library (not part of the C ABI).
#pragma once
#include <vector>

#include "common.cuh"

struct nnb200_gpt_config;      // include/nnb200.h

namespace nnb {

// ---- gpt_step.cu : where a layer's tensors lie in the parameter arena (elements; -1 = absent), for decode.cu
struct DecodeLayer { long long wqkv, bqkv, wo, bo, g1, be1, w1, b1, w2, b2, g2, be2; };
struct DecodeLayout { long long tok_emb, pos_emb, lnf_g, lnf_b, lm_w, lm_b; std::vector<DecodeLayer> layers; };
DecodeLayout decode_layout(const ::nnb200_gpt_config& c);

// ---- gemm_simt.cu : fp32, arbitrary strides, optional batch
int sgemm_strided(const float* A, const float* B, float* C, int M, int N, int K, long long sam, long long sak,
                  long long sbn, long long sbk, long long ldc, int batch, long long batch_a, long long batch_b,
                  long long batch_c, float alpha, const float* bias_n, const float* bias_m, const float* residual,
                  int accumulate, cudaStream_t stream);

// ---- gemm_tcgen05.cu : bf16 operands, fp32 accumulate in TMEM
int gemm_bf16(const bf16* A, const bf16* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
              int a_mn, int b_mn, int c_bf16, float alpha, const float* bias_n, const void* residual, int accumulate,
              cudaStream_t stream);
// first projection of a SwiGLU feed-forward block and its activation in one launch: H1[M, 2 ff] = X W^T + bias (W rows:
// gate, then up), H2[M, ff] = gate * sigmoid(gate) * up, bit-identical to gemm_bf16 followed by act_fwd
bool gemm_swiglu_supported(int M, int ff, int K);
int gemm_bf16_swiglu(const bf16* X, const bf16* W, const float* bias, bf16* H1, bf16* H2, int M, int ff, int K, cudaStream_t stream);
// input gradient of a SwiGLU block's second projection taken through the activation: dH1 = SwiGLU'(H1) * (dY W), the
// product itself not stored; bit-identical to gemm_bf16 followed by act_bwd
bool gemm_swiglu_bwd_supported(int M, int ff, int K);
int gemm_bf16_swiglu_bwd(const bf16* dY, const bf16* W, const bf16* H1, bf16* dH1, int M, int ff, int K, float* colsum_partial,
                         cudaStream_t stream);   // colsum_partial: null, or ceil(M / 128) x 2 ff floats for the column sums per 128 rows
// input gradient of a projection, dX = dY W, and the sums over each 64-column block of dX * other in the same launch
// (the row term of the attention backward pass when dX is the gradient of the attention output and other that output)
bool gemm_rowdot_supported(int M, int N, int K, int S, int H);
int gemm_bf16_dx_rowdot(const bf16* dY, const bf16* W, bf16* dX, const bf16* other, float* dot_out, int M, int N, int K, int S, int H,
                        cudaStream_t stream);
int gemm_device_error(int* code);
int gemm_pair_capacity();
// {next item, CTAs that have left} of (current device, stream), zero between launches (work_counter.cu)
int work_counter_pair(cudaStream_t s, unsigned int** out);
int gemm_clear_device_error();
int gemm_profile_enable(int enable);
int gemm_profile_read(int cls, double* total_ms, double* total_flops, int* launches);   // 0: products, 1: products with an activation in the epilogue

// ---- fused_kernels.cu
template <typename T> int norm_fwd(const T* x, const float* gamma, const float* beta, T* y, float* rinv, float* mean,
                                   int rows, int d, bool layer, cudaStream_t s);
template <typename T> int norm_bwd(const T* g, const T* x, const float* gamma, const float* rinv, const float* mean,
                                   const T* add, T* dx, float* dgamma, float* dbeta, float* scratch, int rows, int d,
                                   bool layer, cudaStream_t s, int* counters = nullptr, float* out_colsum = nullptr,
                                   float* defer_partial = nullptr, bool* deferred = nullptr);
size_t norm_bwd_scratch_floats(int rows, int d);
// Deferred parameter-gradient fold of norm_bwd: with defer_partial (norm_bwd_defer_slot_floats(d) floats, one slot per
// call) the fused kernel leaves its per-block partial sums there and sets *deferred; norm_bwd_fold_deferred later adds
// every slot into its destinations (offsets into the gradient arena, -1 = absent) in one launch.  *deferred stays
// false when the shape takes a path that folds at once; the caller then must not list that slot.
constexpr int kNormFoldMaxSlots = 64;
struct NormFoldSlots { long long dgamma[kNormFoldMaxSlots], dbeta[kNormFoldMaxSlots], osum[kNormFoldMaxSlots]; };
size_t norm_bwd_defer_slot_floats(int d);
int norm_bwd_fold_deferred(const float* partials, const NormFoldSlots& slots, int n, float* G, int d, cudaStream_t s);
// Deferred fold of the column sums, as for norm_bwd: with `defer` (partial = a buffer of colsum_scratch_floats(rows, cols)
// floats of the caller's) the chunk partials are left there, `chunks` and `deferred` are filled in, and
// colsum_fold_deferred adds every listed slot into its destination later.
struct ColsumDefer { float* partial; int chunks; bool deferred; };
constexpr int kColsumFoldMaxSlots = 64;
struct ColsumFoldSlots { long long dst[kColsumFoldMaxSlots], part[kColsumFoldMaxSlots]; int chunks[kColsumFoldMaxSlots], cols[kColsumFoldMaxSlots]; };
int colsum_fold_deferred(const float* partial_base, const ColsumFoldSlots& slots, int n, float* G, cudaStream_t s);
template <typename T> int colsum_accumulate(const T* g, long long ldg, const T* x, const float* gamma, const float* rinv,
                                            const float* mean, int mode, float* out, float* scratch, int rows, int cols,
                                            cudaStream_t s, int* counters = nullptr, ColsumDefer* defer = nullptr);
constexpr int kColsumCounters = 1024;   // ints a caller-provided, zero-initialised counter array must hold
size_t colsum_scratch_floats(int rows, int cols);
template <typename T> int act_fwd(const T* h1, T* h2, int rows, int ff, bool swiglu, cudaStream_t s);
template <typename T> int act_bwd(const T* g, const T* h1, T* dh1, int rows, int ff, bool swiglu, cudaStream_t s,
                                  float* dbias = nullptr, float* scratch = nullptr, int* counters = nullptr,
                                  ColsumDefer* defer = nullptr);
template <typename T> int cross_entropy(T* logits, const int* labels, const float* mask, float grad_scale,
                                        float* loss_vec, float* stats, float* loss_out, int rows, int V, int vocab,
                                        cudaStream_t s);
int adamw_update(float* p, const float* g, float* m, float* v, bf16* shadow, size_t n, float lr, float beta1, float beta2,
                 float eps, float wd, int t_next, const float* gscale, cudaStream_t s);
size_t sumsq_scratch_floats();
int sum_squares(const float* g, size_t n, float pre_scale, float max_norm, float post_scale, float* scratch, float* out,
                cudaStream_t s);
int muon_momentum(const float* g, float* vel, float* u, size_t n, float mu, const float* gscale, cudaStream_t s);
template <typename T> int muon_normalize(const float* u, const float* sumsq, float eps, T* X, size_t n, cudaStream_t s);
template <typename T> int axpby(const T* a, const T* b, T* out, float alpha, float beta, size_t n, cudaStream_t s);
template <typename T> int muon_apply(float* p, const T* X, bf16* shadow, float lr, size_t n, cudaStream_t s);
int f32_to_bf16(const float* in, bf16* out, size_t n, cudaStream_t s);
int bf16_to_f32(const bf16* in, float* out, size_t n, cudaStream_t s);

// ---- embedding.cu
template <typename T> int embed_fwd(const float* tok_emb, const float* pos_table, const int* tokens, T* x, int n_tok,
                                    int seq, int d, int vocab, cudaStream_t s);
template <typename T> int embed_bwd(float* tok_grad, float* pos_grad, const int* tokens, const T* g, void* scratch,
                                    int batch, int seq, int d, int vocab, cudaStream_t s);
size_t embed_bwd_scratch_bytes(int n_tok);
template <typename T> int rope_apply(T* qkv, const float* table, int ntok, int seq, int heads, int dk, long long ld,
                                    bool backward, cudaStream_t s);
void rope_table_host(int seq, int dk, float* out);   // cos (seq, dk/2) then sin (seq, dk/2)
int ids_from_float(const float* ids_seq_major, int* out_batch_major, int seq, int batch, cudaStream_t s);
template <typename T> int logits_to_reference(const T* logits_token_major, float* out_vocab_major, int tokens, int vocab, cudaStream_t s);
int zero_f32(float* p, size_t n, cudaStream_t s);

// ---- attention_simt.cu / attention_mma.cu
template <typename T> int attention_fwd_simt(const T* qkv, T* out, float* lse, const int* doc, int B, int S, int H, int dk,
                                             int alibi, cudaStream_t s);
template <typename T> int attention_bwd_simt(const T* qkv, const T* out, const T* dout, const float* lse, float* dvec,
                                             T* dqkv, const int* doc, int B, int S, int H, int dk, int alibi,
                                             cudaStream_t s);
int attention_dvec_bf16(const bf16* out, const bf16* dout, float* dvec, int B, int S, int H, int dk, cudaStream_t s);
bool attention_mma_supported(int dk, int d);
// attention_tc.cu : tcgen05 forward (head size 64 or 128, seq a multiple of 128).  doc_ranges (may be null): the table
// attention_doc_ranges fills, 2 ints (min, max document id) per 64 rows, with which fully masked blocks are skipped
bool attention_tc_supported(int dk, int S, int d);
int attention_doc_ranges(const int* doc, int B, int S, int* ranges, cudaStream_t s);
int attention_fwd_tc(const bf16* qkv, bf16* out, float* lse, const int* doc, const int* doc_ranges, int B, int S, int H, int dk,
                     int alibi, cudaStream_t s);
int attention_device_error(int* code);
// attention_tc_bwd.cu : tcgen05 backward (same shape limits)
// have_dvec: dvec already holds rowsum(dout * out) per (batch, head, row) (written by gemm_bf16_dx_rowdot).
// colsum_part: null, or (B S / 32) x 3 d floats that receive the column sums of dqkv over each 32 token rows, every
// element written (summed over the rows they are the bias gradient of the QKV projection)
int attention_bwd_tc(const bf16* qkv, const bf16* out, const bf16* dout, const float* lse, float* dvec, bf16* dqkv,
                     const int* doc, const int* doc_ranges, int B, int S, int H, int dk, int alibi, cudaStream_t s,
                     bool have_dvec = false, float* colsum_part = nullptr);
int attention_bwd_device_error(int* code);
// status word of the fused elementwise kernels that wait on bulk copies (reads and clears)
int fused_device_error(int* code);
int attention_fwd_mma(const bf16* qkv, bf16* out, float* lse, const int* doc, int B, int S, int H, int dk, int alibi,
                      cudaStream_t s);
int attention_bwd_mma(const bf16* qkv, const bf16* out, const bf16* dout, const float* lse, float* dvec, bf16* dqkv,
                      const int* doc, int B, int S, int H, int dk, int alibi, cudaStream_t s);

}  // namespace nnb
