/* nnb200.h — C ABI of the B200 (sm_100a) compute library for neuralnet.cpp's GPT training step.
 *
 * Conventions, the ones of the reference ABI (cuda/cuda_kernels.h:1-9, cuda/cuda_kernels.cu:24-55):
 *   - every entry point returns int: 0 = success, positive = cudaError_t, -1 = shape/argument error,
 *     -2 = driver service unavailable; a one-line message goes to stderr;
 *   - the caller owns every buffer; nothing here allocates or frees device memory (the nnb200_rt_*
 *     runtime family at the end is the one exception); results are written to caller-provided outputs; all work is enqueued on `stream` and returns at once;
 *   - pointers are device pointers unless a parameter says "host"; matrices are row-major.
 * There is no CPU fallback: without a CUDA device every compute entry point fails.
 *
 * Section 1 re-exports, symbol for symbol, the fifteen kernels of cuda/cuda_kernels.h so the
 * reference CudaBackend links against this library unchanged.  Sections 2-5 are new entry points in
 * the same style for what the reference CudaEngine leaves unimplemented or composes from many
 * primitive calls.
 */
#ifndef NNB200_H
#define NNB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ===================================================================================== *
 * 1. Engine primitives, fp32 — same signatures as cuda/cuda_kernels.h                    *
 * ===================================================================================== */

/* C = op(A) x op(B).  Replaces cuda_matmul (cuda_kernels.h:27-32). */
int cuda_matmul(const float* A, const float* B, float* C, size_t A_rows, size_t A_cols, size_t B_rows, size_t B_cols,
                int transA, int transB, void* stream);
/* Same; `handle_ptr` is ignored (no cuBLAS handle is needed) and the stream is the one given to
 * nnb200_set_handle_stream.  Replaces cuda_matmul_with_handle (cuda_kernels.h:37-42). */
int cuda_matmul_with_handle(const float* A, const float* B, float* C, size_t A_rows, size_t A_cols, size_t B_rows,
                            size_t B_cols, int transA, int transB, void* handle_ptr);
int nnb200_set_handle_stream(void* stream);
/* Per-batch C_b = op(A_b) x op(B_b), stacked vertically.  Replaces cuda_batched_matmul (:47-52). */
int cuda_batched_matmul(const float* A, const float* B, float* C, size_t A_rows, size_t A_cols, size_t B_rows,
                        size_t B_cols, unsigned int batch, int transA, int transB, void* stream);
/* op: 0 Neg 1 Exp 2 Log 3 Sqrt 4 Rsqrt 5 Abs 6 Tanh.  Replaces cuda_elementwise_unary (:60-63). */
int cuda_elementwise_unary(const float* A, float* out, unsigned int count, unsigned int op, void* stream);
/* op: 0 Add 1 Sub 2 Mul 3 Div 4 Max 5 Min.  Replaces cuda_elementwise_binary (:67-70). */
int cuda_elementwise_binary(const float* A, const float* B, float* out, unsigned int count, unsigned int op, void* stream);
/* out = op(A, s) or op(s, A).  Replaces cuda_elementwise_binary_scalar (:74-78). */
int cuda_elementwise_binary_scalar(const float* A, float* out, unsigned int count, unsigned int op, float scalar,
                                   int scalar_first, void* stream);
/* out = A + s*B.  Replaces cuda_axpy (:81-84). */
int cuda_axpy(const float* A, const float* B, float* out, unsigned int count, float scalar, void* stream);
/* out = cmp(A, b) ? then_v : else; cmp: 0 Lt 1 Le 2 Gt 3 Ge 4 Eq 5 Ne.  Replaces
 * cuda_elementwise_select_scalar_cond (:88-92). */
int cuda_elementwise_select_scalar_cond(const float* A, const float* then_v, float* out, unsigned int count,
                                        unsigned int cmp, float scalar_b, float scalar_else, void* stream);
/* (rows, cols) -> (rows, 1); mode 0 sum, 1 max, 2 min (2 is an extension).  Replaces cuda_reduce_row (:100-103). */
int cuda_reduce_row(const float* A, float* out, unsigned int rows, unsigned int cols, unsigned int mode, void* stream);
/* (rows, cols) -> (1, cols).  Replaces cuda_reduce_col (:107-110). */
int cuda_reduce_col(const float* A, float* out, unsigned int rows, unsigned int cols, unsigned int mode, void* stream);
/* out[r][c] = op(A[r][c], vec[r]).  Replaces cuda_broadcast_row (:118-121). */
int cuda_broadcast_row(const float* A, const float* vec, float* out, unsigned int rows, unsigned int cols,
                       unsigned int op, void* stream);
/* out[r][c] = op(A[r][c], vec[c]).  Replaces cuda_broadcast_col (:124-127). */
int cuda_broadcast_col(const float* A, const float* vec, float* out, unsigned int rows, unsigned int cols,
                       unsigned int op, void* stream);
/* (R, C) -> (C, R).  Replaces cuda_transpose (:134-137). */
int cuda_transpose(const float* A, float* out, unsigned int R, unsigned int C, void* stream);
/* inverse=0: (M, B*N) -> (B*M, N); inverse=1 the way back.  Replaces cuda_rearrange_3d (:142-146). */
int cuda_rearrange_3d(const float* A, float* out, unsigned int M, unsigned int B, unsigned int N, unsigned int inverse,
                      void* stream);
/* out[i] = table[(int)indices[i]], zero row when out of range.  Replaces cuda_gather (:155-158). */
int cuda_gather(const float* table, const float* indices, float* out, unsigned int vocab, unsigned int D,
                unsigned int num, void* stream);
/* dst[(int)indices[i]] += grad[i], rows added in ascending i — bit-identical to the CPU engine's
 * sequential loop (cpu_engine.hpp:203-214), unlike the reference's atomicAdd kernel.  Replaces
 * cuda_scatter_add (:162-165). */
int cuda_scatter_add(float* dst, const float* indices, const float* grad, unsigned int vocab, unsigned int D,
                     unsigned int num, void* stream);

/* ===================================================================================== *
 * 2. Dense contractions                                                                  *
 * ===================================================================================== */

/* D[M,N] = alpha * A[M,K] * B[N,K]^T (+ bias_n[n]) (+ residual[m,n]), or D += ... when accumulate.
 * a_mn_major = 0: A stored (M, K), K contiguous, row stride lda; 1: stored (K, M), M contiguous.
 * b_mn_major = 0: B stored (N, K), K contiguous, row stride ldb; 1: stored (K, N), N contiguous.
 * bf16 version: TMA-fed tcgen05 tiles, fp32 accumulation in TMEM; A, B bf16; D bf16 (c_bf16=1) or
 * fp32; residual has D's type and ldc; accumulate needs fp32 D and adds atomically (split-K).
 * lda, ldb multiples of 8; A, B 16-byte aligned.  Replaces cublasSgemm + broadcast_row(Add) +
 * add_inplace of Linear::forward/backward (compute_layer.hpp:151-195; cuda_kernels.cu:527-563). */
int nnb200_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                     long long ldc, int a_mn_major, int b_mn_major, int c_bf16, float alpha, const float* bias_n,
                     const void* residual, int accumulate, void* stream);
/* First projection of a SwiGLU feed-forward block with its activation, one launch: h1[M, 2 ff] = x[M, K] W[2 ff, K]^T
 * + bias (rows of W: gate, then up) and h2[M, ff] = gate * sigmoid(gate) * up from the bf16-rounded h1, the values
 * nnb200_gemm_bf16 followed by nnb200_activation_forward(swiglu = 1) give, bit for bit.  All operands bf16, bias fp32
 * or NULL.  Needs M > 128, ff a multiple of 128, K a multiple of 8 (nnb200_linear_swiglu_supported: 1 or 0); -1
 * otherwise.  Replaces Linear::forward + SwiGLU::forward inside FeedForward (compute_layer.hpp:151-195, 375-404). */
int nnb200_linear_swiglu_supported(int M, int ff, int K);
int nnb200_linear_swiglu_forward(const void* x, const void* W, const float* bias, void* h1, void* h2, int M, int ff, int K,
                                 void* stream);
/* Input gradient of a SwiGLU block's second projection taken through the activation, one launch:
 * dh1[M, 2 ff] = (dgate | dup) from the product dY[M, K] W[K, ff] (W stored (K, ff), ff contiguous: the (out, in) weight
 * of Linear) and h1[M, 2 ff] = (gate | up); the product is rounded to bf16 and not stored.  The values
 * nnb200_gemm_bf16 followed by nnb200_activation_backward(swiglu = 1) give, bit for bit.  All matrices bf16.  Needs
 * M > 128, ff > 128 a multiple of 64, K a multiple of 8 (nnb200_linear_swiglu_backward_supported: 1 or 0); -1 otherwise.
 * colsum_partial (may be NULL; 16-byte aligned): ceil(M / 128) rows of 2 ff floats, every one written, row r = the column
 * sums of dh1 over matrix rows [128 r, 128 r + 128): summed over r they are the bias gradient of the first projection
 * (Linear::backward's column sum, compute_layer.hpp:188-193), which then needs no pass over dh1.
 * Replaces the input gradient of Linear::backward + SwiGLU::backward (compute_layer.hpp:176-195, 436-445). */
int nnb200_linear_swiglu_backward_supported(int M, int ff, int K);
int nnb200_linear_swiglu_backward(const void* dY, const void* W, const void* h1, void* dh1, int M, int ff, int K,
                                  float* colsum_partial, void* stream);
/* Input gradient of a projection with a row term, one launch: dX[M, N] = dY[M, K] W[K, N] (W stored (K, N), N
 * contiguous: the (out, in) weight of Linear) and dot[(m / S * H + h) * S + m % S] = sum over the 64 columns of block
 * h of dX (as stored, bf16) * other[m, .], H = N / 64.  With dY the gradient of the attention out-projection's output
 * and other the attention output (heads of 64) this leaves rowsum(dO * O) per (batch, head, row) in the layout
 * nnb200_attention_backward keeps its dvec in.  All matrices bf16, dot fp32.  Needs M > 128, N = 64 H > 128, S | M,
 * K a multiple of 8 (nnb200_gemm_bf16_rowdot_supported: 1 or 0); -1 otherwise.  Replaces Linear::backward's input
 * gradient (compute_layer.hpp:176-195) plus a pass the reference does not have as such: its attention backward forms
 * sum_j P_ij dP_ij inside softmax_backward_q / _kv (compute_layer.hpp:1317-1346). */
int nnb200_gemm_bf16_rowdot_supported(int M, int N, int K, int S, int H);
int nnb200_gemm_bf16_rowdot(const void* dY, const void* W, void* dX, const void* other, float* dot, int M, int N, int K,
                            int S, int H, void* stream);
/* Same contract, fp32 operands and fp32 SIMT arithmetic (the check mode). */
int nnb200_gemm_f32(const float* A, const float* B, float* D, int M, int N, int K, long long lda, long long ldb,
                    long long ldc, int a_mn_major, int b_mn_major, float alpha, const float* bias_n,
                    const float* residual, int accumulate, void* stream);
/* Per-launch timing of the tcgen05 GEMM: enable=1 starts recording a CUDA event pair around every
 * GEMM kernel on its launching stream (and resets the totals), enable=0 stops.  _read synchronises
 * on the recorded events and returns (host) the summed kernel time, the summed algorithmic FLOPs
 * (2*M*N*K per launch) and the number of launches.  Only launches on the stream of the first GEMM after enabling
 * are recorded: pairs of launches that overlap on other streams would add up to more than the time that passed. */
int nnb200_gemm_profile(int enable);
int nnb200_gemm_profile_read(double* host_total_ms, double* host_total_flops, int* host_launches);
/* The launches whose epilogue also runs an activation (nnb200_linear_swiglu_forward / _backward) are kept apart from
 * the figures above, because that epilogue outlasts a short main loop: their totals. */
int nnb200_gemm_profile_read_fused(double* host_total_ms, double* host_total_flops, int* host_launches);
/* CTA pairs (two SMs running one 256 x 256 tile with tcgen05.mma.cta_group::2) the device keeps resident at once;
 * 0 when the pair kernel is unavailable or switched off (environment NNB200_GEMM_PAIR=0). */
int nnb200_gemm_pair_capacity(void);
/* Kernels launched by this library since the last reset (host-side counter). */
unsigned long long nnb200_launch_count(int reset);
/* Reads (host) and clears the device-side status word of the tcgen05 GEMM: 0 = no wait ever gave up. */
int nnb200_gemm_status(int* host_code);

/* ===================================================================================== *
 * 3. Fused attention and the fused memory-bound layers (token-major activations)         *
 *    dtype: 0 = fp32, 1 = bf16 for every activation pointer; statistics are fp32.        *
 * ===================================================================================== */

/* Causal, optionally document-masked and ALiBi-biased attention over qkv (tokens, 3*d) = q|k|v,
 * tokens = batch*seq in batch-major order; out (tokens, d); lse (batch*heads*seq).  doc_ids may be
 * NULL.  In bf16, head sizes 64 and 128 with seq a multiple of 128 run on tcgen05 tensor cores.
 * doc_ranges (NULL, or the table nnb200_attention_doc_ranges made of the same doc_ids) lets those
 * kernels skip the key blocks a document mask leaves nothing of; the result is bit-identical either
 * way.  One fused kernel replaces batched_matmul_reduce/_softmax_denom/_softmax_apply, the
 * materialised-score path (compute_layer.hpp:1193-1252; compute_engine.hpp:217-243) and the
 * (batch*heads*seq, seq) mask build_attention_mask fills on the host (compute_layer.hpp:2081-2128). */
int nnb200_attention_forward(const void* qkv, void* out, float* lse, const int32_t* doc_ids, const int32_t* doc_ranges,
                             int batch, int seq, int heads, int head_dim, int alibi, int dtype, void* stream);
/* dqkv (tokens, 3*d) from dout (tokens, d); dvec is scratch (batch*heads*seq floats).  Replaces
 * batched_matmul_softmax_backward_q/_kv and the materialised backward (compute_layer.hpp:1296-1360). */
int nnb200_attention_backward(const void* qkv, const void* out, const void* dout, const float* lse, float* dvec,
                              void* dqkv, const int32_t* doc_ids, const int32_t* doc_ranges, int batch, int seq, int heads,
                              int head_dim, int alibi, int dtype, void* stream);
/* The same on the tcgen05 kernels only (bf16, head size 64 or 128, seq a multiple of 128; -1 otherwise), which also
 * leave the column sums of dqkv over each 32 token rows in colsum_partial ((batch*seq/32) x 3*d floats, every one
 * written): summed over the rows they are the bias gradient of the QKV projection (Linear::backward's column sum,
 * compute_layer.hpp:188-193), which then needs no pass over dqkv.  dqkv is bit-identical to nnb200_attention_backward's. */
int nnb200_attention_backward_bias_partials(const void* qkv, const void* out, const void* dout, const float* lse, float* dvec,
                                            void* dqkv, const int32_t* doc_ids, const int32_t* doc_ranges,
                                            float* colsum_partial, int batch, int seq, int heads, int head_dim, int alibi,
                                            void* stream);
/* ranges[2*(b*seq/64 + k)], [.. + 1] = smallest and largest document id among rows [64k, 64k+64) of
 * sequence b; seq must be a multiple of 64; ranges holds 2*batch*seq/64 ints.  The device-side
 * counterpart of the per-step mask rebuild of CausalSelfAttention (compute_layer.hpp:2226-2246). */
int nnb200_attention_doc_ranges(const int32_t* doc_ids, int batch, int seq, int32_t* ranges, void* stream);

/* y = norm(x) * gamma (+ beta); layer=1 LayerNorm, 0 RMSNorm; eps 1e-5; rinv (rows), mean (rows,
 * LayerNorm only) are saved for backward.  Replaces LayerNorm/RMSNorm::forward
 * (compute_layer.hpp:541-590, 722-755). */
int nnb200_norm_forward(const void* x, const float* gamma, const float* beta, void* y, float* rinv, float* mean,
                        int rows, int d, int layer, int dtype, void* stream);
/* dx = norm-backward(g) (+ add); dgamma += sum g*gamma*n (the reference's formula, including gamma);
 * dbeta += sum g.  scratch: nnb200_colsum_scratch_floats(rows, d) floats.  Replaces
 * LayerNorm/RMSNorm::backward (compute_layer.hpp:592-654, 757-800). */
int nnb200_norm_backward(const void* g, const void* x, const float* gamma, const float* rinv, const float* mean,
                         const void* add, void* dx, float* dgamma, float* dbeta, float* scratch, int rows, int d,
                         int layer, int dtype, void* stream);
size_t nnb200_colsum_scratch_floats(int rows, int cols);
/* out[c] += sum_r g[r][c] (bias gradient of Linear::backward, compute_layer.hpp:190-193). */
int nnb200_bias_grad(const void* g, long long ldg, float* out, float* scratch, int rows, int cols, int dtype, void* stream);

/* Same result as nnb200_bias_grad for callers that cannot supply scratch memory (no counterpart in
 * the reference: its CudaBackend allocates op outputs only and offers kernels no workspace, and
 * hosts with a device-memory budget fixed at start-up must not call cudaMalloc).  The partial sums
 * go to a buffer built into the library — NNB200_BIAS_GRAD_STATIC_MAX_FLOATS floats (1 MiB) that
 * each GPU holds from library load to exit; shapes needing more (ceil(rows/128)*cols floats) are
 * rejected with -1.  Allocates nothing.  The first call on a device looks the buffer's address up;
 * make that call before any stream capture.  All calls on a device share the buffer, so two calls
 * whose kernels may overlap on the GPU (different streams) race: serialise them. */
#define NNB200_BIAS_GRAD_STATIC_MAX_FLOATS 262144
int nnb200_bias_grad_static(const void* g, long long ldg, float* out, int rows, int cols, int dtype, void* stream);

/* swiglu=0: h2 = h1*sigmoid(1.702*h1) on (rows, ff); swiglu=1: h1 (rows, 2ff) = gate|up,
 * h2 = gate*sigmoid(gate)*up.  Replaces GeLU/SwiGLU::forward (compute_layer.hpp:266-295, 375-404). */
int nnb200_activation_forward(const void* h1, void* h2, int rows, int ff, int swiglu, int dtype, void* stream);
int nnb200_activation_backward(const void* g, const void* h1, void* dh1, int rows, int ff, int swiglu, int dtype,
                               void* stream);

/* Softmax cross-entropy over token rows: logits (rows, V) are overwritten by
 * grad_scale*(softmax - onehot)/num_valid; rows with mask < 0.5 or label >= vocab get zero.
 * stats (2 floats): number of valid rows and its reciprocal; loss_out[0] = -sum(loss_vec)/num_valid.
 * Replaces CrossEntropyLoss::forward_sparse + col_softmax_sparse_forward (compute_loss.hpp:229-309;
 * cpu_engine.hpp:948-1006). */
int nnb200_cross_entropy(void* logits, const int32_t* labels, const float* mask, float grad_scale, float* loss_vec,
                         float* stats, float* loss_out, int rows, int V, int vocab, int dtype, void* stream);

/* x[i] = token_emb[tokens[i]] (+ pos_table[i % seq]); zero row for an id out of range.  Replaces
 * the transpose/gather/transpose/add chain of GPTModel::forward (compute_layer.hpp:2792-2809). */
int nnb200_embedding_forward(const float* token_emb, const float* pos_table, const int32_t* tokens, void* x, int tokens_n,
                             int seq, int d, int vocab, int dtype, void* stream);
/* token_grad[tokens[i]] += g[i] in ascending i (bit-exact against the sequential CPU loop);
 * pos_grad[t] += sum_b g[b*seq+t] when pos_grad != NULL.  scratch: nnb200_embedding_scratch_bytes.
 * Replaces scatter_add_rows in GPTModel::backward (compute_layer.hpp:2882-2891, 2573-2580). */
int nnb200_embedding_backward(float* token_grad, float* pos_grad, const int32_t* tokens, const void* g, void* scratch,
                              int batch, int seq, int d, int vocab, int dtype, void* stream);
size_t nnb200_embedding_scratch_bytes(int tokens_n);

/* Token ids as the reference hands them to GPTModel::forward — a (seq, batch) row-major matrix of floats
 * (compute_layer.hpp:2783-2790) — to the int32 batch-major ids the fused step takes: out[b*seq + t] =
 * (int) ids[t*batch + b]; negative or non-finite values become -1 (out of range: zero embedding row). */
int nnb200_ids_from_float(const float* ids_seq_major, int32_t* out_batch_major, int seq, int batch, void* stream);
/* Logits of the fused step, (tokens, vocab) in the step's precision, to the reference's (vocab, tokens) fp32
 * matrix (the Tensor GPTModel::forward returns, compute_layer.hpp:2836-2838). */
int nnb200_logits_to_reference(const void* logits_token_major, float* out_vocab_major, int tokens, int vocab, int dtype,
                               void* stream);
/* p[0..n) = 0 in one launch; p 16-byte aligned.  Replaces the per-tensor engine.zero calls of
 * Layer::zero_grad / Optimizer::zero_grad (compute_layer.hpp:57-65, compute_optimizer.hpp:141-150). */
int nnb200_zero_f32(float* p, size_t n, void* stream);

/* Rotary position encoding (RotaryEmbedding, compute_layer.hpp:876-988).  nnb200_rope_table fills a HOST buffer of
 * seq*head_dim floats: cos (seq, head_dim/2) then sin (seq, head_dim/2), theta = pos / 10000^(2j/head_dim) computed with
 * the reference's float calls; the caller copies it to the device.  nnb200_rope_apply rotates, in place, the Q and K
 * thirds of a token-major buffer whose rows (length ld) start with heads*head_dim Q then K values, token i at sequence
 * position i % seq: x[j] <- x[j] c - x[j+h/2] s, x[j+h/2] <- x[j+h/2] c + x[j] s; backward=1 applies the inverse
 * rotation (to the gradients).  Replaces RotaryEmbedding::apply and the expression program it submits. */
int nnb200_rope_table(int seq, int head_dim, float* host_out);
int nnb200_rope_apply(void* qkv, const float* table, int tokens_n, int seq, int heads, int head_dim, long long ld, int backward,
                      int dtype, void* stream);

/* ===================================================================================== *
 * 4. Optimizers over flat fp32 ranges                                                    *
 * ===================================================================================== */

/* One fused AdamW update of n parameters: p *= (1 - lr*wd); m, v moments; p -= lr*m^/(sqrt(v^)+eps);
 * the gradient is multiplied by *grad_scale_dev first (NULL = 1); shadow (bf16, may be NULL)
 * receives the rounded parameters.  t_next is the 1-based step.  Replaces the sixteen engine
 * calls per tensor of AdamW::step (compute_optimizer.hpp:252-304, 388-412). */
int nnb200_adamw_step(float* p, const float* g, float* m, float* v, void* shadow_bf16, size_t n, float lr, float beta1,
                      float beta2, float eps, float weight_decay, int t_next, const float* grad_scale_dev, void* stream);
/* out[0] = pre_scale^2 * sum g^2, out[1] = its sqrt (the norm of pre_scale*g),
 * out[2] = (max_norm > 0 && norm > max_norm ? max_norm/norm : 1) * pre_scale — the factor that
 * turns g into the clipped, pre-scaled gradient; scratch: nnb200_sumsq_scratch_floats() floats.
 * Deterministic two-stage reduction.  Replaces Optimizer::clip_grad_norm
 * (compute_optimizer.hpp:90-140) without its host synchronisation. */
int nnb200_grad_norm_clip(const float* g, size_t n, float pre_scale, float max_norm, float* scratch, float* out3,
                          void* stream);
size_t nnb200_sumsq_scratch_floats(void);
/* Muon update of one (rows, cols) matrix: v = mu*v + g; u = g + mu*v; X = u/sqrt(|u|^2 + eps^2);
 * ns_steps Newton-Schulz iterations (a,b,c) = (3.4445,-4.7750,2.0315) as GEMMs; p -= lr*X.
 * precision 0: fp32 GEMMs in the stored orientation; 1: bf16 tcgen05 GEMMs on the short side
 * (NS is an odd polynomial, so NS(X^T) = NS(X)^T).  scratch: nnb200_muon_scratch_bytes.  Replaces
 * Muon::step + newton_schulz_orthogonalize (compute_optimizer.hpp:430-497, 517-590). */
int nnb200_muon_step(float* p, const float* g, float* velocity, void* shadow_bf16, int rows, int cols, float lr,
                     float momentum, int ns_steps, float ns_eps, int precision, void* scratch,
                     const float* grad_scale_dev, void* stream);
size_t nnb200_muon_scratch_bytes(int rows, int cols, int precision);
/* nnb200_muon_step on `count` matrices (host arrays of device pointers and shapes), spread round-robin over `lanes`
 * (1..16) auxiliary streams of the library that start behind `stream` and that `stream` waits for at the end: the
 * Newton-Schulz GEMMs of a hidden matrix fill a fraction of the machine, so several matrices run side by side.
 * scratch holds lanes * scratch_bytes_per_lane bytes, scratch_bytes_per_lane >= nnb200_muon_scratch_bytes of every
 * matrix; shadow_bf16 may be NULL.  The updates are independent, so the result equals `count` single calls.
 * Replaces the loop over parameters of Muon::step (compute_optimizer.hpp:546-587). */
int nnb200_muon_step_many(int count, float* const* p, const float* const* g, float* const* velocity, void* const* shadow_bf16,
                          const int* rows, const int* cols, float lr, float momentum, int ns_steps, float ns_eps, int precision,
                          void* scratch, size_t scratch_bytes_per_lane, int lanes, const float* grad_scale_dev, void* stream);
int nnb200_f32_to_bf16(const float* in, void* out, size_t n, void* stream);
int nnb200_bf16_to_f32(const void* in, float* out, size_t n, void* stream);

/* ===================================================================================== *
 * 5. The fused GPT training step                                                         *
 * ===================================================================================== */

typedef struct nnb200_gpt_config {
    int32_t vocab, d_model, heads, layers, d_ff, seq, batch;
    int32_t act;        /* 0 QuickGeLU, 1 SwiGLU          (ActivationType, model_spec.hpp:33-37) */
    int32_t norm;       /* 0 LayerNorm, 1 RMSNorm         (NormType, model_spec.hpp:40-45)       */
    int32_t pos;        /* 0 learned, 1 sinusoidal, 2 ALiBi, 3 rotary (PosEncodingType, model_spec.hpp:24-30) */
    int32_t precision;  /* 0 fp32 check mode, 1 bf16 tensor-core mode with fp32 master weights   */
    int32_t reserved[5];
} nnb200_gpt_config;

/* Parameters live in one fp32 arena (gradients, moments and the bf16 shadow mirror it element for
 * element).  The arena is [vectors and embeddings | hidden matrices]; within it wq|wk|wv are
 * adjacent so the three projections run as one GEMM.  The table lists the tensors in the
 * reference's parameter order (GPTModel::parameters, compute_layer.hpp:2739-2755): offset (in
 * elements), rows, cols.  Returns the number of tensors; arrays may be NULL to query the count. */
int nnb200_gpt_param_table(const nnb200_gpt_config* cfg, long long* offsets, int32_t* rows, int32_t* cols);
long long nnb200_gpt_arena_elems(const nnb200_gpt_config* cfg);
long long nnb200_gpt_matrix_region_begin(const nnb200_gpt_config* cfg);   /* first element of the hidden matrices */
/* Start (elements) of layer l's matrices inside the arena; l = layers gives the end of the arena. */
long long nnb200_gpt_layer_matrix_begin(const nnb200_gpt_config* cfg, int layer);
long long nnb200_gpt_workspace_bytes(const nnb200_gpt_config* cfg);
/* Byte offset of a named buffer inside the workspace, for inspection: 0 logits (tokens, vocab),
 * 1 loss scalar (1 float), 2 gradient w.r.t. the embedded input (tokens, d), 3 CE stats. */
long long nnb200_gpt_workspace_offset(const nnb200_gpt_config* cfg, int which);
/* Fills the constant tables of the workspace (sinusoidal positions or rotary cos/sin).  Call once, and again after
 * the workspace moved. */
int nnb200_gpt_init_workspace(const nnb200_gpt_config* cfg, void* workspace, void* stream);
/* tokens, doc_ids (NULL = none): int32 (batch*seq), batch-major.  Logits are left in the workspace.
 * Replaces GPTModel::forward (compute_layer.hpp:2783-2839). */
int nnb200_gpt_forward(const nnb200_gpt_config* cfg, const float* params, const void* params_bf16, void* workspace,
                       const int32_t* tokens, const int32_t* doc_ids, void* stream);
/* Loss of the logits in the workspace; overwrites them by their gradient times grad_scale
 * (1/accumulation steps, text_train.cpp:1253-1258).  The scalar loss lands in the workspace. */
int nnb200_gpt_loss(const nnb200_gpt_config* cfg, void* workspace, const int32_t* labels, const float* loss_mask,
                    float grad_scale, void* stream);
/* Adds this micro-batch's parameter gradients into `grads` (arena layout).  layer_events (NULL or
 * layers+2 entries, each a cudaEvent_t or NULL): event[l] is recorded when layer l's matrix gradients
 * are final, event[layers] when every gradient is, event[layers+1] when the LM head's weight gradient
 * is (right after the first GEMM).  Replaces GPTModel::backward (compute_layer.hpp:2841-2896). */
int nnb200_gpt_backward(const nnb200_gpt_config* cfg, const float* params, const void* params_bf16, float* grads,
                        void* workspace, const int32_t* tokens, const int32_t* doc_ids, void* const* layer_events,
                        void* stream);

/* Incremental inference with a key/value cache (GPTModel::forward_step, compute_layer.hpp:2906-2950; the per-block
 * step :1426-1511; ALiBi bias of a step :2267-2290).  The decode workspace holds the cache of every layer
 * (layers x {K, V} x seq x d_model, fp32), the position tables and one token's activations; cfg->batch is not used
 * (one sequence).  _init fills the sinusoidal / rotary tables: call once, and again after the workspace moved.
 * _forward_step runs token `token_id` at cache row `cur_len` (0 <= cur_len < seq; rows [0, cur_len) must hold the
 * earlier tokens of the context) with position encoding index `pos`, appends its key and value to the cache and
 * writes the (vocab) fp32 logits to logits_out (device; NULL = left in the workspace).  Weights are read as bf16
 * (params_bf16, bf16 mode) or fp32 (check mode); activations and the cache are fp32 in both. */
long long nnb200_gpt_decode_workspace_bytes(const nnb200_gpt_config* cfg);
int nnb200_gpt_decode_init(const nnb200_gpt_config* cfg, void* workspace, void* stream);
int nnb200_gpt_forward_step(const nnb200_gpt_config* cfg, const float* params, const void* params_bf16, void* workspace, int token_id,
                            int pos, int cur_len, float* logits_out, void* stream);
/* The same step with the token id, the position and the cache length read from device memory (three int32 at
 * step_dev, which the caller fills before the call; they are not validated: 0 <= position, cache length < seq).  Every
 * launch of this call is the same whatever the three values are, so a caller may capture it in a CUDA graph once and
 * replay it per token after updating step_dev.  No counterpart in the reference, which builds its step on the host. */
int nnb200_gpt_forward_step_dev(const nnb200_gpt_config* cfg, const float* params, const void* params_bf16, void* workspace,
                                const int32_t* step_dev, float* logits_out, void* stream);
/* Writes the three values nnb200_gpt_forward_step_dev reads (a one-thread kernel on `stream`: ordered with the step
 * without pinned host memory).  Helper, no counterpart in the reference. */
int nnb200_gpt_decode_set_step(int32_t* step_dev, int token_id, int pos, int cur_len, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Engine primitives in the reference's own layouts (fp32; matrices row-major, batch blocks stacked
 * along rows).  These are the ComputeEngine virtuals the reference's CudaEngine answers "not
 * implemented" to (cuda_engine.hpp:213-261, 461-469); with them the unchanged reference layers run
 * on the device one primitive at a time.  Semantics follow the CPU engine.
 * A_b is (M,K) (stored (K,M) when transA), B_b is (K,N) (stored (N,K) when transB); S = alpha*A_b*B_b
 * + mask, mask (M,N) shared by the batch or NULL. */

/* cuda_batched_matmul with the alpha factor of ComputeEngine::batched_matmul (compute_engine.hpp:72-79). */
int nnb200_batched_matmul(const float* A, const float* B, float* C, size_t A_rows, size_t A_cols, size_t B_rows, size_t B_cols,
                          unsigned int batch, int transA, int transB, float alpha, void* stream);
/* op 0 Sum, 1 Max, 2 Min over the columns (reduce_cols=1, out (batch*M)) or rows (0, out (batch*N)) of S;
 * entries whose mask is -inf are skipped for Sum and Min.  cpu_engine.hpp:426-515. */
int nnb200_bmm_reduce(const float* A, const float* B, const float* mask, float* out, int batch, int M, int N, int K, int op,
                      int transA, int transB, float alpha, int reduce_cols, void* stream);
/* out[b*M+i] = sum_j exp(S_ij - row_max[b*M+i]) over unmasked j.  cpu_engine.hpp:517-590. */
int nnb200_bmm_softmax_denom(const float* A, const float* B, const float* row_max, const float* mask, float* out, int batch,
                             int M, int N, int K, int transA, int transB, float alpha, void* stream);
/* out (batch*M, D) = softmax(S) * V, V (batch*N, D).  cpu_engine.hpp:592-680. */
int nnb200_bmm_softmax_apply(const float* A, const float* B, const float* V, const float* row_max, const float* denom,
                             const float* mask, float* out, int batch, int M, int N, int K, int D, int transA, int transB,
                             float alpha, void* stream);
/* P (batch*M, N) is the gradient w.r.t. the weights.  r_out[b*M+i] = sum_j W_ij P_ij;
 * grad_q (batch*K, M) = alpha * B_b * (W o (P - R))^T.  cpu_engine.hpp:682-790. */
int nnb200_bmm_softmax_backward_q(const float* A, const float* B, const float* P, const float* row_max, const float* denom,
                                  const float* mask, float* grad_q, float* r_out, int batch, int M, int N, int K, int transA,
                                  int transB, float alpha, void* stream);
/* grad_k (batch*K, N) = alpha * A_b^T * (W o (P - R)); grad_v (batch*K, N) = (W^T * G[:, :K])^T with
 * G (batch*M, D), D >= K (the reference sizes grad_v by K).  cpu_engine.hpp:792-915. */
int nnb200_bmm_softmax_backward_kv(const float* A, const float* B, const float* P, const float* G, const float* R,
                                   const float* row_max, const float* denom, const float* mask, float* grad_k, float* grad_v,
                                   int batch, int M, int N, int K, int D, int transA, int transB, float alpha, void* stream);
/* logits (classes, tokens): out[n] = sum_r exp(logits[r][n] - col_max[n]).  cpu_engine.hpp:922-946. */
int nnb200_col_softmax_denom(const float* logits, const float* col_max, float* out, int classes, int tokens, void* stream);
/* Fused sparse cross-entropy on (classes, tokens) logits with float labels: grad (classes, tokens) =
 * inv_num_valid*(softmax - onehot), loss_vec[n] = log-probability of the label; a column whose mask
 * is < 0.5 or whose label is >= vocab_size gets zeros.  cpu_engine.hpp:948-1006. */
int nnb200_col_softmax_sparse_forward(const float* logits, const float* labels, const float* mask, float* grad, float* loss_vec,
                                      int classes, int tokens, int vocab_size, float inv_num_valid, void* stream);

/* Element-wise expression programs: the flat form of the reference's ExprSpec (expr_spec.hpp:30-180).
 * instrs[i] = {op, dst, a.kind, a.idx, b.kind, b.idx, c.kind, c.idx} with the reference's numbering of
 * operators (0-23), operand kinds (0-4) and view kinds (0-8). */
#define NNB200_EXPR_MAX_INPUTS 8
#define NNB200_EXPR_MAX_CONSTS 16
#define NNB200_EXPR_MAX_REGS 16
#define NNB200_EXPR_MAX_INSTRS 64
typedef struct nnb200_expr_program {
    uint32_t num_instrs, num_regs, num_inputs, num_consts;
    uint8_t instrs[NNB200_EXPR_MAX_INSTRS][8];
    uint8_t view_kind[NNB200_EXPR_MAX_INPUTS];
    uint8_t view_negate[NNB200_EXPR_MAX_INPUTS];
    uint32_t view_param[NNB200_EXPR_MAX_INPUTS];
    float consts[NNB200_EXPR_MAX_CONSTS];
} nnb200_expr_program;
/* -1 element-wise, 0 all reductions by row, 1 all by column, -2 mixed (expr_spec_reduce_axis). */
int nnb200_expr_reduce_axis(const nnb200_expr_program* prog);
size_t nnb200_eval_expr_scratch_floats(int rows, int cols);
/* ComputeEngine::eval_expr (vector_out=0: out (rows, cols)) and eval_expr_reduce (vector_out=1: out
 * (rows,1) for a row reduction, (1,cols) for a column reduction).  inputs[k] has shape
 * (input_rows[k], input_cols[k]), checked against views as the CPU engine does; an invalid program or
 * shape prints the reason and returns -1.  cpu_engine.hpp:1280-1659. */
int nnb200_eval_expr(const nnb200_expr_program* prog, const float* const* inputs, const int* input_rows, const int* input_cols,
                     float* out, float* scratch, int rows, int cols, int vector_out, void* stream);

/* Device runtime of the C++ drop-in engine (the one family of entry points that owns memory): device
 * selection, one compute stream, stream-ordered blocks from the device's default memory pool, blocking
 * host<->device copies.  Replaces CudaBackend::initialize, CudaBuffer::allocate/~CudaBuffer,
 * upload_blocking, download_blocking and sync_stream (backend/cuda_backend.hpp:66-125, 207-337).
 * device < 0 picks LOCAL_RANK (one process per GPU) or 0.  The first call wins; later calls only
 * report the device's name, memory and SM count. */
int nnb200_rt_init(int device, char* name_out, size_t name_len, size_t* total_mem, int* sm_count);
int nnb200_rt_device(void);                     /* -1 before nnb200_rt_init */
void* nnb200_rt_stream(void);
int nnb200_rt_alloc(size_t bytes, void** out);  /* valid for work queued on the runtime's stream */
int nnb200_rt_free(void* p);                    /* returns the block once the work queued so far has run */
int nnb200_rt_upload(void* dst, const void* host_src, size_t bytes);
int nnb200_rt_download(void* host_dst, const void* src, size_t bytes);
int nnb200_rt_copy(void* dst, const void* src, size_t bytes);
int nnb200_rt_zero(void* dst, size_t bytes);
int nnb200_rt_sync(void);
/* A pair of CUDA events on the runtime's stream: _stop waits for the queue up to it and returns (host) the device
 * time since _start in milliseconds.  The reference times its loop on the host clock (text_train.cpp:1107). */
int nnb200_rt_timer_start(void);
int nnb200_rt_timer_stop(float* host_ms);

#ifdef __cplusplus
}
#endif
#endif /* NNB200_H */
