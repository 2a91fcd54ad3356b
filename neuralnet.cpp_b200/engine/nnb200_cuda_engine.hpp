// Stand-in for the reference's cuda_engine.hpp: class nn::CudaEngine, a ComputeEngine
// (compute_engine.hpp:60-413) whose every virtual runs on the device through the C ABI of libnnb200.
// It defines the reference header's include guard; force-include it after nnb200_cuda_backend.hpp.
//
// Differences from the reference CudaEngine (cuda_engine.hpp:24-486), by design:
//   - the nine members it answers "not implemented" to (the five fused attention primitives, the two
//     fused cross-entropy primitives, eval_expr, eval_expr_reduce) are implemented, so the reference's
//     layers, losses and expression DSL run unchanged with --cuda;
//   - the *_inplace members write into A's own buffer, as the CPU engine does, instead of rebinding A
//     to a fresh tensor (which detached A from reshape() views of the same buffer);
//   - shapes come from the Tensor, not from the CudaTensor beneath it, so reshape() views work;
//   - shape errors the CPU engine reports are reported here with the same texts.
// Host tensors given to an op are uploaded first (ensure_cuda), as in the reference.
#ifndef NN_CUDA_ENGINE_HPP
#define NN_CUDA_ENGINE_HPP
#ifdef NN_HAS_CUDA

#include <array>
#include <cstring>
#include <limits>

#include "neuralnet.cpp/compute_engine.hpp"

namespace nn
{

class CudaEngine final : public ComputeEngine
{
private:
    CudaBackend& backend_;

    using Err = std::unexpected<Error>;
    static Err fail(std::string msg) { return std::unexpected(Error{std::move(msg)}); }
    [[nodiscard]] void* stream() const noexcept { return backend_.stream_ptr(); }
    [[nodiscard]] static float* ptr(const Tensor& t) noexcept { return t.cuda_tensor().data(); }

    [[nodiscard]] Result<Tensor> alloc(std::size_t rows, std::size_t cols)
    {
        auto r = CudaTensor::create_empty(rows, cols, backend_);
        if (!r) return std::unexpected(r.error());
        return Tensor::from_cuda(std::move(*r));
    }
    // device copy of a host tensor; a device tensor passes through (shares its buffer)
    [[nodiscard]] Result<Tensor> ensure_cuda(const Tensor& t)
    {
        if (t.is_gpu()) return t;
        if (!t.valid()) return fail("ensure_cuda: invalid tensor");
        auto r = CudaTensor::from_matrix(t.cpu_matrix(), backend_);
        if (!r) return std::unexpected(r.error());
        return Tensor::from_cuda(std::move(*r));
    }
    [[nodiscard]] static Result<void> ok(int rc, const char* what) { return cuda_detail::check(rc, what); }
    [[nodiscard]] static bool fits_u32(std::size_t n) noexcept { return n <= std::numeric_limits<std::uint32_t>::max(); }
    [[nodiscard]] static unsigned u32(std::size_t n) noexcept { return static_cast<unsigned>(n); }

    // shapes shared by the five fused attention primitives (cpu_engine.hpp:436-448)
    struct BmmShape { int batch, M, N, K; };
    [[nodiscard]] static Result<BmmShape> bmm_shape(const char* name, const Tensor& A, const Tensor& B, std::size_t batch,
                                                   bool transA, bool transB, const Tensor* mask)
    {
        const std::string n(name);
        if (batch == 0) return fail(n + ": batch must be > 0");
        if (A.rows() % batch != 0 || B.rows() % batch != 0) return fail(n + ": rows not divisible by batch");
        const std::size_t a_rpb = A.rows() / batch, b_rpb = B.rows() / batch;
        const std::size_t M = transA ? A.cols() : a_rpb, K = transA ? a_rpb : A.cols();
        const std::size_t K2 = transB ? B.cols() : b_rpb, N = transB ? b_rpb : B.cols();
        if (K != K2) return fail(n + ": K dimension mismatch");
        if (mask && (mask->rows() != M || mask->cols() != N)) return fail(n + ": mask shape mismatch");
        constexpr std::size_t lim = std::numeric_limits<int>::max();
        if (batch > lim || M > lim || N > lim || K > lim) return fail(n + ": dimension exceeds int range");
        return BmmShape{static_cast<int>(batch), static_cast<int>(M), static_cast<int>(N), static_cast<int>(K)};
    }
    [[nodiscard]] static bool is_col_vector(const Tensor& t, std::size_t rows) noexcept { return t.rows() == rows && t.cols() == 1; }

public:
    explicit CudaEngine(CudaBackend& backend) : backend_(backend) {}

    [[nodiscard]] Device device() const noexcept override { return Device::GPU; }
    [[nodiscard]] Result<void> begin_batch() override { return backend_.begin_batch(); }
    [[nodiscard]] Result<void> end_batch() override { return backend_.end_batch(); }
    [[nodiscard]] Result<void> flush_batch() override { return {}; }
    [[nodiscard]] Result<void> begin_expr() override { return {}; }
    [[nodiscard]] Result<void> end_expr() override { return {}; }

    // ── tensors ────────────────────────────────────────────────────────────────────────────────
    [[nodiscard]] Tensor create_tensor(std::size_t rows, std::size_t cols) override
    {
        auto r = alloc(rows, cols);
        return r ? std::move(*r) : Tensor();
    }
    [[nodiscard]] Result<Tensor> from_matrix(const Matrix& m) override
    {
        auto r = CudaTensor::from_matrix(m, backend_);
        if (!r) return std::unexpected(r.error());
        return Tensor::from_cuda(std::move(*r));
    }
    [[nodiscard]] Result<Matrix> to_matrix(const Tensor& t) override
    {
        if (t.is_cpu()) return Matrix(t.cpu_matrix());
        if (!t.valid()) return fail("to_matrix: invalid tensor");
        Matrix m(t.rows(), t.cols());
        if (auto r = ok(nnb200_rt_download(m.span().data(), ptr(t), t.size() * sizeof(float)), "download"); !r)
            return std::unexpected(r.error());
        return m;
    }
    [[nodiscard]] Result<void> copy_from(Tensor& dst, const Matrix& src) override
    {
        if (dst.rows() != src.rows() || dst.cols() != src.cols()) return fail("copy_from: shape mismatch");
        if (dst.is_cpu())
        {
            dst = Tensor::from_matrix(Matrix(src));
            return {};
        }
        return ok(nnb200_rt_upload(ptr(dst), src.span().data(), src.size() * sizeof(float)), "upload");
    }
    [[nodiscard]] Result<Tensor> clone(const Tensor& src) override
    {
        if (src.is_cpu()) return Tensor::from_matrix(Matrix(src.cpu_matrix()));
        auto out = alloc(src.rows(), src.cols());
        if (!out) return out;
        if (auto r = ok(nnb200_rt_copy(ptr(*out), ptr(src), src.size() * sizeof(float)), "device copy"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<Tensor> slice_rows(const Tensor& src, std::size_t start_row, std::size_t count) override
    {
        auto s = ensure_cuda(src);
        if (!s) return s;
        if (start_row + count > s->rows()) return fail("slice_rows: range out of bounds");
        auto out = alloc(count, s->cols());
        if (!out) return out;
        if (auto r = ok(nnb200_rt_copy(ptr(*out), ptr(*s) + start_row * s->cols(), count * s->cols() * sizeof(float)),
                        "device copy"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<void> insert_rows(Tensor& dst, std::size_t dst_start_row, const Tensor& src) override
    {
        if (dst.is_cpu()) return fail("CudaEngine::insert_rows: dst must be a CUDA tensor");
        auto s = ensure_cuda(src);
        if (!s) return std::unexpected(s.error());
        if (dst.cols() != s->cols()) return fail("insert_rows: column count mismatch");
        if (dst_start_row + s->rows() > dst.rows()) return fail("insert_rows: range out of bounds");
        return ok(nnb200_rt_copy(ptr(dst) + dst_start_row * dst.cols(), ptr(*s), s->size() * sizeof(float)), "device copy");
    }
    [[nodiscard]] Result<Tensor> gather_rows(const Tensor& table, const Tensor& indices) override
    {
        auto t = ensure_cuda(table);
        if (!t) return t;
        auto i = ensure_cuda(indices);
        if (!i) return i;
        if (!fits_u32(t->rows()) || !fits_u32(t->cols()) || !fits_u32(i->size())) return fail("gather_rows: dimension exceeds 32 bits");
        auto out = alloc(i->size(), t->cols());
        if (!out) return out;
        if (auto r = ok(cuda_gather(ptr(*t), ptr(*i), ptr(*out), u32(t->rows()), u32(t->cols()), u32(i->size()), stream()),
                        "cuda_gather"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<void> scatter_add_rows(Tensor& dst, const Tensor& indices, const Tensor& grad) override
    {
        if (!dst.is_gpu()) return fail("scatter_add_rows: dst must be GPU tensor");
        if (dst.cols() != grad.cols()) return fail("scatter_add_rows: column count mismatch");
        auto i = ensure_cuda(indices);
        if (!i) return std::unexpected(i.error());
        auto g = ensure_cuda(grad);
        if (!g) return std::unexpected(g.error());
        if (g->rows() < i->size()) return fail("scatter_add_rows: fewer gradient rows than indices");
        if (!fits_u32(dst.rows()) || !fits_u32(dst.cols()) || !fits_u32(i->size())) return fail("scatter_add_rows: dimension exceeds 32 bits");
        return ok(cuda_scatter_add(ptr(dst), ptr(*i), ptr(*g), u32(dst.rows()), u32(dst.cols()), u32(i->size()), stream()),
                  "cuda_scatter_add");
    }
    [[nodiscard]] Result<Tensor> rearrange_3d(const Tensor& x, std::size_t M, std::size_t B, std::size_t N, bool inverse) override
    {
        auto xs = ensure_cuda(x);
        if (!xs) return xs;
        if (M * B * N != xs->size()) return fail("rearrange_3d: element count mismatch");
        if (!fits_u32(M) || !fits_u32(B) || !fits_u32(N)) return fail("rearrange_3d: dimension exceeds 32 bits");
        auto out = inverse ? alloc(M, B * N) : alloc(B * M, N);
        if (!out) return out;
        if (auto r = ok(cuda_rearrange_3d(ptr(*xs), ptr(*out), u32(M), u32(B), u32(N), inverse ? 1u : 0u, stream()),
                        "cuda_rearrange_3d"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<Tensor> transpose(const Tensor& A) override
    {
        auto a = ensure_cuda(A);
        if (!a) return a;
        if (!fits_u32(a->rows()) || !fits_u32(a->cols())) return fail("transpose: dimension exceeds 32 bits");
        auto out = alloc(a->cols(), a->rows());
        if (!out) return out;
        if (auto r = ok(cuda_transpose(ptr(*a), ptr(*out), u32(a->rows()), u32(a->cols()), stream()), "cuda_transpose"); !r)
            return std::unexpected(r.error());
        return out;
    }

    // ── contractions ───────────────────────────────────────────────────────────────────────────
    [[nodiscard]] Result<Tensor> matmul(const Tensor& A, const Tensor& B, bool transA, bool transB) override
    {
        auto a = ensure_cuda(A);
        if (!a) return a;
        auto b = ensure_cuda(B);
        if (!b) return b;
        const std::size_t M = transA ? a->cols() : a->rows(), K = transA ? a->rows() : a->cols();
        const std::size_t N = transB ? b->rows() : b->cols(), K2 = transB ? b->cols() : b->rows();
        if (K != K2) return fail("matmul: dimension mismatch A=" + A.shape_str() + " B=" + B.shape_str());
        auto out = alloc(M, N);
        if (!out) return out;
        if (auto r = ok(cuda_matmul(ptr(*a), ptr(*b), ptr(*out), a->rows(), a->cols(), b->rows(), b->cols(), transA, transB,
                                    stream()), "cuda_matmul"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<Tensor> batched_matmul(const Tensor& A, const Tensor& B, std::size_t batch, bool transA, bool transB,
                                                Scalar alpha) override
    {
        auto a = ensure_cuda(A);
        if (!a) return a;
        auto b = ensure_cuda(B);
        if (!b) return b;
        auto sh = bmm_shape("batched_matmul", *a, *b, batch, transA, transB, nullptr);
        if (!sh) return std::unexpected(sh.error());
        auto out = alloc(batch * static_cast<std::size_t>(sh->M), static_cast<std::size_t>(sh->N));
        if (!out) return out;
        if (auto r = ok(nnb200_batched_matmul(ptr(*a), ptr(*b), ptr(*out), a->rows(), a->cols(), b->rows(), b->cols(),
                                              u32(batch), transA, transB, alpha, stream()), "nnb200_batched_matmul"); !r)
            return std::unexpected(r.error());
        return out;
    }

    // ── fused attention primitives (cpu_engine.hpp:426-915) ───────────────────────────────────
    [[nodiscard]] Result<Tensor> batched_matmul_reduce(const Tensor& A, const Tensor& B, std::size_t batch, ReduceOp op,
                                                       bool transA, bool transB, Scalar alpha, bool reduce_cols,
                                                       const Tensor* mask) override
    {
        auto a = ensure_cuda(A);
        if (!a) return a;
        auto b = ensure_cuda(B);
        if (!b) return b;
        Tensor mk;
        if (mask) { auto m = ensure_cuda(*mask); if (!m) return m; mk = std::move(*m); }
        auto sh = bmm_shape("batched_matmul_reduce", *a, *b, batch, transA, transB, mask);
        if (!sh) return std::unexpected(sh.error());
        auto out = reduce_cols ? alloc(batch * static_cast<std::size_t>(sh->M), 1) : alloc(batch, static_cast<std::size_t>(sh->N));
        if (!out) return out;
        if (auto r = ok(nnb200_bmm_reduce(ptr(*a), ptr(*b), mask ? ptr(mk) : nullptr, ptr(*out), sh->batch, sh->M, sh->N, sh->K,
                                          static_cast<int>(op), transA, transB, alpha, reduce_cols, stream()),
                        "nnb200_bmm_reduce"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<Tensor> batched_matmul_softmax_denom(const Tensor& A, const Tensor& B, const Tensor& row_max,
                                                              std::size_t batch, bool transA, bool transB, Scalar alpha,
                                                              const Tensor* mask) override
    {
        constexpr const char* name = "batched_matmul_softmax_denom";
        auto a = ensure_cuda(A);
        if (!a) return a;
        auto b = ensure_cuda(B);
        if (!b) return b;
        auto rm = ensure_cuda(row_max);
        if (!rm) return rm;
        Tensor mk;
        if (mask) { auto m = ensure_cuda(*mask); if (!m) return m; mk = std::move(*m); }
        auto sh = bmm_shape(name, *a, *b, batch, transA, transB, mask);
        if (!sh) return std::unexpected(sh.error());
        const std::size_t bm = batch * static_cast<std::size_t>(sh->M);
        if (!is_col_vector(*rm, bm)) return fail(std::string(name) + ": row_max shape mismatch");
        auto out = alloc(bm, 1);
        if (!out) return out;
        if (auto r = ok(nnb200_bmm_softmax_denom(ptr(*a), ptr(*b), ptr(*rm), mask ? ptr(mk) : nullptr, ptr(*out), sh->batch,
                                                 sh->M, sh->N, sh->K, transA, transB, alpha, stream()),
                        "nnb200_bmm_softmax_denom"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<Tensor> batched_matmul_softmax_apply(const Tensor& A, const Tensor& B, const Tensor& V,
                                                              const Tensor& row_max, const Tensor& denom, std::size_t batch,
                                                              bool transA, bool transB, Scalar alpha, const Tensor* mask) override
    {
        constexpr const char* name = "batched_matmul_softmax_apply";
        auto a = ensure_cuda(A);
        if (!a) return a;
        auto b = ensure_cuda(B);
        if (!b) return b;
        auto v = ensure_cuda(V);
        if (!v) return v;
        auto rm = ensure_cuda(row_max);
        if (!rm) return rm;
        auto dn = ensure_cuda(denom);
        if (!dn) return dn;
        Tensor mk;
        if (mask) { auto m = ensure_cuda(*mask); if (!m) return m; mk = std::move(*m); }
        auto sh = bmm_shape(name, *a, *b, batch, transA, transB, mask);
        if (!sh) return std::unexpected(sh.error());
        const std::size_t bm = batch * static_cast<std::size_t>(sh->M), D = v->cols();
        if (v->rows() / batch != static_cast<std::size_t>(sh->N)) return fail(std::string(name) + ": V rows per batch != N");
        if (!is_col_vector(*rm, bm)) return fail(std::string(name) + ": row_max shape mismatch");
        if (!is_col_vector(*dn, bm)) return fail(std::string(name) + ": denom shape mismatch");
        auto out = alloc(bm, D);
        if (!out) return out;
        if (auto r = ok(nnb200_bmm_softmax_apply(ptr(*a), ptr(*b), ptr(*v), ptr(*rm), ptr(*dn), mask ? ptr(mk) : nullptr,
                                                 ptr(*out), sh->batch, sh->M, sh->N, sh->K, static_cast<int>(D), transA, transB,
                                                 alpha, stream()), "nnb200_bmm_softmax_apply"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<Tensor> batched_matmul_softmax_backward_q(const Tensor& A, const Tensor& B, const Tensor& P,
                                                                   const Tensor& row_max, const Tensor& denom,
                                                                   std::size_t batch, bool transA, bool transB, Scalar alpha,
                                                                   Tensor& r_out, const Tensor* mask) override
    {
        constexpr const char* name = "batched_matmul_softmax_backward_q";
        auto a = ensure_cuda(A);
        if (!a) return a;
        auto b = ensure_cuda(B);
        if (!b) return b;
        auto p = ensure_cuda(P);
        if (!p) return p;
        auto rm = ensure_cuda(row_max);
        if (!rm) return rm;
        auto dn = ensure_cuda(denom);
        if (!dn) return dn;
        Tensor mk;
        if (mask) { auto m = ensure_cuda(*mask); if (!m) return m; mk = std::move(*m); }
        auto sh = bmm_shape(name, *a, *b, batch, transA, transB, mask);
        if (!sh) return std::unexpected(sh.error());
        const std::size_t bm = batch * static_cast<std::size_t>(sh->M);
        if (p->rows() != bm || p->cols() != static_cast<std::size_t>(sh->N)) return fail(std::string(name) + ": P shape mismatch");
        if (!is_col_vector(*rm, bm)) return fail(std::string(name) + ": row_max shape mismatch");
        if (!is_col_vector(*dn, bm)) return fail(std::string(name) + ": denom shape mismatch");
        auto out = alloc(batch * static_cast<std::size_t>(sh->K), static_cast<std::size_t>(sh->M));
        if (!out) return out;
        auto rv = alloc(bm, 1);
        if (!rv) return rv;
        if (auto r = ok(nnb200_bmm_softmax_backward_q(ptr(*a), ptr(*b), ptr(*p), ptr(*rm), ptr(*dn), mask ? ptr(mk) : nullptr,
                                                      ptr(*out), ptr(*rv), sh->batch, sh->M, sh->N, sh->K, transA, transB,
                                                      alpha, stream()), "nnb200_bmm_softmax_backward_q"); !r)
            return std::unexpected(r.error());
        r_out = std::move(*rv);
        return out;
    }
    [[nodiscard]] Result<Tensor> batched_matmul_softmax_backward_kv(const Tensor& A, const Tensor& B, const Tensor& P,
                                                                    const Tensor& G, const Tensor& R, const Tensor& row_max,
                                                                    const Tensor& denom, std::size_t batch, bool transA,
                                                                    bool transB, Scalar alpha, Tensor& grad_v_out,
                                                                    const Tensor* mask) override
    {
        constexpr const char* name = "batched_matmul_softmax_backward_kv";
        auto a = ensure_cuda(A);
        if (!a) return a;
        auto b = ensure_cuda(B);
        if (!b) return b;
        auto p = ensure_cuda(P);
        if (!p) return p;
        auto g = ensure_cuda(G);
        if (!g) return g;
        auto rr = ensure_cuda(R);
        if (!rr) return rr;
        auto rm = ensure_cuda(row_max);
        if (!rm) return rm;
        auto dn = ensure_cuda(denom);
        if (!dn) return dn;
        Tensor mk;
        if (mask) { auto m = ensure_cuda(*mask); if (!m) return m; mk = std::move(*m); }
        auto sh = bmm_shape(name, *a, *b, batch, transA, transB, mask);
        if (!sh) return std::unexpected(sh.error());
        const std::size_t bm = batch * static_cast<std::size_t>(sh->M), bk = batch * static_cast<std::size_t>(sh->K);
        if (p->rows() != bm || p->cols() != static_cast<std::size_t>(sh->N)) return fail(std::string(name) + ": P shape mismatch");
        if (g->rows() != bm) return fail(std::string(name) + ": G rows != batch*M");
        if (!is_col_vector(*rr, bm)) return fail(std::string(name) + ": R shape mismatch");
        if (!is_col_vector(*rm, bm)) return fail(std::string(name) + ": row_max shape mismatch");
        if (!is_col_vector(*dn, bm)) return fail(std::string(name) + ": denom shape mismatch");
        // the reference sizes grad_v by K and reads the first K columns of G (cpu_engine.hpp:870-908)
        if (g->cols() < static_cast<std::size_t>(sh->K)) return fail(std::string(name) + ": G has fewer than K columns");
        auto gk = alloc(bk, static_cast<std::size_t>(sh->N));
        if (!gk) return gk;
        auto gv = alloc(bk, static_cast<std::size_t>(sh->N));
        if (!gv) return gv;
        if (auto r = ok(nnb200_bmm_softmax_backward_kv(ptr(*a), ptr(*b), ptr(*p), ptr(*g), ptr(*rr), ptr(*rm), ptr(*dn),
                                                       mask ? ptr(mk) : nullptr, ptr(*gk), ptr(*gv), sh->batch, sh->M, sh->N,
                                                       sh->K, static_cast<int>(g->cols()), transA, transB, alpha, stream()),
                        "nnb200_bmm_softmax_backward_kv"); !r)
            return std::unexpected(r.error());
        grad_v_out = std::move(*gv);
        return gk;
    }

    // ── fused cross-entropy primitives (cpu_engine.hpp:922-1006) ──────────────────────────────
    [[nodiscard]] Result<Tensor> col_softmax_denom(const Tensor& logits, const Tensor& col_max) override
    {
        auto l = ensure_cuda(logits);
        if (!l) return l;
        auto m = ensure_cuda(col_max);
        if (!m) return m;
        if (m->rows() != 1 || m->cols() != l->cols()) return fail("col_softmax_denom: col_max shape mismatch");
        auto out = alloc(1, l->cols());
        if (!out) return out;
        if (auto r = ok(nnb200_col_softmax_denom(ptr(*l), ptr(*m), ptr(*out), static_cast<int>(l->rows()),
                                                 static_cast<int>(l->cols()), stream()), "nnb200_col_softmax_denom"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<Tensor> col_softmax_sparse_forward(const Tensor& logits, const Tensor& labels, const Tensor* mask,
                                                            std::size_t vocab_size, Scalar inv_num_valid,
                                                            Tensor& loss_vec_out) override
    {
        if (vocab_size > (std::size_t{1} << 24))
            return fail("col_softmax_sparse_forward: vocab_size exceeds 2^24 (float labels not exactly representable)");
        auto l = ensure_cuda(logits);
        if (!l) return l;
        auto lb = ensure_cuda(labels);
        if (!lb) return lb;
        Tensor mk;
        if (mask) { auto m = ensure_cuda(*mask); if (!m) return m; mk = std::move(*m); }
        const std::size_t C = l->rows(), N = l->cols();
        if (lb->rows() != 1 || lb->cols() != N) return fail("col_softmax_sparse_forward: labels shape mismatch");
        if (vocab_size > C) return fail("col_softmax_sparse_forward: vocab_size > classes");
        if (mask && (mask->rows() != 1 || mask->cols() != N)) return fail("col_softmax_sparse_forward: mask shape mismatch");
        auto grad = alloc(C, N);
        if (!grad) return grad;
        auto lv = alloc(1, N);
        if (!lv) return lv;
        if (auto r = ok(nnb200_col_softmax_sparse_forward(ptr(*l), ptr(*lb), mask ? ptr(mk) : nullptr, ptr(*grad), ptr(*lv),
                                                          static_cast<int>(C), static_cast<int>(N), static_cast<int>(vocab_size),
                                                          inv_num_valid, stream()), "nnb200_col_softmax_sparse_forward"); !r)
            return std::unexpected(r.error());
        loss_vec_out = std::move(*lv);
        return grad;
    }

    // ── in-place arithmetic: results land in A's own buffer ───────────────────────────────────
private:
    // A on the device; a host A is replaced by its device copy, as the reference does
    [[nodiscard]] Result<void> to_device_inplace(Tensor& A)
    {
        if (A.is_gpu()) return {};
        auto a = ensure_cuda(A);
        if (!a) return std::unexpected(a.error());
        A = std::move(*a);
        return {};
    }
    [[nodiscard]] Result<void> binary_into(const Tensor& a, const Tensor& b, float* out, unsigned op)
    {
        if (!fits_u32(a.size())) return fail("elementwise: element count exceeds 32 bits");
        return ok(cuda_elementwise_binary(ptr(a), ptr(b), out, u32(a.size()), op, stream()), "cuda_elementwise_binary");
    }

public:
    [[nodiscard]] Result<void> add_inplace(Tensor& A, const Tensor& B) override
    {
        if (A.rows() != B.rows() || A.cols() != B.cols()) return fail("add_inplace: shape mismatch");
        if (auto d = to_device_inplace(A); !d) return d;
        auto b = ensure_cuda(B);
        if (!b) return std::unexpected(b.error());
        return binary_into(A, *b, ptr(A), 0);
    }
    [[nodiscard]] Result<void> scale_inplace(Tensor& A, Scalar s) override
    {
        if (auto d = to_device_inplace(A); !d) return d;
        if (!fits_u32(A.size())) return fail("scale_inplace: element count exceeds 32 bits");
        return ok(cuda_elementwise_binary_scalar(ptr(A), ptr(A), u32(A.size()), 2, s, 0, stream()), "cuda_elementwise_binary_scalar");
    }
    [[nodiscard]] Result<void> axpy_inplace(Tensor& A, Scalar scalar, const Tensor& B) override
    {
        if (A.rows() != B.rows() || A.cols() != B.cols()) return fail("axpy_inplace: shape mismatch");
        if (auto d = to_device_inplace(A); !d) return d;
        auto b = ensure_cuda(B);
        if (!b) return std::unexpected(b.error());
        if (!fits_u32(A.size())) return fail("axpy_inplace: element count exceeds 32 bits");
        return ok(cuda_axpy(ptr(A), ptr(*b), ptr(A), u32(A.size()), scalar, stream()), "cuda_axpy");
    }
    [[nodiscard]] Result<void> zero(Tensor& A) override
    {
        if (A.is_cpu())
        {
            if (!A.valid()) return fail("zero: invalid tensor");
            auto z = alloc(A.rows(), A.cols());
            if (!z) return std::unexpected(z.error());
            A = std::move(*z);
        }
        return ok(nnb200_rt_zero(ptr(A), A.size() * sizeof(float)), "device memset");
    }

    // ── reductions and broadcasts ──────────────────────────────────────────────────────────────
private:
    [[nodiscard]] Result<Tensor> reduce(const Tensor& A, bool by_row, unsigned mode)
    {
        auto a = ensure_cuda(A);
        if (!a) return a;
        if (!fits_u32(a->rows()) || !fits_u32(a->cols())) return fail("reduce: dimension exceeds 32 bits");
        auto out = by_row ? alloc(a->rows(), 1) : alloc(1, a->cols());
        if (!out) return out;
        const int rc = by_row ? cuda_reduce_row(ptr(*a), ptr(*out), u32(a->rows()), u32(a->cols()), mode, stream())
                              : cuda_reduce_col(ptr(*a), ptr(*out), u32(a->rows()), u32(a->cols()), mode, stream());
        if (auto r = ok(rc, "cuda_reduce"); !r) return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<void> broadcast(Tensor& A, const Tensor& vec, bool by_row, BinaryOp op)
    {
        if (auto d = to_device_inplace(A); !d) return d;
        auto v = ensure_cuda(vec);
        if (!v) return std::unexpected(v.error());
        if (v->size() != (by_row ? A.rows() : A.cols()))
            return fail(by_row ? "broadcast_row_inplace: vector length != rows" : "broadcast_col_inplace: vector length != cols");
        if (!fits_u32(A.rows()) || !fits_u32(A.cols())) return fail("broadcast: dimension exceeds 32 bits");
        const int rc = by_row ? cuda_broadcast_row(ptr(A), ptr(*v), ptr(A), u32(A.rows()), u32(A.cols()), static_cast<unsigned>(op), stream())
                              : cuda_broadcast_col(ptr(A), ptr(*v), ptr(A), u32(A.rows()), u32(A.cols()), static_cast<unsigned>(op), stream());
        return ok(rc, "cuda_broadcast");
    }

public:
    [[nodiscard]] Result<Tensor> row_reduce_sum(const Tensor& A) override { return reduce(A, true, 0); }
    [[nodiscard]] Result<Tensor> col_reduce_sum(const Tensor& A) override { return reduce(A, false, 0); }
    [[nodiscard]] Result<Tensor> row_reduce_max(const Tensor& A) override { return reduce(A, true, 1); }
    [[nodiscard]] Result<Tensor> col_reduce_max(const Tensor& A) override { return reduce(A, false, 1); }
    [[nodiscard]] Result<void> broadcast_row_inplace(Tensor& A, const Tensor& row_vec, BinaryOp op) override
    {
        return broadcast(A, row_vec, true, op);
    }
    [[nodiscard]] Result<void> broadcast_col_inplace(Tensor& A, const Tensor& col_vec, BinaryOp op) override
    {
        return broadcast(A, col_vec, false, op);
    }

    // ── element-wise ───────────────────────────────────────────────────────────────────────────
    [[nodiscard]] Result<Tensor> elementwise_unary(UnaryOp op, const Tensor& A) override
    {
        auto a = ensure_cuda(A);
        if (!a) return a;
        if (!fits_u32(a->size())) return fail("elementwise_unary: element count exceeds 32 bits");
        auto out = alloc(a->rows(), a->cols());
        if (!out) return out;
        if (auto r = ok(cuda_elementwise_unary(ptr(*a), ptr(*out), u32(a->size()), static_cast<unsigned>(op), stream()),
                        "cuda_elementwise_unary"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<Tensor> elementwise_binary(BinaryOp op, const Tensor& A, const Tensor& B) override
    {
        if (A.rows() != B.rows() || A.cols() != B.cols()) return fail("elementwise_binary: shape mismatch");
        auto a = ensure_cuda(A);
        if (!a) return a;
        auto b = ensure_cuda(B);
        if (!b) return b;
        auto out = alloc(a->rows(), a->cols());
        if (!out) return out;
        if (auto r = binary_into(*a, *b, ptr(*out), static_cast<unsigned>(op)); !r) return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<Tensor> elementwise_binary_scalar(BinaryOp op, const Tensor& A, Scalar s, bool scalar_first) override
    {
        auto a = ensure_cuda(A);
        if (!a) return a;
        if (!fits_u32(a->size())) return fail("elementwise_binary_scalar: element count exceeds 32 bits");
        auto out = alloc(a->rows(), a->cols());
        if (!out) return out;
        if (auto r = ok(cuda_elementwise_binary_scalar(ptr(*a), ptr(*out), u32(a->size()), static_cast<unsigned>(op), s,
                                                       scalar_first ? 1 : 0, stream()), "cuda_elementwise_binary_scalar"); !r)
            return std::unexpected(r.error());
        return out;
    }
    [[nodiscard]] Result<Tensor> elementwise_select_scalar_cond(CompareOp cmp, const Tensor& A, Scalar scalar_b,
                                                                const Tensor& then_t, Scalar scalar_else) override
    {
        if (A.rows() != then_t.rows() || A.cols() != then_t.cols()) return fail("elementwise_select: A and then shape mismatch");
        auto a = ensure_cuda(A);
        if (!a) return a;
        auto t = ensure_cuda(then_t);
        if (!t) return t;
        if (!fits_u32(a->size())) return fail("elementwise_select: element count exceeds 32 bits");
        auto out = alloc(a->rows(), a->cols());
        if (!out) return out;
        if (auto r = ok(cuda_elementwise_select_scalar_cond(ptr(*a), ptr(*t), ptr(*out), u32(a->size()), static_cast<unsigned>(cmp),
                                                            scalar_b, scalar_else, stream()), "cuda_elementwise_select_scalar_cond"); !r)
            return std::unexpected(r.error());
        return out;
    }

    // ── expression programs (cpu_engine.hpp:1280-1659) ────────────────────────────────────────
    [[nodiscard]] Result<Tensor> eval_expr(const ExprSpec& spec, std::span<const Tensor> inputs, std::size_t rows,
                                           std::size_t cols) override
    {
        return eval_expr_impl(spec, inputs, rows, cols, false);
    }
    [[nodiscard]] Result<Tensor> eval_expr_reduce(const ExprSpec& spec, std::span<const Tensor> inputs, std::size_t rows,
                                                  std::size_t cols) override
    {
        return eval_expr_impl(spec, inputs, rows, cols, true);
    }

private:
    [[nodiscard]] Result<Tensor> eval_expr_impl(const ExprSpec& spec, std::span<const Tensor> inputs, std::size_t rows,
                                                std::size_t cols, bool vector_out)
    {
        if (auto v = validate_expr_spec(spec, inputs.size()); !v) return std::unexpected(v.error());
        const int axis = vector_out ? expr_spec_reduce_axis(spec) : -1;
        if (vector_out && axis != 0 && axis != 1) return fail("eval_expr_reduce: expression is not a pure row or column reduction");
        constexpr std::size_t lim = std::numeric_limits<int>::max();
        if (rows > lim || cols > lim) return fail("eval_expr: dimension exceeds int range");

        // flatten the program
        nnb200_expr_program prog{};
        prog.num_instrs = static_cast<std::uint32_t>(spec.instrs.size());
        prog.num_regs = spec.num_regs;
        prog.num_inputs = static_cast<std::uint32_t>(inputs.size());
        prog.num_consts = static_cast<std::uint32_t>(spec.consts.size());
        for (std::size_t i = 0; i < spec.instrs.size(); ++i)
        {
            const ExprInstr& in = spec.instrs[i];
            const std::uint8_t flat[8] = {in.op, in.dst, in.a.kind, in.a.idx, in.b.kind, in.b.idx, in.c.kind, in.c.idx};
            std::memcpy(prog.instrs[i], flat, sizeof(flat));
        }
        for (std::size_t k = 0; k < spec.views.size(); ++k)
        {
            prog.view_kind[k] = spec.views[k].kind;
            prog.view_negate[k] = spec.views[k].negate_first_half;
            prog.view_param[k] = spec.views[k].param;
        }
        for (std::size_t k = 0; k < spec.consts.size(); ++k) prog.consts[k] = spec.consts[k];

        std::array<Tensor, EXPR_MAX_INPUTS> dev;
        const float* in_ptr[EXPR_MAX_INPUTS] = {};
        int in_rows[EXPR_MAX_INPUTS] = {}, in_cols[EXPR_MAX_INPUTS] = {};
        for (std::size_t k = 0; k < inputs.size(); ++k)
        {
            auto d = ensure_cuda(inputs[k]);
            if (!d) return d;
            dev[k] = std::move(*d);
            in_ptr[k] = ptr(dev[k]);
            in_rows[k] = static_cast<int>(dev[k].rows());
            in_cols[k] = static_cast<int>(dev[k].cols());
        }
        auto out = !vector_out ? alloc(rows, cols) : (axis == 0 ? alloc(rows, 1) : alloc(1, cols));
        if (!out) return out;
        auto scratch = alloc(1, nnb200_eval_expr_scratch_floats(static_cast<int>(rows), static_cast<int>(cols)));
        if (!scratch) return scratch;
        if (nnb200_eval_expr(&prog, in_ptr, in_rows, in_cols, ptr(*out), ptr(*scratch), static_cast<int>(rows),
                             static_cast<int>(cols), vector_out ? 1 : 0, stream()) != 0)
            return fail("eval_expr: rejected by the device interpreter (shape or program invalid; reason on stderr)");
        return out;
    }
};

} // namespace nn

#endif // NN_HAS_CUDA
#endif // NN_CUDA_ENGINE_HPP
