// TEST INFRASTRUCTURE: parity of the drop-in CudaEngine against the reference's own CpuEngine.
//
// Every ComputeEngine virtual (compute_engine.hpp:60-413) is run twice on the same seeded inputs: on the
// reference's CpuEngine, compiled from the reference's headers where they lie, and on the CudaEngine of
// this repository (neuralnet.cpp_b200/engine/, force-included in place of the reference's CUDA engine).
// Index and copy work must agree bit for bit; floating-point work within 1e-5 of the largest reference
// magnitude (sums are re-associated on the device).  Exit code 0 = every case agreed.
//
//   engine_check [--seed N] [--verbose]
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <random>
#include <string>
#include <vector>

#include "neuralnet.cpp/cpu_engine.hpp"
#include "neuralnet.cpp/cuda_engine.hpp"

using nn::Matrix;
using nn::Result;
using nn::Scalar;
using nn::Tensor;
namespace ex = nn::expr;

namespace
{
std::mt19937 g_rng(7);
bool g_verbose = false;
int g_failed = 0, g_cases = 0;

Matrix rnd(std::size_t r, std::size_t c, float lo = -1.f, float hi = 1.f)
{
    Matrix m(r, c);
    std::uniform_real_distribution<float> d(lo, hi);
    for (auto& v : m.span()) v = d(g_rng);
    return m;
}

void report(const std::string& name, bool okay, double err)
{
    ++g_cases;
    if (!okay) ++g_failed;
    if (!okay || g_verbose) std::printf("  %-58s %s  err=%.3g\n", name.c_str(), okay ? "OK  " : "FAIL", err);
}

// relative to the largest reference magnitude; tol == 0 asks for bit equality
void compare(const std::string& name, const Matrix& ref, const Matrix& got, double tol)
{
    if (ref.rows() != got.rows() || ref.cols() != got.cols())
    {
        std::printf("  %-58s FAIL  shape (%zu,%zu) vs (%zu,%zu)\n", name.c_str(), ref.rows(), ref.cols(), got.rows(), got.cols());
        ++g_cases;
        ++g_failed;
        return;
    }
    const auto a = ref.span();
    const auto b = got.span();
    double scale = 0, err = 0;
    bool bits = true;
    for (std::size_t i = 0; i < a.size(); ++i)
    {
        scale = std::max(scale, static_cast<double>(std::fabs(a[i])));
        if (std::isnan(a[i]) != std::isnan(b[i])) err = INFINITY;
        else if (!std::isnan(a[i]) && a[i] != b[i])
        {
            if (std::isinf(a[i]) || std::isinf(b[i])) err = INFINITY;
            else err = std::max(err, static_cast<double>(std::fabs(a[i] - b[i])));
        }
        if (std::memcmp(&a[i], &b[i], sizeof(float)) != 0 && !(a[i] == b[i])) bits = false;
    }
    const double rel = err / std::max(scale, 1e-30);
    report(name, tol == 0 ? bits : rel <= tol, rel);
}

struct Pair
{
    nn::CpuEngine& cpu;
    nn::CudaEngine& gpu;

    Tensor up(const Matrix& m)
    {
        auto r = gpu.from_matrix(m);
        if (!r) { std::printf("upload failed: %s\n", r.error().message.c_str()); std::exit(2); }
        return std::move(*r);
    }
    Matrix down(const Tensor& t)
    {
        auto r = gpu.to_matrix(t);
        if (!r) { std::printf("download failed: %s\n", r.error().message.c_str()); std::exit(2); }
        return std::move(*r);
    }
    // op(engine, make) where make(Matrix) gives the engine's own tensor; both must succeed or both fail
    void run(const std::string& name, double tol,
             const std::function<Result<Tensor>(nn::ComputeEngine&, const std::function<Tensor(const Matrix&)>&)>& op)
    {
        auto rc = op(cpu, [](const Matrix& m) { return Tensor::from_matrix(Matrix(m)); });
        auto rg = op(gpu, [this](const Matrix& m) { return up(m); });
        if (!rc || !rg)
        {
            report(name + (rc ? "" : " [both reject]"), !rc && !rg, 0);
            if (rc.has_value() != rg.has_value())
                std::printf("      cpu: %s | cuda: %s\n", rc ? "ok" : rc.error().message.c_str(), rg ? "ok" : rg.error().message.c_str());
            return;
        }
        compare(name, rc->cpu_matrix(), down(*rg), tol);
    }
};

constexpr double kTol = 1e-5;
const float kNegInf = -std::numeric_limits<float>::infinity();

Matrix causal_mask(std::size_t M, std::size_t N, bool with_bias)
{
    Matrix m(M, N);
    for (std::size_t i = 0; i < M; ++i)
        for (std::size_t j = 0; j < N; ++j) m.span()[i * N + j] = j > i ? kNegInf : (with_bias ? -0.25f * static_cast<float>(i - j) : 0.f);
    return m;
}
} // namespace

// ── contractions and the fused attention primitives ─────────────────────────────────────────────
static void check_contractions(Pair& P)
{
    using Mk = std::function<Tensor(const Matrix&)>;
    for (int ta = 0; ta < 2; ++ta)
        for (int tb = 0; tb < 2; ++tb)
        {
            const std::size_t M = 37, K = 53, N = 29;
            const Matrix A = ta ? rnd(K, M) : rnd(M, K), B = tb ? rnd(N, K) : rnd(K, N);
            P.run("matmul tA=" + std::to_string(ta) + " tB=" + std::to_string(tb), kTol,
                  [&](nn::ComputeEngine& e, const Mk& mk) { return e.matmul(mk(A), mk(B), ta, tb); });
            const std::size_t batch = 5;
            const Matrix Ab = ta ? rnd(batch * K, M) : rnd(batch * M, K), Bb = tb ? rnd(batch * N, K) : rnd(batch * K, N);
            P.run("batched_matmul tA=" + std::to_string(ta) + " tB=" + std::to_string(tb), kTol,
                  [&](nn::ComputeEngine& e, const Mk& mk) { return e.batched_matmul(mk(Ab), mk(Bb), batch, ta, tb, 0.37f); });
        }
    const Matrix m45 = rnd(4, 5), m63 = rnd(6, 3);
    P.run("matmul K mismatch", kTol, [&](nn::ComputeEngine& e, const Mk& mk) { return e.matmul(mk(m45), mk(m63), false, false); });

    // attention-shaped: A = Q^T stored (batch*dk, S) with transA, B = K stored (batch*dk, S); S = alpha Q K^T + mask
    const std::size_t batch = 6, S = 45, dk = 16;
    const float alpha = 0.25f;
    const Matrix Q = rnd(batch * dk, S), Kx = rnd(batch * dk, S), V = rnd(batch * S, dk), G = rnd(batch * S, dk);
    const Matrix Pg = rnd(batch * S, S);
    for (int mk_kind = 0; mk_kind < 3; ++mk_kind)
    {
        const Matrix mask = causal_mask(S, S, mk_kind == 2);
        const bool use_mask = mk_kind > 0;
        const std::string tag = mk_kind == 0 ? " nomask" : (mk_kind == 1 ? " causal" : " causal+bias");
        auto mptr = [&](const Mk& mk, Tensor& hold) -> const Tensor* { if (!use_mask) return nullptr; hold = mk(mask); return &hold; };
        for (int op = 0; op < 3; ++op)
            for (int rc = 0; rc < 2; ++rc)
                P.run("bmm_reduce op=" + std::to_string(op) + " cols=" + std::to_string(rc) + tag, kTol,
                      [&](nn::ComputeEngine& e, const Mk& mk) {
                          Tensor hold;
                          return e.batched_matmul_reduce(mk(Q), mk(Kx), batch, static_cast<nn::ReduceOp>(op), true, false, alpha, rc, mptr(mk, hold));
                      });
        // the chain the attention layer runs: max -> denom -> apply -> backward_q -> backward_kv
        auto chain = [&](int stage) {
            return [&, stage](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
                Tensor hold;
                const Tensor* m = mptr(mk, hold);
                Tensor q = mk(Q), k = mk(Kx);
                auto mx = e.batched_matmul_reduce(q, k, batch, nn::ReduceOp::Max, true, false, alpha, true, m);
                if (!mx) return mx;
                auto dn = e.batched_matmul_softmax_denom(q, k, *mx, batch, true, false, alpha, m);
                if (!dn || stage == 0) return dn;
                if (stage == 1) return e.batched_matmul_softmax_apply(q, k, mk(V), *mx, *dn, batch, true, false, alpha, m);
                Tensor r_out;
                auto gq = e.batched_matmul_softmax_backward_q(q, k, mk(Pg), *mx, *dn, batch, true, false, alpha, r_out, m);
                if (!gq || stage == 2) return gq;
                if (stage == 3) return r_out;
                Tensor gv;
                auto gk = e.batched_matmul_softmax_backward_kv(q, k, mk(Pg), mk(G), r_out, *mx, *dn, batch, true, false, alpha, gv, m);
                if (!gk || stage == 4) return gk;
                return gv;
            };
        };
        const char* names[] = {"softmax_denom", "softmax_apply", "softmax_backward_q", "softmax_backward_q r_out", "softmax_backward_kv gradK",
                               "softmax_backward_kv gradV"};
        for (int st = 0; st < 6; ++st) P.run(std::string("bmm_") + names[st] + tag, kTol, chain(st));
    }
    // the other transposition pattern (A (batch*M, K), B stored (batch*N, K)), rectangular
    {
        const std::size_t b2 = 3, M = 20, N = 33, K = 12, D = 12;
        const Matrix A = rnd(b2 * M, K), B = rnd(b2 * N, K), Vv = rnd(b2 * N, D);
        P.run("bmm chain tA=0 tB=1 rectangular", kTol, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
            Tensor a = mk(A), b = mk(B);
            auto mx = e.batched_matmul_reduce(a, b, b2, nn::ReduceOp::Max, false, true, 0.5f, true, nullptr);
            if (!mx) return mx;
            auto dn = e.batched_matmul_softmax_denom(a, b, *mx, b2, false, true, 0.5f, nullptr);
            if (!dn) return dn;
            return e.batched_matmul_softmax_apply(a, b, mk(Vv), *mx, *dn, b2, false, true, 0.5f, nullptr);
        });
        P.run("bmm_reduce mask shape mismatch", kTol, [&](nn::ComputeEngine& e, const Mk& mk) {
            Tensor m = mk(rnd(M, N + 1));
            return e.batched_matmul_reduce(mk(A), mk(B), b2, nn::ReduceOp::Max, false, true, 1.f, true, &m);
        });
    }
}

// ── cross-entropy primitives ─────────────────────────────────────────────────────────────────────
static void check_cross_entropy(Pair& P)
{
    using Mk = std::function<Tensor(const Matrix&)>;
    const std::size_t C = 70, N = 91, vocab = 64;
    const Matrix logits = rnd(C, N, -4.f, 4.f);
    Matrix labels(1, N), mask(1, N);
    std::uniform_int_distribution<int> lab(0, static_cast<int>(vocab) - 1);
    for (std::size_t i = 0; i < N; ++i)
    {
        labels.span()[i] = static_cast<float>(lab(g_rng));
        mask.span()[i] = (i % 5 == 0) ? 0.f : 1.f;
    }
    labels.span()[3] = static_cast<float>(vocab + 2);   // out of the vocabulary -> zero column
    labels.span()[4] = -1.f;                            // negative -> treated as label 0
    P.run("col_softmax_denom", kTol, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        auto mx = e.col_reduce_max(mk(logits));
        if (!mx) return mx;
        return e.col_softmax_denom(mk(logits), *mx);
    });
    for (int with_mask = 0; with_mask < 2; ++with_mask)
        for (int which = 0; which < 2; ++which)
            P.run(std::string("col_softmax_sparse_forward ") + (which ? "loss_vec" : "grad") + (with_mask ? " masked" : ""), kTol,
                  [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
                      Tensor m = mk(mask), lv;
                      auto g = e.col_softmax_sparse_forward(mk(logits), mk(labels), with_mask ? &m : nullptr, vocab, 1.0f / 73.f, lv);
                      if (!g) return g;
                      return which ? lv : *g;
                  });
    P.run("col_softmax_sparse_forward vocab > classes", kTol, [&](nn::ComputeEngine& e, const Mk& mk) {
        Tensor lv;
        return e.col_softmax_sparse_forward(mk(logits), mk(labels), nullptr, C + 1, 1.f, lv);
    });
}

// ── element-wise, reductions, broadcasts, in-place ───────────────────────────────────────────────
static void check_elementwise(Pair& P)
{
    using Mk = std::function<Tensor(const Matrix&)>;
    const std::size_t R = 67, C = 131;
    const Matrix A = rnd(R, C, -2.f, 2.f), B = rnd(R, C, 0.5f, 2.f), Pos = rnd(R, C, 0.1f, 3.f);
    const char* un[] = {"Neg", "Exp", "Log", "Sqrt", "Rsqrt", "Abs", "Tanh"};
    for (int op = 0; op < 7; ++op)
    {
        const Matrix& in = (op >= 2 && op <= 4) ? Pos : A;
        P.run(std::string("elementwise_unary ") + un[op], kTol,
              [&](nn::ComputeEngine& e, const Mk& mk) { return e.elementwise_unary(static_cast<nn::UnaryOp>(op), mk(in)); });
    }
    const char* bn[] = {"Add", "Sub", "Mul", "Div", "Max", "Min"};
    for (int op = 0; op < 6; ++op)
    {
        const auto bop = static_cast<nn::BinaryOp>(op);
        P.run(std::string("elementwise_binary ") + bn[op], kTol, [&](nn::ComputeEngine& e, const Mk& mk) { return e.elementwise_binary(bop, mk(A), mk(B)); });
        for (int first = 0; first < 2; ++first)
            P.run(std::string("elementwise_binary_scalar ") + bn[op] + (first ? " scalar first" : ""), kTol,
                  [&](nn::ComputeEngine& e, const Mk& mk) { return e.elementwise_binary_scalar(bop, mk(B), 1.3f, first); });
        const Matrix rv = rnd(R, 1, 0.5f, 2.f), cv = rnd(1, C, 0.5f, 2.f);
        P.run(std::string("broadcast_row_inplace ") + bn[op], kTol, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
            Tensor a = mk(A);
            if (auto r = e.broadcast_row_inplace(a, mk(rv), bop); !r) return std::unexpected(r.error());
            return a;
        });
        P.run(std::string("broadcast_col_inplace ") + bn[op], kTol, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
            Tensor a = mk(A);
            if (auto r = e.broadcast_col_inplace(a, mk(cv), bop); !r) return std::unexpected(r.error());
            return a;
        });
    }
    P.run("elementwise_binary shape mismatch", kTol, [&](nn::ComputeEngine& e, const Mk& mk) { return e.elementwise_binary(nn::BinaryOp::Add, mk(A), mk(rnd(R, C + 1))); });
    Matrix Q = A;   // quantised so that Eq / Ne / Le / Ge see ties
    for (auto& v : Q.span()) v = std::round(v * 2.f) / 2.f;
    const char* cn[] = {"Lt", "Le", "Gt", "Ge", "Eq", "Ne"};
    for (int c = 0; c < 6; ++c)
        P.run(std::string("elementwise_select_scalar_cond ") + cn[c], 0, [&](nn::ComputeEngine& e, const Mk& mk) {
            return e.elementwise_select_scalar_cond(static_cast<nn::CompareOp>(c), mk(Q), 0.5f, mk(B), -7.f);
        });
    P.run("row_reduce_sum", kTol, [&](nn::ComputeEngine& e, const Mk& mk) { return e.row_reduce_sum(mk(A)); });
    P.run("col_reduce_sum", kTol, [&](nn::ComputeEngine& e, const Mk& mk) { return e.col_reduce_sum(mk(A)); });
    P.run("row_reduce_max", 0, [&](nn::ComputeEngine& e, const Mk& mk) { return e.row_reduce_max(mk(A)); });
    P.run("col_reduce_max", 0, [&](nn::ComputeEngine& e, const Mk& mk) { return e.col_reduce_max(mk(A)); });
    P.run("add_inplace", kTol, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        Tensor a = mk(A);
        if (auto r = e.add_inplace(a, mk(B)); !r) return std::unexpected(r.error());
        return a;
    });
    P.run("scale_inplace", kTol, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        Tensor a = mk(A);
        if (auto r = e.scale_inplace(a, -0.75f); !r) return std::unexpected(r.error());
        return a;
    });
    P.run("axpy_inplace", kTol, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        Tensor a = mk(A);
        if (auto r = e.axpy_inplace(a, 0.3f, mk(B)); !r) return std::unexpected(r.error());
        return a;
    });
    P.run("zero", 0, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        Tensor a = mk(A);
        if (auto r = e.zero(a); !r) return std::unexpected(r.error());
        return a;
    });
    P.run("add_inplace shape mismatch", kTol, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        Tensor a = mk(A);
        if (auto r = e.add_inplace(a, mk(rnd(C, R))); !r) return std::unexpected(r.error());
        return a;
    });
}

// ── index and copy work: bit-exact ───────────────────────────────────────────────────────────────
static void check_index_ops(Pair& P)
{
    using Mk = std::function<Tensor(const Matrix&)>;
    const std::size_t vocab = 50, D = 24, num = 300;
    const Matrix table = rnd(vocab, D);
    Matrix idx(num, 1);
    std::uniform_int_distribution<int> d(0, static_cast<int>(vocab) + 3);   // a few beyond the table
    for (auto& v : idx.span()) v = static_cast<float>(d(g_rng));
    const Matrix grad = rnd(num, D);
    P.run("gather_rows (with out-of-range ids)", 0, [&](nn::ComputeEngine& e, const Mk& mk) { return e.gather_rows(mk(table), mk(idx)); });
    P.run("scatter_add_rows (duplicates, out-of-range ids)", 0, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        Tensor dst = mk(table);
        if (auto r = e.scatter_add_rows(dst, mk(idx), mk(grad)); !r) return std::unexpected(r.error());
        return dst;
    });
    const std::size_t M = 12, B = 5, N = 7;
    const Matrix x = rnd(M, B * N), y = rnd(B * M, N);
    P.run("rearrange_3d forward", 0, [&](nn::ComputeEngine& e, const Mk& mk) { return e.rearrange_3d(mk(x), M, B, N, false); });
    P.run("rearrange_3d inverse", 0, [&](nn::ComputeEngine& e, const Mk& mk) { return e.rearrange_3d(mk(y), M, B, N, true); });
    P.run("rearrange_3d element count mismatch", 0, [&](nn::ComputeEngine& e, const Mk& mk) { return e.rearrange_3d(mk(x), M, B, N + 1, false); });
    const Matrix wide = rnd(33, 65);
    P.run("transpose", 0, [&](nn::ComputeEngine& e, const Mk& mk) { return e.transpose(mk(wide)); });
    const Matrix big = rnd(40, 9), part = rnd(6, 9), fresh = rnd(40, 9);
    P.run("slice_rows", 0, [&](nn::ComputeEngine& e, const Mk& mk) { return e.slice_rows(mk(big), 11, 17); });
    P.run("slice_rows out of bounds", 0, [&](nn::ComputeEngine& e, const Mk& mk) { return e.slice_rows(mk(big), 30, 11); });
    P.run("insert_rows", 0, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        Tensor dst = mk(big);
        if (auto r = e.insert_rows(dst, 20, mk(part)); !r) return std::unexpected(r.error());
        return dst;
    });
    P.run("insert_rows out of bounds", 0, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        Tensor dst = mk(big);
        if (auto r = e.insert_rows(dst, 36, mk(part)); !r) return std::unexpected(r.error());
        return dst;
    });
    P.run("clone is a copy, not an alias", 0, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        Tensor a = mk(big);
        auto c = e.clone(a);
        if (!c) return c;
        if (auto r = e.scale_inplace(a, 2.f); !r) return std::unexpected(r.error());
        return c;
    });
    P.run("copy_from", 0, [&](nn::ComputeEngine& e, const Mk& mk) -> Result<Tensor> {
        Tensor a = mk(big);
        if (auto r = e.copy_from(a, fresh); !r) return std::unexpected(r.error());
        return a;
    });
    // a reshape() view must be read with the view's shape, and an in-place op through the original must show in it
    {
        const Matrix src = rnd(8, 6);
        Tensor t = P.up(src);
        Tensor view = t.reshape(4, 12);
        (void)P.gpu.scale_inplace(t, 3.f);
        Matrix want(4, 12);
        for (std::size_t i = 0; i < 48; ++i) want.span()[i] = src.span()[i] * 3.f;
        compare("reshape view follows in-place update", want, P.down(view), 0);
        auto tr = P.gpu.transpose(view);
        Matrix wt(12, 4);
        for (std::size_t r = 0; r < 4; ++r)
            for (std::size_t c = 0; c < 12; ++c) wt.span()[c * 4 + r] = want.span()[r * 12 + c];
        if (tr) compare("transpose of a reshape view", wt, P.down(*tr), 0);
        else report("transpose of a reshape view", false, 0);
    }
}

// ── expression programs ──────────────────────────────────────────────────────────────────────────
static nn::ExprInstr ins(nn::ExprOp op, std::uint8_t dst, nn::ExprOperand a, nn::ExprOperand b = {}, nn::ExprOperand c = {})
{
    return nn::ExprInstr{static_cast<std::uint8_t>(op), dst, a, b, c};
}

static void check_expr(Pair& P)
{
    using Mk = std::function<Tensor(const Matrix&)>;
    using Op = nn::ExprOp;
    const std::size_t dk = 8, heads = 3, batch = 2, seq = 19;
    const std::size_t R = batch * heads * dk, C = seq;
    const Matrix q = rnd(R, C), cosT = rnd(dk, C), sinT = rnd(dk, C);
    auto eval = [&](const std::string& name, const nn::ExprSpec& spec, std::vector<Matrix> in, std::size_t rows, std::size_t cols,
                    bool reduce = false, double tol = kTol) {
        P.run(name, tol, [&](nn::ComputeEngine& e, const Mk& mk) {
            std::vector<Tensor> ts;
            for (const auto& m : in) ts.push_back(mk(m));
            return reduce ? e.eval_expr_reduce(spec, ts, rows, cols) : e.eval_expr(spec, ts, rows, cols);
        });
    };
    {   // rotary embedding: q*cos + rotate_half(q)*sin, tables tiled by row modulo
        nn::ExprSpec s;
        s.views = {ex::linear(), ex::rotate_half(dk, true), ex::row_mod(dk), ex::row_mod(dk)};
        s.num_regs = 3;
        s.instrs = {ins(Op::Mul, 0, ex::input(0), ex::input(2)), ins(Op::Mul, 1, ex::input(1), ex::input(3)), ins(Op::Add, 2, ex::reg(0), ex::reg(1))};
        eval("eval_expr rotary (RotateHalf + RowMod views)", s, {q, q, cosT, sinT}, R, C);
        s.views[1] = ex::rotate_half(dk, false);
        eval("eval_expr rotary without negation", s, {q, q, cosT, sinT}, R, C);
        s.views[1] = ex::rotate_half(7, true);
        eval("eval_expr RotateHalf odd block", s, {q, q, cosT, sinT}, R, C);
    }
    const std::size_t F = 40, T = 77;
    const Matrix x = rnd(F, T, -2.f, 2.f), gamma = rnd(F, 1, 0.5f, 1.5f), beta = rnd(F, 1);
    {   // RMS norm over the feature rows of each token column: x * rsqrt(colsum(x*x)/F + eps) * gamma
        nn::ExprSpec s;
        s.views = {ex::linear(), ex::row_broadcast()};
        s.consts = {1.0f / static_cast<float>(F), 1e-5f};
        s.num_regs = 5;
        s.instrs = {ins(Op::Mul, 0, ex::input(0), ex::input(0)), ins(Op::ColSum, 1, ex::reg(0)),
                    ins(Op::Mul, 2, ex::reduce(1), ex::cst(0)), ins(Op::Add, 2, ex::reg(2), ex::cst(1)),
                    ins(Op::Rsqrt, 3, ex::reg(2)), ins(Op::Mul, 4, ex::input(0), ex::reg(3)), ins(Op::Mul, 4, ex::reg(4), ex::input(1))};
        eval("eval_expr RMS norm (ColSum instruction)", s, {x, gamma}, F, T);
        // the statistic alone, as a (1, T) vector
        nn::ExprSpec v;
        v.views = {ex::linear()};
        v.consts = s.consts;
        v.num_regs = 4;
        v.instrs = {ins(Op::Mul, 0, ex::input(0), ex::input(0)), ins(Op::ColSum, 1, ex::reg(0)), ins(Op::Mul, 2, ex::reduce(1), ex::cst(0)),
                    ins(Op::Add, 2, ex::reg(2), ex::cst(1)), ins(Op::Rsqrt, 3, ex::reg(2))};
        eval("eval_expr_reduce inverse RMS per column", v, {x}, F, T, true);
        nn::ExprSpec last;
        last.views = {ex::linear()};
        last.num_regs = 2;
        last.instrs = {ins(Op::Abs, 0, ex::input(0)), ins(Op::RowMax, 1, ex::reg(0))};
        eval("eval_expr_reduce ending in RowMax", last, {x}, F, T, true, 0);
        eval("eval_expr ending in a reduction (broadcast back)", last, {x}, F, T, false, 0);
    }
    {   // layer norm with two chained reductions: mean, then variance of the centred value
        nn::ExprSpec s;
        s.views = {ex::linear(), ex::row_broadcast(), ex::row_broadcast()};
        s.consts = {1.0f / static_cast<float>(F), 1e-5f};
        s.num_regs = 8;
        s.instrs = {ins(Op::ColSum, 0, ex::input(0)), ins(Op::Mul, 1, ex::reduce(0), ex::cst(0)), ins(Op::Sub, 2, ex::input(0), ex::reg(1)),
                    ins(Op::Mul, 3, ex::reg(2), ex::reg(2)), ins(Op::ColSum, 4, ex::reg(3)), ins(Op::Mul, 5, ex::reduce(4), ex::cst(0)),
                    ins(Op::Add, 5, ex::reg(5), ex::cst(1)), ins(Op::Rsqrt, 5, ex::reg(5)), ins(Op::Mul, 6, ex::reg(2), ex::reg(5)),
                    ins(Op::Mul, 6, ex::reg(6), ex::input(1)), ins(Op::Add, 7, ex::reg(6), ex::input(2))};
        eval("eval_expr layer norm (chained ColSum)", s, {x, gamma, beta}, F, T);
    }
    {   // column softmax through reduce views of the same input
        nn::ExprSpec s;
        s.views = {ex::linear(), ex::col_reduce_max()};
        s.num_regs = 4;
        s.instrs = {ins(Op::Sub, 0, ex::input(0), ex::input(1)), ins(Op::Exp, 1, ex::reg(0)), ins(Op::ColSum, 2, ex::reg(1)),
                    ins(Op::Div, 3, ex::reg(1), ex::reduce(2))};
        eval("eval_expr column softmax (ColReduceMax view)", s, {x, x}, F, T);
        nn::ExprSpec r;
        r.views = {ex::linear(), ex::row_reduce_max(), ex::row_reduce_sum()};
        r.num_regs = 2;
        r.instrs = {ins(Op::Sub, 0, ex::input(0), ex::input(1)), ins(Op::Div, 1, ex::reg(0), ex::input(2))};
        Matrix xpos = x;   // a sum that stays away from zero, so that the quotient is well conditioned
        for (auto& v : xpos.span()) v = std::fabs(v) + 0.1f;
        eval("eval_expr row reduce views", r, {x, x, xpos}, F, T);
        nn::ExprSpec cv;
        cv.views = {ex::linear(), ex::col_broadcast(), ex::col_reduce_sum()};
        cv.num_regs = 2;
        cv.instrs = {ins(Op::Mul, 0, ex::input(0), ex::input(1)), ins(Op::Sub, 1, ex::reg(0), ex::input(2))};
        eval("eval_expr ColBroadcast + ColReduceSum views", cv, {x, rnd(1, T), x}, F, T);   // inputs are built once, before both runs
    }
    {   // comparisons, select, min/max, the remaining unary operators
        const Matrix y = rnd(F, T, -2.f, 2.f);
        Matrix xq = x;
        for (auto& v : xq.span()) v = std::round(v * 2.f) / 2.f;
        Matrix yq = y;
        for (auto& v : yq.span()) v = std::round(v * 2.f) / 2.f;
        const Op cmps[] = {Op::Lt, Op::Le, Op::Gt, Op::Ge, Op::Eq, Op::Ne};
        for (int c = 0; c < 6; ++c)
        {
            nn::ExprSpec s;
            s.views = {ex::linear(), ex::linear()};
            s.consts = {0.f, 3.f};
            s.num_regs = 4;
            s.instrs = {ins(cmps[c], 0, ex::input(0), ex::input(1)), ins(Op::Max, 1, ex::input(0), ex::cst(0)), ins(Op::Min, 2, ex::input(1), ex::cst(1)),
                        ins(Op::Select, 3, ex::fanout(0), ex::reg(1), ex::reg(2))};
            eval("eval_expr compare " + std::to_string(c) + " + select + max/min", s, {xq, yq}, F, T, false, 0);
        }
        nn::ExprSpec u;
        u.views = {ex::linear()};
        u.consts = {2.5f};
        u.num_regs = 8;
        u.instrs = {ins(Op::Abs, 0, ex::input(0)), ins(Op::Add, 0, ex::reg(0), ex::cst(0)), ins(Op::Log, 1, ex::reg(0)), ins(Op::Sqrt, 2, ex::reg(0)),
                    ins(Op::Tanh, 3, ex::input(0)), ins(Op::Neg, 4, ex::reg(3)), ins(Op::Exp, 5, ex::reg(4)), ins(Op::Add, 6, ex::reg(1), ex::reg(2)),
                    ins(Op::Sub, 7, ex::reg(6), ex::reg(5))};
        eval("eval_expr unary operators", u, {x}, F, T);
    }
    {   // programs both engines must reject
        nn::ExprSpec mixed;
        mixed.views = {ex::linear()};
        mixed.num_regs = 2;
        mixed.instrs = {ins(Op::ColSum, 0, ex::input(0)), ins(Op::RowSum, 1, ex::input(0))};
        eval("eval_expr_reduce mixed axes", mixed, {x}, F, T, true);
        nn::ExprSpec lin;
        lin.views = {ex::linear()};
        lin.num_regs = 2;
        lin.instrs = {ins(Op::ColSum, 0, ex::input(0)), ins(Op::Mul, 1, ex::input(0), ex::reduce(0))};
        eval("eval_expr_reduce output chain reads a Linear input", lin, {x}, F, T, true);
        nn::ExprSpec badreg;
        badreg.views = {ex::linear()};
        badreg.num_regs = 1;
        badreg.instrs = {ins(Op::Neg, 3, ex::input(0))};
        eval("eval_expr dst register out of range", badreg, {x}, F, T);
        nn::ExprSpec shape;
        shape.views = {ex::linear(), ex::row_broadcast()};
        shape.num_regs = 1;
        shape.instrs = {ins(Op::Mul, 0, ex::input(0), ex::input(1))};
        eval("eval_expr RowBroadcast input of the wrong shape", shape, {x, rnd(1, T)}, F, T);
    }
}

int main(int argc, char** argv)
{
    for (int i = 1; i < argc; ++i)
    {
        if (!std::strcmp(argv[i], "--verbose")) g_verbose = true;
        else if (!std::strcmp(argv[i], "--seed") && i + 1 < argc) g_rng.seed(static_cast<unsigned>(std::atoi(argv[++i])));
    }
    auto& backend = nn::CudaBackend::instance();
    if (auto r = backend.initialize(); !r)
    {
        std::printf("engine_check: %s\n", r.error().message.c_str());
        return 3;
    }
    nn::CpuEngine cpu;
    nn::CudaEngine gpu(backend);
    Pair P{cpu, gpu};
    std::printf("engine_check on %s\n", backend.device_props().name);
    check_contractions(P);
    check_cross_entropy(P);
    check_elementwise(P);
    check_index_ops(P);
    check_expr(P);
    (void)gpu.end_batch();
    std::printf("engine_check: %d cases, %d failed\n", g_cases, g_failed);
    return g_failed ? 1 : 0;
}
