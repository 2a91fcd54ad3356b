// TEST INFRASTRUCTURE — not part of the shipped product.
//
// Runs the fused attention and cross-entropy primitives of the unmodified reference CpuEngine
// (include/neuralnet.cpp/cpu_engine.hpp:426-1006) plus gather/scatter-add/rearrange on inputs read
// from a binary file and dumps their outputs, so the numpy restatement in oracle/gpt_oracle.py and
// the CUDA kernels can be pinned primitive by primitive.
//
// Input : i32 I[8] = {batch, M, N, K, D, C, NC, vocab_size}; f32 F[2] = {alpha, inv_num_valid};
//         f32 A(batch*K,M) B(batch*K,N) V(batch*N,D) G(batch*M,D) P(batch*M,N) mask(M,N)
//         logits(C,NC) labels(1,NC) cmask(1,NC)
// Output: m(batch*M) l(batch*M) O(batch*M,D) gradQ(batch*K,M) R(batch*M) gradK(batch*K,N)
//         gradV(batch*K,N) col_denom(NC) ce_grad(C,NC) loss_vec(NC) gathered(NC,NC2=NC) ... see below
#include <cstdint>
#include <fstream>
#include <iostream>
#include <vector>

#include "neuralnet.cpp/nn.hpp"

using namespace nn;

static Tensor read_t(std::ifstream& f, std::size_t r, std::size_t c)
{
    Matrix m(r, c);
    f.read(reinterpret_cast<char*>(m.span().data()), static_cast<std::streamsize>(m.size() * sizeof(Scalar)));
    return Tensor::from_matrix(std::move(m));
}
static void write_t(std::ofstream& f, const Tensor& t)
{
    auto s = t.cpu_matrix().span();
    f.write(reinterpret_cast<const char*>(s.data()), static_cast<std::streamsize>(s.size() * sizeof(Scalar)));
}
#define TAKE(var, expr) auto var##_r = (expr); if (!var##_r) { std::cerr << #expr << ": " << var##_r.error().message << "\n"; return 2; } auto& var = *var##_r

int main(int argc, char** argv)
{
    if (argc < 3) return 1;
    std::ifstream in(argv[1], std::ios::binary);
    std::int32_t I[8]; float F[2];
    in.read(reinterpret_cast<char*>(I), sizeof I);
    in.read(reinterpret_cast<char*>(F), sizeof F);
    const std::size_t batch = I[0], M = I[1], N = I[2], K = I[3], D = I[4], C = I[5], NC = I[6], vocab = I[7];
    const Scalar alpha = F[0], inv_nv = F[1];
    Tensor A = read_t(in, batch * K, M), B = read_t(in, batch * K, N), V = read_t(in, batch * N, D);
    Tensor G = read_t(in, batch * M, D), P = read_t(in, batch * M, N), mask = read_t(in, M, N);
    Tensor logits = read_t(in, C, NC), labels = read_t(in, 1, NC), cmask = read_t(in, 1, NC);
    if (!in) { std::cerr << "ref_prims: short input\n"; return 1; }

    CpuEngine e;
    std::ofstream out(argv[2], std::ios::binary);
    TAKE(m, e.batched_matmul_reduce(A, B, batch, ReduceOp::Max, true, false, alpha, true, &mask));
    TAKE(l, e.batched_matmul_softmax_denom(A, B, m, batch, true, false, alpha, &mask));
    TAKE(O, e.batched_matmul_softmax_apply(A, B, V, m, l, batch, true, false, alpha, &mask));
    Tensor R, gradV, loss_vec;
    TAKE(gq, e.batched_matmul_softmax_backward_q(A, B, P, m, l, batch, true, false, alpha, R, &mask));
    TAKE(gk, e.batched_matmul_softmax_backward_kv(A, B, P, G, R, m, l, batch, true, false, alpha, gradV, &mask));
    TAKE(cmax, e.col_reduce_max(logits));
    TAKE(cden, e.col_softmax_denom(logits, cmax));
    TAKE(ceg, e.col_softmax_sparse_forward(logits, labels, &cmask, vocab, inv_nv, loss_vec));
    // gather rows of `logits` (C, NC) by `labels` (out-of-range ids give zero rows) and scatter them back
    TAKE(gath, e.gather_rows(logits, labels));
    Tensor dst = e.create_tensor(C, NC);
    { auto z = e.zero(dst); if (!z) return 2; }
    { auto s = e.scatter_add_rows(dst, labels, gath); if (!s) { std::cerr << s.error().message << "\n"; return 2; } }
    TAKE(re, e.rearrange_3d(A, K, batch, M, true));   // (batch*K, M) -> (K, batch*M)
    for (const Tensor* t : {&m, &l, &O, &gq, &R, &gk, &gradV, &cden, &ceg, &loss_vec, &gath, &dst, &re})
        write_t(out, *t);
    return out ? 0 : 1;
}
