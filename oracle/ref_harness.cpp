// TEST INFRASTRUCTURE — not part of the shipped product.
//
// Drives the *unmodified* reference headers (neuralnet.cpp: CpuEngine, GPTModel,
// CrossEntropyLoss::forward_sparse, AdamW, Muon, clip_grad_norm, compute_step_lr)
// through the training-loop order of the reference driver (src/text_train.cpp:1107-1334)
// on inputs read from a binary file, and writes per-micro-step losses, optional
// gradients/logits and the final parameters to a binary file.  It is compiled from the
// reference sources where they lie (see oracle/Makefile) into oracle/_ref/ref_gpt and is
// used (1) to generate the golden vectors under tests/golden/, (2) to pin the numpy
// restatement in oracle/gpt_oracle.py and (3) as the timed CPU baseline of bench.py.
//
// Input file (little endian):
//   u32 magic 0x3242424E ("NBB2"), i32 I[32], f32 F[16],
//   i32 n_params, then per parameter {i32 rows, i32 cols, f32 data[rows*cols]} in the
//   reference parameter order (GPTModel::parameters, compute_layer.hpp:2739-2755),
//   then per micro-step: i32 tokens[B*S] (batch-major b*S+t), i32 labels[B*S],
//   f32 loss_mask[B*S], and i32 doc_ids[B*S] when I[10] != 0.
//   I: 0 vocab 1 d_model 2 heads 3 layers 4 d_ff 5 seq 6 batch 7 act(0 GeLU,1 SwiGLU)
//      8 norm(0 LayerNorm,1 RMSNorm) 9 pos(0 learned,1 sinusoidal,2 ALiBi) 10 use_doc_ids
//      11 optimizer steps 12 accum 13 optimizer(0 AdamW, 1 Muon on hidden 2-D + AdamW rest)
//      14 clip enabled 15 cosine schedule 16 warmup 17 total_steps 18 dump grads of step 0
//      19 dump logits of micro-step 0 20 skip final params
//      21 decode: after training, run GPTModel::forward_step over the first I[21] tokens of a token list that follows
//         the batches in the input (i32 count, i32 ids[count]) and dump the (vocab) logits of every step
//      22 generate: GPTModel::generate(those tokens as the prompt, I[22] new tokens, temperature 0) and dump the ids
//   F: 0 lr 1 weight decay 2 clip max norm 3 min_lr 4 muon lr
// Output file: f32 loss[steps*accum]; [grads, reference order]; [logits (V, B*S)];
//   [final params, reference order]; f64 seconds[steps] (wall time per optimizer step);
//   [decode: f32 logits[I[21]][vocab]]; [generate: i32 count, i32 ids[count]].
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <memory>
#include <thread>
#include <vector>

#include "neuralnet.cpp/nn.hpp"
#include "neuralnet.cpp/cli/lr_scheduler.hpp"

using namespace nn;

namespace {
template <typename T>
bool rd(std::ifstream& f, T* p, std::size_t n)
{
    f.read(reinterpret_cast<char*>(p), static_cast<std::streamsize>(n * sizeof(T)));
    return static_cast<bool>(f);
}
void wr_matrix(std::ofstream& f, const Matrix& m)
{
    auto s = m.span();
    f.write(reinterpret_cast<const char*>(s.data()), static_cast<std::streamsize>(s.size() * sizeof(Scalar)));
}
#define CHECK(expr)                                                             \
    do {                                                                        \
        auto&& _r = (expr);                                                     \
        if (!_r) { std::cerr << "ref_gpt: " #expr ": " << _r.error().message << "\n"; return 2; } \
    } while (0)
}  // namespace

int main(int argc, char** argv)
{
    if (argc < 3) { std::cerr << "usage: ref_gpt <in.bin> <out.bin>\n"; return 1; }
    std::ifstream in(argv[1], std::ios::binary);
    if (!in) { std::cerr << "ref_gpt: cannot open " << argv[1] << "\n"; return 1; }
    std::uint32_t magic = 0;
    std::int32_t I[32];
    float F[16];
    if (!rd(in, &magic, 1) || magic != 0x3242424Eu || !rd(in, I, 32) || !rd(in, F, 16))
    { std::cerr << "ref_gpt: bad header\n"; return 1; }

    const std::size_t V = I[0], D = I[1], H = I[2], L = I[3], FF = I[4], S = I[5], B = I[6];
    const auto act = static_cast<ActivationType>(I[7]);
    const auto norm = static_cast<NormType>(I[8]);
    const auto pos = static_cast<PosEncodingType>(I[9]);
    const bool use_doc = I[10] != 0;
    const int steps = I[11], accum = I[12] > 0 ? I[12] : 1, opt_kind = I[13];
    const bool clip = I[14] != 0, dump_grads = I[18] != 0, dump_logits = I[19] != 0, skip_params = I[20] != 0;

    CpuEngine engine;
    auto model_r = build_gpt_model(engine, GptConfig{V, D, S, H, FF, L, pos, act, norm});
    if (!model_r) { std::cerr << model_r.error().message << "\n"; return 2; }
    Model model = std::move(*model_r);

    auto params = model.parameters();
    auto grads = model.param_gradients();
    std::int32_t n_params = 0;
    if (!rd(in, &n_params, 1) || static_cast<std::size_t>(n_params) != params.size())
    { std::cerr << "ref_gpt: parameter count mismatch: file " << n_params << " model " << params.size() << "\n"; return 1; }
    for (auto& p : params)
    {
        std::int32_t rc[2];
        if (!rd(in, rc, 2) || static_cast<std::size_t>(rc[0]) != p.get().rows() || static_cast<std::size_t>(rc[1]) != p.get().cols())
        { std::cerr << "ref_gpt: parameter shape mismatch\n"; return 1; }
        Matrix m(p.get().rows(), p.get().cols());
        if (!rd(in, m.span().data(), m.size())) { std::cerr << "ref_gpt: short parameter data\n"; return 1; }
        CHECK(engine.copy_from(p.get(), m));
    }

    // Optimizers.  opt_kind 1: Muon on the hidden 2-D matrices (wq,wk,wv,wo,fc1,fc2 weights),
    // AdamW on everything else — the split compute_optimizer.hpp:508-511 prescribes.
    std::vector<std::unique_ptr<Optimizer>> opts;
    std::vector<bool> is_muon(params.size(), false);
    if (opt_kind == 1)
    {
        const std::size_t per_norm = (norm == NormType::LayerNorm) ? 2 : 1;
        std::size_t idx = 1 + ((pos == PosEncodingType::Learned) ? 1 : 0);
        for (std::size_t l = 0; l < L; ++l)
        {
            for (int k = 0; k < 4; ++k) { is_muon[idx] = true; idx += 2; }  // wq wk wv wo (W,b)
            idx += per_norm;                                                // norm1
            is_muon[idx] = true; idx += 2;                                  // fc1
            is_muon[idx] = true; idx += 2;                                  // fc2
            idx += per_norm;                                                // norm2
        }
        std::vector<TensorRef> pm, gm, pa, ga;
        for (std::size_t i = 0; i < params.size(); ++i)
        {
            if (is_muon[i]) { pm.push_back(params[i]); gm.push_back(grads[i]); }
            else            { pa.push_back(params[i]); ga.push_back(grads[i]); }
        }
        opts.push_back(std::make_unique<Muon>(engine, pm, gm, F[4]));
        opts.push_back(std::make_unique<AdamW>(engine, pa, ga, F[0], 0.9, 0.999, 1e-8, F[1]));
    }
    else
    {
        opts.push_back(std::make_unique<AdamW>(engine, params, grads, F[0], 0.9, 0.999, 1e-8, F[1]));
    }
    // clip_grad_norm in the reference is per optimizer object; with two optimizers the
    // harness clips through a third, gradient-only view so the norm is global.
    std::unique_ptr<Optimizer> clipper;
    if (clip) clipper = std::make_unique<SGD>(engine, params, grads, Scalar{0});

    cli::StepLrScheduleConfig sched;
    sched.base_lr = F[0]; sched.min_lr = F[3]; sched.warmup_steps = I[16];
    sched.total_steps = I[17]; sched.cosine = I[15] != 0;

    std::ofstream out(argv[2], std::ios::binary);
    std::vector<float> losses;
    std::vector<double> secs;
    std::vector<Matrix> grads_dump;
    Matrix logits_dump;
    CrossEntropyLoss ce;
    const std::size_t N = B * S;
    std::vector<std::int32_t> tok(N), lab(N), doc(N);
    std::vector<float> msk(N);

    for (int step = 0; step < steps; ++step)
    {
        const auto t0 = std::chrono::steady_clock::now();
        if (sched.cosine || sched.warmup_steps > 0)
        {
            const Scalar lr = cli::compute_step_lr(sched, step);
            // the AdamW object follows the schedule; Muon keeps its own lr scaled alike
            if (opt_kind == 1) { opts[0]->set_lr(lr * F[4] / F[0]); opts[1]->set_lr(lr); }
            else opts[0]->set_lr(lr);
        }
        for (int a = 0; a < accum; ++a)
        {
            if (!rd(in, tok.data(), N) || !rd(in, lab.data(), N) || !rd(in, msk.data(), N) || (use_doc && !rd(in, doc.data(), N)))
            { std::cerr << "ref_gpt: short batch data\n"; return 1; }
            Matrix x(S, B);
            for (std::size_t b = 0; b < B; ++b)
                for (std::size_t t = 0; t < S; ++t)
                    x.set_value_unchecked(t, b, static_cast<Scalar>(tok[b * S + t]));
            std::vector<std::size_t> labels(N), doc_ids;
            for (std::size_t i = 0; i < N; ++i) labels[i] = static_cast<std::size_t>(lab[i]);
            if (use_doc) { doc_ids.assign(doc.begin(), doc.end()); model.set_doc_ids(doc_ids); }
            else model.set_doc_ids({});

            auto xt = engine.from_matrix(x);            CHECK(xt);
            CHECK(engine.begin_batch());
            auto logits = model.forward(*xt);           CHECK(logits);
            auto loss = ce.forward_sparse(engine, *logits, labels, std::span<const Scalar>(msk), V);
            CHECK(loss);
            losses.push_back(*loss);
            if (dump_logits && step == 0 && a == 0) { auto m = engine.to_matrix(*logits); CHECK(m); logits_dump = std::move(*m); }
            CHECK(engine.flush_batch());
            auto g = ce.backward();                     CHECK(g);
            if (accum > 1) CHECK(engine.scale_inplace(*g, Scalar{1} / static_cast<Scalar>(accum)));
            auto gi = model.backward(*g);               CHECK(gi);
            CHECK(engine.end_batch());
        }
        if (dump_grads && step == 0)
            for (auto& gr : grads) { auto m = engine.to_matrix(gr.get()); CHECK(m); grads_dump.push_back(std::move(*m)); }
        if (clip) CHECK(clipper->clip_grad_norm(F[2]));
        CHECK(engine.begin_batch());
        for (auto& o : opts) CHECK(o->step());
        for (auto& o : opts) CHECK(o->zero_grad());
        CHECK(engine.end_batch());
        secs.push_back(std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
    }

    out.write(reinterpret_cast<const char*>(losses.data()), static_cast<std::streamsize>(losses.size() * sizeof(float)));
    for (auto& m : grads_dump) wr_matrix(out, m);
    if (dump_logits) wr_matrix(out, logits_dump);
    if (!skip_params)
        for (auto& p : params) { auto m = engine.to_matrix(p.get()); CHECK(m); wr_matrix(out, *m); }
    out.write(reinterpret_cast<const char*>(secs.data()), static_cast<std::streamsize>(secs.size() * sizeof(double)));
    if (I[21] > 0 || I[22] > 0)
    {
        std::int32_t count = 0;
        if (!rd(in, &count, 1) || count <= 0) { std::cerr << "ref_gpt: decode token list missing\n"; return 1; }
        std::vector<std::int32_t> ids(static_cast<std::size_t>(count));
        if (!rd(in, ids.data(), ids.size())) { std::cerr << "ref_gpt: short decode token list\n"; return 1; }
        auto& gpt = static_cast<GPTModel&>(model.layer_at(0));
        if (I[21] > 0)
        {
            std::vector<Tensor> kc, vc;
            for (std::size_t l = 0; l < L; ++l) { kc.push_back(engine.create_tensor(S, D)); vc.push_back(engine.create_tensor(S, D)); }
            for (int t = 0; t < I[21] && t < count; ++t)
            {
                auto lg = gpt.forward_step(engine, static_cast<std::size_t>(ids[t]), static_cast<std::size_t>(t), kc, vc, static_cast<std::size_t>(t));
                CHECK(lg);
                auto m = engine.to_matrix(*lg); CHECK(m);
                wr_matrix(out, *m);
            }
        }
        if (I[22] > 0)
        {
            std::vector<std::size_t> prompt(ids.begin(), ids.end());
            auto gen = gpt.generate(engine, prompt, static_cast<std::size_t>(I[22]), Scalar{0});
            CHECK(gen);
            const std::int32_t n = static_cast<std::int32_t>(gen->size());
            out.write(reinterpret_cast<const char*>(&n), sizeof(n));
            for (auto id : *gen) { const std::int32_t v = static_cast<std::int32_t>(id); out.write(reinterpret_cast<const char*>(&v), sizeof(v)); }
        }
    }
    std::cerr << "ref_gpt: threads=" << std::thread::hardware_concurrency() << " steps=" << steps
              << " last_loss=" << (losses.empty() ? 0.f : losses.back()) << "\n";
    return out ? 0 : 1;
}
