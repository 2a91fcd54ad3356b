// TEST INFRASTRUCTURE: the reference's own GPTModel (its unchanged Layer code, compute_layer.hpp:2646-2896) run once on
// the reference CpuEngine and once on this repository's drop-in CudaEngine, from the same seeded weights and tokens:
// logits, the sparse cross-entropy loss and the gradient of every parameter must agree.
//
// This is the seeded counterpart of the reference's src/gpt_gradcheck.cpp, which draws its weights from
// std::random_device and compares against fp32 central differences, and therefore fails now and then on the
// reference's own CPU engine too (rotary and ALiBi variants about one run in three).  Here nothing is random: a
// failure is a difference between the two engines.  Exit code 0 = every case agreed.
//
//   model_check [--seed N] [--verbose]
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "neuralnet.cpp/nn.hpp"
#include "neuralnet.cpp/cuda_engine.hpp"

using namespace nn;

namespace
{
bool g_verbose = false;
int g_failed = 0, g_cases = 0;

void report(const std::string& name, bool okay, double err)
{
    ++g_cases;
    if (!okay) ++g_failed;
    if (!okay || g_verbose) std::printf("  %-64s %s  err=%.3g\n", name.c_str(), okay ? "OK  " : "FAIL", err);
}
// largest difference relative to the largest reference magnitude
double rel(const Matrix& ref, const Matrix& got)
{
    if (ref.rows() != got.rows() || ref.cols() != got.cols()) return 1e30;
    double worst = 0, scale = 1e-30;
    const auto a = ref.span();
    const auto b = got.span();
    for (std::size_t i = 0; i < a.size(); ++i) { scale = std::max(scale, std::fabs(double(a[i]))); worst = std::max(worst, std::fabs(double(a[i]) - double(b[i]))); }
    return worst / scale;
}

struct Run { Matrix logits; Scalar loss = 0; std::vector<Matrix> grads; bool ok = false; std::string why; };

Run run_on(ComputeEngine& engine, const GptConfig& cfg, std::size_t batch, const std::vector<Matrix>& weights, const Matrix& x,
           const std::vector<std::size_t>& labels, const std::vector<Scalar>& mask, const std::vector<std::size_t>& docs)
{
    Run r;
    auto model_r = build_gpt_model(engine, cfg);
    if (!model_r) { r.why = model_r.error().message; return r; }
    Model model = std::move(*model_r);
    auto params = model.parameters();
    if (params.size() != weights.size()) { r.why = "parameter count"; return r; }
    for (std::size_t i = 0; i < params.size(); ++i)
        if (auto c = engine.copy_from(params[i].get(), weights[i]); !c) { r.why = c.error().message; return r; }
    model.set_doc_ids(docs);
    auto xt = engine.from_matrix(x);
    if (!xt) { r.why = xt.error().message; return r; }
    if (auto b = engine.begin_batch(); !b) { r.why = b.error().message; return r; }
    auto logits = model.forward(*xt);
    if (!logits) { r.why = "forward: " + logits.error().message; return r; }
    CrossEntropyLoss ce;
    auto loss = ce.forward_sparse(engine, *logits, labels, std::span<const Scalar>(mask), cfg.vocab_size);
    if (!loss) { r.why = "loss: " + loss.error().message; return r; }
    r.loss = *loss;
    auto lm = engine.to_matrix(*logits);
    if (!lm) { r.why = lm.error().message; return r; }
    r.logits = std::move(*lm);
    auto g = ce.backward();
    if (!g) { r.why = "loss backward: " + g.error().message; return r; }
    auto gi = model.backward(*g);
    if (!gi) { r.why = "backward: " + gi.error().message; return r; }
    if (auto e = engine.end_batch(); !e) { r.why = e.error().message; return r; }
    for (auto& gr : model.param_gradients())
    {
        auto m = engine.to_matrix(gr.get());
        if (!m) { r.why = m.error().message; return r; }
        r.grads.push_back(std::move(*m));
    }
    r.ok = true;
    (void)batch;
    return r;
}

void check_case(const std::string& name, CpuEngine& cpu, CudaEngine& gpu, const GptConfig& cfg, std::size_t batch, bool with_docs, unsigned seed)
{
    std::mt19937 rng(seed);
    std::normal_distribution<float> nd(0.f, 0.2f);
    std::uniform_int_distribution<std::size_t> tok(0, cfg.vocab_size - 1);
    // shapes of the parameters: ask a throw-away model on the CPU engine
    std::vector<Matrix> weights;
    {
        auto m = build_gpt_model(cpu, cfg);
        if (!m) { report(name + ": build", false, 0); return; }
        for (auto& p : m->parameters())
        {
            Matrix w(p.get().rows(), p.get().cols());
            // gains near one, everything else (biases included: every parameter then has a gradient that matters) N(0, 0.2)
            const bool gain = p.get().cols() == 1 && p.get().rows() == cfg.d_model;
            for (auto& v : w.span()) v = gain ? 1.f + 0.1f * nd(rng) : nd(rng);
            weights.push_back(std::move(w));
        }
    }
    const std::size_t S = cfg.seq_len, N = batch * S;
    Matrix x(S, batch);
    std::vector<std::size_t> labels(N), docs;
    std::vector<Scalar> mask(N, Scalar{1});
    for (std::size_t b = 0; b < batch; ++b)
        for (std::size_t t = 0; t < S; ++t) { x.set_value_unchecked(t, b, static_cast<Scalar>(tok(rng))); labels[b * S + t] = tok(rng); }
    mask[N / 3] = 0;                                           // one masked target, one label out of range
    labels[N / 2] = cfg.vocab_size + 3;
    if (with_docs)
    {
        docs.resize(N);
        for (std::size_t b = 0; b < batch; ++b)
            for (std::size_t t = 0; t < S; ++t) docs[b * S + t] = 1 + (t >= S / 3) + (t >= (2 * S) / 3 + b);
    }
    const Run a = run_on(cpu, cfg, batch, weights, x, labels, mask, docs);
    const Run b = run_on(gpu, cfg, batch, weights, x, labels, mask, docs);
    if (!a.ok || !b.ok) { std::printf("  %s: run failed: cpu '%s' cuda '%s'\n", name.c_str(), a.why.c_str(), b.why.c_str()); report(name, false, 0); return; }
    const double tol = 2e-5;
    double e = rel(a.logits, b.logits);
    report(name + ": logits", e < tol, e);
    e = std::fabs(double(a.loss) - double(b.loss)) / std::max(1e-30, std::fabs(double(a.loss)));
    report(name + ": loss", e < tol, e);
    double worst = 0;
    bool okay = a.grads.size() == b.grads.size();
    for (std::size_t i = 0; okay && i < a.grads.size(); ++i)
    {
        // the key bias has an analytically zero gradient (softmax ignores a per-query shift): both engines hold rounding noise there
        double scale = 0;
        for (auto v : a.grads[i].span()) scale = std::max(scale, std::fabs(double(v)));
        if (scale < 1e-6) continue;
        const double ei = rel(a.grads[i], b.grads[i]);
        if (ei >= 1e-4 && g_verbose) std::printf("    gradient %zu (%zux%zu): %.3g\n", i, a.grads[i].rows(), a.grads[i].cols(), ei);
        worst = std::max(worst, ei);
    }
    report(name + ": parameter gradients", okay && worst < 1e-4, worst);
}
}  // namespace

int main(int argc, char** argv)
{
    unsigned seed = 7;
    for (int i = 1; i < argc; ++i)
    {
        if (!std::strcmp(argv[i], "--verbose")) g_verbose = true;
        else if (!std::strcmp(argv[i], "--seed") && i + 1 < argc) seed = static_cast<unsigned>(std::atoi(argv[++i]));
    }
    if (auto r = CudaBackend::instance().initialize(); !r) { std::printf("model_check: CUDA initialisation failed, no fallback to CPU: %s\n", r.error().message.c_str()); return 2; }
    CpuEngine cpu;
    CudaEngine gpu(CudaBackend::instance());
    std::printf("model_check: reference GPTModel on CpuEngine vs CUDA engine, seed %u\n", seed);
    using P = PosEncodingType; using A = ActivationType; using Nn = NormType;
    //                vocab d   seq heads ff  layers
    check_case("learned / GeLU / LayerNorm", cpu, gpu, GptConfig{48, 32, 12, 4, 64, 2, P::Learned, A::GeLU, Nn::LayerNorm}, 2, false, seed);
    check_case("sinusoidal / SwiGLU / RMSNorm", cpu, gpu, GptConfig{48, 32, 12, 4, 48, 2, P::Sinusoidal, A::SwiGLU, Nn::RMSNorm}, 3, false, seed + 1);
    check_case("ALiBi / SwiGLU / RMSNorm", cpu, gpu, GptConfig{40, 24, 16, 3, 40, 2, P::ALiBi, A::SwiGLU, Nn::RMSNorm}, 2, false, seed + 2);
    check_case("rotary / SwiGLU / RMSNorm", cpu, gpu, GptConfig{40, 32, 16, 4, 40, 2, P::RoPE, A::SwiGLU, Nn::RMSNorm}, 2, false, seed + 3);
    check_case("learned, documents", cpu, gpu, GptConfig{48, 32, 18, 4, 64, 2, P::Learned, A::GeLU, Nn::LayerNorm}, 2, true, seed + 4);
    check_case("ALiBi, documents", cpu, gpu, GptConfig{40, 24, 18, 3, 40, 2, P::ALiBi, A::SwiGLU, Nn::RMSNorm}, 3, true, seed + 5);
    check_case("rotary, documents, 3 layers, batch 3", cpu, gpu, GptConfig{40, 32, 16, 4, 40, 3, P::RoPE, A::SwiGLU, Nn::RMSNorm}, 3, true, seed + 6);
    std::printf("model_check: %d cases, %d failed\n", g_cases, g_failed);
    return g_failed ? 1 : 0;
}
