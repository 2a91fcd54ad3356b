// C++ driver of the fused GPT training step through the reference's own API: Model::add<B200GPTModel>, the
// Optimizer interface (FusedAdamW, FusedMuon), save_model, and the loop order of src/text_train.cpp:1107-1334
// (per micro-batch forward -> sparse cross-entropy -> backward with the logit gradient scaled by 1/accum; per step
// clip -> optimizer step -> zero_grad; learning rate from compute_step_lr).  Built against the unmodified reference
// headers with this repository's drop-in CUDA backend / engine headers force-included (see the Makefile beside it).
//
//   fused_train run <in.bin> <out.bin> [--precision 0|1] [--save model.bin]
//       One training run described by a binary file, results to another.  Input (little endian): u32 magic
//       0x3242424E, i32 I[32], f32 F[16], i32 n_params, per parameter {i32 rows, i32 cols, f32 data} in
//       GPTModel::parameters order, then per micro-batch i32 tokens[B*S] (batch-major), i32 labels[B*S],
//       f32 loss_mask[B*S] and, when I[10] != 0, i32 doc_ids[B*S].
//       I: 0 vocab, 1 d_model, 2 heads, 3 layers, 4 d_ff, 5 seq, 6 batch, 7 activation, 8 norm, 9 position encoding
//       (the reference's enum values), 10 document ids present, 11 optimizer steps, 12 accumulation, 13 optimizer
//       (0 AdamW; 1 Muon on the hidden matrices + AdamW on the rest), 14 clip on, 15 cosine schedule, 16 warm-up steps,
//       17 total steps, 18 dump the gradients of step 0, 19 dump the logits of micro-batch 0, 20 skip the final parameters.
//       F: 0 lr, 1 weight decay, 2 clip norm, 3 minimum lr, 4 Muon lr.
//       21 > 0: after training, GPTModel-style forward_step over the first I[21] tokens of a list that follows the
//       batches (i32 count, i32 ids[count]); 22 > 0: generate I[22] tokens from that list as the prompt, temperature 0.
//       Output: f32 loss per micro-batch; [gradients]; [logits (vocab, tokens)]; [final parameters]; f64 seconds per step;
//       [f32 logits of every decode step (vocab each)]; [i32 count, i32 generated ids].
//   fused_train bench [--steps K] [--warmup W] [--layers L] [--batch B]
//       BASELINE configuration 3 (vocab 8192, d 768, 12 heads, 12 layers, SwiGLU 2048, RMSNorm, ALiBi, seq 1024,
//       micro-batch 16 x accumulation 2, AdamW + cosine schedule, bf16) on synthetic Zipf(1.1) tokens: prints one JSON
//       line with the device-timed milliseconds per step, ids resident on the device and through host matrices.
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "neuralnet.cpp/nn.hpp"
#include "neuralnet.cpp/cli/lr_scheduler.hpp"
#include "nnb200_fused_gpt.hpp"

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

#define TRY(expr)                                                                                    \
    do {                                                                                             \
        auto&& r_ = (expr);                                                                          \
        if (!r_) { std::cerr << "fused_train: " #expr ": " << r_.error().message << "\n"; return 2; } \
    } while (0)

const char* arg_value(int argc, char** argv, const char* name, const char* dflt)
{
    for (int i = 0; i + 1 < argc; ++i)
        if (std::strcmp(argv[i], name) == 0) return argv[i + 1];
    return dflt;
}

// optimizer objects of one run: AdamW over everything, or the Muon split
struct Optimizers {
    std::unique_ptr<FusedAdamW> adamw;
    std::unique_ptr<FusedMuon> muon;
    void set_lr(Scalar lr, Scalar muon_lr) { adamw->set_lr(lr); if (muon) muon->set_lr(muon_lr); }
};

int run_file(int argc, char** argv)
{
    if (argc < 4) { std::cerr << "usage: fused_train run <in.bin> <out.bin> [--precision 0|1] [--save file]\n"; return 1; }
    std::ifstream in(argv[2], std::ios::binary);
    if (!in) { std::cerr << "fused_train: cannot open " << argv[2] << "\n"; return 1; }
    const int precision = std::atoi(arg_value(argc, argv, "--precision", "1"));
    const std::string save_path = arg_value(argc, argv, "--save", "");
    std::uint32_t magic = 0;
    std::int32_t I[32];
    float F[16];
    if (!rd(in, &magic, 1) || magic != 0x3242424Eu || !rd(in, I, 32) || !rd(in, F, 16)) { std::cerr << "fused_train: bad header\n"; return 1; }
    const std::size_t V = I[0], D = I[1], H = I[2], L = I[3], FF = I[4], S = I[5], B = I[6];
    const auto act = static_cast<ActivationType>(I[7]);
    const auto norm = static_cast<NormType>(I[8]);
    const auto pos = static_cast<PosEncodingType>(I[9]);
    const bool use_doc = I[10] != 0;
    const int steps = I[11], accum = I[12] > 0 ? I[12] : 1, opt_kind = I[13];
    const bool clip = I[14] != 0, dump_grads = I[18] != 0, dump_logits = I[19] != 0, skip_params = I[20] != 0;

    TRY(CudaBackend::instance().initialize());
    CudaEngine engine(CudaBackend::instance());
    Model model(engine);
    model.add<B200GPTModel>(engine, GptConfig{V, D, S, H, FF, L, pos, act, norm}, B,
                            precision ? B200Precision::BF16 : B200Precision::FP32Check);
    auto& gpt = static_cast<B200GPTModel&>(model.layer_at(0));
    TRY(gpt.status());

    auto params = model.parameters();
    auto grads = model.param_gradients();
    std::int32_t n_params = 0;
    if (!rd(in, &n_params, 1) || static_cast<std::size_t>(n_params) != params.size())
    { std::cerr << "fused_train: parameter count mismatch: file " << n_params << " model " << params.size() << "\n"; return 1; }
    for (auto& p : params)
    {
        std::int32_t rc[2];
        if (!rd(in, rc, 2) || static_cast<std::size_t>(rc[0]) != p.get().rows() || static_cast<std::size_t>(rc[1]) != p.get().cols())
        { std::cerr << "fused_train: parameter shape mismatch\n"; return 1; }
        Matrix m(p.get().rows(), p.get().cols());
        if (!rd(in, m.span().data(), m.size())) { std::cerr << "fused_train: short parameter data\n"; return 1; }
        TRY(engine.copy_from(p.get(), m));                     // the call load_model makes per parameter
    }

    Optimizers opt;
    opt.adamw = std::make_unique<FusedAdamW>(engine, gpt, F[0], 0.9, 0.999, 1e-8, F[1], /*upto_matrices=*/opt_kind == 1);
    if (opt_kind == 1) opt.muon = std::make_unique<FusedMuon>(engine, gpt, F[4]);

    cli::StepLrScheduleConfig sched;
    sched.base_lr = F[0]; sched.min_lr = F[3]; sched.warmup_steps = I[16];
    sched.total_steps = I[17]; sched.cosine = I[15] != 0;

    std::ofstream out(argv[3], std::ios::binary);
    std::vector<float> losses;
    std::vector<double> secs;
    std::vector<Matrix> grads_dump;
    Matrix logits_dump;
    B200CrossEntropy ce;
    const std::size_t N = B * S;
    std::vector<std::int32_t> tok(N), lab(N), doc(N);
    std::vector<float> msk(N);

    for (int step = 0; step < steps; ++step)
    {
        const auto t0 = std::chrono::steady_clock::now();
        if (sched.cosine || sched.warmup_steps > 0)
        {
            const Scalar lr = cli::compute_step_lr(sched, step);
            opt.set_lr(lr, lr * F[4] / F[0]);
        }
        for (int a = 0; a < accum; ++a)
        {
            if (!rd(in, tok.data(), N) || !rd(in, lab.data(), N) || !rd(in, msk.data(), N) || (use_doc && !rd(in, doc.data(), N)))
            { std::cerr << "fused_train: short batch data\n"; return 1; }
            Matrix x(S, B);
            for (std::size_t b = 0; b < B; ++b)
                for (std::size_t t = 0; t < S; ++t) x.set_value_unchecked(t, b, static_cast<Scalar>(tok[b * S + t]));
            std::vector<std::size_t> labels(N), doc_ids;
            for (std::size_t i = 0; i < N; ++i) labels[i] = static_cast<std::size_t>(lab[i]);
            if (use_doc) { doc_ids.assign(doc.begin(), doc.end()); model.set_doc_ids(doc_ids); }
            else model.set_doc_ids({});

            auto xt = engine.from_matrix(x);            TRY(xt);
            TRY(engine.begin_batch());
            auto logits = model.forward(*xt);           TRY(logits);
            if (dump_logits && step == 0 && a == 0)
            {
                auto lt = gpt.logits(engine);           TRY(lt);
                auto m = engine.to_matrix(*lt);         TRY(m);
                logits_dump = std::move(*m);
            }
            auto loss = ce.forward_sparse(engine, gpt, labels, std::span<const Scalar>(msk), Scalar{1} / static_cast<Scalar>(accum));
            TRY(loss);
            losses.push_back(*loss);
            auto gi = model.backward(*logits);          TRY(gi);
            TRY(engine.end_batch());
        }
        if (dump_grads && step == 0)
            for (auto& gr : grads) { auto m = engine.to_matrix(gr.get()); TRY(m); grads_dump.push_back(std::move(*m)); }
        if (clip) TRY(gpt.compute_grad_scale(F[2]));           // one global norm for both optimizer objects
        TRY(engine.begin_batch());
        if (opt.muon) TRY(opt.muon->step());
        TRY(opt.adamw->step());
        TRY(opt.adamw->zero_grad());
        TRY(engine.end_batch());
        secs.push_back(std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
    }
    TRY(gpt.check_device_status());

    out.write(reinterpret_cast<const char*>(losses.data()), static_cast<std::streamsize>(losses.size() * sizeof(float)));
    for (auto& m : grads_dump) wr_matrix(out, m);
    if (dump_logits) wr_matrix(out, logits_dump);
    if (!skip_params)
        for (auto& p : params) { auto m = engine.to_matrix(p.get()); TRY(m); wr_matrix(out, *m); }
    out.write(reinterpret_cast<const char*>(secs.data()), static_cast<std::streamsize>(secs.size() * sizeof(double)));
    if (I[21] > 0 || I[22] > 0)
    {   // incremental inference: a token list follows the batches; I[21] forward_step logits and / or I[22] generated ids (temperature 0)
        std::int32_t count = 0;
        if (!rd(in, &count, 1) || count <= 0) { std::cerr << "fused_train: decode token list missing\n"; return 1; }
        std::vector<std::int32_t> ids(static_cast<std::size_t>(count));
        if (!rd(in, ids.data(), ids.size())) { std::cerr << "fused_train: short decode token list\n"; return 1; }
        for (int t = 0; t < I[21] && t < count; ++t)
        {
            auto lg = gpt.forward_step(engine, static_cast<std::size_t>(ids[t]), static_cast<std::size_t>(t), static_cast<std::size_t>(t));
            TRY(lg);
            auto m = engine.to_matrix(*lg); TRY(m);
            wr_matrix(out, *m);
        }
        if (I[22] > 0)
        {
            std::vector<std::size_t> prompt(ids.begin(), ids.end());
            auto gen = gpt.generate(engine, prompt, static_cast<std::size_t>(I[22]), Scalar{0});
            TRY(gen);
            const std::int32_t n = static_cast<std::int32_t>(gen->size());
            out.write(reinterpret_cast<const char*>(&n), sizeof(n));
            for (auto id : *gen) { const std::int32_t v = static_cast<std::int32_t>(id); out.write(reinterpret_cast<const char*>(&v), sizeof(v)); }
        }
    }
    if (!save_path.empty())
        TRY(save_model(save_path, model, make_gpt_spec(V, D, S, H, FF, L, pos, act, norm)));
    std::cerr << "fused_train: precision=" << precision << " steps=" << steps << " last_loss=" << (losses.empty() ? 0.f : losses.back()) << "\n";
    return out ? 0 : 1;
}

// Zipf(s) ids by inverse CDF over a precomputed table
std::vector<std::int32_t> zipf_ids(std::mt19937_64& rng, std::size_t vocab, std::size_t n, double s = 1.1)
{
    std::vector<double> cdf(vocab);
    double acc = 0;
    for (std::size_t k = 0; k < vocab; ++k) { acc += 1.0 / std::pow(static_cast<double>(k + 1), s); cdf[k] = acc; }
    std::uniform_real_distribution<double> u(0.0, 1.0);
    std::vector<std::int32_t> ids(n);
    for (auto& id : ids)
    {
        const double x = u(rng) * acc;
        id = static_cast<std::int32_t>(std::min<std::size_t>(static_cast<std::size_t>(std::lower_bound(cdf.begin(), cdf.end(), x) - cdf.begin()), vocab - 1));
    }
    return ids;
}

int run_bench(int argc, char** argv)
{
    const int K = std::max(1, std::atoi(arg_value(argc, argv, "--steps", "10")));
    const int W = std::max(0, std::atoi(arg_value(argc, argv, "--warmup", "3")));
    const std::size_t L = static_cast<std::size_t>(std::atoi(arg_value(argc, argv, "--layers", "12")));
    const std::size_t B = static_cast<std::size_t>(std::atoi(arg_value(argc, argv, "--batch", "16")));
    const std::size_t V = 8192, D = 768, H = 12, FF = 2048, S = 1024;
    const int accum = 2;
    const Scalar base_lr = 6e-4f, min_lr = 6e-5f, wd = 0.01f;

    TRY(CudaBackend::instance().initialize());
    CudaEngine engine(CudaBackend::instance());
    Model model(engine);
    model.add<B200GPTModel>(engine, GptConfig{V, D, S, H, FF, L, PosEncodingType::ALiBi, ActivationType::SwiGLU, NormType::RMSNorm}, B,
                            B200Precision::BF16);
    auto& gpt = static_cast<B200GPTModel&>(model.layer_at(0));
    TRY(gpt.status());
    TRY(gpt.init_parameters(42));
    FusedAdamW opt(engine, gpt, base_lr, 0.9, 0.999, 1e-8, wd);
    B200CrossEntropy ce;
    cli::StepLrScheduleConfig sched;
    sched.base_lr = base_lr; sched.min_lr = min_lr; sched.warmup_steps = 2; sched.total_steps = 1000; sched.cosine = true;

    // a small pool of distinct micro-batches, cycled: S+1 ids per row, x = ids[:S], y = ids[1:]
    const std::size_t N = B * S, pool = static_cast<std::size_t>(accum) * 4;
    std::mt19937_64 rng(1000);
    std::vector<Matrix> xs;
    std::vector<std::vector<std::size_t>> ys;
    std::vector<std::vector<std::int32_t>> xi, yi;
    for (std::size_t p = 0; p < pool; ++p)
    {
        const auto ids = zipf_ids(rng, V, B * (S + 1));
        Matrix x(S, B);
        std::vector<std::size_t> y(N);
        std::vector<std::int32_t> x32(N), y32(N);
        for (std::size_t b = 0; b < B; ++b)
            for (std::size_t t = 0; t < S; ++t)
            {
                x.set_value_unchecked(t, b, static_cast<Scalar>(ids[b * (S + 1) + t]));
                y[b * S + t] = static_cast<std::size_t>(ids[b * (S + 1) + t + 1]);
                x32[b * S + t] = ids[b * (S + 1) + t];
                y32[b * S + t] = ids[b * (S + 1) + t + 1];
            }
        xs.push_back(std::move(x)); ys.push_back(std::move(y)); xi.push_back(std::move(x32)); yi.push_back(std::move(y32));
    }
    // resident copies: ids and labels on the device as int32
    std::vector<Tensor> dev_x, dev_y;
    for (std::size_t p = 0; p < pool; ++p)
    {
        Tensor tx = engine.create_tensor(1, N), ty = engine.create_tensor(1, N);
        if (!tx.valid() || !ty.valid()) { std::cerr << "fused_train: allocation failed\n"; return 2; }
        TRY(cuda_detail::check(nnb200_rt_upload(tx.cuda_tensor().data(), xi[p].data(), N * 4), "upload"));
        TRY(cuda_detail::check(nnb200_rt_upload(ty.cuda_tensor().data(), yi[p].data(), N * 4), "upload"));
        dev_x.push_back(std::move(tx)); dev_y.push_back(std::move(ty));
    }

    float last_loss = 0.f;
    auto run_step = [&](int step, bool resident) -> int {
        opt.set_lr(cli::compute_step_lr(sched, step));
        for (int a = 0; a < accum; ++a)
        {
            const std::size_t p = (static_cast<std::size_t>(step) * accum + a) % pool;
            if (resident)
            {
                auto lg = gpt.forward_device_ids(engine, reinterpret_cast<const std::int32_t*>(dev_x[p].cuda_tensor().data()));  TRY(lg);
                TRY(gpt.loss_device(reinterpret_cast<const std::int32_t*>(dev_y[p].cuda_tensor().data()), nullptr, Scalar{1} / accum));
                auto gi = model.backward(*lg);                   TRY(gi);
            }
            else
            {   // the reference loop: a host matrix of ids in, the scalar loss out, every micro-batch
                auto xt = engine.from_matrix(xs[p]);             TRY(xt);
                auto lg = model.forward(*xt);                    TRY(lg);
                auto loss = ce.forward_sparse(engine, gpt, ys[p], {}, Scalar{1} / accum);   TRY(loss);
                last_loss = static_cast<float>(*loss);
                auto gi = model.backward(*lg);                   TRY(gi);
            }
        }
        TRY(opt.step());
        TRY(opt.zero_grad());
        return 0;
    };
    auto timed = [&](int first, bool resident, float* ms) -> int {
        TRY(cuda_detail::check(nnb200_rt_sync(), "sync"));
        TRY(cuda_detail::check(nnb200_rt_timer_start(), "timer"));
        for (int s = 0; s < K; ++s)
            if (int rc = run_step(first + s, resident)) return rc;
        TRY(cuda_detail::check(nnb200_rt_timer_stop(ms), "timer"));
        return 0;
    };
    for (int s = 0; s < W; ++s)
        if (int rc = run_step(s, true)) return rc;
    nnb200_launch_count(1);
    float ms_res = 0.f, ms_e2e = 0.f;
    if (int rc = timed(W, true, &ms_res)) return rc;
    const unsigned long long launches = nnb200_launch_count(1);
    if (int rc = run_step(W + K, false)) return rc;
    if (int rc = timed(W + K + 1, false, &ms_e2e)) return rc;
    TRY(gpt.check_device_status());
    const double tokens = static_cast<double>(N) * accum;
    std::printf("{\"host\": \"cpp\", \"steps\": %d, \"warmup\": %d, \"layers\": %zu, \"micro_batch\": %zu, \"tokens_per_step\": %.0f, "
                "\"ms_per_step\": %.4f, \"tokens_per_s\": %.1f, \"e2e_ms_per_step\": %.4f, \"e2e_tokens_per_s\": %.1f, "
                "\"gpu_launches\": %llu, \"last_loss\": %.5f}\n",
                K, W, L, B, tokens, ms_res / K, tokens * K / (ms_res * 1e-3), ms_e2e / K, tokens * K / (ms_e2e * 1e-3), launches, last_loss);
    return 0;
}

}  // namespace

int main(int argc, char** argv)
{
    if (argc >= 2 && std::strcmp(argv[1], "run") == 0) return run_file(argc, argv);
    if (argc >= 2 && std::strcmp(argv[1], "bench") == 0) return run_bench(argc, argv);
    std::cerr << "usage: fused_train run <in.bin> <out.bin> [--precision 0|1] [--save file]\n"
                 "       fused_train bench [--steps K] [--warmup W] [--layers L] [--batch B]\n";
    return 1;
}
