// The fused GPT training step behind the reference's own extension points: a Layer, a loss and two Optimizers that
// a program built on neuralnet.cpp uses in place of GPTModel, CrossEntropyLoss, AdamW and Muon, with Model, TensorRef,
// save_model / load_model and the training-loop order (src/text_train.cpp:1107-1334) unchanged.
//
//   nn::Model model(engine);
//   model.add<nn::B200GPTModel>(engine, cfg, batch, nn::B200Precision::BF16);        // Model::add<LayerType>, model_container.hpp:60-65
//   auto& gpt = static_cast<nn::B200GPTModel&>(model.layer_at(0));
//   nn::FusedAdamW opt(engine, gpt, lr);                                            // : nn::Optimizer
//   nn::B200CrossEntropy ce;
//   ... logits = model.forward(x);  loss = ce.forward_sparse(engine, gpt, labels, mask, 1/accum);
//       model.backward(*logits);  opt.set_max_grad_norm(1.0);  opt.step();  opt.zero_grad();
//
// Where GPTModel issues ~40 engine primitives per block (compute_layer.hpp:2783-2896), B200GPTModel::forward and
// ::backward are one call each into libnnb200 (nnb200_gpt_forward / _backward: tcgen05 GEMMs and attention, fused row
// kernels).  Parameters and gradients live in one arena each; parameters() / param_gradients() hand out Tensor views
// into them in GPTModel::parameters order (compute_layer.hpp:2739-2755), so anything written against TensorRef —
// engine.copy_from, to_matrix, save_model, load_model, Optimizer::clip_grad_norm, the reference's own optimizers —
// works on them.  Needs the drop-in backend and engine headers (nnb200_cuda_backend.hpp, nnb200_cuda_engine.hpp)
// force-included before the reference headers, and -DNN_HAS_CUDA.  There is no CPU path: construction fails without
// a CUDA device.
#ifndef NNB200_FUSED_GPT_HPP
#define NNB200_FUSED_GPT_HPP
#ifdef NN_HAS_CUDA

#include <cmath>
#include <random>
#include <span>
#include <string>
#include <vector>

#include "neuralnet.cpp/compute_layer.hpp"
#include "neuralnet.cpp/compute_optimizer.hpp"
#include "neuralnet.cpp/domain_gpt.hpp"
#include "nnb200.h"

namespace nn
{

enum class B200Precision : int
{
    FP32Check = 0,   // fp32 SIMT arithmetic: the mode held to 1e-5 of the CPU engine
    BF16 = 1,        // bf16 tensor-core GEMMs and attention over fp32 master weights: held to 1e-2
};

namespace b200_detail
{
[[nodiscard]] inline std::unexpected<Error> fail(std::string msg) { return std::unexpected(Error{std::move(msg)}); }
[[nodiscard]] inline Result<void> ok(int rc, const char* what) { return cuda_detail::check(rc, what); }

// A block of device memory from the runtime's pool that frees itself; views into it are non-owning CudaBuffers.
class Arena
{
    std::shared_ptr<CudaBuffer> buf_;
    std::size_t floats_ = 0;

public:
    [[nodiscard]] Result<void> allocate(std::size_t floats)
    {
        auto b = CudaBuffer::allocate(floats);
        if (!b) return std::unexpected(b.error());
        buf_ = std::make_shared<CudaBuffer>(std::move(*b));
        floats_ = floats;
        return ok(nnb200_rt_zero(buf_->ptr(), floats * sizeof(float)), "zero");
    }
    [[nodiscard]] float* f32() const noexcept { return buf_ ? static_cast<float*>(buf_->ptr()) : nullptr; }
    [[nodiscard]] void* ptr() const noexcept { return buf_ ? buf_->ptr() : nullptr; }
    [[nodiscard]] std::size_t floats() const noexcept { return floats_; }
    // (rows, cols) fp32 tensor over [offset, offset + rows*cols): shares nothing with the pool, so dropping it frees nothing
    [[nodiscard]] Tensor view(std::size_t offset, std::size_t rows, std::size_t cols) const
    {
        auto vb = std::make_shared<CudaBuffer>(CudaBuffer::borrowed(f32() + offset, rows * cols));
        return Tensor::from_cuda(CudaTensor(std::move(vb), rows, cols));
    }
};
} // namespace b200_detail

class B200GPTModel final : public Layer
{
    nnb200_gpt_config cfg_{};
    std::size_t tokens_ = 0;
    Result<void> init_ = {};
    b200_detail::Arena params_, grads_, shadow_, workspace_, ids_, scal_, sumsq_, decode_ws_;
    std::vector<Tensor> param_views_, grad_views_;
    std::vector<long long> offsets_;
    long long arena_elems_ = 0, matrix_begin_ = 0;
    long long off_logits_ = 0, off_loss_ = 0, off_stats_ = 0;
    bool shadow_stale_ = true;       // parameters were (or may have been) written since the bf16 copy was made
    bool shadow_managed_ = false;    // a fused optimizer keeps the bf16 copy current; otherwise every forward refreshes it
    bool has_docs_ = false;
    bool has_scale_ = false;         // scal_[2] holds the factor (clip, 1/world) the optimizers apply to the gradients
    std::vector<std::int32_t> host_i32_;
    Tensor zero_input_grad_, handle_;

    [[nodiscard]] std::int32_t* ids_dev() const noexcept { return static_cast<std::int32_t*>(ids_.ptr()); }
    [[nodiscard]] std::int32_t* docs_dev() const noexcept { return ids_dev() + tokens_; }
    [[nodiscard]] std::int32_t* labels_dev() const noexcept { return ids_dev() + 2 * tokens_; }
    [[nodiscard]] float* mask_dev() const noexcept { return reinterpret_cast<float*>(ids_dev() + 3 * tokens_); }
    [[nodiscard]] void* stream() const noexcept { return nnb200_rt_stream(); }

    Result<void> build(std::size_t batch, B200Precision prec)
    {
        if (nnb200_rt_device() < 0)
            if (auto r = CudaBackend::instance().initialize(); !r) return r;
        cfg_.batch = static_cast<std::int32_t>(batch);
        cfg_.precision = static_cast<std::int32_t>(prec);
        const int n = nnb200_gpt_param_table(&cfg_, nullptr, nullptr, nullptr);
        if (n <= 0) return b200_detail::fail("B200GPTModel: invalid configuration");
        offsets_.resize(static_cast<std::size_t>(n));
        std::vector<std::int32_t> rows(offsets_.size()), cols(offsets_.size());
        nnb200_gpt_param_table(&cfg_, offsets_.data(), rows.data(), cols.data());
        arena_elems_ = nnb200_gpt_arena_elems(&cfg_);
        matrix_begin_ = nnb200_gpt_matrix_region_begin(&cfg_);
        tokens_ = batch * static_cast<std::size_t>(cfg_.seq);
        const auto elems = static_cast<std::size_t>(arena_elems_);
        if (auto r = params_.allocate(elems); !r) return r;
        if (auto r = grads_.allocate(elems); !r) return r;
        if (prec == B200Precision::BF16)
            if (auto r = shadow_.allocate((elems + 1) / 2); !r) return r;
        const long long ws = nnb200_gpt_workspace_bytes(&cfg_);
        if (ws <= 0) return b200_detail::fail("B200GPTModel: workspace size query failed");
        if (auto r = workspace_.allocate((static_cast<std::size_t>(ws) + 3) / 4); !r) return r;
        if (auto r = ids_.allocate(4 * tokens_); !r) return r;                 // ids | doc ids | labels | loss mask
        if (auto r = scal_.allocate(8); !r) return r;
        if (auto r = sumsq_.allocate(nnb200_sumsq_scratch_floats()); !r) return r;
        if (auto r = b200_detail::ok(nnb200_gpt_init_workspace(&cfg_, workspace_.ptr(), stream()), "nnb200_gpt_init_workspace"); !r) return r;
        off_logits_ = nnb200_gpt_workspace_offset(&cfg_, 0);
        off_loss_ = nnb200_gpt_workspace_offset(&cfg_, 1);
        off_stats_ = nnb200_gpt_workspace_offset(&cfg_, 3);
        param_views_.reserve(offsets_.size());
        grad_views_.reserve(offsets_.size());
        for (std::size_t i = 0; i < offsets_.size(); ++i)
        {
            param_views_.push_back(params_.view(static_cast<std::size_t>(offsets_[i]), rows[i], cols[i]));
            grad_views_.push_back(grads_.view(static_cast<std::size_t>(offsets_[i]), rows[i], cols[i]));
        }
        handle_ = workspace_.view(static_cast<std::size_t>(off_loss_) / 4, 1, 1);
        Matrix z(static_cast<std::size_t>(cfg_.seq), batch);
        auto zt = CudaTensor::from_matrix(z, CudaBackend::instance());
        if (!zt) return std::unexpected(zt.error());
        zero_input_grad_ = Tensor::from_cuda(std::move(*zt));
        return {};
    }

public:
    // The argument list of GPTModel (compute_layer.hpp:2691-2700) followed by the micro-batch size and the precision.
    B200GPTModel(ComputeEngine& /*engine*/, std::size_t vocab_size, std::size_t d_model, std::size_t seq_len,
                 std::size_t num_heads, std::size_t d_ff, std::size_t num_layers, PosEncodingType pos_enc,
                 ActivationType activation, NormType norm_type, std::size_t batch,
                 B200Precision precision = B200Precision::BF16)
    {
        cfg_.vocab = static_cast<std::int32_t>(vocab_size);
        cfg_.d_model = static_cast<std::int32_t>(d_model);
        cfg_.heads = static_cast<std::int32_t>(num_heads);
        cfg_.layers = static_cast<std::int32_t>(num_layers);
        cfg_.d_ff = static_cast<std::int32_t>(d_ff);
        cfg_.seq = static_cast<std::int32_t>(seq_len);
        cfg_.act = static_cast<std::int32_t>(activation);
        cfg_.norm = static_cast<std::int32_t>(norm_type);
        cfg_.pos = static_cast<std::int32_t>(pos_enc);
        if (norm_type != NormType::LayerNorm && norm_type != NormType::RMSNorm)
            init_ = b200_detail::fail("B200GPTModel: LayerNorm or RMSNorm only");
        else
            init_ = build(batch, precision);
    }
    B200GPTModel(ComputeEngine& engine, const GptConfig& c, std::size_t batch, B200Precision precision = B200Precision::BF16)
        : B200GPTModel(engine, c.vocab_size, c.d_model, c.seq_len, c.num_heads, c.d_ff, c.num_layers, c.pos_enc,
                       c.activation, c.norm_type, batch, precision) {}

    // Construction cannot throw (the reference builds with -fno-exceptions): ask here, or let the first forward report it.
    [[nodiscard]] const Result<void>& status() const noexcept { return init_; }
    [[nodiscard]] const nnb200_gpt_config& config() const noexcept { return cfg_; }
    [[nodiscard]] std::size_t tokens_per_batch() const noexcept { return tokens_; }

    // Matrices and embeddings ~ N(0, stddev), biases 0, norm scales 1 (shifts 0): the values the reference harnesses
    // overwrite GPTModel's parameters with.  The same seed gives the same weights in every process.
    [[nodiscard]] Result<void> init_parameters(std::uint64_t seed, Scalar stddev = Scalar{0.02})
    {
        if (!init_) return init_;
        std::mt19937_64 rng(seed);
        std::normal_distribution<float> nd(0.f, static_cast<float>(stddev));
        const bool layer_norm = cfg_.norm == 0;
        std::vector<bool> is_gain(param_views_.size(), false);
        {   // positions of the norm scales in GPTModel::parameters order
            std::size_t i = 1 + (cfg_.pos == 0 ? 1 : 0);
            const std::size_t per_norm = layer_norm ? 2 : 1;
            for (int l = 0; l < cfg_.layers; ++l)
            {
                i += 8; is_gain[i] = true; i += per_norm;      // wq wk wv wo (W, b), then norm1
                i += 4; is_gain[i] = true; i += per_norm;      // fc1, fc2 (W, b), then norm2
            }
            is_gain[i] = true;                                 // ln_f
        }
        for (std::size_t i = 0; i < param_views_.size(); ++i)
        {
            Tensor& t = param_views_[i];
            Matrix m(t.rows(), t.cols());
            auto sp = m.span();
            if (is_gain[i]) for (auto& v : sp) v = Scalar{1};
            else if (t.cols() == 1) for (auto& v : sp) v = Scalar{0};
            else for (auto& v : sp) v = static_cast<Scalar>(nd(rng));
            if (auto r = b200_detail::ok(nnb200_rt_upload(t.cuda_tensor().data(), sp.data(), sp.size_bytes()), "upload"); !r) return r;
        }
        shadow_stale_ = true;
        return {};
    }

    // ── Layer ───────────────────────────────────────────────────────────────────────────────────
    // input: (seq, batch) token ids as floats, host or device (GPTModel::forward, compute_layer.hpp:2783-2790).
    // Returns a (1, 1) handle: the logits stay in the step's workspace, token-major and in the step's precision;
    // logits() converts them to the reference's (vocab, tokens) fp32 matrix when a caller wants to look at them.
    [[nodiscard]] Result<Tensor> forward(ComputeEngine& engine, const Tensor& input) override
    {
        if (!init_) return std::unexpected(init_.error());
        const auto S = static_cast<std::size_t>(cfg_.seq), B = static_cast<std::size_t>(cfg_.batch);
        if (input.rows() != S || input.cols() != B)
            return b200_detail::fail("B200GPTModel::forward: expected a (" + std::to_string(S) + ", " + std::to_string(B) +
                                     ") id matrix, got " + input.shape_str());
        if (input.is_gpu())
        {
            if (auto r = b200_detail::ok(nnb200_ids_from_float(input.cuda_tensor().data(), ids_dev(), cfg_.seq, cfg_.batch, stream()),
                                         "nnb200_ids_from_float"); !r) return std::unexpected(r.error());
        }
        else
        {
            host_i32_.resize(tokens_);
            const Matrix& m = input.cpu_matrix();
            for (std::size_t b = 0; b < B; ++b)
                for (std::size_t t = 0; t < S; ++t)
                {
                    const Scalar v = m.at_unchecked(t, b);
                    host_i32_[b * S + t] = (v >= Scalar{0} && v < Scalar{2147483520.0}) ? static_cast<std::int32_t>(v) : -1;
                }
            if (auto r = b200_detail::ok(nnb200_rt_upload(ids_dev(), host_i32_.data(), tokens_ * 4), "upload ids"); !r) return std::unexpected(r.error());
        }
        return forward_ids(engine);
    }
    // The same with ids already on the device in batch-major int32 order (for drivers that stage their own input).
    [[nodiscard]] Result<Tensor> forward_device_ids(ComputeEngine& engine, const std::int32_t* ids_batch_major)
    {
        if (!init_) return std::unexpected(init_.error());
        if (auto r = b200_detail::ok(nnb200_rt_copy(ids_dev(), ids_batch_major, tokens_ * 4), "copy ids"); !r) return std::unexpected(r.error());
        return forward_ids(engine);
    }

    // grad_output is not read: the gradient of the loss with respect to the logits was left in the workspace by
    // B200CrossEntropy::forward_sparse (already scaled by 1/accumulation, text_train.cpp:1253-1258).  Returns the zero
    // (seq, batch) matrix GPTModel::backward returns for its integer input (compute_layer.hpp:2892-2895).
    [[nodiscard]] Result<Tensor> backward(ComputeEngine& /*engine*/, const Tensor& /*grad_output*/) override
    {
        if (!init_) return std::unexpected(init_.error());
        if (auto r = b200_detail::ok(nnb200_gpt_backward(&cfg_, params_.f32(), shadow_.ptr(), grads_.f32(), workspace_.ptr(), ids_dev(),
                                                         has_docs_ ? docs_dev() : nullptr, nullptr, stream()),
                                     "nnb200_gpt_backward"); !r) return std::unexpected(r.error());
        has_scale_ = false;
        return zero_input_grad_;
    }

    // Handing out mutable references means the caller may write the parameters (copy_from, load_model, a generic
    // optimizer): the bf16 copy is refreshed before the next forward.
    [[nodiscard]] std::vector<TensorRef> parameters() override
    {
        shadow_stale_ = true;
        return {param_views_.begin(), param_views_.end()};
    }
    [[nodiscard]] std::vector<TensorRef> param_gradients() override { return {grad_views_.begin(), grad_views_.end()}; }

    [[nodiscard]] Result<void> zero_grad(ComputeEngine& /*engine*/) override
    {
        if (!init_) return init_;
        has_scale_ = false;
        return b200_detail::ok(nnb200_zero_f32(grads_.f32(), static_cast<std::size_t>(arena_elems_), stream()), "nnb200_zero_f32");
    }

    // Per-token document ids, batch-major, of the next forward / backward (GPTModel::set_doc_ids,
    // compute_layer.hpp:2206-2218): attention stays inside a document; an empty span switches back to plain causal.
    void set_doc_ids(std::span<const std::size_t> ids) override
    {
        has_docs_ = false;
        if (!init_ || ids.size() != tokens_) return;
        host_i32_.resize(tokens_);
        for (std::size_t i = 0; i < tokens_; ++i) host_i32_[i] = static_cast<std::int32_t>(ids[i]);
        has_docs_ = nnb200_rt_upload(docs_dev(), host_i32_.data(), tokens_ * 4) == 0;
    }

    // ── beyond Layer ────────────────────────────────────────────────────────────────────────────
    // The logits of the last forward as the reference returns them: (vocab, tokens) fp32, a fresh tensor.
    [[nodiscard]] Result<Tensor> logits(ComputeEngine& engine)
    {
        if (!init_) return std::unexpected(init_.error());
        Tensor out = engine.create_tensor(static_cast<std::size_t>(cfg_.vocab), tokens_);
        if (!out.valid()) return b200_detail::fail("B200GPTModel::logits: allocation failed");
        const char* src = static_cast<const char*>(workspace_.ptr()) + off_logits_;
        if (auto r = b200_detail::ok(nnb200_logits_to_reference(src, out.cuda_tensor().data(), static_cast<int>(tokens_), cfg_.vocab,
                                                                cfg_.precision, stream()), "nnb200_logits_to_reference"); !r)
            return std::unexpected(r.error());
        return out;
    }

    // Sparse cross-entropy of the logits in the workspace against labels / loss mask given on the host; the logits are
    // overwritten by their gradient times grad_scale.  Used by B200CrossEntropy.
    [[nodiscard]] Result<void> loss_from_host(std::span<const std::size_t> labels, std::span<const Scalar> loss_mask, Scalar grad_scale)
    {
        if (!init_) return init_;
        if (labels.size() != tokens_) return b200_detail::fail("sparse CE: labels size mismatch");
        if (!loss_mask.empty() && loss_mask.size() != tokens_) return b200_detail::fail("sparse CE: mask size mismatch");
        host_i32_.resize(tokens_);
        // a label beyond int32 is out of range for any vocabulary: keep it out of range
        for (std::size_t i = 0; i < tokens_; ++i) host_i32_[i] = labels[i] < 2147483647u ? static_cast<std::int32_t>(labels[i]) : 2147483647;
        if (auto r = b200_detail::ok(nnb200_rt_upload(labels_dev(), host_i32_.data(), tokens_ * 4), "upload labels"); !r) return r;
        if (!loss_mask.empty())
            if (auto r = b200_detail::ok(nnb200_rt_upload(mask_dev(), loss_mask.data(), tokens_ * 4), "upload mask"); !r) return r;
        return loss_device(labels_dev(), loss_mask.empty() ? nullptr : mask_dev(), grad_scale);
    }
    [[nodiscard]] Result<void> loss_device(const std::int32_t* labels, const float* loss_mask, Scalar grad_scale)
    {
        if (!init_) return init_;
        return b200_detail::ok(nnb200_gpt_loss(&cfg_, workspace_.ptr(), labels, loss_mask, static_cast<float>(grad_scale), stream()),
                               "nnb200_gpt_loss");
    }
    // Blocking read of the scalar loss of the last loss_* call (the download CrossEntropyLoss::forward_sparse ends with).
    [[nodiscard]] Result<Scalar> read_loss()
    {
        float v = 0.f;
        const char* src = static_cast<const char*>(workspace_.ptr()) + off_loss_;
        if (auto r = b200_detail::ok(nnb200_rt_download(&v, src, 4), "download loss"); !r) return std::unexpected(r.error());
        return static_cast<Scalar>(v);
    }
    // Number of valid targets of the last loss call (what the driver weights its evaluation average with, text_train.cpp:1455-1463).
    [[nodiscard]] Result<Scalar> read_num_valid()
    {
        float v = 0.f;
        const char* src = static_cast<const char*>(workspace_.ptr()) + off_stats_;
        if (auto r = b200_detail::ok(nnb200_rt_download(&v, src, 4), "download stats"); !r) return std::unexpected(r.error());
        return static_cast<Scalar>(v);
    }

    // Global gradient norm over every tensor (Optimizer::clip_grad_norm, compute_optimizer.hpp:90-140) without its
    // host round trip: leaves on the device the factor pre_scale * (norm > max_norm ? max_norm / norm : 1) that the
    // fused optimizers multiply the gradients by.  max_norm <= 0: no clipping, the factor is pre_scale.
    [[nodiscard]] Result<void> compute_grad_scale(Scalar max_norm, Scalar pre_scale = Scalar{1})
    {
        if (!init_) return init_;
        auto r = b200_detail::ok(nnb200_grad_norm_clip(grads_.f32(), static_cast<std::size_t>(arena_elems_), static_cast<float>(pre_scale),
                                                       static_cast<float>(max_norm > 0 ? max_norm : Scalar{0}), sumsq_.f32(), scal_.f32(), stream()),
                                 "nnb200_grad_norm_clip");
        has_scale_ = static_cast<bool>(r);
        return r;
    }
    [[nodiscard]] const float* grad_scale_dev() const noexcept { return has_scale_ ? scal_.f32() + 2 : nullptr; }
    [[nodiscard]] Result<Scalar> read_grad_norm()
    {
        float v = 0.f;
        if (auto r = b200_detail::ok(nnb200_rt_download(&v, scal_.f32() + 1, 4), "download norm"); !r) return std::unexpected(r.error());
        return static_cast<Scalar>(v);
    }

    // ── inference with a key/value cache ────────────────────────────────────────────────────────
    // GPTModel::forward_step (compute_layer.hpp:2906-2950) without its cache arguments: the cache of every layer lives
    // in the model's own decode workspace (allocated at the first call).  Returns the (vocab, 1) logits.
    [[nodiscard]] Result<Tensor> forward_step(ComputeEngine& engine, std::size_t token_id, std::size_t pos, std::size_t cur_len)
    {
        if (!init_) return std::unexpected(init_.error());
        if (!decode_ws_.ptr())
        {
            const long long n = nnb200_gpt_decode_workspace_bytes(&cfg_);
            if (n <= 0) return b200_detail::fail("B200GPTModel::forward_step: workspace size query failed");
            if (auto r = decode_ws_.allocate((static_cast<std::size_t>(n) + 3) / 4); !r) return std::unexpected(r.error());
            if (auto r = b200_detail::ok(nnb200_gpt_decode_init(&cfg_, decode_ws_.ptr(), stream()), "nnb200_gpt_decode_init"); !r)
                return std::unexpected(r.error());
        }
        if (cfg_.precision == 1 && (shadow_stale_ || !shadow_managed_))
        {
            if (auto r = b200_detail::ok(nnb200_f32_to_bf16(params_.f32(), shadow_.ptr(), static_cast<std::size_t>(arena_elems_), stream()),
                                         "nnb200_f32_to_bf16"); !r) return std::unexpected(r.error());
            shadow_stale_ = false;
        }
        Tensor out = engine.create_tensor(static_cast<std::size_t>(cfg_.vocab), 1);
        if (!out.valid()) return b200_detail::fail("B200GPTModel::forward_step: allocation failed");
        if (auto r = b200_detail::ok(nnb200_gpt_forward_step(&cfg_, params_.f32(), shadow_.ptr(), decode_ws_.ptr(), static_cast<int>(token_id),
                                                             static_cast<int>(pos), static_cast<int>(cur_len), out.cuda_tensor().data(), stream()),
                                     "nnb200_gpt_forward_step"); !r) return std::unexpected(r.error());
        return out;
    }

    // GPTModel::generate (compute_layer.hpp:2952-3096), same arguments: prompt into the cache (its last seq tokens), then
    // per new token softmax-sampling of the last logits on the host at `temperature` (0 = arg max), stop at eos_token_id
    // once min_new_tokens were produced, and a rebuild of the cache from the last seq-1 tokens when it is full.
    [[nodiscard]] Result<std::vector<std::size_t>> generate(ComputeEngine& engine, const std::vector<std::size_t>& prompt,
                                                            std::size_t max_new_tokens, Scalar temperature = 1.0,
                                                            std::size_t eos_token_id = static_cast<std::size_t>(-1),
                                                            std::size_t min_new_tokens = 0)
    {
        const auto seq = static_cast<std::size_t>(cfg_.seq), vocab = static_cast<std::size_t>(cfg_.vocab);
        std::vector<std::size_t> context(prompt), generated;
        std::mt19937_64 rng{std::random_device{}()};
        std::uniform_real_distribution<Scalar> dist(0.0, 1.0);
        std::size_t cur_len = 0;
        Tensor last;
        auto fill = [&](std::size_t start) -> Result<void> {
            for (std::size_t i = start; i < context.size(); ++i)
            {
                auto r = forward_step(engine, context[i], cur_len, cur_len);
                if (!r) return std::unexpected(r.error());
                last = std::move(*r);
                ++cur_len;
            }
            return {};
        };
        if (auto r = fill(context.size() > seq ? context.size() - seq : 0); !r) return std::unexpected(r.error());
        for (std::size_t step = 0; step < max_new_tokens; ++step)
        {
            if (cur_len >= seq)
            {
                cur_len = 0;
                const std::size_t keep = seq - 1;
                if (auto r = fill(context.size() > keep ? context.size() - keep : 0); !r) return std::unexpected(r.error());
            }
            if (!last.valid()) return b200_detail::fail("B200GPTModel::generate: empty prompt");
            auto lm = engine.to_matrix(last);
            if (!lm) return std::unexpected(lm.error());
            std::vector<Scalar> p(vocab);
            for (std::size_t v = 0; v < vocab; ++v) p[v] = lm->at_unchecked(v, 0);
            if (temperature > 0.0 && temperature != 1.0) for (auto& v : p) v /= temperature;
            Scalar mx = p[0];
            for (std::size_t v = 1; v < vocab; ++v) mx = std::max(mx, p[v]);
            Scalar sum = 0;
            for (auto& v : p) { v = std::exp(v - mx); sum += v; }
            for (auto& v : p) v /= sum;
            std::size_t next = 0;
            if (temperature > 0.0)
            {
                const Scalar r = dist(rng);
                Scalar cum = 0;
                next = vocab - 1;
                for (std::size_t v = 0; v < vocab; ++v) { cum += p[v]; if (r <= cum) { next = v; break; } }
            }
            else
            {
                Scalar best = p[0];
                for (std::size_t v = 1; v < vocab; ++v) if (p[v] > best) { best = p[v]; next = v; }
            }
            context.push_back(next);
            if (step >= min_new_tokens && next == eos_token_id) break;
            generated.push_back(next);
            auto r = forward_step(engine, next, cur_len, cur_len);
            if (!r) return std::unexpected(r.error());
            last = std::move(*r);
            ++cur_len;
        }
        return generated;
    }

    // Status word of the device-side bounded waits (tcgen05 GEMM and attention kernels): an error if one ever gave up.
    [[nodiscard]] Result<void> check_device_status()
    {
        int code = 0;
        if (auto r = b200_detail::ok(nnb200_gemm_status(&code), "nnb200_gemm_status"); !r) return r;
        if (code != 0) return b200_detail::fail("a device-side wait timed out (status " + std::to_string(code) + ")");
        return {};
    }

    // for the fused optimizers
    [[nodiscard]] float* params_f32() const noexcept { return params_.f32(); }
    [[nodiscard]] float* grads_f32() const noexcept { return grads_.f32(); }
    [[nodiscard]] void* shadow_bf16() const noexcept { return shadow_.ptr(); }
    [[nodiscard]] long long arena_elems() const noexcept { return arena_elems_; }
    [[nodiscard]] long long matrix_region_begin() const noexcept { return matrix_begin_; }
    [[nodiscard]] const std::vector<long long>& offsets() const noexcept { return offsets_; }
    [[nodiscard]] const std::vector<Tensor>& parameter_views() const noexcept { return param_views_; }
    void set_shadow_managed(bool managed) noexcept { shadow_managed_ = managed; }
    void shadow_is_current() noexcept { shadow_stale_ = false; }

private:
    [[nodiscard]] Result<Tensor> forward_ids(ComputeEngine& /*engine*/)
    {
        if (cfg_.precision == 1 && (shadow_stale_ || !shadow_managed_))
        {
            if (auto r = b200_detail::ok(nnb200_f32_to_bf16(params_.f32(), shadow_.ptr(), static_cast<std::size_t>(arena_elems_), stream()),
                                         "nnb200_f32_to_bf16"); !r) return std::unexpected(r.error());
            shadow_stale_ = false;
        }
        if (auto r = b200_detail::ok(nnb200_gpt_forward(&cfg_, params_.f32(), shadow_.ptr(), workspace_.ptr(), ids_dev(),
                                                        has_docs_ ? docs_dev() : nullptr, stream()), "nnb200_gpt_forward"); !r)
            return std::unexpected(r.error());
        return handle_;
    }
};

// CrossEntropyLoss::forward_sparse (compute_loss.hpp:229-309) for the fused model: same arguments, with the model in
// place of the logits tensor (they never leave its workspace) and the 1/accumulation factor the driver otherwise
// applies to the gradient afterwards (text_train.cpp:1253-1258).  The gradient needs no backward() call: it replaces
// the logits in place and B200GPTModel::backward picks it up.
class B200CrossEntropy
{
public:
    [[nodiscard]] Result<Scalar> forward_sparse(ComputeEngine& /*engine*/, B200GPTModel& model, std::span<const std::size_t> labels,
                                                std::span<const Scalar> loss_mask = {}, Scalar grad_scale = Scalar{1})
    {
        if (auto r = model.loss_from_host(labels, loss_mask, grad_scale); !r) return std::unexpected(r.error());
        return model.read_loss();
    }
};

// AdamW::step (compute_optimizer.hpp:388-412) over the model's arena in one launch, bias correction, decoupled decay
// of every parameter and the bf16 copy of the updated weights included.  With `upto_matrices` it covers only the
// embeddings, head and vectors — the AdamW half of the Muon split (compute_optimizer.hpp:508-511).
class FusedAdamW final : public Optimizer
{
    B200GPTModel& model_;
    b200_detail::Arena m_, v_;
    Result<void> init_ = {};
    Scalar lr_, beta1_, beta2_, eps_, wd_, max_norm_ = Scalar{0};
    std::size_t t_ = 0, n_ = 0;

public:
    FusedAdamW(ComputeEngine& engine, B200GPTModel& model, Scalar lr, Scalar beta1 = 0.9, Scalar beta2 = 0.999,
               Scalar eps = 1e-8, Scalar weight_decay = 0.01, bool upto_matrices = false)
        : Optimizer(engine, model.parameters(), model.param_gradients()), model_(model), lr_(lr), beta1_(beta1), beta2_(beta2),
          eps_(eps), wd_(weight_decay)
    {
        n_ = static_cast<std::size_t>(upto_matrices ? model.matrix_region_begin() : model.arena_elems());
        if (auto r = m_.allocate(n_); !r) init_ = r;
        else if (auto r2 = v_.allocate(n_); !r2) init_ = r2;
        model_.set_shadow_managed(true);
    }
    void set_lr(Scalar lr) override { lr_ = lr; }
    // step() clips to this global norm first (0 = off); the norm covers every gradient of the model
    void set_max_grad_norm(Scalar max_norm) { max_norm_ = max_norm; }
    [[nodiscard]] std::size_t steps_done() const noexcept { return t_; }

    [[nodiscard]] Result<void> step() override
    {
        if (!init_) return init_;
        if (max_norm_ > 0 && model_.grad_scale_dev() == nullptr)
            if (auto r = model_.compute_grad_scale(max_norm_); !r) return r;
        ++t_;
        auto r = b200_detail::ok(nnb200_adamw_step(model_.params_f32(), model_.grads_f32(), m_.f32(), v_.f32(), model_.shadow_bf16(), n_,
                                                   static_cast<float>(lr_), static_cast<float>(beta1_), static_cast<float>(beta2_),
                                                   static_cast<float>(eps_), static_cast<float>(wd_), static_cast<int>(t_),
                                                   model_.grad_scale_dev(), nnb200_rt_stream()), "nnb200_adamw_step");
        if (r && n_ == static_cast<std::size_t>(model_.arena_elems())) model_.shadow_is_current();
        return r;
    }
    [[nodiscard]] Result<void> zero_grad() override { return model_.zero_grad(engine_); }
};

// Muon::step + newton_schulz_orthogonalize (compute_optimizer.hpp:430-497, 517-590) on the hidden matrices of every
// block (wq, wk, wv, wo, fc1, fc2): momentum, Nesterov direction, normalisation and the Newton-Schulz iterations as
// tensor-core GEMMs in bf16 mode.  Pair it with FusedAdamW(..., upto_matrices = true) for everything else.
class FusedMuon final : public Optimizer
{
    B200GPTModel& model_;
    b200_detail::Arena velocity_, scratch_;
    Result<void> init_ = {};
    Scalar lr_, momentum_, ns_eps_;
    int ns_steps_;
    // the hidden matrices as arrays of device pointers / shapes, and the streams ("lanes") they are spread over: the
    // Newton-Schulz GEMMs of one matrix fill only a fraction of the machine
    std::vector<float*> p_, g_, v_;
    std::vector<void*> sh_;
    std::vector<int> rows_, cols_;
    std::size_t lane_bytes_ = 0;
    int lanes_ = 1;

public:
    FusedMuon(ComputeEngine& engine, B200GPTModel& model, Scalar lr, Scalar momentum = 0.95f, std::size_t ns_steps = 5,
              Scalar ns_eps = 1e-7f)
        : Optimizer(engine, model.parameters(), model.param_gradients()), model_(model), lr_(lr), momentum_(momentum), ns_eps_(ns_eps),
          ns_steps_(static_cast<int>(ns_steps))
    {
        const auto begin = static_cast<std::size_t>(model.matrix_region_begin());
        const auto total = static_cast<std::size_t>(model.arena_elems());
        std::size_t worst = 0;
        const auto& views = model.parameter_views();
        if (auto r = velocity_.allocate(total - begin); !r) { init_ = r; return; }
        char* shadow = static_cast<char*>(model.shadow_bf16());
        for (std::size_t i = 0; i < views.size(); ++i)
        {
            const auto off = static_cast<std::size_t>(model.offsets()[i]);
            if (off < begin) continue;
            worst = std::max(worst, nnb200_muon_scratch_bytes(static_cast<int>(views[i].rows()), static_cast<int>(views[i].cols()), model.config().precision));
            p_.push_back(model.params_f32() + off);
            g_.push_back(model.grads_f32() + off);
            v_.push_back(velocity_.f32() + (off - begin));
            sh_.push_back(shadow ? shadow + 2 * off : nullptr);
            rows_.push_back(static_cast<int>(views[i].rows()));
            cols_.push_back(static_cast<int>(views[i].cols()));
        }
        lane_bytes_ = (worst + 255) / 256 * 256;
        lanes_ = static_cast<int>(std::max<std::size_t>(1, std::min<std::size_t>(8, p_.size())));
        if (auto r2 = scratch_.allocate(lane_bytes_ * static_cast<std::size_t>(lanes_) / 4); !r2) init_ = r2;
        model_.set_shadow_managed(true);
    }
    void set_lr(Scalar lr) override { lr_ = lr; }

    [[nodiscard]] Result<void> step() override
    {
        if (!init_) return init_;
        if (auto r = b200_detail::ok(nnb200_muon_step_many(static_cast<int>(p_.size()), p_.data(), g_.data(), v_.data(),
                                                           model_.shadow_bf16() ? sh_.data() : nullptr, rows_.data(), cols_.data(),
                                                           static_cast<float>(lr_), static_cast<float>(momentum_), ns_steps_,
                                                           static_cast<float>(ns_eps_), model_.config().precision, scratch_.ptr(), lane_bytes_,
                                                           lanes_, model_.grad_scale_dev(), nnb200_rt_stream()), "nnb200_muon_step_many"); !r) return r;
        model_.shadow_is_current();      // the AdamW half, stepped before or after, keeps its own range current
        return {};
    }
    [[nodiscard]] Result<void> zero_grad() override { return model_.zero_grad(engine_); }
};

} // namespace nn

#endif // NN_HAS_CUDA
#endif // NNB200_FUSED_GPT_HPP
