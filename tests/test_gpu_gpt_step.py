"""GPU parity of the fused GPT training step against golden vectors of the reference CPU engine
(tests/golden/, produced by oracle/_ref/ref_gpt) — through the C ABI, in fp32 check mode (1e-5) and
in bf16 tensor-core mode (1e-2), the two bars the target states."""
import os

import numpy as np
import pytest

from tests.golden_io import (FULL_CASES, GOLDEN, GPT_CASES, global_rel_err, key_bias_indices, load_full_case, load_gpt_case,
                             rel_err, sample_indices, sample_tensors)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nnb():
    from tests import gpu_util
    return gpu_util.nnb


def _run(nnb, case, precision, record_logits=False):
    """The loop of src/text_train.cpp:1107-1334 on the GPU trainer.  Returns (losses, first grads,
    final params, first logits)."""
    import torch
    from oracle import gpt_oracle as go
    c, kw = case["cfg"], dict(case["kw"])
    cfg = nnb.GptConfig(c.vocab, c.d_model, c.heads, c.layers, c.d_ff, c.seq, c.batch, c.act, c.norm, c.pos, precision)
    muon = kw.get("optimizer", 0) == go.OPT_MUON_SPLIT
    tr = nnb.GptTrainer(cfg, lr=kw["lr"], weight_decay=kw.get("wd", 0.01), muon=muon, muon_lr=kw.get("muon_lr", 0.02))
    tr.load_params(case["params"])
    steps, accum = kw["steps"], kw.get("accum", 1)
    losses, first, logits = [], None, None
    it = iter(case["batches"])
    for step in range(steps):
        lr = kw["lr"]
        mlr = kw.get("muon_lr", 0.02)
        if kw.get("cosine") or kw.get("warmup", 0) > 0:
            lr = float(go.step_lr(kw["lr"], kw.get("min_lr", 0.0), kw.get("warmup", 0), kw.get("total_steps", 1),
                                  kw.get("cosine", False), step))
            mlr = lr * kw.get("muon_lr", 0.02) / kw["lr"]
        for a in range(accum):
            mb = next(it)
            tr.forward(mb["tokens"], mb["doc_ids"])
            if record_logits and step == 0 and a == 0:
                torch.cuda.synchronize()
                logits = tr.logits().float().cpu().numpy().copy()
            tr.loss_and_grad(mb["labels"], mb["mask"], 1.0 / accum)
            tr.backward()
            losses.append(float(tr.loss_tensor().item()))
        if step == 0:
            first = tr.get_grads()
        tr.optimizer_step(clip=kw.get("clip"), lr=lr, muon_lr=mlr)
    torch.cuda.synchronize()
    tr.check_device_status()
    return np.array(losses, np.float32), first, tr.get_params(), logits


@pytest.mark.parametrize("name", GPT_CASES)
def test_check_mode_matches_reference(nnb, name):
    case = load_gpt_case(name)
    losses, grads, params, logits = _run(nnb, case, nnb.FP32, record_logits=True)
    assert rel_err(logits, case["logits"].T) < 1e-5
    assert rel_err(losses, case["losses"]) < 1e-5
    skip = key_bias_indices(case["cfg"])
    assert global_rel_err(grads, case["grads"], skip) < 1e-5
    assert global_rel_err(params, case["final"], skip) < 1e-5
    for i, (p, pr) in enumerate(zip(params, case["final"])):
        if i not in skip:
            assert global_rel_err([p], [pr]) < 2e-4, i


@pytest.mark.parametrize("name", ["tile_rms_swiglu_alibi", "tile_docs_learned", "rms_swiglu_sin_clip", "docs_muon"])
def test_bf16_mode_matches_reference(nnb, name):
    case = load_gpt_case(name)
    if case["cfg"].d_model % 8 or case["cfg"].d_ff % 8 or case["cfg"].vocab % 8:
        pytest.skip("bf16 mode needs dimensions in multiples of 8")
    losses, grads, params, logits = _run(nnb, case, nnb.BF16, record_logits=True)
    assert rel_err(losses, case["losses"]) < 1e-2
    skip = key_bias_indices(case["cfg"])
    assert global_rel_err(params, case["final"], skip) < 1e-2
    assert global_rel_err(grads, case["grads"], skip) < 5e-2      # single bf16 backward: looser, reported


def _full_case_or_skip(name):
    if not os.path.isfile(os.path.join(GOLDEN, f"gpt_{name}.npz")):
        pytest.skip(f"golden gpt_{name}.npz not generated")
    return load_full_case(name)


def _check_full(case, got, tol, grad_tol, key_bias_tol, logits_l2_tol=None):
    """Losses, the logits sample, gradient / parameter samples and per-tensor norms of a full-width case against the
    reference CPU engine's.  The key-bias gradient is analytically zero (softmax does not see a per-query shift of
    the scores): instead of leaving it out silently, its norm must be negligible beside the query bias's."""
    from oracle import gpt_oracle as go
    losses, grads, params, logits = got
    cfg = case["cfg"]
    assert rel_err(losses, case["losses"]) < tol
    lg = logits.reshape(-1)
    lg = lg[sample_indices(lg.size, 4 * 4096)]
    if logits_l2_tol is None:
        assert np.abs(lg - case["logits_sample"]).max() < tol * case["logits_absmax"]
    else:
        # bf16 mode: every logit is itself rounded to bf16 (4e-3 relative) after up to twelve layers of bf16 arithmetic,
        # so single elements near zero are not held to a fraction of the largest logit; the sample as a whole is
        assert global_rel_err([lg], [case["logits_sample"]]) < logits_l2_tol
        assert np.abs(lg - case["logits_sample"]).max() < 5 * tol * case["logits_absmax"]
    names = [n for n, _, _ in go.param_shapes(cfg)]
    skip = key_bias_indices(cfg)
    assert global_rel_err(sample_tensors(grads), case["grads"], skip) < grad_tol
    assert global_rel_err(sample_tensors(params), case["final"], skip) < tol
    gn = np.array([np.linalg.norm(g.astype(np.float64)) for g in grads])
    pn = np.array([np.linalg.norm(p.astype(np.float64)) for p in params])
    for i, n in enumerate(names):
        if i in skip:
            j = names.index(n.replace("wk.b", "wq.b"))
            assert gn[i] <= key_bias_tol * gn[j], (n, gn[i], gn[j])
            assert case["g_norms"][i] <= 1e-6 * case["g_norms"][j]           # and so it is in the reference
            continue
        assert abs(gn[i] - case["g_norms"][i]) <= grad_tol * case["g_norms"][i] + 1e-12, (n, gn[i], case["g_norms"][i])
        assert abs(pn[i] - case["p1_norms"][i]) <= tol * case["p1_norms"][i] + 1e-12, (n, pn[i], case["p1_norms"][i])


@pytest.mark.parametrize("name", FULL_CASES)
def test_full_width_check_mode_matches_reference(nnb, name):
    """BASELINE configurations 2, 3 and 4 at the model shapes the benchmark runs (configuration 2 at full size;
    configuration 3 with micro-batch 2 x accumulation 2 and the cosine schedule; configuration 4 two layers deep, one
    packed row, Muon split), fp32 check mode against the reference CPU engine within 1e-5."""
    import torch
    case = _full_case_or_skip(name)
    _check_full(case, _run(nnb, case, nnb.FP32, record_logits=True), 1e-5, 1e-5, 1e-6)
    torch.cuda.empty_cache()


@pytest.mark.parametrize("name", FULL_CASES)
def test_full_width_bf16_mode_matches_reference(nnb, name):
    """The same cases on the bf16 tensor-core path (tcgen05 GEMMs and attention) within 1e-2 of the reference CPU
    engine; the gradient of a single bf16 backward pass is held to 5e-2."""
    import torch
    case = _full_case_or_skip(name)
    _check_full(case, _run(nnb, case, nnb.BF16, record_logits=True), 1e-2, 5e-2, 5e-2, logits_l2_tol=2e-2)
    torch.cuda.empty_cache()


def test_embedding_gradient_bit_exact_in_check_mode(nnb):
    """scatter_add_rows is index work: given the same row gradients the embedding gradient must be
    bit-identical to the sequential sum.  The trainer exposes the input gradient; re-add it on the
    host in ascending order and compare with the arena bit for bit."""
    import torch
    from oracle import gpt_oracle as go
    case = load_gpt_case("ln_gelu_learned")
    c = case["cfg"]
    cfg = nnb.GptConfig(c.vocab, c.d_model, c.heads, c.layers, c.d_ff, c.seq, c.batch, c.act, c.norm, c.pos, nnb.FP32)
    tr = nnb.GptTrainer(cfg)
    tr.load_params(case["params"])
    mb = case["batches"][0]
    tr.micro_step(mb["tokens"], mb["labels"], mb["mask"])
    torch.cuda.synchronize()
    n = c.batch * c.seq
    o = tr._off["grad_x0"]
    gx = tr.workspace[o:o + n * c.d_model * 4].view(torch.float32).view(n, c.d_model).cpu().numpy()
    tok = np.zeros((c.vocab, c.d_model), np.float32)
    pos = np.zeros((c.seq, c.d_model), np.float32)
    go.scatter_add_rows(tok, mb["tokens"].astype(np.float32), gx)
    go.scatter_add_rows(pos, np.tile(np.arange(c.seq), c.batch).astype(np.float32), gx)
    grads = tr.get_grads()
    assert np.array_equal(grads[0], tok)
    assert np.array_equal(grads[1], pos)


def test_config1_twenty_steps_check_mode(nnb):
    """BASELINE configuration 1 (vocab 512, d 128, 4 heads, 2 layers, FFN 512 GeLU, LayerNorm, learned
    positions, seq 128, batch 8, AdamW lr 1e-3 wd 0.01, 20 steps) against the reference loss curve."""
    import torch
    from oracle import gpt_oracle as go
    z = np.load(os.path.join(GOLDEN, "gpt_c1_20steps.npz"))
    c = go.GptConfig(*[int(v) for v in z["cfg"]])
    cfg = nnb.GptConfig(c.vocab, c.d_model, c.heads, c.layers, c.d_ff, c.seq, c.batch, c.act, c.norm, c.pos, nnb.FP32)
    tr = nnb.GptTrainer(cfg, lr=1e-3, weight_decay=0.01)
    tr.load_params(go.init_params(c, 42))
    losses = []
    for i in range(20):
        tr.micro_step(z["tokens"][i], z["labels"][i], z["mask"][i])
        losses.append(tr.loss_tensor().clone())
        tr.optimizer_step()
    torch.cuda.synchronize()
    losses = torch.cat(losses).cpu().numpy()
    assert rel_err(losses, z["losses"]) < 1e-5
    norms = np.array([np.linalg.norm(p.astype(np.float64)) for p in tr.get_params()])
    keep = [i for i in range(len(norms)) if i not in key_bias_indices(c)]
    assert np.allclose(norms[keep], z["p1_norms"][keep], rtol=1e-4)
    assert global_rel_err([tr.get_params()[-4]], [z["p1_ln_f_gamma"]]) < 1e-5


def test_config1_bf16_mode_loss_curve(nnb):
    import torch
    from oracle import gpt_oracle as go
    z = np.load(os.path.join(GOLDEN, "gpt_c1_20steps.npz"))
    c = go.GptConfig(*[int(v) for v in z["cfg"]])
    cfg = nnb.GptConfig(c.vocab, c.d_model, c.heads, c.layers, c.d_ff, c.seq, c.batch, c.act, c.norm, c.pos, nnb.BF16)
    tr = nnb.GptTrainer(cfg, lr=1e-3, weight_decay=0.01)
    tr.load_params(go.init_params(c, 42))
    losses = []
    for i in range(20):
        tr.micro_step(z["tokens"][i], z["labels"][i], z["mask"][i])
        losses.append(tr.loss_tensor().clone())
        tr.optimizer_step()
    torch.cuda.synchronize()
    tr.check_device_status()
    assert rel_err(torch.cat(losses).cpu().numpy(), z["losses"]) < 1e-2


def test_document_mask_invariance_full_seq(nnb):
    """Property of src/doc_attn_test.cpp at a larger size: with document ids, logits of later documents
    do not depend on tokens of earlier ones (<= 1e-4); without, they do (> 1e-2)."""
    import torch
    from oracle import gpt_oracle as go
    c = go.GptConfig(512, 128, 2, 2, 256, 512, 2, go.ACT_SWIGLU, go.NORM_RMS, go.POS_LEARNED)
    cfg = nnb.GptConfig(c.vocab, c.d_model, c.heads, c.layers, c.d_ff, c.seq, c.batch, c.act, c.norm, c.pos, nnb.FP32)
    tr = nnb.GptTrainer(cfg)
    tr.load_params(go.init_params(c, 7, std=0.2))
    r = np.random.default_rng(0)
    t1 = r.integers(0, c.vocab, c.tokens).astype(np.int32)
    t2 = t1.copy()
    t2[:100] = (t2[:100] + 17) % c.vocab                   # first document of row 0
    docs = np.ones((c.batch, c.seq), np.int32)
    docs[:, 100:] = 2
    docs[:, 300:] = 3
    docs = docs.reshape(-1)

    def logits(tok, d):
        tr.forward(tok, d)
        torch.cuda.synchronize()
        return tr.logits().float().cpu().numpy().copy()
    a, b = logits(t1, docs), logits(t2, docs)
    assert np.abs(a[100:] - b[100:]).max() <= 1e-4
    a, b = logits(t1, None), logits(t2, None)
    assert np.abs(a[100:512] - b[100:512]).max() > 1e-2


def _packed_doc_ids(rng, batch, seq, mean_len):
    """Rows packed with documents whose lengths are geometric(mean_len): ids 1, 2, ... along each row."""
    docs = np.zeros((batch, seq), np.int32)
    for b in range(batch):
        pos, k = 0, 1
        while pos < seq:
            n = int(rng.geometric(1.0 / mean_len))
            docs[b, pos:pos + n] = k
            pos, k = pos + n, k + 1
    return docs


def test_packed_document_shape_bf16_muon(nnb):
    """The packed-document configuration at its full width (vocab 16384, d 1024, 16 heads, SwiGLU 2816, RMSNorm,
    learned positions, seq 2048, geometric(300) documents), two layers deep, in bf16 mode on the tensor-core kernels:
    (1) logits outside a document do not change at all when that document's tokens change (masked keys contribute an
    exact zero, every other kernel works per token), while the document's own logits do; (2) Muon + AdamW steps with
    clipping on one batch lower the loss and leave the device status word clear."""
    import torch
    cfg = nnb.GptConfig(16384, 1024, 16, 2, 2816, 2048, 2, nnb.ACT_SWIGLU, nnb.NORM_RMS, nnb.POS_LEARNED, nnb.BF16)
    tr = nnb.GptTrainer(cfg, lr=1e-3, weight_decay=0.01, muon=True, muon_lr=0.02)
    tr.init_params_normal(seed=11, std=0.02)
    r = np.random.default_rng(4)
    n = 2 * 2048
    docs = _packed_doc_ids(r, 2, 2048, 300)
    assert docs[0].max() >= 3                                   # several documents per row
    t1 = r.integers(0, 16384, n).astype(np.int32)
    victim = (docs[0] == 2)                                     # second document of row 0
    t2 = t1.copy()
    t2[:2048][victim] = (t2[:2048][victim] + 101) % 16384
    flat_docs = docs.reshape(-1)

    def logits(tok):
        tr.forward(tok, flat_docs)
        torch.cuda.synchronize()
        return tr.logits().float().cpu().numpy().copy()
    a, b = logits(t1), logits(t2)
    outside = np.ones(n, bool)
    outside[:2048] = ~victim
    assert np.array_equal(a[outside], b[outside])
    assert np.abs(a[~outside] - b[~outside]).max() > 1e-3
    labels = np.roll(t1, -1).astype(np.int32)
    losses = []
    for _ in range(4):
        tr.forward(t1, flat_docs)
        tr.loss_and_grad(labels, None, 1.0)
        tr.backward()
        losses.append(float(tr.loss_tensor().item()))
        tr.optimizer_step(clip=1.0)
    torch.cuda.synchronize()
    tr.check_device_status()
    assert all(np.isfinite(losses)) and losses[-1] < losses[0] - 0.05, losses


def test_config2_full_size_bf16_follows_check_mode(nnb):
    """The 1-GPU configuration at full size (vocab 4096, d 384, 6 heads, 6 layers, SwiGLU 1024, RMSNorm, sinusoidal,
    seq 256, batch 32, Zipf(1.1) tokens, AdamW 6e-4, clip 1.0): the bf16 tensor-core path and the fp32 check path
    (different GEMM, attention and reduction kernels) start from the same weights and see the same batches; their
    per-step losses stay within 1e-2 relative, and the loss falls."""
    import torch
    r = np.random.default_rng(21)
    ranks = np.arange(1, 4097, dtype=np.float64)
    p = ranks ** -1.1
    p /= p.sum()
    steps, n = 6, 32 * 256
    ids = r.choice(4096, size=(steps, 32, 257), p=p).astype(np.int32)
    curves = {}
    for prec in (nnb.FP32, nnb.BF16):
        cfg = nnb.GptConfig(4096, 384, 6, 6, 1024, 256, 32, nnb.ACT_SWIGLU, nnb.NORM_RMS, nnb.POS_SINUSOIDAL, prec)
        tr = nnb.GptTrainer(cfg, lr=6e-4, weight_decay=0.01)
        tr.init_params_normal(seed=42, std=0.02)
        losses = []
        for s in range(steps):
            tok = np.ascontiguousarray(ids[s, :, :-1]).reshape(n)
            lab = np.ascontiguousarray(ids[s, :, 1:]).reshape(n)
            tr.forward(tok)
            tr.loss_and_grad(lab, None, 1.0)
            tr.backward()
            losses.append(float(tr.loss_tensor().item()))
            tr.optimizer_step(clip=1.0)
        torch.cuda.synchronize()
        tr.check_device_status()
        curves[prec] = np.array(losses)
        del tr
    a, b = curves[nnb.FP32], curves[nnb.BF16]
    assert np.all(np.abs(a - b) <= 1e-2 * np.abs(a)), (a, b)
    assert a[-1] < a[0] - 0.1, a


def test_config3_full_size_bf16_follows_check_mode(nnb):
    """The benchmark configuration at full size (vocab 8192, d 768, 12 heads, 12 layers, SwiGLU 2048, RMSNorm, ALiBi,
    seq 1024, micro-batch 16 x accumulation 2, AdamW with a falling learning rate): bf16 tensor-core path against
    the fp32 check path on the same weights and batches, per-micro-batch losses within 1e-2 relative."""
    import torch
    r = np.random.default_rng(33)
    ranks = np.arange(1, 8193, dtype=np.float64)
    p = ranks ** -1.1
    p /= p.sum()
    steps, accum, n = 3, 2, 16 * 1024
    ids = r.choice(8192, size=(steps * accum, 16, 1025), p=p).astype(np.int32)
    curves = {}
    for prec in (nnb.FP32, nnb.BF16):
        cfg = nnb.GptConfig(8192, 768, 12, 12, 2048, 1024, 16, nnb.ACT_SWIGLU, nnb.NORM_RMS, nnb.POS_ALIBI, prec)
        tr = nnb.GptTrainer(cfg, lr=3e-4, weight_decay=0.01)
        tr.init_params_normal(seed=42, std=0.02)
        losses = []
        for s in range(steps):
            for a in range(accum):
                i = s * accum + a
                tok = np.ascontiguousarray(ids[i, :, :-1]).reshape(n)
                lab = np.ascontiguousarray(ids[i, :, 1:]).reshape(n)
                tr.micro_step(tok, lab, None, None, grad_scale=1.0 / accum, last=(a == accum - 1))
                losses.append(float(tr.loss_tensor().item()))
            tr.optimizer_step(lr=3e-4 * (1.0 - 0.2 * s))
        torch.cuda.synchronize()
        tr.check_device_status()
        curves[prec] = np.array(losses)
        del tr
        torch.cuda.empty_cache()
    a, b = curves[nnb.FP32], curves[nnb.BF16]
    assert np.all(np.abs(a - b) <= 1e-2 * np.abs(a)), (a, b)
    assert a[-1] < a[0], a
