"""The numpy restatement (oracle/gpt_oracle.py) against golden vectors from the reference CPU engine."""
import os

import numpy as np
import pytest

from oracle import gpt_oracle as go
from tests.golden_io import (GOLDEN, GPT_CASES, global_rel_err, key_bias_indices, load_gpt_case,
                             rel_err)

TOL = 1e-5   # fp32 check-mode bar: per-step loss and parameter values within 1e-5 relative


@pytest.mark.parametrize("name", GPT_CASES)
def test_training_matches_reference(name):
    c = load_gpt_case(name)
    losses, model, first = go.train(c["cfg"], c["params"], c["batches"], keep_first_grads=True, **c["kw"])
    assert rel_err(losses, c["losses"]) < TOL
    skip = key_bias_indices(c["cfg"])
    for i, (g, gr) in enumerate(zip(first, c["grads"])):
        if i not in skip:
            assert rel_err(g, gr) < 2e-5, go.param_shapes(c["cfg"])[i]
    # parameters: 1e-5 relative L2 on the whole set; per tensor 1e-4 relative L2, because Adam divides
    # by sqrt(v) and so turns rounding differences of near-zero gradient elements into +-lr steps
    assert global_rel_err(model.params, c["final"], skip) < TOL
    for i, (p, pr) in enumerate(zip(model.params, c["final"])):
        if i not in skip:
            assert global_rel_err([p], [pr]) < 1e-4, go.param_shapes(c["cfg"])[i]


@pytest.mark.parametrize("name", GPT_CASES)
def test_forward_logits_match_reference(name):
    c = load_gpt_case(name)
    m = go.GptOracle(c["cfg"], c["params"])
    logits = m.forward(c["batches"][0]["tokens"], c["batches"][0]["doc_ids"])
    assert rel_err(logits, c["logits"]) < TOL


def test_config1_twenty_steps():
    z = np.load(os.path.join(GOLDEN, "gpt_c1_20steps.npz"))
    cfg = go.GptConfig(*[int(v) for v in z["cfg"]])
    params = go.init_params(cfg, 42)
    assert np.allclose([np.linalg.norm(p.astype(np.float64)) for p in params], z["p0_norms"], rtol=1e-9)
    mbs = [{"tokens": z["tokens"][i], "labels": z["labels"][i], "mask": z["mask"][i], "doc_ids": None}
           for i in range(20)]
    losses, model, _ = go.train(cfg, params, mbs, steps=20, lr=1e-3, wd=0.01)
    assert rel_err(losses, z["losses"]) < TOL
    norms = np.array([np.linalg.norm(p.astype(np.float64)) for p in model.params])
    skip = key_bias_indices(cfg)
    keep = [i for i in range(len(norms)) if i not in skip]
    assert np.allclose(norms[keep], z["p1_norms"][keep], rtol=1e-4)
    assert global_rel_err([model.params[-1]], [z["p1_lm_head_b"]]) < 1e-4
    assert global_rel_err([model.params[-3]], [z["p1_ln_f_beta"]]) < 1e-4
    assert global_rel_err([model.params[-4]], [z["p1_ln_f_gamma"]]) < TOL


def test_primitives_match_reference():
    z = np.load(os.path.join(GOLDEN, "prims.npz"))
    batch, M, N, K, D, C, NC, vocab = [int(v) for v in z["dims"]]
    alpha, inv_nv = z["scal"]
    A, B, V, G, P, mask = z["A"], z["B"], z["V"], z["G"], z["P"], z["mask"]
    m = go.bmm_reduce_max(A, B, batch, alpha, mask)
    l = go.bmm_softmax_denom(A, B, m, batch, alpha, mask)
    O = go.bmm_softmax_apply(A, B, V, m, l, batch, alpha, mask)
    gq, R = go.bmm_softmax_backward_q(A, B, P, m, l, batch, alpha, mask)
    gk, gv = go.bmm_softmax_backward_kv(A, B, P, G, R, m, l, batch, alpha, mask)
    for got, key in ((m, "m"), (l, "l"), (O, "O"), (gq, "gradQ"), (R, "R"), (gk, "gradK"), (gv, "gradV")):
        assert np.allclose(got, z["out_" + key], rtol=1e-5, atol=1e-6), key
    logits, labels, cmask = z["logits"], z["labels"], z["cmask"]
    assert np.allclose(go.col_softmax_denom(logits, logits.max(axis=0)), z["out_col_denom"], rtol=1e-6)
    grad, lv = go.col_softmax_sparse_forward(logits, labels, cmask, vocab, inv_nv)
    assert np.allclose(grad, z["out_ce_grad"], rtol=1e-5, atol=1e-7)
    assert np.allclose(lv, z["out_loss_vec"], rtol=1e-5, atol=1e-7)
    # gather / scatter-add / rearrange are index work: bit-exact
    gath = go.gather_rows(logits, labels)
    assert np.array_equal(gath, z["out_gathered"])
    dst = np.zeros((C, NC), np.float32)
    go.scatter_add_rows(dst, labels, gath)
    assert np.array_equal(dst, z["out_scattered"])
    assert np.array_equal(go.rearrange_3d(A, K, batch, M, inverse=True), z["out_rearranged"])


def test_attention_mask_and_doc_invariance():
    """Properties the reference pins in src/doc_mask_test.cpp and src/doc_attn_test.cpp."""
    slopes = go.alibi_slopes(4)
    assert slopes[0] == 1.0 and np.isclose(slopes[1], 0.25)
    doc = np.array([1, 1, 1, 2, 2, 2, 2, 3])
    m = go.build_attention_mask(1, 8, 4, True, slopes, doc).reshape(4, 8, 8)
    assert m[1, 2, 0] == np.float32(-0.25 * 2) and np.isneginf(m[1, 3, 2]) and np.isneginf(m[0, 0, 1])
    cfg = go.GptConfig(32, 16, 2, 1, 32, 8, 2, go.ACT_SWIGLU, go.NORM_RMS, go.POS_LEARNED)
    params = go.init_params(cfg, 7, std=0.3)
    rng = np.random.default_rng(0)
    t1 = rng.integers(0, 32, 16)
    t2 = t1.copy()
    t2[:3] = (t2[:3] + 5) % 32          # change document A of row 0 only
    docs = np.concatenate([doc, doc])
    l1 = go.GptOracle(cfg, params).forward(t1, docs)
    l2 = go.GptOracle(cfg, params).forward(t2, docs)
    assert np.abs(l1[:, 3:8] - l2[:, 3:8]).max() <= 1e-4       # document B, C untouched
    l3 = go.GptOracle(cfg, params).forward(t1, None)
    l4 = go.GptOracle(cfg, params).forward(t2, None)
    assert np.abs(l3[:, 3:8] - l4[:, 3:8]).max() > 1e-2
