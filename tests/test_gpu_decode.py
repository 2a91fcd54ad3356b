"""Incremental inference with a key/value cache (nnb200_gpt_forward_step, GptTrainer.forward_step / generate) against
golden vectors of the reference's GPTModel::forward_step and GPTModel::generate (tests/golden/decode.npz, made by
tests/golden/make_golden.py from oracle/_ref/ref_gpt), and against the training-time forward pass of the same tokens."""
import os

import numpy as np
import pytest

from oracle import gpt_oracle as go
from tests.golden_io import GOLDEN, rel_err

pytestmark = pytest.mark.gpu

CASES = ["ln_gelu_learned", "rms_swiglu_sin", "rms_swiglu_alibi", "rms_swiglu_rope"]


@pytest.fixture(scope="module")
def nnb():
    from tests import gpu_util
    return gpu_util.nnb


def _load(name):
    z = np.load(os.path.join(GOLDEN, "decode.npz"))
    cfg = go.GptConfig(*[int(v) for v in z[name + "_cfg"]])
    params = go.init_params(cfg, 42, std=0.2)
    chk = float(sum(np.abs(p.astype(np.float64)).sum() for p in params))
    assert abs(chk - float(z[name + "_p0_checksum"][0])) <= 1e-9 * chk, "numpy RNG stream changed: regenerate goldens"
    return cfg, params, z[name + "_tokens"], z[name + "_logits"], z[name + "_generated"]


def _trainer(nnb, c, params, precision):
    cfg = nnb.GptConfig(c.vocab, c.d_model, c.heads, c.layers, c.d_ff, c.seq, c.batch, c.act, c.norm, c.pos, precision)
    tr = nnb.GptTrainer(cfg)
    tr.load_params(params)
    return tr


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("precision,tol", [(0, 1e-5), (1, 2e-2)])     # bf16 weights N(0, 0.2): ten times the training init, largest-logit norm
def test_forward_step_matches_reference(nnb, name, precision, tol):
    import torch
    c, params, tokens, want, _ = _load(name)
    tr = _trainer(nnb, c, params, nnb.FP32 if precision == 0 else nnb.BF16)
    got = []
    for t, tok in enumerate(tokens):
        got.append(tr.forward_step(int(tok), t, t).clone())
    torch.cuda.synchronize()
    got = torch.stack(got).cpu().numpy()
    assert rel_err(got, want) < tol


@pytest.mark.parametrize("name", CASES)
def test_forward_step_equals_full_forward(nnb, name):
    """What the reference's attn_consistency_test checks on its Vulkan engine: the logits of token t computed step by
    step from the cache equal column t of the full causal forward pass over the same tokens (check mode, 1e-5)."""
    import torch
    c, params, tokens, _, _ = _load(name)
    tr = _trainer(nnb, c, params, nnb.FP32)
    tr.forward(tokens.astype(np.int32))
    torch.cuda.synchronize()
    full = tr.logits().float().cpu().numpy().copy()          # (tokens, vocab)
    steps = torch.stack([tr.forward_step(int(tok), t, t).clone() for t, tok in enumerate(tokens)]).cpu().numpy()
    assert rel_err(steps, full) < 1e-5


@pytest.mark.parametrize("name", CASES)
def test_generate_greedy_matches_reference(nnb, name):
    """Temperature 0 (arg max) generation from a 10-token prompt, past the end of the window (sliding-window rebuild)."""
    c, params, tokens, _, want = _load(name)
    tr = _trainer(nnb, c, params, nnb.FP32)
    got = tr.generate([int(t) for t in tokens[:10]], c.seq + 6, temperature=0.0)
    assert got == [int(v) for v in want]


def test_generate_sampling_and_eos(nnb):
    c, params, tokens, _, _ = _load("rms_swiglu_alibi")
    tr = _trainer(nnb, c, params, nnb.BF16)
    a = tr.generate([1, 2, 3], 12, temperature=0.8, rng=np.random.default_rng(5))
    b = tr.generate([1, 2, 3], 12, temperature=0.8, rng=np.random.default_rng(5))
    assert a == b and len(a) == 12 and all(0 <= t < c.vocab for t in a)
    greedy = tr.generate([1, 2, 3], 8, temperature=0.0)
    cut = tr.generate([1, 2, 3], 8, temperature=0.0, eos_token_id=greedy[3])
    assert cut == greedy[:greedy.index(greedy[3])]           # stops before the first occurrence of the end token


@pytest.mark.parametrize("pos", [0, 2, 3])                  # learned, ALiBi, rotary
def test_forward_step_long_context_crosses_attention_chunks(nnb, pos):
    """The decode attention splits the cache into chunks of 32 rows and merges the partial softmaxes: 300 steps in a
    320-token window (ten chunks) against the full causal forward pass of the same tokens (check mode, 1e-5), with
    the CUDA-graph replay and with plain launches."""
    import torch
    c = go.GptConfig(64, 64, 2, 2, 96, 320, 1, 1, 1, pos)       # vocab, d, heads, layers, ff, seq, batch, SwiGLU, RMSNorm
    params = go.init_params(c, 7, std=0.2)
    tokens = np.random.default_rng(11).integers(0, c.vocab, c.seq).astype(np.int32)
    tr = _trainer(nnb, c, params, nnb.FP32)
    tr.forward(tokens)
    torch.cuda.synchronize()
    full = tr.logits().float().cpu().numpy().copy()[:300]
    graph = torch.stack([tr.forward_step(int(tok), t, t).clone() for t, tok in enumerate(tokens[:300])]).cpu().numpy()
    assert rel_err(graph, full) < 1e-5
    plain = torch.stack([tr.forward_step(int(tok), t, t, graph=False).clone() for t, tok in enumerate(tokens[:300])]).cpu().numpy()
    assert np.array_equal(plain, graph)
