"""TEST INFRASTRUCTURE — CPU restatement (numpy, float32) of the neuralnet.cpp GPT training step.

This module is the parity oracle.  Only the tests, the smoke check and the CPU-baseline leg of
the benchmark may import it; the product (the CUDA library) never does.

Every function restates the arithmetic of the reference's CPU path and cites the file:line it
follows (paths are relative to the reference project root).  Tensors keep the reference layout:
activations are 2-D row-major ``(features, batch*seq)`` matrices whose columns are batch-major
``i = b*seq + t`` (include/neuralnet.cpp/compute_layer.hpp:2788-2809); weights are ``(out, in)``.

Parity status: pinned.  ``tests/golden/*.npz`` hold outputs of the unmodified reference CPU engine
(built by ``oracle/Makefile`` into ``oracle/_ref/ref_gpt``) and ``tests/test_oracle_golden.py``
checks this restatement against them.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

F32 = np.float32

ACT_GELU, ACT_SWIGLU = 0, 1
NORM_LAYER, NORM_RMS = 0, 1
POS_LEARNED, POS_SINUSOIDAL, POS_ALIBI, POS_ROPE = 0, 1, 2, 3
OPT_ADAMW, OPT_MUON_SPLIT = 0, 1


@dataclasses.dataclass
class GptConfig:
    """Mirror of nn::GptConfig (include/neuralnet.cpp/domain_gpt.hpp:29-39) plus batch."""
    vocab: int
    d_model: int
    heads: int
    layers: int
    d_ff: int
    seq: int
    batch: int
    act: int = ACT_GELU
    norm: int = NORM_LAYER
    pos: int = POS_LEARNED

    @property
    def d_k(self) -> int:
        return self.d_model // self.heads

    @property
    def tokens(self) -> int:
        return self.batch * self.seq


# --------------------------------------------------------------------------------------
# parameters
# --------------------------------------------------------------------------------------
def param_shapes(cfg: GptConfig) -> List[Tuple[str, int, int]]:
    """Parameter order exposed to the optimizer: GPTModel::parameters
    (compute_layer.hpp:2739-2755), GPTBlock (:2336-2346), AttentionBase (:1109-1119),
    FeedForward (:1642-1648), Linear {W, b} (:145-148), LayerNorm {gamma, beta} (:519-522),
    RMSNorm {gamma} (:704-707)."""
    d, ff, V, S = cfg.d_model, cfg.d_ff, cfg.vocab, cfg.seq
    out: List[Tuple[str, int, int]] = [("token_emb", V, d)]
    if cfg.pos == POS_LEARNED:
        out.append(("pos_emb", S, d))

    def norm(prefix):
        r = [(prefix + ".gamma", d, 1)]
        if cfg.norm == NORM_LAYER:
            r.append((prefix + ".beta", d, 1))
        return r

    fc1_out = 2 * ff if cfg.act == ACT_SWIGLU else ff
    for l in range(cfg.layers):
        p = f"blk{l}."
        for w in ("wq", "wk", "wv", "wo"):
            out += [(p + w + ".W", d, d), (p + w + ".b", d, 1)]
        out += norm(p + "norm1")
        out += [(p + "fc1.W", fc1_out, d), (p + "fc1.b", fc1_out, 1)]
        out += [(p + "fc2.W", d, ff), (p + "fc2.b", d, 1)]
        out += norm(p + "norm2")
    out += norm("ln_f")
    out += [("lm_head.W", V, d), ("lm_head.b", V, 1)]
    return out


def init_params(cfg: GptConfig, seed: int = 42, std: float = 0.02) -> List[np.ndarray]:
    """Seeded synthetic weights: every >=2-D parameter ~ N(0, std); biases 0; gamma 1; beta 0.
    (The reference's own Linear init is not reproducible — compute_layer.hpp:108 — so parity runs
    overwrite every parameter, as src/gpt_gradcheck.cpp:85-99 does.)"""
    rng = np.random.default_rng(seed)
    ps = []
    for name, r, c in param_shapes(cfg):
        if name.endswith(".gamma"):
            ps.append(np.ones((r, c), F32))
        elif c == 1:
            ps.append(np.zeros((r, c), F32))
        else:
            ps.append((rng.standard_normal((r, c)) * std).astype(F32))
    return ps


def muon_mask(cfg: GptConfig) -> List[bool]:
    """True for the hidden 2-D matrices (wq, wk, wv, wo, fc1, fc2 weights) that Muon owns in the
    split the reference prescribes (compute_optimizer.hpp:508-511)."""
    return [n.startswith("blk") and n.endswith(".W") for n, _, _ in param_shapes(cfg)]


def sinusoidal_table(seq: int, d: int) -> np.ndarray:
    """SinusoidalPositionEncoder (compute_layer.hpp:2604-2622): float arithmetic throughout."""
    pe = np.empty((seq, d), F32)
    i = np.arange(d)
    expo = (2 * (i // 2)).astype(F32) / F32(d)
    denom = np.power(F32(10000.0), expo, dtype=F32)
    for pos in range(seq):
        angle = F32(pos) / denom
        pe[pos] = np.where(i % 2 == 0, np.sin(angle, dtype=F32), np.cos(angle, dtype=F32))
    return pe


def rope_tables(seq: int, d_k: int):
    """RotaryEmbedding::fill_pos_column_ (compute_layer.hpp:886-902): cos/sin tables (d_k, seq) with
    theta = pos / 10000^(2j/d_k) in fp32, rows j and j + d_k/2 alike."""
    half = d_k // 2
    j = np.arange(half, dtype=F32)
    inv = np.power(F32(10000), (F32(2) * j) / F32(d_k)).astype(F32)          # std::pow(float, float)
    theta = (np.arange(seq, dtype=F32)[None, :] / inv[:, None]).astype(F32)
    c, s_ = np.cos(theta).astype(F32), np.sin(theta).astype(F32)
    return np.concatenate([c, c], axis=0), np.concatenate([s_, s_], axis=0)


def rope_apply(x, cos, sin, backward=False):
    """RotaryEmbedding::apply (compute_layer.hpp:926-945) on (BH, d_k, S): x*cos +/- rotate_half(x)*sin, where
    rotate_half reads the other half of the head dimension and negates what it puts into the first half."""
    half = x.shape[1] // 2
    rot = np.concatenate([-x[:, half:], x[:, :half]], axis=1)
    out = x * cos[None] - rot * sin[None] if backward else x * cos[None] + rot * sin[None]
    return out.astype(F32)


def alibi_slopes(heads: int) -> np.ndarray:
    """m_h = 2^(-8h/H), h from 0 (compute_layer.hpp:2179-2187)."""
    h = np.arange(heads, dtype=F32)
    return np.power(F32(2.0), F32(-8.0) * h / F32(heads), dtype=F32)


# --------------------------------------------------------------------------------------
# engine primitives restated (cpu_engine.hpp)
# --------------------------------------------------------------------------------------
def gather_rows(table: np.ndarray, idx: np.ndarray) -> np.ndarray:
    """cpu_engine.hpp:125-179 — out[i] = table[(size_t)idx[i]], zero row when out of range."""
    idx = np.asarray(idx).reshape(-1)
    ii = idx.astype(np.int64)
    ok = (idx >= 0) & (ii < table.shape[0])
    out = np.zeros((ii.size, table.shape[1]), F32)
    out[ok] = table[ii[ok]]
    return out


def scatter_add_rows(dst: np.ndarray, idx: np.ndarray, grad: np.ndarray) -> None:
    """cpu_engine.hpp:184-216 — dst[idx[i]] += grad[i], sequential in ascending i (fp32), indices
    out of range skipped.  np.add.at applies the updates unbuffered in index order."""
    idx = np.asarray(idx).reshape(-1)
    ii = idx.astype(np.int64)
    ok = (idx >= 0) & (ii < dst.shape[0])
    np.add.at(dst, ii[ok], grad[ok])


def rearrange_3d(x: np.ndarray, M: int, B: int, N: int, inverse: bool = False) -> np.ndarray:
    """(M, B*N) -> (B*M, N) and back (compute_engine.hpp:163-170)."""
    if not inverse:
        return np.ascontiguousarray(x.reshape(M, B, N).transpose(1, 0, 2)).reshape(B * M, N)
    return np.ascontiguousarray(x.reshape(B, M, N).transpose(1, 0, 2)).reshape(M, B * N)


def build_attention_mask(batch, seq, heads, use_alibi, slopes, doc_ids=None) -> np.ndarray:
    """build_attention_mask (compute_layer.hpp:2081-2128): (batch*heads*seq, seq) additive mask;
    allowed = j<=i and same document; bias -slope*(i-j) where allowed, -inf elsewhere."""
    i = np.arange(seq)[:, None]
    j = np.arange(seq)[None, :]
    causal = j <= i
    dist = (i - j).astype(F32)
    out = np.empty((batch, heads, seq, seq), F32)
    for b in range(batch):
        allowed = causal
        if doc_ids is not None:
            d = np.asarray(doc_ids[b * seq:(b + 1) * seq])
            allowed = causal & (d[:, None] == d[None, :])
        for h in range(heads):
            bias = (-slopes[h] * dist) if use_alibi else np.zeros((seq, seq), F32)
            out[b, h] = np.where(allowed, bias, F32(-np.inf))
    return out.reshape(batch * heads * seq, seq)


def _scores(A, B, batch, alpha, mask):
    """alpha * A_b^T B_b + mask for transA=true, transB=false; A (batch*K, M), B (batch*K, N)."""
    K = A.shape[0] // batch
    s = np.einsum("bkm,bkn->bmn", A.reshape(batch, K, -1), B.reshape(batch, K, -1)).astype(F32)
    s = F32(alpha) * s
    if mask is not None:
        M, N = s.shape[1], s.shape[2]
        if mask.shape[0] == M:          # shared (M, N) mask
            s = s + mask[None]
        else:                           # stacked (batch*M, N)
            s = s + mask.reshape(batch, M, N)
    return s


def bmm_reduce_max(A, B, batch, alpha, mask=None):
    """batched_matmul_reduce(op=Max, reduce_cols) — cpu_engine.hpp:426-532."""
    return _scores(A, B, batch, alpha, mask).max(axis=2).reshape(-1, 1)


def bmm_softmax_denom(A, B, row_max, batch, alpha, mask=None):
    """batched_matmul_softmax_denom — cpu_engine.hpp:535-604."""
    s = _scores(A, B, batch, alpha, mask)
    return np.exp(s - row_max.reshape(batch, -1, 1)).sum(axis=2, dtype=F32).reshape(-1, 1)


def bmm_softmax_apply(A, B, V, row_max, denom, batch, alpha, mask=None):
    """batched_matmul_softmax_apply — cpu_engine.hpp:607-699.  V is (batch*N, D)."""
    s = _scores(A, B, batch, alpha, mask)
    W = np.exp(s - row_max.reshape(batch, -1, 1)) / denom.reshape(batch, -1, 1)
    D = V.shape[1]
    return np.einsum("bmn,bnd->bmd", W, V.reshape(batch, -1, D)).astype(F32).reshape(-1, D)


def bmm_softmax_backward_q(A, B, P, row_max, denom, batch, alpha, mask=None):
    """batched_matmul_softmax_backward_q — cpu_engine.hpp:702-801.  Returns (gradQ (batch*K, M), R)."""
    s = _scores(A, B, batch, alpha, mask)
    W = np.exp(s - row_max.reshape(batch, -1, 1)) / denom.reshape(batch, -1, 1)
    Pm = P.reshape(W.shape)
    R = (W * Pm).sum(axis=2, dtype=F32)
    dS = W * (Pm - R[..., None])
    K = B.shape[0] // batch
    gq = F32(alpha) * np.einsum("bmn,bkn->bkm", dS, B.reshape(batch, K, -1))
    return gq.astype(F32).reshape(batch * K, -1), R.reshape(-1, 1)


def bmm_softmax_backward_kv(A, B, P, G, R, row_max, denom, batch, alpha, mask=None):
    """batched_matmul_softmax_backward_kv — cpu_engine.hpp:804-915.  G is (batch*M, D).
    Returns (gradK (batch*K, N), gradV (batch*K, N)): the reference sizes gradV by K and reads the
    first K columns of G (cpu_engine.hpp:870-908); the layer always calls it with D == K."""
    s = _scores(A, B, batch, alpha, mask)
    W = np.exp(s - row_max.reshape(batch, -1, 1)) / denom.reshape(batch, -1, 1)
    Pm = P.reshape(W.shape)
    dS = W * (Pm - R.reshape(batch, -1, 1))
    K = A.shape[0] // batch
    gk = F32(alpha) * np.einsum("bmn,bkm->bkn", dS, A.reshape(batch, K, -1))
    D = G.shape[1]
    gv = np.einsum("bmn,bmd->bdn", W, G.reshape(batch, -1, D)[:, :, :K])
    return gk.astype(F32).reshape(batch * K, -1), gv.astype(F32).reshape(batch * K, -1)


def col_softmax_denom(logits, col_max):
    """cpu_engine.hpp:922-945."""
    return np.exp(logits - col_max.reshape(1, -1)).sum(axis=0, dtype=F32).reshape(1, -1)


def col_softmax_sparse_forward(logits, labels, mask, vocab_size, inv_num_valid):
    """cpu_engine.hpp:948-1006 — per column: max, denom, grad = inv_nv*softmax - inv_nv*onehot,
    loss_vec = logit[label] - max - log(denom); invalid columns (mask < 0.5 or label >= vocab) are zero."""
    C, N = logits.shape
    lab_f = np.asarray(labels, F32).reshape(-1)
    lab = np.where(lab_f >= 0, lab_f, 0).astype(np.int64)
    valid = lab < vocab_size
    if mask is not None:
        valid &= np.asarray(mask, F32).reshape(-1) >= 0.5
    mv = logits.max(axis=0)
    e = np.exp(logits - mv[None, :], dtype=F32)
    denom = e.sum(axis=0, dtype=F32)
    inv = F32(inv_num_valid)
    grad = (inv * e / denom[None, :]).astype(F32)
    cols = np.nonzero(valid)[0]
    grad[lab[cols], cols] -= inv
    grad[:, ~valid] = 0
    loss_vec = np.zeros((1, N), F32)
    loss_vec[0, cols] = logits[lab[cols], cols] - mv[cols] - np.log(denom[cols], dtype=F32)
    return grad, loss_vec


def ce_forward_sparse(logits, labels, loss_mask, vocab_size):
    """CrossEntropyLoss::forward_sparse (compute_loss.hpp:229-309): returns (loss, grad_logits)."""
    labels = np.asarray(labels).reshape(-1)
    N = logits.shape[1]
    masked = np.zeros(N, bool) if loss_mask is None else (np.asarray(loss_mask, F32).reshape(-1) < 0.5)
    num_valid = int(np.count_nonzero(~masked & (labels < vocab_size)))
    inv = F32(1.0) / F32(num_valid) if num_valid > 0 else F32(0)
    m = None if loss_mask is None else np.where(masked, F32(0), F32(1))
    grad, loss_vec = col_softmax_sparse_forward(logits, labels.astype(F32), m, vocab_size, inv)
    total = loss_vec.sum(dtype=F32)
    loss = -total / F32(num_valid) if num_valid > 0 else F32(0)
    return F32(loss), grad


# --------------------------------------------------------------------------------------
# layers (compute_layer.hpp)
# --------------------------------------------------------------------------------------
EPS_NORM = F32(1e-5)       # compute_layer.hpp:495,687
GELU_BETA = F32(1.702)     # compute_layer.hpp:259


def _sigmoid(x):
    # 1 / (1 + exp(-x)) in the op order of GeLU::forward / SwiGLU::forward (compute_layer.hpp:270-290,385-392)
    return (F32(1) / (F32(1) + np.exp(-x, dtype=F32))).astype(F32)


class _Norm:
    """LayerNorm (compute_layer.hpp:541-654) / RMSNorm (:722-800), normalising down columns."""

    def __init__(self, kind, gamma, beta=None):
        self.kind, self.gamma, self.beta = kind, gamma, beta

    def forward(self, x):
        F = x.shape[0]
        inv_f = F32(1) / F32(F)
        if self.kind == NORM_RMS:
            s = (x * x).sum(axis=0, dtype=F32) * inv_f
            self.rinv = (F32(1) / np.sqrt(s + EPS_NORM, dtype=F32)).astype(F32)
            self.n = (x * self.rinv[None, :]).astype(F32)
            return (self.n * self.gamma).astype(F32)
        mean = x.sum(axis=0, dtype=F32) * inv_f
        diff = x - mean[None, :]
        var = (diff * diff).sum(axis=0, dtype=F32) * inv_f
        self.rinv = (F32(1) / np.sqrt(var + EPS_NORM, dtype=F32)).astype(F32)
        self.n = (diff * self.rinv[None, :]).astype(F32)
        return (self.n * self.gamma + self.beta).astype(F32)

    def backward(self, g):
        """Returns (grad_x, grad_gamma, grad_beta|None).  grad_gamma = sum_tokens g*gamma*n —
        the reference multiplies by gamma (compute_layer.hpp:789-797, :636-644); reproduced."""
        F = g.shape[0]
        inv_f = F32(1) / F32(F)
        gg = g * self.gamma
        ggn = gg * self.n
        if self.kind == NORM_RMS:
            m = ggn.sum(axis=0, dtype=F32) * inv_f
            gx = (gg - m[None, :] * self.n) * self.rinv[None, :]
            return gx.astype(F32), ggn.sum(axis=1, dtype=F32).reshape(-1, 1), None
        mean_g = gg.sum(axis=0, dtype=F32) * inv_f
        mean_gn = ggn.sum(axis=0, dtype=F32) * inv_f
        gx = (gg - mean_g[None, :] - self.n * mean_gn[None, :]) * self.rinv[None, :]
        return (gx.astype(F32), ggn.sum(axis=1, dtype=F32).reshape(-1, 1),
                g.sum(axis=1, dtype=F32).reshape(-1, 1))


class GptOracle:
    """GPTModel forward/backward (compute_layer.hpp:2783-2896) with gradient accumulation into
    ``self.grads`` exactly as Linear::backward / scatter_add_rows accumulate (+=)."""

    def __init__(self, cfg: GptConfig, params: Sequence[np.ndarray]):
        self.cfg = cfg
        self.shapes = param_shapes(cfg)
        assert len(params) == len(self.shapes)
        self.params = [np.array(p, F32).reshape(r, c) for p, (_, r, c) in zip(params, self.shapes)]
        self.index = {n: i for i, (n, _, _) in enumerate(self.shapes)}
        self.grads = [np.zeros_like(p) for p in self.params]
        self.slopes = alibi_slopes(cfg.heads)
        self.sin_table = sinusoidal_table(cfg.seq, cfg.d_model) if cfg.pos == POS_SINUSOIDAL else None
        self.rope = rope_tables(cfg.seq, cfg.d_k) if cfg.pos == POS_ROPE else None

    def p(self, name):
        return self.params[self.index[name]]

    def g(self, name):
        return self.grads[self.index[name]]

    def zero_grad(self):
        for g in self.grads:
            g[...] = 0

    # -- pieces ------------------------------------------------------------------
    def _norm(self, prefix):
        beta = self.p(prefix + ".beta") if self.cfg.norm == NORM_LAYER else None
        return _Norm(self.cfg.norm, self.p(prefix + ".gamma"), beta)

    def _norm_backward(self, prefix, layer, g):
        gx, gg, gb = layer.backward(g)
        self.g(prefix + ".gamma")[...] += gg
        if gb is not None:
            self.g(prefix + ".beta")[...] += gb
        return gx

    def _linear(self, name, x):
        # Linear::forward (compute_layer.hpp:151-169)
        return (self.p(name + ".W") @ x + self.p(name + ".b")).astype(F32)

    def _linear_backward(self, name, x, gy):
        # Linear::backward (compute_layer.hpp:172-195)
        self.g(name + ".W")[...] += (gy @ x.T).astype(F32)
        self.g(name + ".b")[...] += gy.sum(axis=1, dtype=F32).reshape(-1, 1)
        return (self.p(name + ".W").T @ gy).astype(F32)

    def _attention_mask(self, doc_ids):
        c = self.cfg
        return build_attention_mask(c.batch, c.seq, c.heads, c.pos == POS_ALIBI, self.slopes,
                                    doc_ids).reshape(c.batch * c.heads, c.seq, c.seq)

    def _attn_forward(self, prefix, x, mask, cache):
        # AttentionBase::forward (compute_layer.hpp:1133-1269); the two-pass and the materialised
        # branch compute the same softmax(QK^T/sqrt(dk) + mask) V.
        c = self.cfg
        BH, S, dk = c.batch * c.heads, c.seq, c.d_k
        q = rearrange_3d(self._linear(prefix + "wq", x), c.d_model, c.batch, S).reshape(BH, dk, S)
        k = rearrange_3d(self._linear(prefix + "wk", x), c.d_model, c.batch, S).reshape(BH, dk, S)
        v = rearrange_3d(self._linear(prefix + "wv", x), c.d_model, c.batch, S).reshape(BH, dk, S)
        if self.rope is not None:                                  # compute_layer.hpp:1178-1185
            q, k = rope_apply(q, *self.rope), rope_apply(k, *self.rope)
        scale = F32(1) / np.sqrt(F32(dk))
        s = scale * np.einsum("bki,bkj->bij", q, k).astype(F32) + mask
        s = s - s.max(axis=2, keepdims=True)
        e = np.exp(s, dtype=F32)
        a = (e / e.sum(axis=2, keepdims=True, dtype=F32)).astype(F32)
        o = np.einsum("bkj,bij->bki", v, a).astype(F32)            # O = V A^T
        concat = rearrange_3d(o.reshape(BH * dk, S), c.d_model, c.batch, S, inverse=True)
        cache.update(x=x, q=q, k=k, v=v, a=a, concat=concat, scale=scale)
        return self._linear(prefix + "wo", concat)

    def _attn_backward(self, prefix, gy, cache):
        # AttentionBase::backward (compute_layer.hpp:1271-1412)
        c = self.cfg
        BH, S, dk = c.batch * c.heads, c.seq, c.d_k
        q, k, v, a, scale = cache["q"], cache["k"], cache["v"], cache["a"], cache["scale"]
        gc = self._linear_backward(prefix + "wo", cache["concat"], gy)
        go = rearrange_3d(gc, c.d_model, c.batch, S).reshape(BH, dk, S)
        gv = np.einsum("bki,bij->bkj", go, a).astype(F32)
        ga = np.einsum("bki,bkj->bij", go, v).astype(F32)
        gs = a * (ga - (a * ga).sum(axis=2, keepdims=True, dtype=F32))   # Softmax::backward (:851-861)
        gq = scale * np.einsum("bkj,bij->bki", k, gs).astype(F32)
        gk = scale * np.einsum("bki,bij->bkj", q, gs).astype(F32)
        if self.rope is not None:                                  # compute_layer.hpp:1365-1372
            gq, gk = rope_apply(gq, *self.rope, backward=True), rope_apply(gk, *self.rope, backward=True)
        back = lambda t: rearrange_3d(t.reshape(BH * dk, S), c.d_model, c.batch, S, inverse=True)
        x = cache["x"]
        gx = self._linear_backward(prefix + "wq", x, back(gq))
        gx = gx + self._linear_backward(prefix + "wk", x, back(gk))
        gx = gx + self._linear_backward(prefix + "wv", x, back(gv))
        return gx.astype(F32)

    def _ffn_forward(self, prefix, x, cache):
        # FeedForward::forward (compute_layer.hpp:1658-1672), GeLU (:266-295), SwiGLU (:375-404)
        c = self.cfg
        h1 = self._linear(prefix + "fc1", x)
        if c.act == ACT_SWIGLU:
            gate, up = h1[:c.d_ff], h1[c.d_ff:]
            s = _sigmoid(gate)
            h2 = (gate * s * up).astype(F32)
            cache.update(ffn_x=x, gate=gate, up=up, sig=s, h2=h2)
        else:
            s = _sigmoid(GELU_BETA * h1)
            h2 = (h1 * s).astype(F32)
            cache.update(ffn_x=x, h1=h1, sig=s, h2=h2)
        return self._linear(prefix + "fc2", h2)

    def _ffn_backward(self, prefix, gy, cache):
        c = self.cfg
        g2 = self._linear_backward(prefix + "fc2", cache["h2"], gy)
        s = cache["sig"]
        one = F32(1)
        if c.act == ACT_SWIGLU:
            gate, up = cache["gate"], cache["up"]
            g_gate = g2 * up * (s * (one + gate * (one - s)))      # compute_layer.hpp:436-441
            g_up = g2 * gate * s                                   # :442-445
            g1 = np.concatenate([g_gate, g_up], axis=0).astype(F32)
        else:
            h1 = cache["h1"]
            g1 = (g2 * (s * (one + (GELU_BETA * h1) * (one - s)))).astype(F32)   # :310-337
        return self._linear_backward(prefix + "fc1", cache["ffn_x"], g1)

    # -- model -------------------------------------------------------------------
    def forward(self, tokens, doc_ids=None):
        """tokens: batch-major ids (B*S,).  Returns logits (V, B*S)."""
        c = self.cfg
        tokens = np.asarray(tokens).reshape(-1)
        assert tokens.size == c.tokens
        self.tokens = tokens
        x = gather_rows(self.p("token_emb"), tokens.astype(F32)).T.copy()    # (d, N)
        self.pos_idx = np.tile(np.arange(c.seq), c.batch).astype(F32)
        if c.pos == POS_LEARNED:
            x = x + gather_rows(self.p("pos_emb"), self.pos_idx).T
        elif c.pos == POS_SINUSOIDAL:
            x = x + gather_rows(self.sin_table, self.pos_idx).T
        x = x.astype(F32)
        mask = self._attention_mask(doc_ids)
        self.caches = []
        for l in range(c.layers):
            pfx = f"blk{l}."
            cache: Dict[str, object] = {}
            n1 = self._norm(pfx + "norm1")
            a = self._attn_forward(pfx, n1.forward(x), mask, cache)
            r2 = (x + a).astype(F32)
            n2 = self._norm(pfx + "norm2")
            f = self._ffn_forward(pfx, n2.forward(r2), cache)
            x = (r2 + f).astype(F32)
            cache.update(n1=n1, n2=n2)
            self.caches.append(cache)
        self.lnf = self._norm("ln_f")
        self.lnf_out = self.lnf.forward(x)
        return self._linear("lm_head", self.lnf_out)

    def backward(self, grad_logits):
        c = self.cfg
        g = self._linear_backward("lm_head", self.lnf_out, grad_logits)
        g = self._norm_backward("ln_f", self.lnf, g)
        for l in reversed(range(c.layers)):
            pfx = f"blk{l}."
            cache = self.caches[l]
            gff = self._ffn_backward(pfx, g, cache)
            gr1 = (g + self._norm_backward(pfx + "norm2", cache["n2"], gff)).astype(F32)
            gsa = self._attn_backward(pfx, gr1, cache)
            g = (gr1 + self._norm_backward(pfx + "norm1", cache["n1"], gsa)).astype(F32)
        gT = np.ascontiguousarray(g.T)                                        # (N, d)
        if c.pos == POS_LEARNED:
            scatter_add_rows(self.g("pos_emb"), self.pos_idx, gT)             # :2573-2580
        scatter_add_rows(self.g("token_emb"), self.tokens.astype(F32), gT)    # :2887-2891
        self.grad_x0 = gT


# --------------------------------------------------------------------------------------
# optimizers (compute_optimizer.hpp) and schedule (cli/lr_scheduler.hpp)
# --------------------------------------------------------------------------------------
def step_lr(base_lr, min_lr, warmup, total, cosine, step):
    """compute_step_lr (cli/lr_scheduler.hpp:89-114), float arithmetic."""
    base_lr, min_lr = F32(base_lr), F32(min_lr)
    if warmup > 0 and step < warmup:
        return F32(base_lr * F32(step + 1) / F32(warmup))
    if cosine:
        cs = total - warmup
        if cs <= 0:
            return base_lr
        p = F32(step - warmup) / F32(cs)
        p = F32(min(max(p, F32(0)), F32(1)))
        return F32(min_lr + F32(0.5) * (base_lr - min_lr) * (F32(1) + F32(math.cos(F32(np.pi) * p))))
    return base_lr


def clip_grad_norm(grads, max_norm):
    """Optimizer::clip_grad_norm (compute_optimizer.hpp:90-140): scale = max_norm/norm, no eps,
    applied only when norm > max_norm.  Returns the norm."""
    if max_norm <= 0 or not grads:
        return F32(0)
    total = F32(0)
    for g in grads:
        total = F32(total + (g * g).sum(axis=1, dtype=F32).sum(dtype=F32))
    norm = F32(np.sqrt(total))
    if norm > F32(max_norm):
        scale = F32(max_norm) / norm
        for g in grads:
            g *= scale
    return norm


class AdamW:
    """Adam::adam_update_ + AdamW::step (compute_optimizer.hpp:252-304, 388-412): decay every
    parameter by (1 - lr*wd), then Adam with eps added after the sqrt; beta 0.9/0.999, eps 1e-8."""

    def __init__(self, params, grads, lr, wd=0.01, beta1=0.9, beta2=0.999, eps=1e-8):
        self.params, self.grads = params, grads
        self.lr, self.wd = F32(lr), F32(wd)
        self.b1, self.b2, self.eps = F32(beta1), F32(beta2), F32(eps)
        self.t = 0
        self.m = [np.zeros_like(p) for p in params]
        self.v = [np.zeros_like(p) for p in params]

    def step(self):
        t = self.t + 1
        inv_bc1 = F32(1) / (F32(1) - F32(np.power(self.b1, F32(t), dtype=F32)))
        inv_bc2 = F32(1) / (F32(1) - F32(np.power(self.b2, F32(t), dtype=F32)))
        decay = F32(1) - self.lr * self.wd
        for p, g, m, v in zip(self.params, self.grads, self.m, self.v):
            if self.wd != 0:
                p *= decay
            m *= self.b1
            m += (F32(1) - self.b1) * g
            v *= self.b2
            v += (g * g) * (F32(1) - self.b2)
            ratio = (m * inv_bc1) / (np.sqrt(v * inv_bc2, dtype=F32) + self.eps)
            p += ratio * (-self.lr)
        self.t = t


def newton_schulz(G, steps=5, eps=1e-7):
    """newton_schulz_orthogonalize (compute_optimizer.hpp:430-497): X = G/sqrt(|G|^2 + eps^2);
    5x {A = X X^T; B = b A + c A^2; X = a X + B X}; stored orientation, no transpose."""
    a, b, c = F32(3.4445), F32(-4.7750), F32(2.0315)
    nsq = (G * G).sum(axis=1, dtype=F32).sum(dtype=F32)
    X = (G * (F32(1) / np.sqrt(nsq + F32(eps) * F32(eps), dtype=F32))).astype(F32)
    for _ in range(steps):
        A = (X @ X.T).astype(F32)
        Bm = (b * A + c * (A @ A).astype(F32)).astype(F32)
        X = ((Bm @ X).astype(F32) + a * X).astype(F32)
    return X


class Muon:
    """Muon::step (compute_optimizer.hpp:517-590): v = mu*v + g; Nesterov u = g + mu*v; 2-D tensors
    take p -= lr * NS(u), others p -= lr * u; mu 0.95; no shape scaling."""

    def __init__(self, params, grads, lr, momentum=0.95, ns_steps=5, ns_eps=1e-7):
        self.params, self.grads = params, grads
        self.lr, self.mu = F32(lr), F32(momentum)
        self.ns_steps, self.ns_eps = ns_steps, ns_eps
        self.vel = [np.zeros_like(p) for p in params]

    def step(self):
        for p, g, v in zip(self.params, self.grads, self.vel):
            v *= self.mu
            v += g
            u = (g + self.mu * v).astype(F32)
            if p.shape[0] > 1 and p.shape[1] > 1:
                u = newton_schulz(u, self.ns_steps, self.ns_eps)
            p += (-self.lr) * u


def train(cfg: GptConfig, params, micro_batches, *, steps, accum=1, lr=1e-3, wd=0.01,
          optimizer=OPT_ADAMW, muon_lr=0.02, clip=None, cosine=False, warmup=0, total_steps=1,
          min_lr=0.0, keep_first_grads=False):
    """The training-loop order of src/text_train.cpp:1107-1334.  ``micro_batches`` is a list of
    dicts {tokens, labels, mask, doc_ids|None}, ``steps*accum`` long.  Returns
    (losses[steps*accum], model, first_window_grads|None)."""
    model = GptOracle(cfg, params)
    if optimizer == OPT_MUON_SPLIT:
        mm = muon_mask(cfg)
        pm = [p for p, f in zip(model.params, mm) if f]
        gm = [g for g, f in zip(model.grads, mm) if f]
        pa = [p for p, f in zip(model.params, mm) if not f]
        ga = [g for g, f in zip(model.grads, mm) if not f]
        opts = [Muon(pm, gm, muon_lr), AdamW(pa, ga, lr, wd)]
    else:
        opts = [AdamW(model.params, model.grads, lr, wd)]
    losses, first = [], None
    it = iter(micro_batches)
    for step in range(steps):
        if cosine or warmup > 0:
            cur = step_lr(lr, min_lr, warmup, total_steps, cosine, step)
            if optimizer == OPT_MUON_SPLIT:
                opts[0].lr = F32(cur * F32(muon_lr) / F32(lr))
                opts[1].lr = cur
            else:
                opts[0].lr = cur
        for _ in range(accum):
            mb = next(it)
            logits = model.forward(mb["tokens"], mb.get("doc_ids"))
            loss, grad = ce_forward_sparse(logits, mb["labels"], mb.get("mask"), cfg.vocab)
            losses.append(loss)
            if accum > 1:
                grad = grad * (F32(1) / F32(accum))       # text_train.cpp:1253-1258
            model.backward(grad.astype(F32))
        if keep_first_grads and step == 0:
            first = [g.copy() for g in model.grads]
        if clip is not None:
            clip_grad_norm(model.grads, clip)
        for o in opts:
            o.step()
        model.zero_grad()
    return np.array(losses, F32), model, first


# --------------------------------------------------------------------------------------
# synthetic inputs (shapes and distributions of the benchmark configurations)
# --------------------------------------------------------------------------------------
def zipf_tokens(rng: np.random.Generator, vocab: int, n: int, s: float = 1.1) -> np.ndarray:
    """Token ids Zipf(s) over [0, vocab) by inverse CDF."""
    w = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    cdf = np.cumsum(w) / w.sum()
    return np.minimum(np.searchsorted(cdf, rng.random(n)), vocab - 1).astype(np.int32)


def packed_doc_ids(rng: np.random.Generator, batch: int, seq: int, mean_len: float = 300.0) -> np.ndarray:
    """Each row packs documents with geometric(mean_len) lengths; ids are 1-based per row
    (0 is the padding id in src/text_train.cpp:1159-1161)."""
    out = np.zeros((batch, seq), np.int32)
    for b in range(batch):
        t, d = 0, 1
        while t < seq:
            ln = int(rng.geometric(1.0 / mean_len))
            out[b, t:t + ln] = d
            t += ln
            d += 1
    return out.reshape(-1)


def make_batches(cfg: GptConfig, n: int, seed: int, dist: str = "uniform", docs: bool = False):
    """n micro-batches: per row S+1 ids, x = ids[:S], y = ids[1:], mask all ones."""
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n):
        total = cfg.batch * (cfg.seq + 1)
        ids = (rng.integers(0, cfg.vocab, total, dtype=np.int32) if dist == "uniform"
               else zipf_tokens(rng, cfg.vocab, total)).reshape(cfg.batch, cfg.seq + 1)
        mb = {"tokens": ids[:, :-1].reshape(-1).copy(), "labels": ids[:, 1:].reshape(-1).copy(),
              "mask": np.ones(cfg.tokens, F32), "doc_ids": None}
        if docs:
            mb["doc_ids"] = packed_doc_ids(rng, cfg.batch, cfg.seq,
                                           mean_len=max(2.0, min(300.0, cfg.seq / 3)))
        out.append(mb)
    return out
