"""C-ABI parity of the reference-layout engine primitives (the ComputeEngine virtuals the reference's CUDA
engine leaves unimplemented): against tests/golden/prims.npz, which the reference CPU engine produced, and
against the numpy restatement at larger seeded sizes.  fp32; tolerance 1e-5 of the largest reference value."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import gpt_oracle as go
from tests.golden_io import GOLDEN

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def g():
    import tests.gpu_util as gu
    return gu


def close(got, want, tol=TOL):
    want = np.asarray(want, np.float32)
    assert got.shape == want.shape, (got.shape, want.shape)
    scale = max(float(np.abs(want).max()), 1e-30)
    err = float(np.abs(got.astype(np.float64) - want).max()) / scale
    assert err <= tol, err


def attention_chain(g, A, B, V, G, P, mask, batch, M, N, K, D, alpha):
    """max -> denom -> apply -> backward_q -> backward_kv through the C ABI, transA=1 / transB=0 as the layer calls it."""
    dA, dB, dV, dG, dP = (g.dev(x) for x in (A, B, V, G, P))
    dmask = g.dev(mask) if mask is not None else None
    mp = g.ptr(dmask) if mask is not None else None
    z = lambda *s: g.dev(np.zeros(s, np.float32))
    m, l, O, gq, R, gk, gv = z(batch * M, 1), z(batch * M, 1), z(batch * M, D), z(batch * K, M), z(batch * M, 1), z(batch * K, N), z(batch * K, N)
    s = g.stream()
    g.call("nnb200_bmm_reduce", g.ptr(dA), g.ptr(dB), mp, g.ptr(m), batch, M, N, K, 1, 1, 0, C.c_float(alpha), 1, s)
    g.call("nnb200_bmm_softmax_denom", g.ptr(dA), g.ptr(dB), g.ptr(m), mp, g.ptr(l), batch, M, N, K, 1, 0, C.c_float(alpha), s)
    g.call("nnb200_bmm_softmax_apply", g.ptr(dA), g.ptr(dB), g.ptr(dV), g.ptr(m), g.ptr(l), mp, g.ptr(O), batch, M, N, K, D, 1, 0,
           C.c_float(alpha), s)
    g.call("nnb200_bmm_softmax_backward_q", g.ptr(dA), g.ptr(dB), g.ptr(dP), g.ptr(m), g.ptr(l), mp, g.ptr(gq), g.ptr(R), batch, M, N, K,
           1, 0, C.c_float(alpha), s)
    g.call("nnb200_bmm_softmax_backward_kv", g.ptr(dA), g.ptr(dB), g.ptr(dP), g.ptr(dG), g.ptr(R), g.ptr(m), g.ptr(l), mp, g.ptr(gk),
           g.ptr(gv), batch, M, N, K, D, 1, 0, C.c_float(alpha), s)
    return [g.host(t) for t in (m, l, O, gq, R, gk, gv)]


def test_attention_primitives_match_reference_golden(g):
    z = np.load(os.path.join(GOLDEN, "prims.npz"))
    batch, M, N, K, D = (int(v) for v in z["dims"][:5])
    got = attention_chain(g, z["A"], z["B"], z["V"], z["G"], z["P"], z["mask"], batch, M, N, K, D, float(z["scal"][0]))
    for arr, name in zip(got, ("m", "l", "O", "gradQ", "R", "gradK", "gradV")):
        close(arr, z["out_" + name])


@pytest.mark.parametrize("batch,M,N,K,D,masked", [(4, 64, 64, 32, 32, True), (2, 150, 150, 64, 64, True), (3, 40, 70, 16, 16, False),
                                                  (1, 130, 257, 8, 8, False)])
def test_attention_primitives_match_oracle(g, batch, M, N, K, D, masked):
    r = np.random.default_rng(batch * 1000 + M)
    f = lambda *s: r.standard_normal(s).astype(np.float32)
    A, B, V, G, P = f(batch * K, M), f(batch * K, N), f(batch * N, D), f(batch * M, D), f(batch * M, N)
    mask = np.where(np.arange(N)[None, :] <= np.arange(M)[:, None], 0.0, -np.inf).astype(np.float32) if masked else None
    alpha = 1.0 / np.sqrt(K)
    m, l, O, gq, R, gk, gv = attention_chain(g, A, B, V, G, P, mask, batch, M, N, K, D, float(alpha))
    wm = go.bmm_reduce_max(A, B, batch, alpha, mask)
    wl = go.bmm_softmax_denom(A, B, wm, batch, alpha, mask)
    close(m, wm)
    close(l, wl)
    close(O, go.bmm_softmax_apply(A, B, V, wm, wl, batch, alpha, mask))
    wq, wR = go.bmm_softmax_backward_q(A, B, P, wm, wl, batch, alpha, mask)
    close(gq, wq)
    close(R, wR)
    wk, wv = go.bmm_softmax_backward_kv(A, B, P, G, wR, wm, wl, batch, alpha, mask)
    close(gk, wk)
    close(gv, wv)


@pytest.mark.parametrize("op", [0, 1, 2])
@pytest.mark.parametrize("reduce_cols", [0, 1])
def test_bmm_reduce_all_ops_both_axes(g, op, reduce_cols):
    """Sum and Min skip entries whose mask is -inf; Max does not (cpu_engine.hpp:470-515)."""
    r = np.random.default_rng(op * 2 + reduce_cols)
    batch, M, N, K = 3, 33, 47, 12
    A, B = r.standard_normal((batch * M, K)).astype(np.float32), r.standard_normal((batch * N, K)).astype(np.float32)   # transA=0, transB=1
    mask = np.where(r.random((M, N)) < 0.3, -np.inf, r.standard_normal((M, N))).astype(np.float32)
    S = 0.5 * np.einsum("bmk,bnk->bmn", A.reshape(batch, M, K), B.reshape(batch, N, K)) + mask[None]
    live = np.isfinite(mask)[None]
    axis = 2 if reduce_cols else 1
    if op == 0:
        want = np.where(live, S, 0).sum(axis=axis)
    elif op == 1:
        want = np.maximum(S.max(axis=axis), np.finfo(np.float32).min)
    else:
        want = np.where(live, S, np.finfo(np.float32).max).min(axis=axis)
    out = g.dev(np.zeros(want.size, np.float32))
    g.call("nnb200_bmm_reduce", g.ptr(g.dev(A)), g.ptr(g.dev(B)), g.ptr(g.dev(mask)), g.ptr(out), batch, M, N, K, op, 0, 1, C.c_float(0.5),
           reduce_cols, g.stream())
    close(g.host(out).reshape(want.shape), want.astype(np.float32), 2e-5)


def test_cross_entropy_primitives_match_reference_golden(g):
    z = np.load(os.path.join(GOLDEN, "prims.npz"))
    logits, labels, cmask = z["logits"], z["labels"], z["cmask"]
    Cn, N = logits.shape
    vocab, inv_nv = int(z["dims"][7]), float(z["scal"][1])
    dl = g.dev(logits)
    cmax = g.dev(logits.max(axis=0).astype(np.float32))
    den = g.dev(np.zeros((1, N), np.float32))
    g.call("nnb200_col_softmax_denom", g.ptr(dl), g.ptr(cmax), g.ptr(den), Cn, N, g.stream())
    close(g.host(den), z["out_col_denom"])
    grad, lv = g.dev(np.zeros((Cn, N), np.float32)), g.dev(np.zeros((1, N), np.float32))
    g.call("nnb200_col_softmax_sparse_forward", g.ptr(dl), g.ptr(g.dev(labels)), g.ptr(g.dev(cmask)), g.ptr(grad), g.ptr(lv), Cn, N, vocab,
           C.c_float(inv_nv), g.stream())
    close(g.host(grad), z["out_ce_grad"])
    close(g.host(lv), z["out_loss_vec"])


def test_cross_entropy_primitive_large_vocab_matches_oracle(g):
    r = np.random.default_rng(3)
    Cn, N, vocab = 4099, 333, 4096
    logits = (r.standard_normal((Cn, N)) * 3).astype(np.float32)
    labels = r.integers(0, vocab + 40, (1, N)).astype(np.float32)
    mask = (r.random((1, N)) > 0.2).astype(np.float32)
    want_g, want_lv = go.col_softmax_sparse_forward(logits, labels, mask, vocab, np.float32(1 / 250))
    grad, lv = g.dev(np.zeros((Cn, N), np.float32)), g.dev(np.zeros((1, N), np.float32))
    g.call("nnb200_col_softmax_sparse_forward", g.ptr(g.dev(logits)), g.ptr(g.dev(labels)), g.ptr(g.dev(mask)), g.ptr(grad), g.ptr(lv), Cn, N,
           vocab, C.c_float(1 / 250), g.stream())
    close(g.host(grad), want_g)
    close(g.host(lv), np.asarray(want_lv).reshape(1, N))
    with pytest.raises(Exception):
        g.call("nnb200_col_softmax_sparse_forward", g.ptr(g.dev(logits)), g.ptr(g.dev(labels)), None, g.ptr(grad), g.ptr(lv), Cn, N, Cn + 1,
               C.c_float(1.0), g.stream())


class ExprProgram(C.Structure):
    """struct nnb200_expr_program (include/nnb200.h)."""
    _fields_ = [("num_instrs", C.c_uint32), ("num_regs", C.c_uint32), ("num_inputs", C.c_uint32), ("num_consts", C.c_uint32),
                ("instrs", (C.c_uint8 * 8) * 64), ("view_kind", C.c_uint8 * 8), ("view_negate", C.c_uint8 * 8),
                ("view_param", C.c_uint32 * 8), ("consts", C.c_float * 16)]


def make_program(instrs, views, consts, num_regs):
    p = ExprProgram()
    p.num_instrs, p.num_regs, p.num_inputs, p.num_consts = len(instrs), num_regs, len(views), len(consts)
    for i, ins in enumerate(instrs):
        for j, v in enumerate(list(ins) + [0] * (8 - len(ins))):
            p.instrs[i][j] = v
    for k, (kind, neg, prm) in enumerate(views):
        p.view_kind[k], p.view_negate[k], p.view_param[k] = kind, neg, prm
    for k, c in enumerate(consts):
        p.consts[k] = c
    return p


def run_expr(g, prog, inputs, rows, cols, vector_out=0, out_shape=None):
    devs = [g.dev(x) for x in inputs]
    ptrs = (C.c_void_p * 8)(*[g.ptr(d).value for d in devs])
    ir = (C.c_int * 8)(*[x.shape[0] for x in inputs])
    ic = (C.c_int * 8)(*[x.shape[1] for x in inputs])
    out = g.dev(np.zeros(out_shape or (rows, cols), np.float32))
    scratch = g.dev(np.zeros(int(g.call("nnb200_eval_expr_scratch_floats", rows, cols)), np.float32))
    g.call("nnb200_eval_expr", C.byref(prog), ptrs, ir, ic, g.ptr(out), g.ptr(scratch), rows, cols, vector_out, g.stream())
    return g.host(out)


REG, INPUT, CONST, REDUCE = 0, 1, 2, 4
MUL, ADD, RSQRT, COLSUM = 9, 7, 4, 20


def test_eval_expr_rms_norm_program(g):
    """x * rsqrt(colsum(x*x)/F + eps) * gamma on the reference layout (features, tokens) — RMSNorm::forward
    (compute_layer.hpp:722-760) as one expression program."""
    r = np.random.default_rng(4)
    F, T = 96, 300
    x, gamma = r.standard_normal((F, T)).astype(np.float32), r.uniform(0.5, 1.5, (F, 1)).astype(np.float32)
    instrs = [(MUL, 0, INPUT, 0, INPUT, 0), (COLSUM, 1, REG, 0), (MUL, 2, REDUCE, 1, CONST, 0), (ADD, 2, REG, 2, CONST, 1),
              (RSQRT, 3, REG, 2), (MUL, 4, INPUT, 0, REG, 3), (MUL, 4, REG, 4, INPUT, 1)]
    prog = make_program(instrs, [(0, 0, 0), (7, 0, 0)], [1.0 / F, 1e-5], 5)
    got = run_expr(g, prog, [x, gamma], F, T)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=0, keepdims=True) + 1e-5) * gamma
    close(got, want.astype(np.float32))
    assert g.call("nnb200_expr_reduce_axis", C.byref(prog)) == 1
    stat = make_program(instrs[:5], [(0, 0, 0)], [1.0 / F, 1e-5], 4)
    got = run_expr(g, stat, [x], F, T, vector_out=1, out_shape=(1, T))
    close(got, (1 / np.sqrt((x.astype(np.float64) ** 2).mean(axis=0, keepdims=True) + 1e-5)).astype(np.float32))


def test_eval_expr_rotary_views(g):
    """q*cos + rotate_half(q)*sin with the tables tiled by row modulo (RotaryEmbedding, compute_layer.hpp:884-988)."""
    r = np.random.default_rng(5)
    dk, blocks, T = 16, 6, 50
    q = r.standard_normal((dk * blocks, T)).astype(np.float32)
    cos, sin = r.standard_normal((dk, T)).astype(np.float32), r.standard_normal((dk, T)).astype(np.float32)
    prog = make_program([(MUL, 0, INPUT, 0, INPUT, 2), (MUL, 1, INPUT, 1, INPUT, 3), (ADD, 2, REG, 0, REG, 1)],
                        [(0, 0, 0), (1, 1, dk), (2, 0, dk), (2, 0, dk)], [], 3)
    got = run_expr(g, prog, [q, q, cos, sin], dk * blocks, T)
    qb = q.reshape(blocks, dk, T)
    rot = np.concatenate([-qb[:, dk // 2:], qb[:, :dk // 2]], axis=1)
    want = qb * cos[None] + rot * sin[None]
    assert np.array_equal(got, want.reshape(dk * blocks, T).astype(np.float32)) or np.abs(got - want.reshape(got.shape)).max() < 1e-6


def test_eval_expr_rejects_invalid_programs(g):
    x = np.zeros((4, 4), np.float32)
    bad_dst = make_program([(0, 3, INPUT, 0)], [(0, 0, 0)], [], 1)
    with pytest.raises(Exception):
        run_expr(g, bad_dst, [x], 4, 4)
    reg_on_reduce = make_program([(COLSUM, 0, INPUT, 0), (MUL, 1, INPUT, 0, REG, 0)], [(0, 0, 0)], [], 2)
    with pytest.raises(Exception):
        run_expr(g, reg_on_reduce, [x], 4, 4)
    shape = make_program([(MUL, 0, INPUT, 0, INPUT, 1)], [(0, 0, 0), (7, 0, 0)], [], 1)
    with pytest.raises(Exception):
        run_expr(g, shape, [x, np.zeros((1, 4), np.float32)], 4, 4)
