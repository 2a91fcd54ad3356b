"""GPU parity of the engine primitives (the fifteen cuda_* symbols of the reference ABI) against numpy
and the oracle restatement, on the shapes the reference's own probes use (src/matmul_probe.cpp,
src/matmul_fusion_test.cpp) plus ragged and empty cases.  Index work is compared bit for bit."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    from tests import gpu_util
    return gpu_util


def _rng(seed=7):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("tA,tB", [(0, 0), (1, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(4, 6, 5), (70, 33, 129), (128, 64, 64)])
def test_matmul_trans_combos(g, tA, tB, M, N, K):
    r = _rng()
    A = r.standard_normal((K, M) if tA else (M, K)).astype(np.float32)
    B = r.standard_normal((N, K) if tB else (K, N)).astype(np.float32)
    want = (A.T if tA else A).astype(np.float64) @ (B.T if tB else B).astype(np.float64)
    a, b = g.dev(A), g.dev(B)
    c = g.dev(np.zeros((M, N), np.float32))
    g.call("cuda_matmul", g.ptr(a), g.ptr(b), g.ptr(c), A.shape[0], A.shape[1], B.shape[0], B.shape[1], tA, tB, g.stream())
    assert np.allclose(g.host(c), want, atol=1e-4)      # the reference probe's bound (matmul_probe.cpp, 1e-4)
    c2 = g.dev(np.zeros((M, N), np.float32))
    g.call("nnb200_set_handle_stream", g.stream())
    g.call("cuda_matmul_with_handle", g.ptr(a), g.ptr(b), g.ptr(c2), A.shape[0], A.shape[1], B.shape[0], B.shape[1], tA, tB, None)
    assert np.array_equal(g.host(c2), g.host(c))


def test_matmul_shape_error(g):
    a = g.dev(np.zeros((3, 4), np.float32))
    assert g.nnb.lib.cuda_matmul(g.ptr(a), g.ptr(a), g.ptr(a), 3, 4, 3, 4, 0, 0, g.stream()) == -1


@pytest.mark.parametrize("tA,tB", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_batched_matmul(g, tA, tB):
    r = _rng(3)
    batch, M, N, K = 3, 5, 7, 4
    A = r.standard_normal((batch, K, M) if tA else (batch, M, K)).astype(np.float32)
    B = r.standard_normal((batch, N, K) if tB else (batch, K, N)).astype(np.float32)
    want = np.stack([(A[i].T if tA else A[i]) @ (B[i].T if tB else B[i]) for i in range(batch)])
    a, b = g.dev(A.reshape(-1, A.shape[2])), g.dev(B.reshape(-1, B.shape[2]))
    c = g.dev(np.zeros((batch * M, N), np.float32))
    g.call("cuda_batched_matmul", g.ptr(a), g.ptr(b), g.ptr(c), a.shape[0], a.shape[1], b.shape[0], b.shape[1], batch, tA, tB, g.stream())
    assert np.allclose(g.host(c).reshape(batch, M, N), want, atol=1e-4)


def test_elementwise_family(g):
    r = _rng(11)
    n = 1000 + 3                                       # not a multiple of the vector width
    A = (r.random(n) + 0.1).astype(np.float32)
    B = (r.random(n) + 0.1).astype(np.float32)
    a, b, o = g.dev(A), g.dev(B), g.dev(np.zeros(n, np.float32))
    unary = [lambda x: -x, np.exp, np.log, np.sqrt, lambda x: 1 / np.sqrt(x), np.abs, np.tanh]
    for op, f in enumerate(unary):
        g.call("cuda_elementwise_unary", g.ptr(a), g.ptr(o), n, op, g.stream())
        assert np.allclose(g.host(o), f(A), rtol=2e-6, atol=1e-7), op
    binary = [np.add, np.subtract, np.multiply, np.divide, np.maximum, np.minimum]
    for op, f in enumerate(binary):
        g.call("cuda_elementwise_binary", g.ptr(a), g.ptr(b), g.ptr(o), n, op, g.stream())
        assert np.allclose(g.host(o), f(A, B), rtol=1e-6), op
        g.call("cuda_elementwise_binary_scalar", g.ptr(a), g.ptr(o), n, op, C.c_float(0.7), 0, g.stream())
        assert np.allclose(g.host(o), f(A, np.float32(0.7)), rtol=1e-6), op
        g.call("cuda_elementwise_binary_scalar", g.ptr(a), g.ptr(o), n, op, C.c_float(0.7), 1, g.stream())
        assert np.allclose(g.host(o), f(np.float32(0.7), A), rtol=1e-6), op
    g.call("cuda_axpy", g.ptr(a), g.ptr(b), g.ptr(o), n, C.c_float(-0.25), g.stream())
    assert np.allclose(g.host(o), A - 0.25 * B, rtol=1e-6)
    cmps = [np.less, np.less_equal, np.greater, np.greater_equal, np.equal, np.not_equal]
    for cmp, f in enumerate(cmps):
        g.call("cuda_elementwise_select_scalar_cond", g.ptr(a), g.ptr(b), g.ptr(o), n, cmp, C.c_float(0.5), C.c_float(-3.0), g.stream())
        assert np.array_equal(g.host(o), np.where(f(A, np.float32(0.5)), B, np.float32(-3.0))), cmp
    assert g.nnb.lib.cuda_elementwise_unary(g.ptr(a), g.ptr(o), n, 9, g.stream()) == -1
    g.call("cuda_elementwise_unary", g.ptr(a), g.ptr(o), 0, 0, g.stream())     # empty input is a no-op


@pytest.mark.parametrize("rows,cols", [(1, 1), (5, 7), (33, 1000), (1030, 65)])
def test_reduce_and_broadcast(g, rows, cols):
    r = _rng(5)
    A = r.standard_normal((rows, cols)).astype(np.float32)
    a = g.dev(A)
    orow, ocol = g.dev(np.zeros(rows, np.float32)), g.dev(np.zeros(cols, np.float32))
    for mode, f in enumerate([np.sum, np.max, np.min]):
        g.call("cuda_reduce_row", g.ptr(a), g.ptr(orow), rows, cols, mode, g.stream())
        assert np.allclose(g.host(orow), f(A.astype(np.float64), axis=1), atol=1e-4 * max(1, cols) ** 0.5)
        g.call("cuda_reduce_col", g.ptr(a), g.ptr(ocol), rows, cols, mode, g.stream())
        assert np.allclose(g.host(ocol), f(A.astype(np.float64), axis=0), atol=1e-4 * max(1, rows) ** 0.5)
    rv, cv = r.standard_normal(rows).astype(np.float32), r.standard_normal(cols).astype(np.float32)
    o = g.dev(np.zeros((rows, cols), np.float32))
    g.call("cuda_broadcast_row", g.ptr(a), g.ptr(g.dev(rv)), g.ptr(o), rows, cols, 0, g.stream())
    assert np.array_equal(g.host(o), A + rv[:, None])
    g.call("cuda_broadcast_col", g.ptr(a), g.ptr(g.dev(cv)), g.ptr(o), rows, cols, 2, g.stream())
    assert np.array_equal(g.host(o), A * cv[None, :])


@pytest.mark.parametrize("R,Cc", [(1, 1), (16, 17), (100, 37), (64, 256)])
def test_transpose(g, R, Cc):
    A = _rng(1).standard_normal((R, Cc)).astype(np.float32)
    o = g.dev(np.zeros((Cc, R), np.float32))
    g.call("cuda_transpose", g.ptr(g.dev(A)), g.ptr(o), R, Cc, g.stream())
    assert np.array_equal(g.host(o), A.T)


def test_rearrange_3d_roundtrip_and_golden(g):
    from oracle import gpt_oracle as go
    M, B, N = 6, 4, 9
    A = _rng(2).standard_normal((M, B * N)).astype(np.float32)
    o = g.dev(np.zeros((B * M, N), np.float32))
    g.call("cuda_rearrange_3d", g.ptr(g.dev(A)), g.ptr(o), M, B, N, 0, g.stream())
    assert np.array_equal(g.host(o), go.rearrange_3d(A, M, B, N))
    back = g.dev(np.zeros((M, B * N), np.float32))
    g.call("cuda_rearrange_3d", g.ptr(o), g.ptr(back), M, B, N, 1, g.stream())
    assert np.array_equal(g.host(back), A)


def test_gather_scatter_bit_exact_vs_reference_golden(g):
    """Inputs and expected outputs come from the reference CPU engine (tests/golden/prims.npz)."""
    import os
    from tests.golden_io import GOLDEN
    z = np.load(os.path.join(GOLDEN, "prims.npz"))
    logits, labels = z["logits"], z["labels"]
    Cn, NC = logits.shape
    out = g.dev(np.zeros((NC, NC), np.float32))
    g.call("cuda_gather", g.ptr(g.dev(logits)), g.ptr(g.dev(labels)), g.ptr(out), Cn, NC, NC, g.stream())
    assert np.array_equal(g.host(out), z["out_gathered"])
    dst = g.dev(np.zeros((Cn, NC), np.float32))
    g.call("cuda_scatter_add", g.ptr(dst), g.ptr(g.dev(labels)), g.ptr(out), Cn, NC, NC, g.stream())
    assert np.array_equal(g.host(dst), z["out_scattered"])


def test_scatter_add_order_is_sequential(g):
    """Many collisions: the fp32 sum must equal the ascending-i sequential sum bit for bit."""
    from oracle import gpt_oracle as go
    r = _rng(9)
    vocab, D, num = 37, 70, 5000
    idx = r.integers(-2, vocab + 3, num).astype(np.float32)        # includes out-of-range ids
    grad = (r.standard_normal((num, D)) * 10 ** r.uniform(-3, 3, (num, 1))).astype(np.float32)
    want = r.standard_normal((vocab, D)).astype(np.float32)
    dst = g.dev(want.copy())
    go.scatter_add_rows(want, idx, grad)
    g.call("cuda_scatter_add", g.ptr(dst), g.ptr(g.dev(idx)), g.ptr(g.dev(grad)), vocab, D, num, g.stream())
    assert np.array_equal(g.host(dst), want)
