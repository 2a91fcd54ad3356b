"""Host-side logic of the data-parallel path on CPU ranks (gloo, world size 2): the gradient buckets tile the
arena, a bucket-wise sum-all-reduce equals one all-reduce of the whole arena, and folding 1/world into the
gradient scale reproduces the single-replica gradient when every rank holds the same data."""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry


def _layout(cfg_args):
    nnb = entry.load_package()
    cfg = nnb.GptConfig(*cfg_args).c_struct()
    L = cfg_args[3]
    layer_begin = [int(nnb.call("nnb200_gpt_layer_matrix_begin", C.byref(cfg), l)) for l in range(L + 1)]
    return layer_begin, int(nnb.call("nnb200_gpt_matrix_region_begin", C.byref(cfg))), int(nnb.call("nnb200_gpt_arena_elems", C.byref(cfg)))


def _lm_head(cfg_args):
    """(start, end) of lm_head.W in the arena: the last but one tensor of the reference's parameter order."""
    nnb = entry.load_package()
    cfg = nnb.GptConfig(*cfg_args).c_struct()
    n = nnb.call("nnb200_gpt_param_table", C.byref(cfg), None, None, None)
    offs, rows, cols = (C.c_longlong * n)(), (C.c_int32 * n)(), (C.c_int32 * n)()
    nnb.call("nnb200_gpt_param_table", C.byref(cfg), offs, rows, cols)
    return int(offs[n - 2]), int(offs[n - 2]) + int(rows[n - 2]) * int(cols[n - 2])


CFG = (96, 48, 6, 3, 80, 12, 4, 1, 1, 2, 0)


def test_buckets_tile_the_arena():
    nnb = entry.load_package()
    from neuralnet_cpp_b200.trainer import gradient_buckets
    layer_begin, matrix_begin, total = _layout(CFG)
    assert layer_begin[0] == matrix_begin and layer_begin[-1] == total
    L = len(layer_begin) - 1
    for lm in (None, _lm_head(CFG)):
        order = gradient_buckets(layer_begin, matrix_begin, lm)
        spans = sorted((lo, hi) for _, lo, hi in order)
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        # issue order: (LM head weight first, behind its own event;) last layer first; vectors / embeddings last
        first_layer = order[1] if lm else order[0]
        assert first_layer == (L - 1, layer_begin[-2], layer_begin[-1])
        assert order[-1][0] == L and order[-1][2] == matrix_begin
        if lm:
            assert order[0] == (L + 1, lm[0], lm[1]) and 0 < lm[0] < lm[1] < matrix_begin
        else:
            assert order[-1] == (L, 0, matrix_begin)


def _worker(rank, world, port, layer_begin, matrix_begin, total, lm, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    entry.load_package()
    from neuralnet_cpp_b200.trainer import gradient_buckets
    rng = np.random.default_rng(100 + rank)
    grads = torch.from_numpy(rng.standard_normal(total).astype(np.float32))
    whole = grads.clone()
    dist.all_reduce(whole)
    for _, lo, hi in gradient_buckets(layer_begin, matrix_begin, lm):
        dist.all_reduce(grads[lo:hi])
    same = torch.equal(grads, whole)
    # identical data on every rank: sum * (1/world) is exact for world = 2
    g1 = torch.from_numpy(np.random.default_rng(7).standard_normal(total).astype(np.float32))
    g = g1.clone()
    dist.all_reduce(g)
    exact = torch.equal(g * (1.0 / world), g1)
    q.put((rank, same, exact))
    dist.destroy_process_group()


def test_bucketed_all_reduce_world2_gloo():
    layer_begin, matrix_begin, total = _layout(CFG)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, layer_begin, matrix_begin, total, _lm_head(CFG), q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(same and exact for _, same, exact in results)
