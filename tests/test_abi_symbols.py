"""CPU-side checks of the drop-in boundary: the shared library loads and exports every entry point
that include/nnb200.h declares (no compute calls are made without a GPU), the ctypes table covers
them all, and the host-side layout queries agree with the reference parameter order."""
import ctypes as C
import os
import re

import pytest

import __graft_entry__ as entry

HEADER = os.path.join(entry.ROOT, "include", "nnb200.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"(?:\b(?:int|size_t|long long|unsigned long long)\s+|\bvoid\s*\*\s*)((?:cuda|nnb200)_\w+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    nnb = entry.load_package()
    names = declared_functions()
    assert len(names) >= 50
    for n in names:
        assert hasattr(nnb.lib, n), f"{n} is declared in include/nnb200.h but not exported"


def test_reference_abi_symbols_present():
    """The fifteen symbols of the reference's cuda/cuda_kernels.h:27-165."""
    ref = ["cuda_matmul", "cuda_matmul_with_handle", "cuda_batched_matmul", "cuda_elementwise_unary",
           "cuda_elementwise_binary", "cuda_elementwise_binary_scalar", "cuda_axpy",
           "cuda_elementwise_select_scalar_cond", "cuda_reduce_row", "cuda_reduce_col", "cuda_broadcast_row",
           "cuda_broadcast_col", "cuda_transpose", "cuda_rearrange_3d", "cuda_gather", "cuda_scatter_add"]
    names = declared_functions()
    for n in ref:
        assert n in names


def test_ctypes_table_covers_header():
    nnb = entry.load_package()
    from neuralnet_cpp_b200 import _lib
    assert set(declared_functions()) == set(_lib.SIGNATURES)


@pytest.mark.parametrize("act,norm,pos", [(0, 0, 0), (1, 1, 1), (1, 1, 2), (1, 0, 0)])
def test_param_table_matches_reference_order(act, norm, pos):
    """Shapes in the reference's parameter order (GPTModel::parameters) — compared with the oracle's
    list, which the reference harness verified tensor by tensor when the goldens were made."""
    nnb = entry.load_package()
    from oracle import gpt_oracle as go
    cfg = nnb.GptConfig(80, 32, 4, 3, 48, 16, 2, act, norm, pos, 0).c_struct()
    n = nnb.call("nnb200_gpt_param_table", C.byref(cfg), None, None, None)
    offs, rows, cols = (C.c_longlong * n)(), (C.c_int32 * n)(), (C.c_int32 * n)()
    nnb.call("nnb200_gpt_param_table", C.byref(cfg), offs, rows, cols)
    want = go.param_shapes(go.GptConfig(80, 32, 4, 3, 48, 16, 2, act, norm, pos))
    assert [(rows[i], cols[i]) for i in range(n)] == [(r, c) for _, r, c in want]
    spans = sorted((offs[i], offs[i] + rows[i] * cols[i]) for i in range(n))
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))          # tensors do not overlap
    assert spans[-1][1] <= nnb.call("nnb200_gpt_arena_elems", C.byref(cfg))
    assert all(o % 8 == 0 for o, _ in spans)                            # 16-byte aligned in bf16: TMA-safe


def test_invalid_config_is_rejected():
    nnb = entry.load_package()
    bad = nnb.GptConfig(80, 30, 4, 1, 48, 16, 2).c_struct()             # d_model not divisible by heads
    assert nnb.lib.nnb200_gpt_param_table(C.byref(bad), None, None, None) == -1
