"""ctypes binding of libnnb200.so — the C ABI declared in include/nnb200.h.

The library is the product; there is no Python or CPU fallback.  Importing this module without
the built library raises, and every compute call raises on a non-zero status.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnnb200.so")


class NnbError(RuntimeError):
    """A C-ABI call returned a non-zero status (positive: cudaError_t, -1: argument error)."""


class GptConfigC(C.Structure):
    """struct nnb200_gpt_config (include/nnb200.h)."""
    _fields_ = [(n, C.c_int32) for n in ("vocab", "d_model", "heads", "layers", "d_ff", "seq", "batch", "act",
                                          "norm", "pos", "precision")] + [("reserved", C.c_int32 * 5)]


def _load():
    if not os.path.isfile(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C neuralnet.cpp_b200/csrc` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). There is no fallback path.")
    return C.CDLL(LIB_PATH)


lib = _load()

_p, _i, _u, _f, _ll, _sz = C.c_void_p, C.c_int, C.c_uint, C.c_float, C.c_longlong, C.c_size_t
_cfgp = C.POINTER(GptConfigC)

# name -> argument types; every function returns int unless listed in _RET
SIGNATURES = {
    "cuda_matmul": [_p, _p, _p, _sz, _sz, _sz, _sz, _i, _i, _p],
    "cuda_matmul_with_handle": [_p, _p, _p, _sz, _sz, _sz, _sz, _i, _i, _p],
    "nnb200_set_handle_stream": [_p],
    "cuda_batched_matmul": [_p, _p, _p, _sz, _sz, _sz, _sz, _u, _i, _i, _p],
    "cuda_elementwise_unary": [_p, _p, _u, _u, _p],
    "cuda_elementwise_binary": [_p, _p, _p, _u, _u, _p],
    "cuda_elementwise_binary_scalar": [_p, _p, _u, _u, _f, _i, _p],
    "cuda_axpy": [_p, _p, _p, _u, _f, _p],
    "cuda_elementwise_select_scalar_cond": [_p, _p, _p, _u, _u, _f, _f, _p],
    "cuda_reduce_row": [_p, _p, _u, _u, _u, _p],
    "cuda_reduce_col": [_p, _p, _u, _u, _u, _p],
    "cuda_broadcast_row": [_p, _p, _p, _u, _u, _u, _p],
    "cuda_broadcast_col": [_p, _p, _p, _u, _u, _u, _p],
    "cuda_transpose": [_p, _p, _u, _u, _p],
    "cuda_rearrange_3d": [_p, _p, _u, _u, _u, _u, _p],
    "cuda_gather": [_p, _p, _p, _u, _u, _u, _p],
    "cuda_scatter_add": [_p, _p, _p, _u, _u, _u, _p],
    "nnb200_gemm_bf16": [_p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _f, _p, _p, _i, _p],
    "nnb200_gemm_f32": [_p, _p, _p, _i, _i, _i, _ll, _ll, _ll, _i, _i, _f, _p, _p, _i, _p],
    "nnb200_gemm_status": [C.POINTER(C.c_int)],
    "nnb200_gemm_profile": [_i],
    "nnb200_gemm_profile_read": [C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_int)],
    "nnb200_gemm_profile_read_fused": [C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_int)],
    "nnb200_launch_count": [_i],
    "nnb200_attention_forward": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "nnb200_attention_backward": [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "nnb200_attention_backward_bias_partials": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p],
    "nnb200_attention_doc_ranges": [_p, _i, _i, _p, _p],
    "nnb200_muon_step_many": [_i, _p, _p, _p, _p, _p, _p, _f, _f, _i, _f, _i, _p, _sz, _i, _p, _p],
    "nnb200_gpt_decode_workspace_bytes": [_cfgp],
    "nnb200_gpt_decode_init": [_cfgp, _p, _p],
    "nnb200_gpt_forward_step": [_cfgp, _p, _p, _p, _i, _i, _i, _p, _p],
    "nnb200_gpt_forward_step_dev": [_cfgp, _p, _p, _p, _p, _p, _p],
    "nnb200_gpt_decode_set_step": [_p, _i, _i, _i, _p],
    "nnb200_ids_from_float": [_p, _p, _i, _i, _p],
    "nnb200_logits_to_reference": [_p, _p, _i, _i, _i, _p],
    "nnb200_zero_f32": [_p, _sz, _p],
    "nnb200_rt_timer_start": [],
    "nnb200_rt_timer_stop": [C.POINTER(C.c_float)],
    "nnb200_norm_forward": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p],
    "nnb200_norm_backward": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p],
    "nnb200_colsum_scratch_floats": [_i, _i],
    "nnb200_bias_grad": [_p, _ll, _p, _p, _i, _i, _i, _p],
    "nnb200_bias_grad_static": [_p, _ll, _p, _i, _i, _i, _p],
    "nnb200_activation_forward": [_p, _p, _i, _i, _i, _i, _p],
    "nnb200_linear_swiglu_supported": [_i, _i, _i],
    "nnb200_gemm_bf16_rowdot_supported": [_i, _i, _i, _i, _i],
    "nnb200_linear_swiglu_backward_supported": [_i, _i, _i],
    "nnb200_linear_swiglu_backward": [_p, _p, _p, _p, _i, _i, _i, _p, _p],
    "nnb200_gemm_bf16_rowdot": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p],
    "nnb200_linear_swiglu_forward": [_p, _p, _p, _p, _p, _i, _i, _i, _p],
    "nnb200_activation_backward": [_p, _p, _p, _i, _i, _i, _i, _p],
    "nnb200_cross_entropy": [_p, _p, _p, _f, _p, _p, _p, _i, _i, _i, _i, _p],
    "nnb200_embedding_forward": [_p, _p, _p, _p, _i, _i, _i, _i, _i, _p],
    "nnb200_embedding_backward": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p],
    "nnb200_embedding_scratch_bytes": [_i],
    "nnb200_adamw_step": [_p, _p, _p, _p, _p, _sz, _f, _f, _f, _f, _f, _i, _p, _p],
    "nnb200_grad_norm_clip": [_p, _sz, _f, _f, _p, _p, _p],
    "nnb200_sumsq_scratch_floats": [],
    "nnb200_muon_step": [_p, _p, _p, _p, _i, _i, _f, _f, _i, _f, _i, _p, _p, _p],
    "nnb200_muon_scratch_bytes": [_i, _i, _i],
    "nnb200_f32_to_bf16": [_p, _p, _sz, _p],
    "nnb200_bf16_to_f32": [_p, _p, _sz, _p],
    "nnb200_gpt_param_table": [_cfgp, C.POINTER(_ll), C.POINTER(C.c_int32), C.POINTER(C.c_int32)],
    "nnb200_gpt_arena_elems": [_cfgp],
    "nnb200_gpt_matrix_region_begin": [_cfgp],
    "nnb200_gpt_layer_matrix_begin": [_cfgp, _i],
    "nnb200_gpt_workspace_bytes": [_cfgp],
    "nnb200_gpt_workspace_offset": [_cfgp, _i],
    "nnb200_gpt_init_workspace": [_cfgp, _p, _p],
    "nnb200_gpt_forward": [_cfgp, _p, _p, _p, _p, _p, _p],
    "nnb200_gpt_loss": [_cfgp, _p, _p, _p, _f, _p],
    "nnb200_gpt_backward": [_cfgp, _p, _p, _p, _p, _p, _p, _p, _p],
    # engine primitives in the reference's layouts
    "nnb200_batched_matmul": [_p, _p, _p, _sz, _sz, _sz, _sz, _u, _i, _i, _f, _p],
    "nnb200_bmm_reduce": [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "nnb200_bmm_softmax_denom": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _p],
    "nnb200_bmm_softmax_apply": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _p],
    "nnb200_bmm_softmax_backward_q": [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _p],
    "nnb200_bmm_softmax_backward_kv": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _p],
    "nnb200_col_softmax_denom": [_p, _p, _p, _i, _i, _p],
    "nnb200_col_softmax_sparse_forward": [_p, _p, _p, _p, _p, _i, _i, _i, _f, _p],
    "nnb200_expr_reduce_axis": [_p],
    "nnb200_eval_expr_scratch_floats": [_i, _i],
    "nnb200_eval_expr": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _p],
    # device runtime of the C++ engine
    "nnb200_rt_init": [_i, _p, _sz, _p, _p],
    "nnb200_rt_device": [],
    "nnb200_rt_stream": [],
    "nnb200_rt_alloc": [_sz, _p],
    "nnb200_rt_free": [_p],
    "nnb200_rt_upload": [_p, _p, _sz],
    "nnb200_rt_download": [_p, _p, _sz],
    "nnb200_rt_copy": [_p, _p, _sz],
    "nnb200_rt_zero": [_p, _sz],
    "nnb200_rt_sync": [],
    "nnb200_gemm_pair_capacity": [],
    "nnb200_rope_table": [_i, _i, _p],
    "nnb200_rope_apply": [_p, _p, _i, _i, _i, _i, _ll, _i, _i, _p],
}
_RET = {
    "nnb200_launch_count": C.c_ulonglong,
    "nnb200_colsum_scratch_floats": _sz, "nnb200_embedding_scratch_bytes": _sz, "nnb200_sumsq_scratch_floats": _sz,
    "nnb200_muon_scratch_bytes": _sz, "nnb200_gpt_arena_elems": _ll, "nnb200_gpt_matrix_region_begin": _ll,
    "nnb200_gpt_layer_matrix_begin": _ll, "nnb200_gpt_workspace_bytes": _ll, "nnb200_gpt_workspace_offset": _ll,
    "nnb200_gpt_decode_workspace_bytes": _ll,
    "nnb200_eval_expr_scratch_floats": _sz, "nnb200_rt_stream": C.c_void_p,
}
# functions whose int return value is a count, not a status
_COUNT = {"nnb200_gpt_param_table"}
# functions that return a plain value (negative values are answers, not errors)
_VALUE = {"nnb200_gemm_pair_capacity", "nnb200_linear_swiglu_supported", "nnb200_gemm_bf16_rowdot_supported", "nnb200_linear_swiglu_backward_supported", "nnb200_expr_reduce_axis", "nnb200_rt_device", "nnb200_rt_stream"}

for _name, _args in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.argtypes = _args
    _fn.restype = _RET.get(_name, C.c_int)


def call(name, *args):
    """Calls a status-returning entry point and raises NnbError on failure."""
    rc = getattr(lib, name)(*args)
    if name in _VALUE:
        return rc
    if name in _RET or name in _COUNT:
        if rc < 0:
            raise NnbError(f"{name} rejected its arguments ({rc})")
        return rc
    if rc != 0:
        raise NnbError(f"{name} failed with status {rc}")
    return 0
