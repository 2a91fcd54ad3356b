"""Helpers for the GPU parity tests: device buffers through torch, calls through the C ABI."""
import ctypes as C

import numpy as np
import torch

import __graft_entry__ as entry

nnb = entry.load_package()
call = nnb.call

# Device tensors made by dev() stay referenced until the test ends (tests/conftest.py clears the
# list): a temporary passed as `ptr(dev(x))` would otherwise be freed, and its memory handed to the
# next allocation, before the kernel that reads it has even been enqueued.
_keep = []


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    if dtype is not None:
        t = t.to(dtype)
    _keep.append(t)
    return t


def release():
    _keep.clear()


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def host(t):
    torch.cuda.synchronize()
    return t.detach().float().cpu().numpy() if t.dtype == torch.bfloat16 else t.detach().cpu().numpy()


def bf16_round(a):
    """fp32 array rounded to bf16 and back (what a bf16 kernel sees of an fp32 input)."""
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()


def gemm_status():
    code = C.c_int(0)
    call("nnb200_gemm_status", C.byref(code))
    return code.value
