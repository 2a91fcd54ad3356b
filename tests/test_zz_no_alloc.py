"""The scratch-free bias-gradient entry point (nnb200_bias_grad_static) against the entry point that
takes caller scratch, through the C ABI.  It exists for hosts that cannot allocate device memory
for a kernel's workspace — the reference's CudaBackend only allocates op outputs, and services with
a fixed memory budget must not call cudaMalloc mid-run.  The two calls in a row check that what the
first call left in the shared built-in buffer does not leak into the second.
This file is named to be collected last."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [0, 1])
def test_static_scratch_matches_caller_scratch_twice(dtype):
    import torch
    from tests import gpu_util as g
    r = np.random.default_rng(12)
    tdt = torch.bfloat16 if dtype else torch.float32
    warm = torch.zeros(256, 64, dtype=tdt, device="cuda")
    warm_out = torch.zeros(64, device="cuda")
    # the first call on a device looks the built-in buffer's address up and loads the kernels: keep that out of the count
    g.call("nnb200_bias_grad_static", g.ptr(warm), 64, g.ptr(warm_out), 256, 64, dtype, g.stream())
    torch.cuda.synchronize()
    for rows, cols in ((3000, 777), (515, 96)):            # second call is smaller: stale partials stay behind
        gy = r.standard_normal((rows, cols)).astype(np.float32)
        t = g.dev(gy, tdt)
        base = r.standard_normal(cols).astype(np.float32)
        want, got = g.dev(base.copy()), g.dev(base.copy())
        scratch = torch.zeros(int(g.call("nnb200_colsum_scratch_floats", rows, cols)), device="cuda")
        g.call("nnb200_bias_grad", g.ptr(t), cols, g.ptr(want), g.ptr(scratch), rows, cols, dtype, g.stream())
        # free bytes of the device as the driver sees them: a cudaMalloc inside the library (which torch's own
        # counters would not see) would lower it
        torch.cuda.synchronize()
        before = torch.cuda.mem_get_info()[0]
        g.call("nnb200_bias_grad_static", g.ptr(t), cols, g.ptr(got), rows, cols, dtype, g.stream())
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] >= before
        assert np.array_equal(g.host(got), g.host(want))     # same kernels, same order: bit-identical
        ref = base + g.host(t).astype(np.float64).sum(axis=0)
        assert np.allclose(g.host(got), ref, atol=1e-3)


def test_static_scratch_rejects_oversize():
    import torch
    from tests import gpu_util as g
    t = torch.zeros(8, device="cuda")
    rc = g.nnb.lib.nnb200_bias_grad_static(g.ptr(t), 1 << 20, g.ptr(t), 1 << 20, 4096, 0, g.stream())
    assert rc == -1
    # a row stride shorter than a row would sum overlapping rows: rejected
    assert g.nnb.lib.nnb200_bias_grad_static(g.ptr(t), 2, g.ptr(t), 2, 4, 0, g.stream()) == -1
