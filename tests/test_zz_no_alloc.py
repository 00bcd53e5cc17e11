"""psb_reduce_sum_static — the entry point for callers that cannot allocate device memory.

Some users of the kernel library run where cudaMalloc is off limits: inside a host application
that owns all of HBM, in a latency-critical loop, or from plain C with no allocator to borrow
from.  For them the library exports one reduction whose scratch space is a fixed array inside
the library itself.  This test calls it through its exported C symbol (ctypes, no Python
wrapper) and checks, on two calls in a row with different inputs, that it returns what the
ordinary entry point psb_reduce_sum returns with caller-provided scratch.  It is collected
last so that a run stopping at the first failure has already exercised everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from parameter_server_b200.ops._native import lib as kernels_lib

    lib = kernels_lib()             # builds the library first when it is missing or out of date
    lib.psb_reduce_sum_static.restype = C.c_int
    lib.psb_reduce_sum_static.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p]
    return lib


def test_static_scratch_reduction_matches_regular_entry_point():
    from parameter_server_b200.ops.reduce import reduce_sum

    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device=dev).manual_seed(11)
    out = torch.zeros(1, dtype=torch.float64, device=dev)
    cases = [(3_000_001, 0, "sum_log1p_inv"), (123_457, 3, "sum_logistic")]
    for n, op, name in cases:                       # two calls in a row share the built-in scratch
        x = torch.randn(n, generator=g, device=dev)
        if op == 0:
            x = torch.exp(x)
        rc = lib.psb_reduce_sum_static(x.data_ptr(), n, op, out.data_ptr(), stream)
        assert rc == 0
        got = out.item()
        want = reduce_sum(x, name).item()
        assert got == pytest.approx(want, rel=1e-9)
        ref = (torch.log1p(1 / x.double()) if op == 0 else torch.nn.functional.softplus(-x.double())).sum().item()
        assert got == pytest.approx(ref, rel=1e-9)


def test_static_scratch_reduction_rejects_oversized_input():
    lib = _lib()
    out = torch.zeros(1, dtype=torch.float64, device="cuda")
    x = torch.zeros(8, device="cuda")
    rc = lib.psb_reduce_sum_static(x.data_ptr(), (1 << 31) + 1, 0, out.data_ptr(), None)
    assert rc != 0   # refused before any launch; nothing was read
    torch.cuda.synchronize()
