"""The entry point that allocates nothing (infurnace_b200/csrc/linear_skinny_static.h).

Some callers of the few-rows product cannot ask CUDA for memory when they call it: a plug-in whose
host application owns all device memory through its own pool, or a serving loop in which
cudaMalloc's device-wide synchronisation is not allowed.  For them the library carries the
product's split-k scratch inside its own device image.  This test calls that entry point through
its exported C symbol, twice in a row with different inputs (the scratch keeps what the first call
left in it), and compares each result with the ordinary entry point's, which takes its scratch from
the caller, and with the plain statement of the product in float64, so that the test stands on its
own.  It runs last, so that a run that stops at the first failure has seen every other test.
"""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from infurnace_b200.kernels.build import load_library
    lib = load_library("linear_skinny_static")
    lib.ifb_linear_skinny_static.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    lib.ifb_linear_skinny_static.restype = c_int
    lib.ifb_linear_skinny_static_need.argtypes = [c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    lib.ifb_linear_skinny_static_need.restype = None
    return lib


@pytest.mark.parametrize("n,o,k,splits,epilogue,out_dtype", [(8, 4096, 1024, 4, 0, torch.bfloat16),
                                                            (3, 1000, 3072, 7, 1, torch.bfloat16),
                                                            (64, 1024, 2048, 5, 0, torch.float32),
                                                            (1, 333, 136, 1, 0, torch.float32)])
def test_static_scratch_entry_point_matches_the_ordinary_one(n, o, k, splits, epilogue, out_dtype):
    from infurnace_b200.kernels import load_cuda_kernels
    K = load_cuda_kernels()
    lib = _library()
    stream = torch.cuda.current_stream().cuda_stream
    code = 1 if out_dtype == torch.bfloat16 else 0
    g = torch.Generator().manual_seed(n * 7 + o)
    free_before = None
    for call in range(2):
        x = torch.randn((n, k), generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(((2 if epilogue else 1) * o, k), generator=g) * k ** -0.5).to(torch.bfloat16).cuda()
        want = torch.full((n, o), float("nan"), dtype=out_dtype, device="cuda")
        K._linear_skinny(x, w, want, n, o, k, epilogue, splits=splits)
        got = torch.full((n, o), float("nan"), dtype=out_dtype, device="cuda")
        torch.cuda.synchronize()
        if call == 1:
            free_before = torch.cuda.mem_get_info()[0]
        status = lib.ifb_linear_skinny_static(x.data_ptr(), w.data_ptr(), got.data_ptr(), code, n, o, k, epilogue, splits,
                                              stream)
        assert status == 0
        torch.cuda.synchronize()
        if call == 1:
            assert torch.cuda.mem_get_info()[0] >= free_before        # the second call took no device memory
        # the same kernel with the same split: the two agree to the last bit, which is well inside the
        # tolerance the kernel tests use against the plain product
        torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2 if out_dtype == torch.bfloat16 else 2e-4,
                                   atol=2e-3 if out_dtype == torch.bfloat16 else 1e-4)
        assert torch.equal(got, want)
        # and both are the product: against the plain statement in float64
        from kernel_refs import ReferenceKernels
        ref = torch.empty((n, o), dtype=torch.float64)
        ReferenceKernels(torch.float64).linear(x.cpu(), w.cpu(), ref, "silu_gate" if epilogue else "none")
        torch.testing.assert_close(got.cpu().double(), ref, rtol=1.6e-2 if out_dtype == torch.bfloat16 else 2e-4,
                                   atol=2e-3 if out_dtype == torch.bfloat16 else 1e-4)


def test_sizes_beyond_the_scratch_are_refused():
    lib = _library()
    floats, counters = ctypes.c_longlong(), ctypes.c_longlong()
    lib.ifb_linear_skinny_static_need(64, 151936, 0, 2, ctypes.byref(floats), ctypes.byref(counters))
    assert floats.value > (1 << 20)
    x = torch.zeros((64, 1024), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((151936, 1024), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((64, 151936), dtype=torch.float32, device="cuda")
    status = lib.ifb_linear_skinny_static(x.data_ptr(), w.data_ptr(), out.data_ptr(), 0, 64, 151936, 1024, 0, 2,
                                          torch.cuda.current_stream().cuda_stream)
    assert status == 2                                                 # IFB_ERR_SIZE: nothing was launched
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0
