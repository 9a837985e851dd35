"""The matrix product that allocates nothing (`plm_gemm_tc_static`), called the way its users call it:
through the exported C symbol of the kernel library, with nothing but input and output pointers.

Its users are programs that cannot ask for device memory when they need the product (their memory
was planned and handed out at start-up, or they run inside somebody else's budget), so the partial
sums of the split-K product live in an array inside the library.  The test checks that the result is
the one of the ordinary entry point (which takes a caller-allocated workspace), twice in a row,
because the second call finds the first call's partial sums still in the array, and that a problem
too large for the array is refused in words instead of being run.

The file's name makes pytest collect it last: if it fails, a run that stops at the first failure has
run everything else before.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _symbols():
    from picolm_b200.csrc.build import load_library
    lib = load_library("gemm_tc")
    vp, i, l = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
    lib.plm_gemm_tc_static.argtypes = [vp, vp, vp, i, i, i, i, l, l, l, vp, vp]
    lib.plm_gemm_tc_static.restype = i
    lib.plm_gemm_tc_static_strerror.argtypes = [i]
    lib.plm_gemm_tc_static_strerror.restype = ctypes.c_char_p
    return lib


@pytest.mark.parametrize("T,F,K,out_dtype", [(8, 3072, 2048, torch.bfloat16), (33, 264, 1024, torch.float32),
                                              (64, 2048, 8192, torch.float32), (1, 4096, 512, torch.bfloat16)])
def test_static_scratch_entry_matches_the_ordinary_one_twice(T, F, K, out_dtype):
    from util import gemm_tc_workspace
    lib = _symbols()
    torch.manual_seed(T + F + K)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # set-up call: looks up the scratch array's address on this device, launches nothing
    assert lib.plm_gemm_tc_static(None, None, None, 0, 0, 0, 0, 0, 0, 0, None, stream) == 0
    code = 0 if out_dtype == torch.float32 else 1
    for round_ in range(2):                                # the second call inherits the first one's partial sums
        x = (torch.randn(T, K) / K ** 0.25).to(torch.bfloat16).to(DEV)
        w = (torch.randn(F, K) / K ** 0.25).to(torch.bfloat16).to(DEV)
        want = gemm_tc_workspace(x, w, out_dtype)          # the existing entry point, workspace from torch
        got = torch.full((T, F), float("nan"), dtype=out_dtype, device=DEV)
        before = torch.cuda.memory_allocated()
        rc = lib.plm_gemm_tc_static(x.data_ptr(), w.data_ptr(), got.data_ptr(), code, T, F, K, K, K, F, None, stream)
        assert rc == 0, lib.plm_gemm_tc_static_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # same kernels, same split of K, same order of the partial sums: the same numbers
        assert torch.equal(got, want), f"call {round_}: max |diff| {(got.float() - want.float()).abs().max().item()}"
        ref = x.double().cpu() @ w.double().cpu().t()
        tol = dict(atol=2e-3, rtol=1e-4) if out_dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
        assert torch.allclose(got.double().cpu(), ref, **tol)


def test_static_scratch_entry_refuses_what_does_not_fit():
    lib = _symbols()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    T, F, K = 64, 37760, 512                               # two splits of 64 x 37760 partial sums: 4.6 Mi floats > 4 Mi
    x = torch.zeros(T, K, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(F, K, dtype=torch.bfloat16, device=DEV)
    out = torch.full((T, F), 7.0, dtype=torch.float32, device=DEV)
    rc = lib.plm_gemm_tc_static(x.data_ptr(), w.data_ptr(), out.data_ptr(), 0, T, F, K, K, K, F, None, stream)
    assert rc == -6
    assert b"exceed" in lib.plm_gemm_tc_static_strerror(rc)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())                        # refused before anything ran
    rc = lib.plm_gemm_tc_static(x.data_ptr(), w.data_ptr(), out.data_ptr(), 5, T, 128, K, K, K, 128, None, stream)
    assert rc == -1 and b"element type" in lib.plm_gemm_tc_static_strerror(rc)
