"""The matrix product's no-allocation entry point, called through its exported C symbol.

Collected last on purpose: if it fails, a run that stops at the first failure has already
run everything else. It builds its own inputs and loads the library itself, so it passes
alone in a fresh process as well as after the other tests.
"""

from __future__ import annotations

import ctypes
import math
from ctypes import c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def library():
    from llm_inference_b200.csrc import build

    lib = ctypes.CDLL(str(build.build_kernels()))
    lib.b200_last_error.restype = ctypes.c_char_p
    lib.b200_skinny_gemm_static.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    lib.b200_skinny_gemm_static.restype = c_int
    lib.b200_skinny_gemm_static_capacity_floats.restype = ctypes.c_longlong
    lib.b200_skinny_gemm.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_int, c_void_p]
    lib.b200_skinny_gemm.restype = c_int
    lib.b200_skinny_gemm_scratch.argtypes = [c_int, c_int, c_int, ctypes.POINTER(c_int64), ctypes.POINTER(c_int)]
    lib.b200_skinny_gemm_scratch.restype = None
    return lib


def existing_entry_point(lib, w, x, out, epilogue):
    """The entry point whose scratch the caller allocates (here: with torch)."""
    m, k = x.shape
    n = w.shape[0]
    floats, counters = c_int64(0), c_int(0)
    lib.b200_skinny_gemm_scratch(m, n, k, ctypes.byref(floats), ctypes.byref(counters))
    scratch = torch.empty(max(floats.value, 1), dtype=torch.float32, device="cuda")
    counter = torch.zeros(max(counters.value, 1), dtype=torch.int32, device="cuda")
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    status = lib.b200_skinny_gemm(
        c_void_p(w.data_ptr()), c_void_p(x.data_ptr()), c_void_p(out.data_ptr()), m, n, k, epilogue,
        c_void_p(scratch.data_ptr()), c_int64(scratch.numel()), c_void_p(counter.data_ptr()), counter.numel(), stream,
    )
    assert status == 0, lib.b200_last_error().decode()
    return floats.value


@pytest.mark.parametrize("m,n,k,epilogue", [(8, 1536, 8960, 0), (13, 1024, 4096, 1), (5, 2048, 1536, 2)])
def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row(library, m, n, k, epilogue):
    lib = library
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    out_dtype = torch.float32 if epilogue == 1 else torch.bfloat16
    out_cols = n // 2 if epilogue == 2 else n
    used_scratch = 0
    for call in range(2):  # the second call finds the first call's leftovers in the shared array
        torch.manual_seed(100 * call + m)
        x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") / math.sqrt(k)).to(torch.bfloat16)
        want = torch.full((m, out_cols), float("nan"), device="cuda", dtype=out_dtype)
        used_scratch = existing_entry_point(lib, w, x, want, epilogue)
        got = torch.full((m, out_cols), float("nan"), device="cuda", dtype=out_dtype)
        status = lib.b200_skinny_gemm_static(
            c_void_p(w.data_ptr()), c_void_p(x.data_ptr()), c_void_p(got.data_ptr()), m, n, k, epilogue, stream
        )
        assert status == 0, lib.b200_last_error().decode()
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        # Same plan, same order of additions: in fact the two agree to the last bit.
        assert torch.equal(got, want)
        reference = x.double() @ w.double().T
        if epilogue == 2:
            g, u = reference[:, 0::2], reference[:, 1::2]
            reference = g / (1 + torch.exp(-g)) * u
        torch.testing.assert_close(got.double(), reference, atol=2e-2, rtol=2e-2)
    if (m, n, k) == (8, 1536, 8960):
        assert used_scratch > 0  # this shape really goes through the scratch memory


def test_static_scratch_entry_point_refuses_what_does_not_fit(library):
    lib = library
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    m, n, k = 16, 4400, 18944
    floats, counters = c_int64(0), c_int(0)
    lib.b200_skinny_gemm_scratch(m, n, k, ctypes.byref(floats), ctypes.byref(counters))
    assert floats.value > lib.b200_skinny_gemm_static_capacity_floats()
    x = torch.zeros(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(n, k, device="cuda", dtype=torch.bfloat16)
    out = torch.full((m, n), 7.0, device="cuda", dtype=torch.bfloat16)
    status = lib.b200_skinny_gemm_static(c_void_p(w.data_ptr()), c_void_p(x.data_ptr()), c_void_p(out.data_ptr()), m, n, k, 0, stream)
    message = lib.b200_last_error().decode()
    assert status != 0 and "static scratch holds" in message and str(floats.value) in message
    torch.cuda.synchronize()
    assert torch.all(out == 7.0)  # nothing was launched
    # More rows than the kernel takes is refused as well.
    status = lib.b200_skinny_gemm_static(c_void_p(w.data_ptr()), c_void_p(x.data_ptr()), c_void_p(out.data_ptr()), 17, n, k, 0, stream)
    assert status != 0 and "unsupported shape" in lib.b200_last_error().decode()
