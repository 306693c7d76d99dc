"""The matrix product for callers that cannot allocate device memory.

Some users of the kernel library run where cudaMalloc is not theirs to call: inside another
program's process with a fixed memory budget, or in a loop that must never take the allocator's
locks.  For them the library exports srlm_gemm_tn_tcgen05_static, whose split-K scratch is a
device array inside the library itself.  This test calls it through its exported C symbol (not
through the Python wrapper), twice in a row, and compares it with the entry point that takes a
workspace.  It is collected last so that a run that stops at the first failure has run every
other test before it.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_BYTES = 65536 + (8 << 20)


def library():
    from safetyraise_lmengine_b200.csrc.build import build_kernels
    lib = C.CDLL(build_kernels())
    lib.srlm_last_error.restype = C.c_char_p
    return lib


def call_static(lib, a, w, out, splits):
    flag = C.c_int(-1)
    status = lib.srlm_gemm_tn_tcgen05_static(
        C.c_void_p(a.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(out.data_ptr()),
        C.c_int(0 if out.dtype == torch.float32 else 1), C.c_int(a.shape[0]), C.c_int(w.shape[0]),
        C.c_int(a.shape[1]), C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)), C.c_longlong(out.stride(0)),
        C.c_int(splits), C.byref(flag), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return status, flag.value


@pytest.mark.parametrize("M, N, K, splits, odt", [(8, 4096, 4096, 4, torch.bfloat16), (33, 640, 1024, 3, torch.float32),
                                                  (64, 2560, 2048, 1, torch.bfloat16)])
def test_static_scratch_gemm_matches_the_workspace_one(M, N, K, splits, odt):
    from safetyraise_lmengine_b200.kernels import ops
    lib = library()
    g = torch.Generator(device=DEV).manual_seed(M + N)
    a = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device=DEV, generator=g).to(torch.bfloat16)
    want = torch.empty(M, N, device=DEV, dtype=odt)
    ops.gemm_tn_tcgen05(a, w, want, splits=splits)
    assert ops.gemm_error_flag(a.device) == 0
    ref = a.double() @ w.double().T
    tol = dict(rtol=1e-4, atol=2e-4 * math.sqrt(K)) if odt == torch.float32 else dict(rtol=1e-2, atol=1e-2 * math.sqrt(K))
    mem_before = torch.cuda.memory_allocated()
    for _ in range(2):                                   # the second call meets the first one's leftovers
        got = torch.full((M, N), float("nan"), device=DEV, dtype=odt)
        status, flag = call_static(lib, a, w, got, splits)
        assert status == 0, lib.srlm_last_error().decode()
        assert flag == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)                   # same kernel, same order of sums
        assert torch.allclose(got.double(), ref, **tol)
        del got
    assert torch.cuda.memory_allocated() == mem_before


def test_static_scratch_gemm_refuses_what_does_not_fit():
    lib = library()
    M, N, K, splits = 64, 24576, 4096, 4                # 4 * 64 * 24576 * 4 bytes = 25 MB of partial sums
    assert 65536 + splits * M * N * 4 > SCRATCH_BYTES
    a = torch.zeros(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(N, K, device=DEV, dtype=torch.bfloat16)
    out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    status, _ = call_static(lib, a, w, out, splits)
    assert status < 0 and b"scratch" in lib.srlm_last_error()
    torch.cuda.synchronize()
    assert torch.all(out == 7.0)                         # nothing ran
    status, flag = call_static(lib, a, w, out, 1)        # without split-K it needs no scratch at all
    assert status == 0 and flag == 0 and torch.all(out == 0)
