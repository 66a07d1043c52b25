"""The allocation-free linear entry point, called the way a C program would call it.

Some users of the kernel library cannot allocate device memory: a plug-in inside
a serving process that has already given all free memory to its KV cache, or a
plain C host without a tensor library. ``ab200_linear_bf16_noalloc`` serves them
from a scratch array built into the library instead of a caller-supplied
workspace. This test reaches it through its exported C symbol (ctypes, raw
pointers, no wrapper from the package), compares it with the regular entry point
on two calls in a row that share the built-in scratch, and checks that an
oversized problem is refused with a readable reason.

The file name sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""

import ctypes
import math
from ctypes import c_int, c_longlong, c_size_t, c_void_p, c_char_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from arcticinference_b200 import build
    lib = ctypes.CDLL(str(build.build_kernels()))
    P, I, LL, SZ = c_void_p, c_int, c_longlong, c_size_t
    lib.ab200_linear_bf16_noalloc.restype = I
    lib.ab200_linear_bf16_noalloc.argtypes = [P, LL, P, LL, P, LL, I, I, I, P, P, LL, I, I, P, P]
    lib.ab200_linear_bf16.restype = I
    lib.ab200_linear_bf16.argtypes = [P, LL, P, LL, P, LL, I, I, I, P, P, LL, I, P, SZ, I, P, P]
    lib.ab200_linear_bf16_noalloc_fits.restype = I
    lib.ab200_linear_bf16_noalloc_fits.argtypes = [I, I, I]
    lib.ab200_noalloc_last_error.restype = c_char_p
    lib.ab200_noalloc_last_error.argtypes = []
    return lib


def _case(M, N, K, seed):
    g = torch.Generator(device="cuda:0").manual_seed(seed)
    x = torch.randn(M, K, device="cuda:0", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda:0", generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = torch.randn(N, device="cuda:0", generator=g).to(torch.bfloat16)
    r = torch.randn(M, N, device="cuda:0", generator=g).to(torch.bfloat16)
    return x, w, b, r


def test_noalloc_linear_matches_regular_entry_point():
    torch.cuda.set_device(0)
    lib = _lib()
    status = torch.zeros(8, dtype=torch.int32, device="cuda:0")
    workspace = torch.empty(32 << 20, dtype=torch.uint8, device="cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second reuses the scratch the first dirtied
    for seed, (M, N, K, splits) in enumerate([(24, 1024, 4096, 4), (7, 2048, 2048, 0)]):
        x, w, b, r = _case(M, N, K, seed)
        out_new = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda:0")
        out_old = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda:0")
        assert lib.ab200_linear_bf16_noalloc_fits(M, N, K) == 1
        rc = lib.ab200_linear_bf16_noalloc(
            x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out_new.data_ptr(),
            out_new.stride(0), M, N, K, b.data_ptr(), r.data_ptr(), r.stride(0), 0, splits,
            status.data_ptr(), stream)
        assert rc == 0, lib.ab200_noalloc_last_error()
        rc = lib.ab200_linear_bf16(
            x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out_old.data_ptr(),
            out_old.stride(0), M, N, K, b.data_ptr(), r.data_ptr(), r.stride(0), 0,
            workspace.data_ptr(), workspace.numel(), splits, status.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0
        ref = (x.float() @ w.float().t() + b.float() + r.float())
        err = (out_new.float() - out_old.float()).abs()
        tol = 4e-2 + 2e-2 * out_old.float().abs()
        assert bool((err <= tol).all()), float(err.max())
        err_ref = (out_new.float() - ref).abs()
        assert bool((err_ref <= 4e-2 + 2e-2 * ref.abs()).all()), float(err_ref.max())


def test_noalloc_linear_refuses_oversized_problem():
    torch.cuda.set_device(0)
    lib = _lib()
    M, N, K = 256, 65536, 64   # worst-case scratch 8*M*N*4 bytes = 512 MiB > built-in 32 MiB
    assert lib.ab200_linear_bf16_noalloc_fits(M, N, K) == 0
    x = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda:0")
    w = torch.zeros(8, K, dtype=torch.bfloat16, device="cuda:0")  # never read: the call is refused
    out = torch.zeros(8, dtype=torch.bfloat16, device="cuda:0")
    rc = lib.ab200_linear_bf16_noalloc(x.data_ptr(), K, w.data_ptr(), K, out.data_ptr(), N, M, N, K,
                                       None, None, 0, 0, 0, None,
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == -6
    assert b"scratch" in lib.ab200_noalloc_last_error()
