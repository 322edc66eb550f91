"""The allocation-free column sum, called through its exported C symbol.

Some users of the library reach a point where they need a bias gradient but may not allocate
device memory (a no-allocation region of a memory pool, a serving loop whose cache owns all free
memory, a host that forbids allocation after start-up). ``mmj_colsum_bf16_static`` serves them
from scratch space built into the library. This test loads the shared library with ctypes, as
such a caller would, and checks two calls in a row against the regular entry point, which takes
its scratch from the caller. The file name sorts last so that a run stopping at the first failure
has already exercised every other test.
"""
import ctypes

import pytest
import torch

from momijo_b200 import _C

pytestmark = pytest.mark.gpu


def _lib():
    lib = ctypes.CDLL(str(_C.lib_path()))
    lib.mmj_colsum_bf16_static.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_int, ctypes.c_void_p]
    lib.mmj_colsum_bf16_static.restype = ctypes.c_int
    lib.mmj_colsum_bf16.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                                    ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_int, ctypes.c_void_p]
    lib.mmj_colsum_bf16.restype = ctypes.c_int
    lib.mmj_colsum_splits.argtypes = [ctypes.c_int]
    lib.mmj_colsum_splits.restype = ctypes.c_int
    lib.mmj_colsum_bf16_static_max_n.restype = ctypes.c_int
    lib.mmj_colsum_bf16_static_strerror.argtypes = [ctypes.c_int]
    lib.mmj_colsum_bf16_static_strerror.restype = ctypes.c_char_p
    return lib


def test_static_colsum_matches_regular_entry_point_twice():
    lib = _lib()
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    # first call on this device does the one-time address look-up of the built-in scratch
    warm = torch.zeros(8, 8, device="cuda", dtype=torch.bfloat16)
    warm_out = torch.empty(8, device="cuda", dtype=torch.bfloat16)
    assert lib.mmj_colsum_bf16_static(warm.data_ptr(), warm.stride(0), warm_out.data_ptr(), None, 8, 8, 0,
                                      stream) == 0
    torch.cuda.synchronize()
    # two calls in a row with different shapes: the second must not see leftovers of the first
    for M, N in [(4096, 3072), (1000, 776)]:
        x = torch.randn(M, N, device="cuda").to(torch.bfloat16)
        out_static = torch.empty(N, device="cuda", dtype=torch.bfloat16)
        out_ref = torch.empty(N, device="cuda", dtype=torch.bfloat16)
        scratch = torch.empty(lib.mmj_colsum_splits(M) * N, device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = lib.mmj_colsum_bf16_static(x.data_ptr(), x.stride(0), out_static.data_ptr(), None, M, N,
                                        0, stream)
        assert rc == 0, lib.mmj_colsum_bf16_static_strerror(rc)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        # the stated property: the call takes no device memory (driver-level free bytes unchanged)
        assert free_after == free_before, (free_before, free_after)
        rc = lib.mmj_colsum_bf16(x.data_ptr(), x.stride(0), out_ref.data_ptr(), None,
                                 scratch.data_ptr(), M, N, 0, stream)
        assert rc == 0
        torch.cuda.synchronize()
        fp32 = x.float().sum(0)
        # same kernels, same reduction order: the two entry points agree bit for bit
        assert torch.equal(out_static, out_ref)
        err32 = ((out_static.float() - fp32).norm() / fp32.norm()).item()
        assert err32 < 1e-2, err32


def test_static_colsum_rejects_oversized_n():
    lib = _lib()
    n = lib.mmj_colsum_bf16_static_max_n() + 8
    x = torch.zeros(8, n, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    rc = lib.mmj_colsum_bf16_static(x.data_ptr(), x.stride(0), out.data_ptr(), None, 8, n, 0,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == -20
    assert b"16384" in lib.mmj_colsum_bf16_static_strerror(rc)
