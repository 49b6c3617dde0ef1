"""The allocation-free column-sum entry point, called through its exported C symbol exactly as
a C host would: two calls in a row must match the regular entry point (which is given caller
scratch), and an oversized problem must be refused with a message instead of touching memory.
Collected last so that a run that stops at the first failure has already run everything else."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from kharon_b200 import _native
    lib = C.CDLL(str(_native.cuda_lib_path()))     # plain dlopen + symbol lookup, no Python wrapper
    lib.kh_colsum_noalloc.restype = C.c_int
    lib.kh_colsum_noalloc.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.kh_colsum.restype = C.c_int
    lib.kh_colsum.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.kh_colsum_scratch_elems.restype = C.c_long
    lib.kh_colsum_scratch_elems.argtypes = [C.c_int, C.c_int]
    lib.kh_cuda_last_error.restype = C.c_char_p
    return lib


def test_noalloc_colsum_matches_regular_entry_point_twice():
    lib = _lib()
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    st = torch.cuda.current_stream().cuda_stream
    for rows, N in [(4096, 2048), (777, 328)]:          # the second call reuses the array after a different shape
        x = torch.randn(rows, N, device=dev).bfloat16()
        want = torch.full((N,), 0.5, device=dev)
        scratch = torch.zeros(lib.kh_colsum_scratch_elems(rows, N), device=dev)
        assert lib.kh_colsum(x.data_ptr(), x.stride(0), want.data_ptr(), scratch.data_ptr(), rows, N, 1, st) == 0
        for _ in range(2):
            got = torch.full((N,), 0.5, device=dev)
            before = torch.cuda.memory_allocated(dev)
            rc = lib.kh_colsum_noalloc(x.data_ptr(), x.stride(0), got.data_ptr(), rows, N, 1, st)
            assert rc == 0, lib.kh_cuda_last_error()
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated(dev) == before
            ref = 0.5 + x.float().sum(0)
            assert torch.equal(got, want)                 # same kernel, same order: same bits
            assert ((got - ref).norm() / ref.norm()).item() < 1e-5


def test_noalloc_colsum_rejects_oversized_problem():
    lib = _lib()
    dev = torch.device("cuda", 0)
    x = torch.zeros(64, 8, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(8, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    # claimed shape needs more partial floats than the built-in array holds: refused before any launch
    rc = lib.kh_colsum_noalloc(x.data_ptr(), 70000, out.data_ptr(), 1 << 20, 69000, 0, st)
    assert rc == -1
    assert b"built-in scratch" in lib.kh_cuda_last_error() or b"exceeds" in lib.kh_cuda_last_error()
