"""The allocation-free column sum (csrc/kernels/no_alloc_api.h), called through its exported C
symbol the way a non-Python caller would, must agree with the scratch-taking entry point.

Some callers of this library cannot allocate device memory (a callback running where the
framework's allocator must not be touched, a process with a fixed memory budget), so the
variant keeps its scratch inside the library image. Two calls in a row check that the shared
scratch, which keeps the previous call's contents, does not leak into the next result.
This file is collected near the end so that a failure here hides as few other tests as possible.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_colsum_no_alloc_matches_scratch_entry_point(cuda):
    from coccl_b200 import _lib
    lib = _lib.lib()
    fn = lib.cocclkColSumNoAlloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    err = lib.cocclkNoAllocLastError
    err.restype = C.c_char_p
    stream = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(11)
    for call, (M, N) in enumerate([(1000, 4096), (333, 1024)]):   # second call is smaller: stale scratch beyond it
        x = torch.randn(M, N, device=cuda, dtype=torch.bfloat16)
        ref = torch.zeros(N, device=cuda)
        sc = torch.empty(lib.cocclkColSumBlocks(M) * N, device=cuda)
        assert lib.cocclkColSum(x.data_ptr(), ref.data_ptr(), 0, sc.data_ptr(), M, N, stream) == 0
        out = torch.full((N,), 7.0, device=cuda)
        before = torch.cuda.memory_allocated()
        rc = fn(x.data_ptr(), out.data_ptr(), 0, M, N, stream)
        assert rc == 0, err().decode()
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert torch.allclose(out, ref, atol=1e-5, rtol=1e-5), (call, (out - ref).abs().max().item())
        assert torch.allclose(out, x.float().sum(0), atol=2e-2, rtol=2e-2)
        # accumulate mode adds to what is there
        rc = fn(x.data_ptr(), out.data_ptr(), 1, M, N, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(out, 2 * ref, atol=1e-4, rtol=1e-5)
    # sizes beyond the built-in scratch are refused with a message, nothing is launched
    big = torch.zeros(8, 16384 + 8, device=cuda, dtype=torch.bfloat16)
    o = torch.zeros(16384 + 8, device=cuda)
    assert fn(big.data_ptr(), o.data_ptr(), 0, 8, 16384 + 8, stream) == -2
    assert b"exceeds" in err()
    assert fn(big.data_ptr(), o.data_ptr(), 0, 8, 12, stream) == -1
