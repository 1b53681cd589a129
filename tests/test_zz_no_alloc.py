"""The allocation-free bias gradient (csrc/bias_grad_noalloc.h) against the ordinary entry point.

Some users of the library cannot allocate device memory where they call it: inside a stream capture, under a fully
committed memory budget, or in a host that must stay off the allocator lock.  For them ``llmc_bias_grad_noalloc``
keeps its scratch in a fixed array inside the library.  This test calls the exported C symbol directly, twice in a
row (the second call finds the first call's partial sums still in the array), and compares with ``llmc_bias_grad``.
It lives in its own file, collected last, so a failure here cannot hide another test's result.
"""
import ctypes

import pytest
import torch

from llmc_b200 import _lib
from llmc_b200.ops import kernels as KN

pytestmark = pytest.mark.gpu


def _noalloc():
    lib = _lib.cuda()
    fn = lib.llmc_bias_grad_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return fn


def test_noalloc_bias_grad_matches_and_repeats():
    fn = _noalloc()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator().manual_seed(5)
    # two different shapes back to back: the second call must not be disturbed by what the first left in the scratch
    for rows, OC, acc in [(1000, 776, 1), (4096, 3072, 0)]:
        dout = torch.randn(rows, OC, generator=g).to(torch.bfloat16).cuda()
        db0 = torch.randn(OC, generator=g).to(torch.bfloat16).cuda()
        want = db0.clone()
        KN.bias_grad(want, dout, accumulate=bool(acc))
        got = db0.clone()
        rc = fn(got.data_ptr(), dout.data_ptr(), rows, OC, acc, stream)
        assert rc == 0
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs()
        tol = 5e-2 + 1e-2 * want.float().abs()
        assert (err <= tol).all(), "max err %g" % err.max().item()
        # and the same call again gives the same bits
        again = db0.clone()
        assert fn(again.data_ptr(), dout.data_ptr(), rows, OC, acc, stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(again, got)


def test_noalloc_bias_grad_rejects_oversize():
    fn = _noalloc()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    x = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    assert fn(x.data_ptr(), x.data_ptr(), 1, (1 << 20) + 8, 0, stream) == -1      # wider than the built-in scratch
    assert fn(x.data_ptr(), x.data_ptr(), 1, 12, 0, stream) == -1                 # not a multiple of 8
    wide = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    assert fn(x.data_ptr(), wide.data_ptr() + 2, 1, 8, 0, stream) == -1           # dout not aligned to 16 bytes: refused before any launch
    assert fn(x.data_ptr(), None, 1, 8, 0, stream) == -1                          # null pointer
    torch.cuda.synchronize()
