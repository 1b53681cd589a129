"""Failure detection on the device without faulting it: a wait on a peer flag that nobody ever raises must give up after
its limit, record ST_FLAG_TIMEOUT in the status word and leave the context usable."""
import ctypes

import pytest
import torch

from llmc_b200 import _lib
from llmc_b200.ops import kernels as KN
from llmc_b200.parallel import p2p

pytestmark = pytest.mark.gpu


def test_peer_flag_wait_times_out_and_reports():
    lib = p2p._cfg_lib()
    lib.llmc_p2p_set_wait_cycles.restype = ctypes.c_int
    lib.llmc_p2p_set_wait_cycles.argtypes = [ctypes.c_longlong]
    assert _lib.read_status() == 0
    sig = torch.zeros(lib.llmc_p2p_signal_words(), dtype=torch.int64, device="cuda")
    ptrs = p2p._ptr_array([sig.data_ptr(), sig.data_ptr()])       # a "two rank" group whose second rank never signals
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    try:
        assert lib.llmc_p2p_set_wait_cycles(400_000_000) == 0      # about a fifth of a second
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        assert lib.llmc_p2p_wait(ptrs, 0, 2, 0, 1, stream) == 0    # waits for sequence number 1 from both ranks
        t1.record()
        torch.cuda.synchronize()
        assert 20.0 < t0.elapsed_time(t1) < 5000.0
        status = _lib.read_status(clear=True)
        assert status >> 24 == 2, hex(status)                      # ST_FLAG_TIMEOUT
        assert (status & 0xFFF) in (0x740, 0x741)
    finally:
        lib.llmc_p2p_set_wait_cycles(0)
    # the context is intact: an ordinary kernel still runs and the status word is clean again
    x = torch.ones(8 * 1024, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(x)
    KN.residual_add(out, x, x)
    assert (out == 2).all()
    assert _lib.read_status() == 0
