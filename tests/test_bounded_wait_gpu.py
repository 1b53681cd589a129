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
        assert lib.llmc_p2p_wait(ptrs, 0, 2, 0, 0, 1, stream) == 0    # waits for sequence number 1 of group 0 from both ranks
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


class _NeverReady:
    """Flags of an all-gather that never completes (nobody raises them)."""

    def __init__(self, flags, n):
        self.flags_ptr, self.n, self.seq = flags.data_ptr(), n, 1

    def wait(self):
        raise AssertionError("the two-SM kernel polls inside the kernel")


def test_gemm_waiting_for_gathered_weights_gives_up_and_reports(monkeypatch):
    """The GEMM that consumes an all-gather polls the peers' flags inside the kernel; with flags that never rise every CTA gives up
    after the limit, nothing is loaded or stored, the status word says where, and the next GEMM runs normally."""
    lib = p2p._cfg_lib()
    lib.llmc_p2p_set_wait_cycles.restype = ctypes.c_int
    lib.llmc_p2p_set_wait_cycles.argtypes = [ctypes.c_longlong]
    monkeypatch.setattr(KN, "TWO_SM_MIN_TILES", 1)
    assert _lib.read_status() == 0
    M, N, K_ = 512, 512, 256
    g = torch.Generator().manual_seed(0)
    a = torch.randn(M, K_, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K_, generator=g) * 0.05).to(torch.bfloat16).cuda()
    out = torch.full((M, N), 3.0, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(8, dtype=torch.int64, device="cuda")
    try:
        assert lib.llmc_p2p_set_wait_cycles(300_000_000) == 0
        KN.matmul_forward(out, a, w, None, ready=_NeverReady(flags, 2))
        torch.cuda.synchronize()
        status = _lib.read_status(clear=True)
        assert status >> 24 == 2, hex(status)                      # ST_FLAG_TIMEOUT
        assert (status & 0xFF0) == 0x9F0, hex(status)
        assert (out == 3.0).all()                                  # nothing was written
    finally:
        lib.llmc_p2p_set_wait_cycles(0)
    # flags that are already up: the same entry point computes the product
    flags.fill_(1)
    KN.matmul_forward(out, a, w, None, ready=_NeverReady(flags, 2))
    ref = a.float() @ w.float().t()
    assert (out.float() - ref).abs().max().item() < 0.05 + 0.02 * ref.abs().max().item()
    assert _lib.read_status() == 0
