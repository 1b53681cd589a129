"""CPU matmul micro-benchmark: the plain loop nest against the register-tiled one of the C++ host library
(the role of dev/cpu/matmul_forward.c in the reference), checked against torch.matmul.

    python -m llmc_b200.bench_cpu_matmul [--bt 256] [--c 768] [--oc 3072] [--threads 4]
"""
import argparse
import ctypes
import sys
import time

import torch

from . import _lib


def _fn(name):
    f = getattr(_lib.host(), name)
    f.restype = None
    f.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4
    return f


def matmul(kind, inp, weight, bias, threads=1):
    BT, C = inp.shape
    OC = weight.shape[0]
    out = torch.empty(BT, OC)
    _fn("llmc_cpu_matmul_" + kind)(out.data_ptr(), inp.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                                    BT, C, OC, threads)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--bt", type=int, default=256)
    ap.add_argument("--c", type=int, default=768)
    ap.add_argument("--oc", type=int, default=3072)
    ap.add_argument("--threads", type=int, default=4)
    ap.add_argument("--repeat", type=int, default=3)
    a = ap.parse_args(argv)
    g = torch.Generator().manual_seed(0)
    inp, w, b = torch.randn(a.bt, a.c, generator=g), torch.randn(a.oc, a.c, generator=g) * 0.02, torch.randn(a.oc, generator=g)
    ref = inp @ w.t() + b
    flops = 2.0 * a.bt * a.c * a.oc
    for kind in ("naive", "tiled"):
        best = float("inf")
        for _ in range(a.repeat):
            t0 = time.perf_counter()
            out = matmul(kind, inp, w, b, a.threads)
            best = min(best, time.perf_counter() - t0)
        err = (out - ref).abs().max().item()
        print("%-6s %8.2f ms  %7.2f GFLOP/s  max error %.2e" % (kind, best * 1e3, flops / best / 1e9, err))
    return 0


if __name__ == "__main__":
    sys.exit(main())
