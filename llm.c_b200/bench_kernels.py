"""Kernel-versus-library micro-benchmarks on one GPU: every tensor-core kernel of this library next to the library kernel the
reference would call for the same operation (the role of the cuBLASLt / cuDNN arms in the reference's dev/cuda/matmul_forward.cu
and dev/cuda/attention_forward.cu benchmark mains).

    python -m llmc_b200.bench_kernels gemm        # forward / dgrad / wgrad of the GPT-2 124M shapes against torch.matmul (cuBLAS)
    python -m llmc_b200.bench_kernels attention   # flash attention forward / backward against torch SDPA (flash and cuDNN backends)
    python -m llmc_b200.bench_kernels all

Timing: CUDA events around each call on the launching stream, median of `--iters` runs after `--warmup` runs, a 256 MiB buffer
written between runs to flush the L2.  Library kernels only ever see tensors of this GPU.  Output is a plain table; fractions
are of the bf16 matmul peak given by --peak-tflops (default: the measured burst figure of this machine class, 1656).
"""
import argparse
import sys

import torch
import torch.nn.functional as F

from .ops import kernels as K

DEV = "cuda"


def timeit(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def row(out, what, shape, flops, t_ours, t_lib, lib, peak):
    tf_o, tf_l = flops / t_ours / 1e9, flops / t_lib / 1e9 if t_lib else 0.0
    print("%-10s %-28s ours %8.3f ms %7.0f TFLOP/s (%.2f of peak) | %-14s %8.3f ms %7.0f TFLOP/s | ours/lib speed %.2f"
          % (what, shape, t_ours, tf_o, tf_o / peak, lib, t_lib, tf_l, (t_lib / t_ours) if t_lib else float("nan")), file=out, flush=True)


def bench_gemm(a, out=sys.stdout):
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=DEV)
    M = a.tokens
    shapes = [("qkv", M, 2304, 768), ("attproj", M, 768, 768), ("fc", M, 3072, 768), ("fcproj", M, 768, 3072), ("lmhead", M, 50304, 768)]
    for name, M_, N, Kd in shapes:
        x = torch.randn(M_, Kd, device=DEV, dtype=torch.bfloat16)
        w = torch.randn(N, Kd, device=DEV, dtype=torch.bfloat16) * 0.02
        b = torch.randn(N, device=DEV, dtype=torch.bfloat16)
        y = torch.empty(M_, N, device=DEV, dtype=torch.bfloat16)
        fl = 2.0 * M_ * N * Kd
        shape = "M=%d N=%d K=%d" % (M_, N, Kd)
        t1 = timeit(lambda: K.matmul_forward(y, x, w, b), a.iters, a.warmup, flush)
        t2 = timeit(lambda: torch.addmm(b, x, w.t(), out=y), a.iters, a.warmup, flush)
        row(out, "fwd+bias", shape, fl, t1, t2, "torch.addmm", a.peak_tflops)
        if name == "fc":
            pre = torch.empty_like(y)
            t1 = timeit(lambda: K.matmul_forward(y, x, w, b, pre_gelu=pre), a.iters, a.warmup, flush)
            t2 = timeit(lambda: F.gelu(torch.addmm(b, x, w.t(), out=pre), approximate="tanh"), a.iters, a.warmup, flush)
            row(out, "fwd+gelu", shape, fl, t1, t2, "addmm + gelu", a.peak_tflops)
        dy = torch.randn(M_, N, device=DEV, dtype=torch.bfloat16)
        dx = torch.empty(M_, Kd, device=DEV, dtype=torch.bfloat16)
        t1 = timeit(lambda: K.matmul_dgrad(dx, dy, w), a.iters, a.warmup, flush)
        t2 = timeit(lambda: torch.matmul(dy, w, out=dx), a.iters, a.warmup, flush)
        row(out, "dgrad", shape, fl, t1, t2, "torch.matmul", a.peak_tflops)
        dw = torch.zeros(N, Kd, device=DEV, dtype=torch.bfloat16)
        t1 = timeit(lambda: K.matmul_wgrad(dw, dy, x, True), a.iters, a.warmup, flush)
        t2 = timeit(lambda: dw.addmm_(dy.t(), x), a.iters, a.warmup, flush)
        row(out, "wgrad +=", shape, fl, t1, t2, "addmm_", a.peak_tflops)
        del x, w, y, dy, dx, dw


def bench_attention(a, out=sys.stdout):
    from torch.nn.attention import SDPBackend, sdpa_kernel
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=DEV)
    for B, T, NH, hs in [(16, 1024, 12, 64), (64, 1024, 12, 64), (16, 2048, 12, 64), (16, 1024, 12, 128), (16, 2048, 8, 128)]:
        qkv = torch.randn(B, T, 3 * NH * hs, device=DEV, dtype=torch.bfloat16)
        dout = torch.randn(B, T, NH * hs, device=DEV, dtype=torch.bfloat16)
        o = torch.empty(B, T, NH * hs, device=DEV, dtype=torch.bfloat16)
        lse = torch.empty(B, NH, T, device=DEV)
        dqkv = torch.empty_like(qkv)
        causal = 4.0 * B * NH * T * T * hs / 2            # two products over the lower triangle
        shape = "B=%d T=%d NH=%d HS=%d" % (B, T, NH, hs)
        t_f = timeit(lambda: K.attention_forward(o, lse, qkv, B, T, NH), a.iters, a.warmup, flush)
        t_b = timeit(lambda: K.attention_backward(dqkv, dout, qkv, o, lse, B, T, NH), a.iters, a.warmup, flush)
        q5 = qkv.view(B, T, 3, NH, hs)
        q, k, v = [q5[:, :, i].transpose(1, 2).detach().requires_grad_(True) for i in range(3)]
        go = dout.view(B, T, NH, hs).transpose(1, 2)
        for backend, label in ((SDPBackend.FLASH_ATTENTION, "sdpa flash"), (SDPBackend.CUDNN_ATTENTION, "sdpa cudnn")):
            try:
                with sdpa_kernel(backend):
                    t_lf = timeit(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True), a.iters, a.warmup, flush)
                    y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
                    t_lb = timeit(lambda: torch.autograd.grad(y, (q, k, v), go, retain_graph=True), a.iters, a.warmup, flush)
            except Exception as e:      # a backend that this build or this shape does not support
                print("%-10s %-28s %s unavailable: %s" % ("attention", shape, label, str(e).splitlines()[0][:80]), file=out, flush=True)
                continue
            row(out, "attn fwd", shape, causal, t_f, t_lf, label, a.peak_tflops)
            row(out, "attn bwd", shape, 2.5 * causal, t_b, t_lb, label, a.peak_tflops)
        del qkv, dout, o, lse, dqkv


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("what", choices=["gemm", "attention", "all"])
    ap.add_argument("--tokens", type=int, default=65536, help="rows of the GEMM problems (B*T of the training step)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--peak-tflops", type=float, default=1656.0)
    a = ap.parse_args(argv)
    if a.what in ("gemm", "all"):
        bench_gemm(a)
    if a.what in ("attention", "all"):
        bench_attention(a)
    from . import _lib
    print("kernel status 0x%x" % _lib.read_status())
    return 0


if __name__ == "__main__":
    sys.exit(main())
