"""Runs a small, fixed case of one operator a few times so that a profiler can capture it:

    ncu --set full --clock-control none -k regex:<kernel> -s <skip> -c <n> -o out python -m llmc_b200.profile_kernels <op>

Cases are larger than the 126 MB L2 but hold well under 2 GB on the device, so a capture ends by itself within a minute
or two.  ``python -m llmc_b200.profile_kernels list`` prints the operators.  With ``--time`` the operator is timed
with CUDA events instead (L2 flushed between iterations) and its achieved bandwidth / FLOP rate is printed.
(Counterpart of the reference's profile_gpt2.cu / dev/cuda benchmark mains.)
"""
import sys

import torch

from .ops import kernels as K

DEV = "cuda"


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def case(op):
    """Returns (callable, algorithmic bytes, flops) for the operator."""
    M, C = 16384, 768
    if op in ("gemm_fwd", "gemm_gelu", "gemm_dgrad", "gemm_dgelu", "gemm_wgrad"):
        N, Kd = 3072, 768
        a, w, b = _bf(M, Kd), _bf(N, Kd, scale=0.02), _bf(N)
        out, pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16), torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        dout, dinp, dw = _bf(M, N), torch.empty(M, Kd, device=DEV, dtype=torch.bfloat16), torch.zeros(N, Kd, device=DEV, dtype=torch.bfloat16)
        pre_in = _bf(M, N)
        w2 = _bf(Kd, N, scale=0.02)
        big_out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        flops = 2.0 * M * N * Kd
        io = 2.0 * (M * Kd + N * Kd + M * N)
        fns = {
            "gemm_fwd": (lambda: K.matmul_forward(out, a, w, b), io),
            "gemm_gelu": (lambda: K.matmul_forward(out, a, w, b, pre_gelu=pre), io + 2.0 * M * N),
            "gemm_dgrad": (lambda: K.matmul_dgrad(dinp, dout, w), io),
            "gemm_dgelu": (lambda: K.matmul_dgrad(big_out, a, w2, pre_gelu=pre_in), io + 2.0 * M * N),
            "gemm_wgrad": (lambda: K.matmul_wgrad(dw, dout, a, True), io + 2.0 * N * Kd),
        }
        fn, bytes_ = fns[op]
        return fn, bytes_, flops
    if op == "gemm_tf32":
        Mt, Nt, Kt = 8192, 3072, 768
        a32, b32, bias32 = torch.randn(Mt, Kt, device=DEV), torch.randn(Nt, Kt, device=DEV) * 0.02, torch.randn(Nt, device=DEV)
        d32 = torch.empty(Mt, Nt, device=DEV)
        return (lambda: K.gemm_tf32(d32, a32, b32, bias32)), 4.0 * (Mt * Kt + Nt * Kt + Mt * Nt), 2.0 * Mt * Nt * Kt
    if op == "gemm_fwd_1cta":
        # a problem with too few 256 x 256 tiles for the two-SM kernel: runs on the single-CTA kernel (128 x 256 tiles)
        Ms, Ns, Ks = 2048, 2304, 768
        a, w, b = _bf(Ms, Ks), _bf(Ns, Ks, scale=0.02), _bf(Ns)
        out = torch.empty(Ms, Ns, device=DEV, dtype=torch.bfloat16)
        return (lambda: K.matmul_forward(out, a, w, b)), 2.0 * (Ms * Ks + Ns * Ks + Ms * Ns), 2.0 * Ms * Ns * Ks
    if op in ("attn_fwd", "attn_bwd"):
        B, T, NH = 16, 1024, 12
        qkv, dout = _bf(B, T, 3 * NH * 64), _bf(B, T, NH * 64)
        out = torch.empty(B, T, NH * 64, device=DEV, dtype=torch.bfloat16)
        lse = torch.empty(B, NH, T, device=DEV)
        dqkv = torch.empty_like(qkv)
        K.attention_forward(out, lse, qkv, B, T, NH)
        causal = 4.0 * B * NH * T * T * 64 / 2
        if op == "attn_fwd":
            return (lambda: K.attention_forward(out, lse, qkv, B, T, NH)), 2.0 * (qkv.numel() + out.numel()), causal
        return (lambda: K.attention_backward(dqkv, dout, qkv, out, lse, B, T, NH)), 2.0 * (2 * qkv.numel() + 2 * out.numel()), 2.5 * causal      # five products per tile pair
    if op in ("ln_fwd", "fused_residual", "ln_bwd", "ln_bwd_colsum"):
        N = 65536
        x, y, w, b, dy = _bf(N, C), _bf(N, C), _bf(C) + 1, _bf(C), _bf(N, C)
        out, res = torch.empty_like(x), torch.empty_like(x)
        mean, rstd = torch.empty(N, device=DEV), torch.empty(N, device=DEV)
        dx, dw, db = _bf(N, C), _bf(C), _bf(C)
        K.layernorm_forward(out, mean, rstd, x, w, b)
        fns = {
            "ln_fwd": (lambda: K.layernorm_forward(out, mean, rstd, x, w, b), 2.0 * 2 * N * C),
            "fused_residual": (lambda: K.fused_residual_forward(res, out, mean, rstd, x, y, w, b), 2.0 * 4 * N * C),
            "ln_bwd": (lambda: K.layernorm_backward(dx, dw, db, dy, x, w, mean, rstd, True, True), 2.0 * 4 * N * C),
            "ln_bwd_colsum": (lambda: K.layernorm_backward(dx, dw, db, dy, x, w, mean, rstd, True, True, dcolsum=b, accumulate_dcol=False),
                              2.0 * 4 * N * C),
        }
        fn, bytes_ = fns[op]
        return fn, bytes_, 0.0
    if op == "classifier":
        N, V, Vp = 8192, 50257, 50304
        logits = _bf(N, Vp)
        losses = torch.zeros(N, device=DEV)
        tgt = torch.randint(0, V, (N,), device=DEV, dtype=torch.int32)
        return (lambda: K.fused_classifier(logits, losses, tgt, 1.0 / N, V, True, False)), 2.0 * 2 * N * Vp, 0.0
    if op in ("encoder_fwd", "encoder_bwd"):
        B, T, V = 64, 1024, 50257
        tok = torch.randint(0, V, (B, T), device=DEV, dtype=torch.int32)
        wte, wpe = _bf(50304, C), _bf(T, C)
        out, dout = torch.empty(B, T, C, device=DEV, dtype=torch.bfloat16), _bf(B, T, C)
        dwte, dwpe = torch.zeros(50304, C, device=DEV, dtype=torch.bfloat16), torch.zeros(T, C, device=DEV, dtype=torch.bfloat16)
        if op == "encoder_fwd":
            return (lambda: K.encoder_forward(out, tok, wte, wpe)), 2.0 * 2 * B * T * C, 0.0
        return (lambda: K.encoder_backward(dwte, dwpe, dout, tok, True, True, 1)), 2.0 * 3 * B * T * C, 0.0
    if op in ("adamw", "norm"):
        n = 64 * 1024 * 1024
        p, g = _bf(n, scale=0.02), _bf(n, scale=0.01)
        master, m, v = p.float(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
        nsq = torch.ones(1, device=DEV)
        views = [dict(p_base=0, p_stride=n, o_base=0, o_stride=n, n=n, L=1, wd=0.1, seed=7)]
        if op == "adamw":
            return (lambda: K.adamw_update(p, master, g, m, v, views, 1e-3, 0.9, 0.95, 1e-8, 1, 1.0, nsq, 1.0)), n * (2 + 2 + 2 + 3 * 8.0), 0.0
        return (lambda: K.global_norm_sq(nsq, g, views)), 2.0 * n, 0.0
    if op == "bias_grad":
        dout, db = _bf(65536, 3072), _bf(3072)
        return (lambda: K.bias_grad(db, dout, True)), 2.0 * dout.numel(), 0.0
    if op == "gelu":
        x = _bf(65536 * 3072)
        out = torch.empty_like(x)
        return (lambda: K.gelu_forward(out, x)), 4.0 * x.numel(), 0.0
    if op in ("rms_fwd", "rms_fused_residual", "rms_bwd"):
        N, Cw = 16384, 4096
        x, y, w, dy = _bf(N, Cw), _bf(N, Cw), _bf(Cw) + 1, _bf(N, Cw)
        out, res, dx, dw = torch.empty_like(x), torch.empty_like(x), _bf(N, Cw), _bf(Cw)
        rstd = torch.empty(N, device=DEV)
        K.rmsnorm_forward(out, rstd, x, w, 1e-5)
        fns = {
            "rms_fwd": (lambda: K.rmsnorm_forward(out, rstd, x, w, 1e-5), 2.0 * 2 * N * Cw),
            "rms_fused_residual": (lambda: K.rmsnorm_fused_residual_forward(res, out, rstd, x, y, w, 1e-5), 2.0 * 4 * N * Cw),
            "rms_bwd": (lambda: K.rmsnorm_backward(dx, dw, dy, x, w, rstd, True, True), 2.0 * 4 * N * Cw),
        }
        fn, bytes_ = fns[op]
        return fn, bytes_, 0.0
    if op in ("rope_fwd", "rope_bwd"):
        from .models import llama3
        B, T, NH, NKV, HS = 4, 4096, 32, 8, 128
        cfg = llama3.LlamaConfig(max_seq_len=T, num_heads=NH, num_kv_heads=NKV, channels=NH * HS)
        freqs = llama3.rope_table(cfg).to(DEV)
        raw, packed = _bf(B * T, (NH + 2 * NKV) * HS), _bf(B * T, 3 * NH * HS)
        nbytes = 2.0 * (raw.numel() + packed.numel())
        if op == "rope_fwd":
            return (lambda: K.rope_forward(packed, raw, freqs, T, NH, NKV)), nbytes, 0.0
        return (lambda: K.rope_backward(raw, packed, freqs, T, NH, NKV)), nbytes, 0.0
    if op in ("swiglu_fwd", "swiglu_bwd"):
        N, H = 16384, 14336
        x12, h, dh, dx12 = _bf(N, 2 * H), _bf(N, H), _bf(N, H), torch.empty(N, 2 * H, device=DEV, dtype=torch.bfloat16)
        if op == "swiglu_fwd":
            return (lambda: K.swiglu_forward(h, x12)), 2.0 * 3 * N * H, 0.0
        return (lambda: K.swiglu_backward(dx12, dh, x12)), 2.0 * 5 * N * H, 0.0
    if op in ("skinny_gemm", "skinny_gemm_wide"):
        # a decoding step of LLaMA-3 8B: 4 rows against the fused MLP up-projection (235 MB of weights) or the QKV projection
        Mr, Kd, Nw = 4, 4096, (28672 if op == "skinny_gemm" else 6144 * 8)
        x, w = _bf(Mr, Kd), _bf(Nw, Kd, scale=0.02)
        out = torch.empty(Mr, Nw, device=DEV, dtype=torch.bfloat16)
        return (lambda: K.matmul_skinny(out, x, w)), 2.0 * (Nw * Kd + Mr * Kd + Mr * Nw), 2.0 * Mr * Nw * Kd
    if op == "cached_attention":
        # 32 rows decoding at position 4095 with 32 query heads over 8 cached heads of width 128 (537 MB of cache read)
        B, Tmax, NH, NKV, HS = 32, 4096, 32, 8, 128
        kc, vc = _bf(B, Tmax, NKV, HS), _bf(B, Tmax, NKV, HS)
        q, out = _bf(B, NH * HS), torch.empty(B, NH * HS, device=DEV, dtype=torch.bfloat16)
        return (lambda: K.cached_attention(out, q, kc, vc, 1, Tmax - 1, NH, NKV)), 2.0 * (kc.numel() + vc.numel()), 0.0
    raise SystemExit("unknown operator %r" % op)


OPS = ["gemm_fwd", "gemm_gelu", "gemm_dgrad", "gemm_dgelu", "gemm_wgrad", "attn_fwd", "attn_bwd", "ln_fwd", "fused_residual", "ln_bwd", "ln_bwd_colsum",
       "classifier", "encoder_fwd", "encoder_bwd", "adamw", "norm", "bias_grad", "gelu", "rms_fwd", "rms_fused_residual", "rms_bwd", "rope_fwd",
       "rope_bwd", "swiglu_fwd", "swiglu_bwd", "gemm_tf32", "gemm_fwd_1cta", "skinny_gemm", "skinny_gemm_wide", "cached_attention"]


def main(argv):
    if not argv or argv[0] == "list":
        print("\n".join(OPS))
        return 0
    timing = "--time" in argv
    ops = [a for a in argv if not a.startswith("--")]
    if ops == ["all"]:
        ops = OPS
    from . import _lib
    for op in ops:
        fn, nbytes, flops = case(op)
        if not timing:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
        else:
            flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=DEV)
            for _ in range(3):
                fn()
            ts = []
            for _ in range(10):
                flush.zero_()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record(); fn(); e.record()
                torch.cuda.synchronize()
                ts.append(s.elapsed_time(e))
            ts.sort()
            t = ts[len(ts) // 2]
            msg = "%-16s %9.3f us  %8.1f GB/s (algorithmic)" % (op, t * 1e3, nbytes / t / 1e6)
            if flops:
                msg += "  %8.1f TFLOP/s" % (flops / t / 1e9)
            print(msg, flush=True)
        del fn
        torch.cuda.empty_cache()
    print("kernel status 0x%x" % _lib.read_status())
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
