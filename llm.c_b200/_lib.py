"""ctypes bindings of the two native libraries (see build.py).

``cuda()`` returns the kernel library and raises if it is missing on a machine that has a GPU:
there is no silent PyTorch fallback for device tensors.  ``host()`` returns the host runtime.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_uint, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIBDIR = os.path.join(HERE, "lib")

_cuda = None
_host = None


class TensorView(Structure):
    _fields_ = [("p_base", c_longlong), ("p_stride", c_longlong), ("o_base", c_longlong), ("o_stride", c_longlong),
                ("n", c_longlong), ("L", c_int), ("wd", c_float), ("seed", c_uint), ("pad", c_int)]


class TensorTable(Structure):
    _fields_ = [("t", TensorView * 16), ("count", c_int)]


def _load(name, builder):
    path = os.path.join(LIBDIR, name)
    from . import build as _b
    try:
        getattr(_b, builder)()          # no-op when the stored source hash matches
    except Exception:
        if not os.path.exists(path):    # no compiler on this machine and no prebuilt library
            raise
    return ctypes.CDLL(path)


def cuda():
    global _cuda
    if _cuda is not None:
        return _cuda
    if os.environ.get("LLMC_DEBUG_CHECKS") == "1":
        # the kernels with their debug checks on (alignment of every 16-byte access, id ranges): see build.build_cuda_debug
        lib = _load("libllmc_b200_debug.so", "build_cuda_debug")
    else:
        lib = _load("libllmc_b200.so", "build_cuda")
    P, I, L, F, U, S = c_void_p, c_int, c_longlong, c_float, c_uint, c_void_p
    U64 = ctypes.c_ulonglong
    sigs = {
        "llmc_status_read": (I, [I, POINTER(c_uint)]),
        "llmc_tensormap_cache_clear": (None, []),
        "llmc_device_sm_count": (I, []),
        "llmc_debug_checks_enabled": (I, []),
        "llmc_alloc_device_or_managed": (I, [POINTER(c_void_p), ctypes.c_size_t, I, POINTER(c_int)]),
        "llmc_free_device_or_managed": (I, [P]),
        "llmc_gemm": (I, [P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, P, I, S]),
        "llmc_gemm2": (I, [P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, P, S]),
        "llmc_gemm2_after_flags": (I, [P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, P, P, I, U64, S]),
        "llmc_gemm2_workspace": (None, [I, I, I, POINTER(c_longlong), POINTER(c_int)]),
        "llmc_gemm2_pick_splits": (I, [I, I, I, I]),
        "llmc_gemm_workspace": (None, [I, I, I, POINTER(c_longlong), POINTER(c_int)]),
        "llmc_gemm_pick_splits": (I, [I, I, I, I]),
        "llmc_layernorm_fwd": (I, [P, P, P, P, P, P, I, I, S]),
        "llmc_fused_residual_fwd": (I, [P, P, P, P, P, P, P, P, I, I, S]),
        "llmc_layernorm_bwd_scratch": (L, [I, I]),
        "llmc_layernorm_bwd": (I, [P, P, P, P, P, P, P, P, P, I, I, I, I, P, I, S]),
        "llmc_encoder_fwd": (I, [P, P, P, P, I, I, I, I, S]),
        "llmc_encoder_bwd": (I, [P, P, P, P, I, I, I, I, I, I, U, S]),
        "llmc_fused_classifier": (I, [P, P, P, F, I, I, I, I, I, S]),
        "llmc_gelu_fwd": (I, [P, P, L, S]),
        "llmc_gemm_tf32": (I, [P, P, P, P, I, I, I, I, I, I, I, S]),
        "llmc_rmsnorm_fwd": (I, [P, P, P, P, I, I, F, S]),
        "llmc_rmsnorm_fused_residual_fwd": (I, [P, P, P, P, P, P, I, I, F, S]),
        "llmc_rmsnorm_bwd_scratch": (L, [I, I]),
        "llmc_rmsnorm_bwd": (I, [P, P, P, P, P, P, P, I, I, I, I, S]),
        "llmc_rope_fwd": (I, [P, P, P, L, I, I, I, I, S]),
        "llmc_rope_bwd": (I, [P, P, P, L, I, I, I, I, S]),
        "llmc_swiglu_fwd": (I, [P, P, L, I, S]),
        "llmc_swiglu_bwd": (I, [P, P, P, L, I, S]),
        "llmc_rope_cache": (I, [P, P, P, P, P, I, I, I, I, I, I, I, I, P, S]),
        "llmc_skinny_gemm": (I, [P, P, P, I, I, I, I, I, I, S]),
        "llmc_cached_attention": (I, [P, P, P, P, I, I, I, I, I, I, I, P, P, S]),
        "llmc_cached_attention_workspace": (L, [I, I, I, I, I, I]),
        "llmc_gelu_bwd_inplace": (I, [P, P, L, S]),
        "llmc_residual_add": (I, [P, P, P, L, S]),
        "llmc_bias_grad_scratch": (L, [I, I]),
        "llmc_bias_grad": (I, [P, P, P, I, I, I, S]),
        "llmc_norm_sq_scratch": (I, []),
        "llmc_sum_f32": (I, [P, P, I, F, S]),
        "llmc_global_norm_sq": (I, [P, P, P, POINTER(TensorTable), S]),
        "llmc_adamw": (I, [P, P, P, P, P, POINTER(TensorTable), F, F, F, F, I, F, P, F, S]),
        "llmc_params_from_master": (I, [P, P, POINTER(TensorTable), S]),
        "llmc_master_from_params": (I, [P, P, POINTER(TensorTable), S]),
        "llmc_attention_fwd": (I, [P, P, P, I, I, I, I, S]),
        "llmc_attention_bwd": (I, [P, P, P, P, P, P, I, I, I, I, S]),
        "llmc_attention_bwd_workspace": (L, [I, I, I, I]),
        # full-precision operator set (csrc/fp32_ops.cu)
        "llmc_f32_gelu_fwd": (I, [P, P, L, S]),
        "llmc_f32_gelu_bwd": (I, [P, P, L, S]),
        "llmc_f32_residual_add": (I, [P, P, P, L, S]),
        "llmc_f32_encoder_fwd": (I, [P, P, P, P, I, I, I, I, S]),
        "llmc_f32_encoder_bwd": (I, [P, P, P, P, I, I, I, I, I, I, S]),
        "llmc_f32_layernorm_fwd": (I, [P, P, P, P, P, P, P, P, I, I, S]),
        "llmc_f32_layernorm_bwd_scratch": (L, [I, I]),
        "llmc_f32_layernorm_bwd": (I, [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, S]),
        "llmc_f32_bias_grad_scratch": (L, [I, I]),
        "llmc_f32_bias_grad": (I, [P, P, P, I, I, I, S]),
        "llmc_f32_classifier": (I, [P, P, P, F, I, I, I, I, I, S]),
        "llmc_f32_permute_qkv": (I, [P, P, I, I, I, I, I, S]),
        "llmc_f32_permute_heads": (I, [P, P, I, I, I, I, I, S]),
        "llmc_f32_softmax_causal": (I, [P, P, P, F, L, I, S]),
        "llmc_f32_softmax_causal_bwd": (I, [P, P, F, L, I, S]),
        "llmc_f32_adamw": (I, [P, P, P, P, P, L, L, L, L, L, I, F, F, F, I, F, F, F, P, F, S]),
        "llmc_f32_sumsq_partials_per_slice": (I, []),
        "llmc_f32_sumsq": (I, [P, P, L, L, L, I, S]),
        "llmc_f32_copy_slices": (I, [P, P, L, L, L, L, L, I, S]),
    }
    for name, (res, args) in sigs.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
    _cuda = lib
    return lib


def host():
    global _host
    if _host is None:
        override = os.environ.get("LLMC_HOST_LIB")          # e.g. a sanitizer build of csrc/host/host.cpp (see the tests)
        _host = ctypes.CDLL(override) if override else _load("libllmc_host.so", "build_host")
    return _host


class KernelError(RuntimeError):
    pass


def check(rc, what):
    if rc != 0:
        raise KernelError("%s failed with code %d" % (what, rc))


def read_status(clear=True):
    """Synchronises the device and returns the status word (0 = no kernel reported an error)."""
    out = c_uint(0)
    check(cuda().llmc_status_read(1 if clear else 0, ctypes.byref(out)), "llmc_status_read")
    return out.value
