"""Operators of the framework.

Every operator writes into caller-provided output tensors (the model owns flat, preallocated
buffers) and exists in two implementations with the same signature:

* ``kernels``    the hand-written sm_100a CUDA kernels (device tensors),
* ``reference``  a plain PyTorch fp32 restatement (CPU tensors; also the numerics oracle of the tests).

* ``kernels_fp32``  the full-precision kernels of the GPT-2 operator set (fp32 device tensors, the legacy ``-dt fp32`` mode).

The functions exported here dispatch on the device and type of their first tensor argument: bf16 device tensors go
to the sm_100a kernels and never fall back to PyTorch (if the kernel library is missing the call raises); fp32 device
tensors go to ``kernels_fp32`` (operators of the LLaMA family, which that module does not have, and the matmuls' IEEE fp32
form run on PyTorch's library kernels on the device); host tensors go to the restatement.
"""
import torch

from . import kernels, kernels_fp32, reference

_NAMES = [
    "encoder_forward", "encoder_backward", "layernorm_forward", "fused_residual_forward", "layernorm_backward",
    "matmul_forward", "matmul_dgrad", "matmul_wgrad", "bias_grad", "attention_forward", "attention_backward",
    "fused_classifier", "gelu_forward", "gelu_backward_inplace", "residual_add", "global_norm_sq", "adamw_update",
    "params_from_master", "master_from_params", "sum_scaled",
    "rmsnorm_forward", "rmsnorm_fused_residual_forward", "rmsnorm_backward", "rope_forward", "rope_backward",
    "swiglu_forward", "swiglu_backward", "rope_cache", "cached_attention", "matmul_skinny",
]


# operators whose first argument is an fp32 statistic or master copy in every mode: the second argument decides
_DECIDED_BY_SECOND = {"global_norm_sq", "master_from_params"}
# operators on fp32 statistics only: the device alone decides
_DECIDED_BY_DEVICE = {"sum_scaled"}


def _dispatch(name):
    k, r = getattr(kernels, name), getattr(reference, name)
    which = 1 if name in _DECIDED_BY_SECOND else 0

    by_device = name in _DECIDED_BY_DEVICE

    f32 = getattr(kernels_fp32, name, None)

    def op(*args, **kwargs):
        t = args[which]
        if t.is_cuda:
            if by_device or t.dtype != torch.float32:
                return k(*args, **kwargs)
            if f32 is not None:
                return f32(*args, **kwargs)
        return r(*args, **kwargs)

    op.__name__ = name
    op.__doc__ = k.__doc__
    return op


for _n in _NAMES:
    globals()[_n] = _dispatch(_n)
del _n
