"""Operators of the framework.

Every operator writes into caller-provided output tensors (the model owns flat, preallocated
buffers) and exists in two implementations with the same signature:

* ``kernels``    the hand-written sm_100a CUDA kernels (device tensors),
* ``reference``  a plain PyTorch fp32 restatement (CPU tensors; also the numerics oracle of the tests).

The functions exported here dispatch on the device of their first tensor argument.  A device tensor
never falls back to PyTorch: if the kernel library is missing the call raises.
"""
from . import kernels, reference

_NAMES = [
    "encoder_forward", "encoder_backward", "layernorm_forward", "fused_residual_forward", "layernorm_backward",
    "matmul_forward", "matmul_dgrad", "matmul_wgrad", "bias_grad", "attention_forward", "attention_backward",
    "fused_classifier", "gelu_forward", "gelu_backward_inplace", "residual_add", "global_norm_sq", "adamw_update",
    "params_from_master", "master_from_params",
    "rmsnorm_forward", "rmsnorm_fused_residual_forward", "rmsnorm_backward", "rope_forward", "rope_backward",
    "swiglu_forward", "swiglu_backward",
]


def _dispatch(name):
    k, r = getattr(kernels, name), getattr(reference, name)

    def op(first, *args, **kwargs):
        return (k if first.is_cuda else r)(first, *args, **kwargs)

    op.__name__ = name
    op.__doc__ = k.__doc__
    return op


for _n in _NAMES:
    globals()[_n] = _dispatch(_n)
del _n
