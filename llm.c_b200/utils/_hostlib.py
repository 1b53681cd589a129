"""Typed access to the C++ host runtime (csrc/host/host.cpp)."""
import ctypes
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

from .. import _lib

_configured = None


class HostError(RuntimeError):
    pass


def lib():
    global _configured
    if _configured is not None:
        return _configured
    L = _lib.host()
    P, I, LL, F, U = c_void_p, c_int, c_longlong, c_float, c_uint
    sig = {
        "llmc_host_last_error": (c_char_p, []),
        "llmc_rng_new": (P, [U]), "llmc_rng_free": (None, [P]), "llmc_rng_u32": (U, [P]), "llmc_rng_f32": (F, [P]),
        "llmc_rng_uniform": (None, [P, P, LL, F, F]), "llmc_rng_normal": (None, [P, P, LL, F, F]),
        "llmc_rng_permutation": (None, [P, P, I]), "llmc_rng_get_state": (None, [P, P]), "llmc_rng_set_state": (None, [P, P]),
        "llmc_dl_new": (P, [c_char_p, LL, LL, I, I, I]), "llmc_dl_free": (None, [P]), "llmc_dl_next": (I, [P, P, P]),
        "llmc_dl_reset": (I, [P]), "llmc_dl_resume": (I, [P, LL, LL]), "llmc_dl_prefetch": (I, [P, P, P]), "llmc_dl_wait": (I, [P]),
        "llmc_dl_get": (LL, [P, I]), "llmc_dl_get_shuffle_state": (None, [P, P, P, P]),
        "llmc_dl_set_shuffle_state": (I, [P, P, LL, P, LL, P]),
        "llmc_eval_new": (P, [c_char_p, LL, LL, I, I]), "llmc_eval_free": (None, [P]), "llmc_eval_reset": (I, [P]),
        "llmc_eval_next_batch": (I, [P, P, P, P]), "llmc_eval_stat_losses": (I, [P, P, P]), "llmc_eval_get": (I, [P, I]),
        "llmc_tokenizer_new": (P, [c_char_p]), "llmc_tokenizer_free": (None, [P]), "llmc_tokenizer_vocab": (I, [P]),
        "llmc_tokenizer_eot": (I, [P]), "llmc_tokenizer_decode": (I, [P, U, P, I]),
        "llmc_random_u32": (U, [POINTER(c_ulonglong)]), "llmc_random_f32": (F, [POINTER(c_ulonglong)]),
        "llmc_sample_softmax": (I, [P, I, F]),
        "llmc_learning_rate": (F, [I, I, F, I, I, F]),
        "llmc_outlier_new": (P, []), "llmc_outlier_free": (None, [P]), "llmc_outlier_update": (c_double, [P, c_double]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _configured = L
    return L


def last_error():
    return lib().llmc_host_last_error().decode("utf-8", "replace")


def check(rc, what):
    if rc != 0:
        raise HostError("%s: %s" % (what, last_error()))
