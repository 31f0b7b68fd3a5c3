"""ctypes binding of libadamas_b200.so (the C ABI declared in include/adamas_b200.h).

There is no CPU or PyTorch fallback: if the library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p, POINTER

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# ADAMAS_B200_LIBRARY names a library built elsewhere (e.g. a build with extra compile flags)
LIB_PATH = os.environ.get("ADAMAS_B200_LIBRARY") or os.path.join(_PKG_DIR, "libadamas_b200.so")

OK, ERR_INVALID, ERR_CUDA, ERR_STATE = 0, 1, 2, 3
F16, BF16 = 0, 1
METRIC_L1, METRIC_XOR = 0, 1
VAL_F16, VAL_U16 = 0, 1

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing. Build it with `python adamas_b200/build.py` (needs nvcc); "
        "adamas_b200 has no fallback implementation.")

lib = ctypes.CDLL(LIB_PATH)

_P = c_void_p
_I = c_int
_L = c_int64
_F = c_float
_FP = POINTER(c_float)

# name -> argument types; every function returns int except where noted
SIGNATURES = {
    "adamas_hadamard_transform": [_P, _P, _L, _I, _F, _I, _P],
    "adamas_bucketize_pack": [_P, _P, _L, _I, _FP, _I, _P],
    "adamas_append_decode": [_P, _P, _P, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _FP, _I, _P],
    "adamas_append_decode_fused": [_P, _P, _P, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _FP, _I, _P],
    "adamas_apply_rope_in_place": [_P, _P, _L, _I, _I, _I, _L, _F, _F, _I, _P],
    "adamas_append_decode_rope_fused": [_P, _P, _P, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _FP, _F, _F,
                                        _P, _F, _I, _P],
    "adamas_append_prefill": [_P, _P, _P, _L, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _F, _FP, _I, _P],
    "adamas_estimate": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _L, _I, _I, _I, _P, _I, _P],
    "adamas_topk": [_P, _I, _L, _I, _P, _L, _I, _I, _I, _P, _P, _L, _P],
    "adamas_decode_handler_create": [POINTER(c_void_p)],
    "adamas_decode_handler_destroy": [_P],
    "adamas_decode_begin_forward": [_P, _L, _I, _I, _I, _I, _I, _I, _P],
    "adamas_decode_end_forward": [_P],
    "adamas_decode_forward": [_P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _F, _P],
    "adamas_decode_forward_partial": [_P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _F, _P],
    "adamas_decode_forward_static": [_P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P],
    "adamas_select_attend": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _P, _L, _F,
                             _P],
    "adamas_select_attend_slices": [_I, _I, _I, POINTER(c_int)],
    "adamas_decode_step": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I,
                           _P, _L, _P, _P, _L, _F, _FP, _F, _F, _P, _F, _F, _P],
    "adamas_decode_step_dev": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                               _P, _L, _P, _P, _L, _F, _FP, _F, _F, _P, _F, _F, _P],
    "adamas_dense_step_dev": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                              _F, _FP, _F, _F, _P, _F, _F, _P],
    "adamas_seq_len_advance": [_P, _I, _I, _P],
    "adamas_decode_step_batch_dev": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I,
                                     _P, _L, _P, _P, _L, _F, _FP, _F, _F, _P, _F, _F, _P],
    "adamas_dense_step_batch_dev": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                                    _F, _FP, _F, _F, _P, _F, _F, _P],
    "adamas_dist_histograms": [_P, _L, _I, _I, _I, _P, _P],
    "adamas_hist_rowsum": [_P, _I, _I, _P, _P],
    "adamas_global_cut": [_P, _I, _I, _I, _I, _P, _P],
    "adamas_apply_rope_table_in_place": [_P, _P, _L, _I, _I, _I, _L, _P, _F, _I, _P],
    "adamas_append_estimate": [_P, _P, _P, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P, _L, _F, _FP,
                               _P, _I, _P],
    "adamas_merge_states": [_P, _P, _I, _I, _I, _P, _P, _I, _P],
    "adamas_device_error": [POINTER(ctypes.c_uint), _I],
    "adamas_set_pdl": [_I],
    "adamas_set_max_cluster": [_I],
    "adamas_set_fused_append": [_I],
    "adamas_set_estimate_blocks_per_sm": [_I],
}

for _name, _args in SIGNATURES.items():
    try:
        _fn = getattr(lib, _name)
    except AttributeError as exc:
        raise ImportError(f"{LIB_PATH} does not export {_name}: it is stale, rebuild it with "
                          "`python adamas_b200/build.py --force`") from exc
    _fn.argtypes = _args
    _fn.restype = c_int
lib.adamas_abi_version.argtypes = []
lib.adamas_abi_version.restype = c_int
lib.adamas_last_error.argtypes = []
lib.adamas_last_error.restype = c_char_p

ABI_VERSION = 4
HIST_WORDS_PER_HEAD = 16 * 512 + 16 * 132
if lib.adamas_abi_version() != ABI_VERSION:
    raise ImportError(f"{LIB_PATH} has ABI version {lib.adamas_abi_version()}, expected {ABI_VERSION}; rebuild it")


def last_error() -> str:
    return lib.adamas_last_error().decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    """Turn a non-zero status into RuntimeError, the exception type the reference's bindings
    raise through TORCH_CHECK (adamas/ops/csrc/estimate.cu:77-83)."""
    if status != OK:
        raise RuntimeError(f"{what} failed: {last_error()}")


def device_error(clear: bool = True) -> int:
    """Error flags raised by kernels on the current device (0 = none); synchronises."""
    flags = ctypes.c_uint(0)
    check(lib.adamas_device_error(ctypes.byref(flags), int(clear)), "adamas_device_error")
    return flags.value


def thresholds_arg(thresholds):
    if thresholds is None:
        return None
    arr = (c_float * 3)(*[float(t) for t in thresholds])
    return arr
