"""ctypes binding of libfsa_sm100.so (the C ABI in include/fsa_sm100.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libfsa_sm100.so")

FSA_OK = 0
FSA_ERR_BAD_ARG = -1
FSA_ERR_UNSUPPORTED = -2
FSA_ERR_WORKSPACE = -3
FSA_ERR_CUDA = -4
FSA_ERR_DEVICE_STATUS = -5
FSA_ERR_STATIC_LIMIT = -6

DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1}

_lib = None

# name -> (restype, argtypes); every symbol include/fsa_sm100.h declares
SIGNATURES = {
    "fsa_version": (c_int, []),
    "fsa_error_string": (c_char_p, [c_int]),
    "fsa_last_cuda_error": (c_int, []),
    "fsa_last_cuda_error_line": (c_int, []),
    "fsa_profile_enable": (c_int, [c_int]),
    "fsa_profile_read": (c_int, [c_int, POINTER(c_float), POINTER(c_int)]),
    "fsa_sel_index_bytes": (c_int, [c_int64, c_int, c_int, c_int, c_int, c_int, POINTER(c_int64)]),
    "fsa_sel_fwd_scratch_bytes": (c_int, [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_int64)]),
    "fsa_sel_fwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_int64, c_int64, c_int64, c_int64, c_float, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64,
         c_void_p, c_int64, c_void_p],
    ),
    "fsa_sel_fwd_static": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_int64, c_int64, c_int64, c_int64, c_float, c_void_p, c_int64, c_int64, c_void_p, c_void_p],
    ),
    "fsa_sel_bwd_scratch_bytes": (c_int, [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_int64)]),
    "fsa_sel_bwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
         c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
         c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p],
    ),
    "fsa_range_attn_bytes": (c_int, [c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_int64),
                                     POINTER(c_int64), POINTER(c_int64)]),
    "fsa_range_attn_fwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int,
         c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_float, c_void_p, c_int64, c_int64, c_void_p,
         c_void_p, c_int64, c_void_p, c_int64, c_void_p],
    ),
    "fsa_range_attn_bwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
         c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
         c_int64, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p],
    ),
    "fsa_range_attn_fwd_dense": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int,
         c_int64, c_int64, c_int64, c_int64, c_float, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p],
    ),
    "fsa_range_attn_index": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p]),
    "fsa_linear_compress_fwd": (
        c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "fsa_linear_compress_bwd": (
        c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                c_void_p, c_void_p]),
    "fsa_select_topk_fused": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int,
         c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    ),
    "fsa_select_topk_seq": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_int,
         c_int, c_int, c_void_p, c_void_p],
    ),
    "fsa_rope": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int,
                         c_void_p, c_void_p]),
    "fsa_gate_proj_mix_scratch_bytes": (c_int64, [c_int64, c_int]),
    "fsa_gate_proj_mix_fwd": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p,
                                      c_void_p, c_void_p]),
    "fsa_gate_proj_mix_bwd": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                      c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "fsa_gate_mix_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "fsa_gate_mix_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p]),
    "fsa_decode_attn_partial": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_float, c_void_p, c_void_p, c_void_p, c_int64, c_void_p],
    ),
    "fsa_decode_read_status": (c_int, [c_void_p]),
    "fsa_decode_finish": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p]),
    "fsa_lse_merge": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "fsa_decode_select_topk": (
        c_int,
        [c_void_p, c_int64, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_int, c_int, c_void_p, c_void_p],
    ),
    "fsa_decode_cmp_ranges": (
        c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fsa_decode_ranges": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    ),
    "fsa_read_status": (c_int, [c_void_p, c_void_p, POINTER(c_int)]),
    "fsa_debug_wait_timeout": (c_int, [c_void_p, c_void_p]),
    "fsa_sel_index_geometry": (c_int, [c_int64, c_int, c_int, c_int, c_int, c_int, POINTER(c_int64), POINTER(c_int), POINTER(c_int)]),
    "fsa_sel_index_dump": (
        c_int,
        [c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
}


def lib() -> ctypes.CDLL:
    """Load the shared library once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python flash-sparse-attention_b200/build.py` "
                "(there is no fallback implementation)"
            )
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class FsaError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc == FSA_OK:
        return
    L = lib()
    msg = L.fsa_error_string(rc).decode()
    if rc == FSA_ERR_CUDA:
        msg += f" (cudaError {L.fsa_last_cuda_error()} at fsa_api.cu:{L.fsa_last_cuda_error_line()})"
    if rc in (FSA_ERR_BAD_ARG, FSA_ERR_UNSUPPORTED):
        raise ValueError(f"{what}: {msg}")
    raise FsaError(f"{what}: {msg}")


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def current_stream(device) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)
