"""ctypes binding of ``tilerl_b200/_C.so`` (the sm_100a kernels and the C++ runtime).

Every entry point takes raw device pointers plus the CUDA stream handle and
returns a ``cudaError_t`` as int; :func:`check` turns a non-zero code into an
exception.  Launches go to ``torch.cuda.current_stream()``, so they are captured
by ``torch.cuda.graph`` like any torch op.  There is no silent fallback: asking for
the library on a machine where it cannot be loaded raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_longlong, c_void_p
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
# TRL_TRACE_LIB=1 loads the timeline build (``python -m tilerl_b200.build --trace``) instead,
# TRL_BOUNDS_LIB=1 the build with checked table indices (``python -m tilerl_b200.build --bounds``)
_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                     "_C_trace.so" if os.environ.get("TRL_TRACE_LIB") == "1" else
                     ("_C_bounds.so" if os.environ.get("TRL_BOUNDS_LIB") == "1" else "_C.so"))

P, I, L, F = c_void_p, c_int, c_long, c_float

_SIGS = {
    "trl_gemv_nvfp4": [P, I, P, P, P, P, F, P, I, P, I, I, I, I, I, P],
    "trl_gemv_bf16": [P, I, P, P, F, P, I, P, I, I, I, I, I, P],
    "trl_set_pdl": [I],
    "trl_trace_read": [P, I, I],
    "trl_error_read": [P, I],
    "trl_attn_prep": [P, I, P, P, P, P, P, P, P, I, I, I, I, I, F, F, I, I, P],
    "trl_attn_paged": [P, P, I, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, F, I, P],
    "trl_gdn": [P, I, P, P, P, P, P, P, P, P, P, P, P, P, P, L, L, L, P, P, P, P, P, P, P,
                I, I, I, I, I, I, I, F, P],
    "trl_quant_act_fp8": [P, I, P, F, P, P, I, I, I, P],
    "trl_gemm_fp8": [P, P, P, P, P, I, P, I, I, I, I, I, P],
    "trl_gemv_fp8": [P, I, P, P, P, F, P, I, P, I, I, I, I, I, P],
    "trl_gdn_decode": [P, I, P, P, P, P, P, P, P, P, P, P, L, L, L, P, I, I, I, I, I, F, P],
    "trl_embedding": [P, P, P, I, I, I, P],
    "trl_gather_rows": [P, P, P, I, I, P],
    "trl_rmsnorm": [P, P, P, I, I, F, P],
    "trl_swiglu": [P, P, L, P],
    "trl_argmax": [P, I, I, I, P, P, P],
    "trl_argmax_stage1": [P, I, I, I, P, P, P],
    "trl_sample_softmax": [P, I, P, P, P, P, P, I, I, P],
    # host runtime (csrc/runtime.cpp)
    "trl_pager_create": [I], "trl_pager_destroy": [P], "trl_pager_alloc": [P], "trl_pager_alloc_many": [P, I, P],
    "trl_pager_incref": [P, I], "trl_pager_release": [P, I], "trl_pager_free_count": [P],
    "trl_pager_refcount": [P, I], "trl_pager_refs": [P, P, I],
    "trl_batch_ints": [c_longlong, I, I],
    "trl_batch_fill": [I, P, P, P, P, P, P, P, I, I, P, c_longlong],
    "trl_gemm_trace_read": [P, I],
    "trl_gemv2_set_trigger": [I],
    "trl_gdn_set_wy": [I],
    "trl_gdn_set_mma": [I],
    "trl_sample_nucleus": [P, I, P, P, P, P, P, P, P, I, I, P],
    "trl_attn_decode_mma": [P, P, I, P, P, P, I, I, P, P, P, P, P, P, I, I, I, I, I, I, F, I, P],
    "trl_gemv2_chain": [P, I, I, P, P, I, I, I, P],
    "trl_attn_decode_fused": [P, I, P, P, P, P, P, P, P, I, I, P, P, P, P, P, P, I, I, I, I, I, F, F, I, F, I, P],
    "trl_quest_scores": [P, P, P, P, I, I, I, I, P],
    "trl_topk_pages": [P, I, I, P, P],
    "trl_page_mean": [P, P, P, I, I, I, P],
    "trl_index_scores": [P, P, P, I, I, I, P],
    "trl_spec_accept": [P, P, P, P, P, P, I, I, P],
    "trl_gemv_nvfp4_mma": [P, I, P, P, P, P, F, P, I, P, I, I, I, I, I, P],
    "trl_attn_prep_fp8": [P, I, P, P, P, P, P, P, P, P, P, I, I, I, I, I, F, F, I, P],
    "trl_attn_paged_fp8": [P, P, I, P, P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, F, I, P],
    "trl_attn_prefill_fp8": [P, P, I, P, P, P, P, P, I, P, P, P, P, I, I, I, I, I, F, I, P],
    "trl_attn_prefill": [P, P, I, P, P, P, I, I, P, P, P, P, I, I, I, I, I, F, I, P],
    "trl_lora_add": [P, I, P, F, P, P, P, P, I, I, I, I, I, F, P],
    "trl_adamw": [P, P, P, P, P, L, F, F, F, F, F, I, F, P],
    "trl_quant_nvfp4": [P, I, L, L, P, P, P, P, I, P],
    "trl_dequant_nvfp4": [P, P, P, P, L, L, P],
    "trl_add": [P, P, P, L, P],
    "trl_decode_advance": [P, P, P, P, P, P, I, I, P, I, P, P],
}


_RESTYPE = {"trl_set_pdl": None, "trl_gdn_set_wy": None, "trl_gemv2_set_trigger": None, "trl_gdn_set_mma": None, "trl_pager_create": c_void_p, "trl_pager_destroy": None,
            "trl_batch_ints": c_longlong, "trl_batch_fill": c_longlong}


def loadable() -> bool:
    """The library file exists (the host runtime in it needs no GPU)."""
    return os.path.exists(_PATH)


def lib_path() -> str:
    return _PATH


def available() -> bool:
    return os.path.exists(_PATH) and torch.cuda.is_available()


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not os.path.exists(_PATH):
            raise RuntimeError(f"{_PATH} is missing: run `python -m tilerl_b200.build`")
        _LIB = ctypes.CDLL(_PATH)
        for name, sig in _SIGS.items():
            fn = getattr(_LIB, name, None)
            if fn is None:
                continue
            fn.argtypes = sig
            fn.restype = _RESTYPE.get(name, c_int)
    return _LIB


def register(name: str, sig) -> None:
    """Declare the signature of an entry point defined by another source file."""
    _SIGS[name] = sig
    if _LIB is not None and hasattr(_LIB, name):
        fn = getattr(_LIB, name)
        fn.argtypes = sig
        fn.restype = c_int


class KernelError(RuntimeError):
    pass


def check(code: int, what: str = "") -> None:
    if code != 0:
        raise KernelError(f"{what or 'kernel'} failed with cudaError {code}")


def ptr(t) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def read_error(clear: bool = True):
    """(code, a, b, c) of the device error word; code 0 = none."""
    out = (c_int * 4)()
    check(lib().trl_error_read(out, int(clear)), "trl_error_read")
    return tuple(out)


launch_count = 0


def count(n: int = 1) -> None:
    global launch_count
    launch_count += n
