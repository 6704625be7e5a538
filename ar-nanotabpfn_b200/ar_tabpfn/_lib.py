"""ctypes binding of libartab_b200.so (the C ABI declared in include/artab.h).

The library is the product: there is no Python or CPU fallback.  Importing this
module never fails, but the first call that needs the library raises if it is
not built (``python ar-nanotabpfn_b200/build.py``) or no CUDA device is present.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

F32, BF16 = 0, 1
ETIMEOUT = -5
DEBUG_WAIT_CYCLES, DEBUG_DROP_SCORE_COMMITS = 0, 1
MARK_TARGET, MARK_CONTEXT, MARK_BUFFER = 0, 1, 2
MAX_SPLITS = 16

_fp = C.c_void_p  # every device pointer travels as void*


class LayerWeights(C.Structure):
    _fields_ = [(n, _fp) for n in ("wf_t", "ln1_g", "ln1_b", "wqkv_t", "wo_t", "ln2_g", "ln2_b", "w1_t", "b1",
                                   "w2_t", "b2", "ln3_g", "ln3_b", "tc_wo", "tc_w1", "tc_w2", "tc_wf", "tc_wqkv")] + \
               [("tc_lo", C.c_int32), ("tc_reserved", C.c_int32)]


class Model(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("d_model", "n_heads", "head_dim", "d_ff", "n_layers", "n_comp",
                                          "n_ar_tokens", "reserved")] + \
               [(n, _fp) for n in ("wx", "bx", "wy", "by", "marker", "ar_tokens", "lnf_g", "lnf_b", "wa_t", "ba",
                                   "wb_t", "bb", "mean_bias", "std_bias", "weight_bias", "tc_wa", "tc_wb")] + \
               [("tc_head_lo", C.c_int32), ("tc_reserved", C.c_int32), ("layers", C.POINTER(LayerWeights))]


class State(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("dtype", "n_streams", "n_groups", "n_ctx", "n_ctx_pad", "max_buf",
                                          "buffer_len", "max_rows", "max_splits", "reserved")] + \
               [(n, _fp) for n in ("k_ctx", "v_ctx", "kv_buf", "x", "x1", "attn", "q", "o_part", "lse_part",
                                   "status")]


_LIB: Optional[C.CDLL] = None
LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "libartab_b200.so")

_i, _p = C.c_int, C.c_void_p
_SIGNATURES = {
    "artab_prefill": (_i, [C.POINTER(Model), C.POINTER(State), _p, _p, _i, _p]),
    "artab_decode_step": (_i, [C.POINTER(Model), C.POINTER(State), _p, _i, _i, _i, _p, _p, _p, _p, _p, _p]),
    "artab_decode_embedded": (_i, [C.POINTER(Model), C.POINTER(State), _p, _i, _i, _p, _p]),
    "artab_teacher_forcing": (_i, [C.POINTER(Model), C.POINTER(State), _p, _p, _i, _i, _p, _p]),
    "artab_forward_masked": (_i, [C.POINTER(Model), C.POINTER(State), _p, _p, _p, _p, _i, _i, _i, _p, _p, _p]),
    "artab_context_attention": (_i, [_i, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p]),
    "artab_context_attention_noalloc": (_i, [_i, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p]),
    "artab_buffer_attention_merge": (_i, [_i, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i, _i, _p, _p]),
    "artab_buffer_attention_merge_ragged": (_i, [_i, _p, _p, _i, _i, _i, _i, _i, _p, _i, _p, _p, _i, _i, _p, _p,
                                                _p]),
    "artab_buffer_attention_merge_visible": (_i, [_i, _p, _p, _i, _i, _i, _i, _i, _p, _i, _p, _p, _p, _i, _i, _p, _p,
                                                  _p]),
    "artab_kv_append": (_i, [_i, _p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "artab_embed": (_i, [C.POINTER(Model), _p, _p, _p, _i, _i, _i, _p, _p]),
    "artab_head_logpdf": (_i, [C.POINTER(Model), _p, _p, _i, _p, _p]),
    "artab_head_sample": (_i, [C.POINTER(Model), _p, _p, _p, _i, _p, _p, _p, _p]),
    "artab_plan_splits": (_i, [_i, _i, _i, _i, _i, _i]),
    "artab_profile_enable": (None, [_i]),
    "artab_set_dependent_launch": (None, [_i]),
    "artab_debug_set": (_i, [_i, C.c_longlong]),
    "artab_profile_read": (_i, [C.POINTER(C.c_double), C.POINTER(C.c_int64), _i]),
    "artab_launch_count": (C.c_int64, []),
    "artab_launch_count_reset": (None, []),
    "artab_last_error": (C.c_char_p, []),
    "artab_version": (C.c_char_p, []),
}


def load_library(path: Optional[str] = None) -> C.CDLL:
    """dlopen the library and attach argument types (no CUDA call is made)."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise RuntimeError(
            f"{p} is missing: build it with `python ar-nanotabpfn_b200/build.py` "
            "(there is no fallback implementation)")
    lib = C.CDLL(p)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _LIB = lib
    return lib


def lib() -> C.CDLL:
    """The loaded library; raises unless a CUDA device is usable."""
    if not torch.cuda.is_available():
        raise RuntimeError("ar_tabpfn (B200 build) needs a CUDA device; there is no CPU fallback")
    return load_library()


class ArtabError(RuntimeError):
    pass


def check(rc: int) -> None:
    """Map a negative return code to the exception the reference would raise."""
    if rc == 0:
        return
    msg = load_library().artab_last_error().decode()
    if rc in (-1, -2):
        raise ValueError(msg)
    raise ArtabError(f"artab error {rc}: {msg}")


PROFILE_KINDS = ("embed", "dense_chain", "context_attention", "buffer_merge", "kv_append")


def profile_read():
    """{kind: (milliseconds, launches)} recorded since artab_profile_enable(1); sync first."""
    n = len(PROFILE_KINDS)
    ms = (C.c_double * n)()
    cnt = (C.c_int64 * n)()
    load_library().artab_profile_read(ms, cnt, n)
    return {k: (ms[i], cnt[i]) for i, k in enumerate(PROFILE_KINDS)}


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise ValueError(f"unsupported cache dtype {dtype} (float32 or bfloat16)")
