"""ctypes binding of libdram_attention_b200.so (the C ABI declared in
include/dram_attention_b200.h).  There is no fallback: if the library is missing
the import of any operator fails with instructions to build it."""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_longlong, c_size_t, c_void_p, POINTER

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdram_attention_b200.so")

DA_F32, DA_F16, DA_BF16 = 0, 1, 2
STATUS_BAD_PAGE_ID, STATUS_LRU_OVERFLOW, STATUS_BAD_POSITION, STATUS_WAIT_TIMEOUT = 1, 2, 4, 8
_STATUS_TEXT = {
    STATUS_BAD_PAGE_ID: "a listed page id was outside the DRAM page range",
    STATUS_LRU_OVERFLOW: "more distinct non-resident pages requested than evictable slots",
    STATUS_BAD_POSITION: "start_pos - dram_kv_cache_size is outside the local window",
    STATUS_WAIT_TIMEOUT: "a bounded wait on an asynchronous copy ran out",
}

_DTYPES = {torch.float32: DA_F32, torch.float16: DA_F16, torch.bfloat16: DA_BF16}

_SIGNATURES = {
    "da_version": (c_int, []),
    "da_error_string": (c_char_p, [c_int]),
    "da_trace_bytes": (c_size_t, []),
    "da_trace_set": (c_int, [c_void_p]),
    "da_score_pages": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_void_p]),
    "da_topk_pages": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "da_topk_pages_wide": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "da_lru_update": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_int, c_int, c_void_p, c_void_p, c_size_t, c_int, c_void_p, c_void_p]),
    "da_prefill_attention_supported": (c_int, [c_int, c_int]),
    "da_prefill_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                     c_longlong, c_longlong, c_int, c_void_p, c_void_p]),
    "da_rope_qk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                           c_void_p]),
    "da_decode_attention_push_next": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int]),
    "da_gather_heads_buffer_bytes": (c_size_t, [c_int, c_int]),
    "da_gather_heads": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                                c_void_p]),
    "da_decode_attention_fetch": (c_int, [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p,
                                          c_void_p, c_void_p, c_longlong, c_longlong, c_int, c_void_p, c_void_p,
                                          c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p,
                                          c_int, c_int, c_int, c_int, c_void_p]),
    "da_fetch_pages": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                               c_size_t, c_void_p]),
    "da_decode_attention_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "da_decode_attention": (c_int, [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_longlong,
                                    c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                    c_void_p, c_void_p, c_size_t, c_void_p, c_int, c_int, c_int, c_int,
                                    c_void_p]),
    "da_decode_attention_tokens_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "da_decode_attention_tokens": (c_int, [c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p,
                                           c_longlong, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                           c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_int, c_int,
                                           c_int, c_int, c_void_p]),
    "da_decode_attention_phased_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "da_decode_attention_phased_supported": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "da_decode_attention_phased": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                           c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p,
                                           c_void_p, c_void_p, c_longlong, c_longlong, c_int, c_void_p, c_void_p,
                                           c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p,
                                           c_int, c_int, c_int, c_int, c_void_p]),
    "da_decode_attention_static_capacity": (c_size_t, []),
    "da_decode_attention_static": (c_int, [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_longlong,
                                           c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "da_build_pages": (c_int, [c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p,
                               c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dram_attention_b200.build` "
                "(needs nvcc; there is no non-CUDA fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code: int, what: str = "") -> None:
    if code != 0:
        text = lib().da_error_string(code).decode()
        raise RuntimeError(f"dram_attention_b200 {what} failed ({code}): {text}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; expected float32, float16 or bfloat16") from None


def stream_ptr() -> int:
    """cudaStream_t of torch's current stream."""
    return torch.cuda.current_stream().cuda_stream


def status_message(bits: int) -> str:
    return "; ".join(t for b, t in _STATUS_TEXT.items() if bits & b)


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device (got {t.device}); "
                           "dram_attention_b200 has no CPU path")
