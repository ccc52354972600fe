"""ctypes binding of libb200lmk.so (declared in include/b200lmk.h).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint8, c_void_p

import torch

LIB_PATH = os.environ.get("B200LMK_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib",
                                                          "libb200lmk.so")

LMK_F32, LMK_F16, LMK_BF16 = 0, 1, 2
LMK_OK, LMK_ERR_INVALID, LMK_ERR_UNSUPPORTED, LMK_ERR_CUDA, LMK_ERR_WORKSPACE, LMK_ERR_DEVICE = 0, -1, -2, -3, -4, -5
PATH_AUTO, PATH_GENERAL, PATH_TCGEN05 = 0, 1, 2
ROTARY_NONE, ROTARY_HALF, ROTARY_INTERLEAVED, ROTARY_HALF_SYM = 0, 1, 2, 3

_DTYPES = {torch.float32: LMK_F32, torch.float16: LMK_F16, torch.bfloat16: LMK_BF16}


class CacheDesc(Structure):
    _fields_ = [("stride_b", c_int64), ("stride_h", c_int64), ("stride_block", c_int64), ("stride_row", c_int64),
                ("n_blocks", c_int), ("ring_start", c_int), ("block", c_int), ("top_k", c_int), ("pos_base", c_int)]


I64x3 = c_int64 * 3
I64x4 = c_int64 * 4

PROTOTYPES = {
    "lmk_version": (c_int, []),
    "lmk_last_error": (c_char_p, []),
    "lmk_device_status": (c_int, [POINTER(c_int), c_int]),
    "lmk_debug_set_max_ctas": (None, [c_int]),
    "lmk_attn_tcgen05_supported": (c_int, [c_int] * 7),
    "lmk_attn_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int, c_int, c_int, c_int, c_int, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64),
                             c_int, c_float, c_int, c_int, c_void_p]),
    "lmk_attn_bwd_workspace": (c_size_t, [c_int] * 8),
    "lmk_attn_bwd": (c_int, [c_void_p] * 10 + [c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_int,
                                               POINTER(c_int64), POINTER(c_int64), POINTER(c_int64),
                                               c_int, c_float, c_int, c_int, c_void_p]),
    "lmk_attn_bwd_static_max_rows": (c_size_t, []),
    "lmk_attn_bwd_static": (c_int, [c_void_p] * 10 + [c_int, c_int, c_int, c_int, c_int,
                                                      POINTER(c_int64), POINTER(c_int64), POINTER(c_int64),
                                                      c_int, c_float, c_int, c_int, c_void_p]),
    "lmk_attn_mask_supported": (c_int, [c_int] * 6),
    "lmk_attn_mask_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_int, c_int, POINTER(c_int64), POINTER(c_int64),
                                  POINTER(c_int64), c_int, c_float, c_int, c_void_p]),
    "lmk_attn_mask_bwd_workspace": (c_size_t, [c_int] * 4),
    "lmk_attn_mask_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64] + [c_void_p] * 7 +
                          [c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_int, POINTER(c_int64), POINTER(c_int64),
                           POINTER(c_int64), c_int, c_float, c_int, c_void_p]),
    "lmk_grouped_softmax_fwd": (c_int, [c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64), c_void_p,
                                        POINTER(c_int64), c_void_p, POINTER(c_int64), c_void_p, c_void_p, c_int,
                                        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "lmk_grouped_softmax_bwd": (c_int, [c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64), c_void_p,
                                        POINTER(c_int64), c_void_p, POINTER(c_int64), c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "lmk_grouped_softmax_causal_fwd": (c_int, [c_void_p, POINTER(c_int64), c_void_p, c_int64, c_void_p, c_int, c_int,
                                               c_int, c_int, c_int, c_int, c_void_p]),
    "lmk_grouped_softmax_causal_bwd": (c_int, [c_void_p, POINTER(c_int64), c_void_p, c_int64, c_void_p, c_void_p, c_int,
                                               c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "lmk_cache_store": (c_int, [c_void_p, c_void_p, POINTER(c_int64), c_void_p, c_void_p, POINTER(CacheDesc),
                                POINTER(CacheDesc), c_void_p, POINTER(c_int64), c_int, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_void_p]),
    "lmk_rotary_apply": (c_int, [c_void_p, c_void_p, POINTER(c_int64), POINTER(c_int64), c_void_p, c_void_p, c_int,
                                 c_int64, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "lmk_chunk_prepare": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64),
                                  c_void_p, c_void_p, c_int, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_void_p, POINTER(c_int64), c_int64, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_void_p]),
    "lmk_landmark_scores_workspace": (c_size_t, [c_int] * 6),
    "lmk_landmark_scores": (c_int, [c_void_p, c_void_p, POINTER(CacheDesc), c_void_p, c_void_p, c_int, c_int,
                                    c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_size_t,
                                    c_void_p]),
    "lmk_topk_sorted": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int64, c_int,
                                c_int, c_int, c_void_p]),
    "lmk_gather_kv": (c_int, [c_void_p, c_void_p, POINTER(CacheDesc), POINTER(CacheDesc), c_void_p, c_void_p,
                              c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                              c_void_p]),
    "lmk_selected_logits": (c_int, [c_void_p, c_void_p, POINTER(CacheDesc), c_void_p, c_void_p, c_void_p, c_int,
                                    c_int, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_float, c_int,
                                    c_void_p]),
    "lmk_selected_attend": (c_int, [c_void_p, c_void_p, POINTER(CacheDesc), c_void_p, POINTER(CacheDesc), c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_int,
                                    c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "lmk_selected_pv": (c_int, [c_void_p, c_int64, c_int64, c_void_p, POINTER(CacheDesc), c_void_p, c_void_p, c_int,
                                c_int, c_int, c_int, c_int, c_void_p]),
}

_lib = None
c_void_p = c_void_p          # re-exported for callers that pass raw stream handles


def lib():
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m landmark_attention_b200.build` "
                               "(there is no fallback path)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def device_status(clear: bool = True) -> int:
    """Status word of the current device (0 = healthy); a non-zero value names the bounded wait that expired."""
    v = c_int(0)
    rc = lib().lmk_device_status(ctypes.byref(v), int(clear))
    if rc != LMK_ERR_DEVICE:          # LMK_ERR_DEVICE only says that the word is non-zero; the caller gets the value
        check(rc, "lmk_device_status")
    return v.value


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype not in _DTYPES:
        raise AssertionError(f"unsupported dtype {t.dtype}")
    return _DTYPES[t.dtype]


def ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr(device):
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def strides3(t: torch.Tensor):
    assert t.dim() == 4 and t.stride(3) == 1
    return I64x3(t.stride(0), t.stride(1), t.stride(2))


def strides4_broadcast(t: torch.Tensor, shape):
    """Element strides of `t` expanded to 4-D `shape` (0 where broadcast)."""
    t = t.expand(shape)
    return t, I64x4(*t.stride())


def check(rc: int, what: str):
    """Turn a status code into the exception class the reference raises for the same mistake."""
    if rc == LMK_OK:
        return
    msg = lib().lmk_last_error().decode()
    if rc == LMK_ERR_INVALID:
        raise AssertionError(f"{what}: {msg}")
    if rc == LMK_ERR_UNSUPPORTED:
        raise NotImplementedError(f"{what}: {msg}")
    raise RuntimeError(f"{what} failed ({rc}): {msg}")


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise AssertionError("landmark_attention_b200 runs on CUDA tensors only (no CPU path)")
