"""ctypes binding of libphasorkv_b200.so (the C ABI declared in include/phasorkv_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_uint32, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libphasorkv_b200.so")

PAGE_TOKENS = 128
MAX_WIDTH = 256
QUERY_TERMS = 4
NOALLOC_MAX_PARTS = 320
F32, BF16, F64 = 0, 1, 2
ATTN_SCORES_ONLY, ATTN_SIMT, ATTN_PACKED_OUT, ATTN_EARLY_STREAM, ATTN_TAIL_WRITTEN, ATTN_QUERY_READY = 1, 2, 4, 8, 16, 32
EXCHANGE_PUSH, EXCHANGE_MERGE = 1, 2


class PhasorKVError(RuntimeError):
    pass


class Layer(ctypes.Structure):
    _fields_ = [("d_model", c_int32), ("n_q", c_int32), ("n_kv", c_int32), ("head_dim", c_int32),
                ("R", c_int32), ("R_s", c_int32), ("n_slow", c_int32),
                ("attn_scale", c_float), ("second", c_float),
                ("Bw_dev", c_void_p), ("A_re_dev", c_void_p), ("A_im_dev", c_void_p), ("A_s_dev", c_void_p),
                ("freq_dev", c_void_p), ("slow_dev", c_void_p), ("inv_freq_dev", c_void_p), ("Bw_bf16x3_dev", c_void_p),
                ("second_blocks_dev", c_void_p)]


class Exchange(ctypes.Structure):
    _fields_ = [("world", c_int32), ("rank", c_int32), ("batch", c_int32), ("n_q", c_int32), ("head_dim", c_int32),
                ("n_cta", c_int32), ("peer_data_dev", c_void_p), ("epoch_dev", c_void_p)]


class LayerHost(ctypes.Structure):
    """struct pkv_layer_host: host arrays for pkv_layer_create."""
    _fields_ = [("d_model", c_int32), ("n_q", c_int32), ("n_kv", c_int32), ("head_dim", c_int32), ("R", c_int32),
                ("R_s", c_int32), ("n_slow", c_int32), ("attn_scale", c_float), ("second", c_float),
                ("B_re", c_void_p), ("B_im", c_void_p), ("B_s", c_void_p), ("A_re", c_void_p), ("A_im", c_void_p),
                ("A_s", c_void_p), ("freq", c_void_p), ("slow", c_void_p), ("inv_freq", c_void_p)]


class Cache(ctypes.Structure):
    _fields_ = [("latent_dev", c_void_p), ("v_dev", c_void_p), ("n_pages", c_int32), ("W", c_int32),
                ("n_kv", c_int32), ("head_dim", c_int32), ("vq_dev", c_void_p), ("v_bits", c_int32)]


#: name -> (restype, argtypes); the complete exported surface of include/phasorkv_b200.h
SIGNATURES = {
    "pkv_abi_version": (c_int32, []),
    "pkv_status_string": (c_char_p, [c_int32]),
    "pkv_last_cuda_error": (c_int32, []),
    "pkv_device_check": (c_int32, []),
    "pkv_latent_page_bytes": (c_int64, [c_int32]),
    "pkv_v_page_bytes": (c_int64, [c_int32, c_int32]),
    "pkv_query_operand_bytes": (c_int64, [c_int32]),
    "pkv_quantize_rows": (c_int32, [POINTER(Cache), c_void_p, c_void_p, c_int32, c_float, c_void_p]),
    "pkv_quantize_rows_tiered": (c_int32, [POINTER(Cache), c_void_p, c_void_p, c_int32, c_void_p, c_void_p]),
    "pkv_cache_read_tiered": (c_int32, [POINTER(Cache), c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "pkv_cache_write": (c_int32, [POINTER(Layer), POINTER(Cache), c_void_p, c_int32, c_void_p, c_void_p, c_void_p,
                                  c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "pkv_write_scratch_floats": (c_int64, [c_int32, c_int32]),
    "pkv_v_write": (c_int32, [POINTER(Cache), c_void_p, c_void_p, c_int32, c_void_p]),
    "pkv_cache_read": (c_int32, [POINTER(Cache), c_void_p, c_int32, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "pkv_layer_create": (c_int32, [POINTER(LayerHost), POINTER(POINTER(Layer))]),
    "pkv_layer_destroy": (c_int32, [POINTER(Layer)]),
    "pkv_quantize_nvfp4": (c_int32, [POINTER(Cache), c_void_p, c_void_p, c_int32, c_float, c_void_p]),
    "pkv_dequant": (c_int32, [POINTER(Cache), c_void_p, c_int32, c_float, c_void_p, c_void_p]),
    "pkv_status_read": (c_int32, [c_void_p, c_void_p, c_void_p]),
    "pkv_set_scale_round_up": (c_int32, [c_int32]),
    "pkv_absorb": (c_int32, [POINTER(Layer), c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p]),
    "pkv_decode_prologue": (c_int32, [POINTER(Layer), POINTER(Cache), c_void_p, c_int32, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p]),
    "pkv_decode_attn": (c_int32, [POINTER(Layer), POINTER(Cache), c_void_p, c_void_p, c_int32, c_void_p, c_int32,
                                  c_int32, c_uint32, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "pkv_absorb_sync": (c_int32, [POINTER(Layer), c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "pkv_decode_prologue_sync": (c_int32, [POINTER(Layer), POINTER(Cache), c_void_p, c_int32, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p]),
    "pkv_decode_attn_sync": (c_int32, [POINTER(Layer), POINTER(Cache), c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_int32,
                                       c_int32, c_uint32, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "pkv_decode_attn_q": (c_int32, [POINTER(Layer), POINTER(Cache), c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_int32,
                                    c_int32, c_uint32, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "pkv_decode_attn_noalloc": (c_int32, [POINTER(Layer), POINTER(Cache), c_void_p, c_void_p, c_int32, c_void_p, c_int32,
                                          c_int32, c_void_p, c_void_p, c_void_p]),
    "pkv_exchange_merge": (c_int32, [POINTER(Exchange), c_void_p, c_void_p, c_uint32, c_void_p, c_void_p]),
    "pkv_merge_exchange": (c_int32, [POINTER(Exchange), c_void_p, c_int64, c_int64, c_int32, c_void_p, c_void_p, c_void_p]),
    "pkv_exact_partial": (c_int32, [POINTER(Layer), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p,
                                    c_void_p]),
    "pkv_merge_exact": (c_int32, [c_void_p, c_int64, c_int64, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p,
                                  c_void_p]),
    "pkv_scores_exact": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p]),
    "pkv_write_rows_f64": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_int32,
                                     c_void_p, c_void_p]),
    "pkv_absorb_rows_f64": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                      c_int32, c_int32, c_void_p, c_void_p, c_int32, c_void_p, c_void_p]),
    "pkv_vq_page_bytes": (c_int64, [c_int32, c_int32]),
    "pkv_vq_write": (c_int32, [POINTER(Cache), c_void_p, c_void_p, c_int32, c_void_p]),
    "pkv_vq_read": (c_int32, [POINTER(Cache), c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "pkv_read_probe": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p]),
    "pkv_merge": (c_int32, [c_void_p, c_int64, c_int64, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p,
                            c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """dlopen the library (once) and attach the prototypes. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise PhasorKVError(f"{LIB_PATH} is missing: build it with `python -m phasorkv_b200.build`")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        lib = load()
        msg = lib.pkv_status_string(int(status)).decode()
        extra = f" (cudaError {lib.pkv_last_cuda_error()})" if status == -3 else ""
        raise PhasorKVError(f"{what}: {msg}{extra}")


def ptr(t) -> c_void_p:
    """Device (or host) address of a torch tensor, or NULL."""
    return c_void_p(0 if t is None else t.data_ptr())


def current_stream() -> c_void_p:
    import torch
    return c_void_p(torch.cuda.current_stream().cuda_stream)
