"""ctypes binding of the C ABI declared in ``include/nanopd_b200.h``."""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p, POINTER
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libnanopd_b200.so"

NPD_OK = 0
NPD_ERR_INVALID_ARG, NPD_ERR_UNSUPPORTED, NPD_ERR_CUDA, NPD_ERR_WORKSPACE = 1, 2, 3, 4
NPD_DTYPE_F16, NPD_DTYPE_BF16, NPD_DTYPE_F32 = 0, 1, 2
NPD_STATUS_BAD_BLOCK_ID, NPD_STATUS_BAD_POSITION, NPD_STATUS_WAIT_TIMEOUT = 1, 2, 4
NPD_DECODE_KV_INTERLEAVED = 2

# name -> (restype, argtypes); the order mirrors include/nanopd_b200.h
SIGNATURES = {
    "npd_version": (c_int, []),
    "npd_last_error": (c_char_p, []),
    "npd_read_status": (c_int, [c_void_p, POINTER(c_int32), c_void_p]),
    "npd_kv_store": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                             c_int64, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "npd_decode_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int]),
    "npd_paged_decode_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                           c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                           c_int64, c_int64, c_int, c_void_p, c_size_t, c_int, c_void_p]),
    "npd_decode_static_scratch_bytes": (c_size_t, []),
    "npd_paged_decode_attention_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                                  c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                                  c_int64, c_int64, c_int, c_void_p, c_int, c_void_p]),
    "npd_prefill_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int]),
    "npd_paged_prefill_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            POINTER(c_int32), POINTER(c_int32), POINTER(c_int32),
                                            c_int64, c_float, c_int64, c_int64, c_int64, c_int64, c_int64,
                                            c_int64, c_int64, c_int64, c_int, c_void_p, c_size_t, c_int, c_void_p]),
    "npd_kv_migrate": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                               c_int64, c_int64, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                               c_int, c_void_p, c_void_p]),
    "npd_testing_kv_migrate_withheld": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                                c_int64, c_int64, c_int, c_int64, c_int64, c_int64, c_int64, c_int64,
                                                c_int64, c_int, c_void_p, c_void_p, c_int64, c_int64]),
    "npd_qk_norm_rope_store": (c_int, [c_void_p] * 8 + [c_float] + [c_void_p] * 4 + [c_int64] * 14 +
                               [c_int, c_void_p, c_void_p]),
    "npd_top_k_sample_workspace_bytes": (c_int64, [c_int64, c_int64, c_int]),
    "npd_top_k_sample": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p,
                                 c_int64, c_void_p]),
    "npd_enable_peer_access": (c_int, [c_int]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the library once; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m nanopd_b200._build` "
                "(needs nvcc; the library targets sm_100a).  There is no CPU fallback.")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(rc: int) -> None:
    """Turns a non-zero return code into RuntimeError, the error type the reference's
    TORCH_CHECKs surface in Python (nanoPD/paged_attention/csrc/attention/paged_attention_ops.cu:18-22)."""
    if rc != NPD_OK:
        msg = load().npd_last_error()
        raise RuntimeError(f"nanopd_b200 error {rc}: {msg.decode() if msg else 'unknown'}")
