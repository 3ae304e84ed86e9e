"""ctypes binding of libdsa_b200.so (the C ABI declared in include/dsa_b200.h).

There is no fallback: if the shared library is missing the first use raises,
telling the caller to build it.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdsa_b200.so")

_lock = threading.Lock()
_lib = None

# name -> (restype, argtypes); kept in step with include/dsa_b200.h
SIGNATURES = {
    "dsa_version": (c_int, []),
    "dsa_last_error_string": (c_char_p, []),
    "dsa_fp8_quant_per_block": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
    "dsa_rope_fp8_quant": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p,
                                   c_void_p, c_void_p]),
    "dsa_indexer_logits": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                   c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "dsa_indexer_logits_paged": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                         c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                                         c_void_p, c_void_p]),
    "dsa_topk_select": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "dsa_indexer_topk_workspace_bytes": (c_size_t, [c_int, c_int]),
    "dsa_indexer_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                 c_int, c_int, c_int, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "dsa_sparse_mla_prefill": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                       c_void_p, c_void_p]),
    "dsa_block_sparse_mha": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                     c_int, c_int, c_float, c_void_p, c_void_p]),
    "dsa_sparse_mla_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "dsa_sparse_mla_decode_paged": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
                                            c_int, c_int, c_int, c_float, c_void_p, c_size_t, c_void_p, c_void_p]),
    "dsa_test_indexer_logits_general": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                c_void_p]),
    "dsa_test_topk_select_two_pass": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                              c_void_p]),
    "dsa_test_bounded_wait": (c_int, [c_int, c_void_p, c_void_p]),
    "dsa_indexer_topk_static_max_bytes": (c_size_t, []),
    "dsa_indexer_topk_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                        c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
}


class DsaError(RuntimeError):
    """A C-ABI call returned a negative status."""


def load():
    """Load the library once and set the prototypes.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -m llmdivedeep_b200.build` "
                    "(needs nvcc with sm_100a support). There is no CPU fallback.")
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        msg = load().dsa_last_error_string().decode()
        raise DsaError(f"libdsa_b200 error {rc}: {msg}")
