"""ctypes binding of libtq_b200.so (the C ABI declared in include/tq_b200.h).

There is no CPU or PyTorch fallback: if the shared library has not been built
(`python transformers-turboquant_b200/build.py`) importing this module raises.
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtq_b200.so")

TQ_OK = 0
TQ_F32, TQ_BF16, TQ_F16 = 0, 1, 2
TQ_MODE_FP32, TQ_MODE_BF16 = 0, 1


class TurboQuantError(RuntimeError):
    """A libtq_b200 entry point returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"libtq_b200 status {status}: {message}")
        self.status = status


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found: build the CUDA library first with "
        "`python transformers-turboquant_b200/build.py` (needs nvcc; no GPU required to build)")

lib = C.CDLL(LIB_PATH)

_p, _i, _l, _f, _z = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/tq_b200.h declaration by declaration
SIGNATURES = {
    "tq_version": (_i, []),
    "tq_last_error": (C.c_char_p, []),
    "tq_device_fault_count": (_i, [_p, C.POINTER(C.c_int64)]),
    "tq_selftest_wait_expiry": (_i, [_p, _l, C.POINTER(C.c_int64)]),
    "tq_trace_enable": (_i, [_i]),
    "tq_trace_read": (_i, [C.POINTER(C.c_int64), _i, C.POINTER(C.c_int)]),
    "tq_profile_begin": (_i, [_i]),
    "tq_profile_end": (_i, [C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "tq_pack_bits": (_i, [_p, _l, _i, _i, _p, _p]),
    "tq_unpack_bits": (_i, [_p, _l, _i, _i, _p, _p]),
    "tq_quantize_rotated": (_i, [_p, _l, _i, _p, _i, _p, _p]),
    "tq_dequantize": (_i, [_p, _l, _i, _p, _i, _p, _p]),
    "tq_constants_bytes": (_z, [_i, _i]),
    "tq_prepare_constants": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _p, _z, _p]),
    "tq_compress_kv": (_i, [_p, _p, _i, _l, _l, _l, _i, _l, _l, _l, _l, _l, _l, _p, _i, _p, _p, _p, _p, _p, _p,
                            _l, _l, _i, _p]),
    "tq_attention_prepared_workspace_bytes": (_z, [_l, _l, _l, _l, _l, _l, _i, _i]),
    "tq_attention_fwd_prepared": (_i, [_p, _i, _l, _l, _l, _i, _l, _l, _l, _l, _l, _l, _p, _p, _p, _p, _p, _p,
                                       _p, _i, _f, _i, _p, _l, _l, _p, _l, _l, _l, _p, _z, _i, _p]),
    "tq_compress_keys": (_i, [_p, _i, _l, _l, _l, _i, _l, _l, _l, _p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _p]),
    "tq_compress_values": (_i, [_p, _i, _l, _l, _l, _i, _l, _l, _l, _p, _p, _i, _p, _p, _i, _p]),
    "tq_append_keys": (_i, [_p, _i, _l, _l, _l, _i, _l, _l, _l, _p, _p, _p, _p, _i, _p, _p, _p, _p, _l, _l, _i, _p]),
    "tq_append_values": (_i, [_p, _i, _l, _l, _l, _i, _l, _l, _l, _p, _p, _i, _p, _p, _l, _l, _i, _p]),
    "tq_decompress_values": (_i, [_p, _p, _l, _i, _p, _p, _i, _p, _p]),
    "tq_attention_scores": (_i, [_p, _i, _l, _l, _l, _i, _l, _l, _l, _l, _l, _p, _p, _p, _p, _p, _p, _p, _i,
                                 _p, _p, _z, _i, _p]),
    "tq_prepare_queries": (_i, [_p, _i, _l, _l, _l, _i, _l, _l, _l, _p, _p, _p, _p, _z, _i, _p]),
    "tq_attention_workspace_bytes": (_z, [_l, _l, _l, _i, _i]),
    "tq_attention_fwd": (_i, [_p, _i, _l, _l, _l, _i, _l, _l, _l, _l, _l, _p, _p, _p, _p, _p, _p, _p, _p, _p,
                              _p, _p, _i, _f, _i, _p, _l, _l, _p, _l, _l, _l, _p, _z, _i, _p]),
    "tq_attention_fwd_cached": (_i, [_p, _i, _l, _l, _l, _i, _l, _l, _l, _l, _l, _l, _p, _p, _p, _p, _p, _p, _p, _p, _p,
                                     _p, _p, _i, _f, _i, _p, _l, _l, _p, _l, _l, _l, _p, _z, _p]),
    "tq_rope": (_i, [_p, _p, _i, _l, _l, _l, _l, _i, _l, _l, _l, _l, _l, _l, _p, _p, _l, _l, _p, _p, _p]),
    "tq_static_scratch_bytes": (_z, []),
    "tq_attention_fwd_static": (_i, [_p, _i, _l, _l, _l, _i, _l, _l, _l, _l, _l, _p, _p, _p, _p, _p, _p, _p, _p, _p,
                                     _p, _p, _i, _f, _i, _p, _l, _l, _p, _l, _l, _l, _i, _p]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here means the library and the header disagree
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.tq_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    if status != TQ_OK:
        raise TurboQuantError(status, last_error())


def version() -> int:
    return int(lib.tq_version())
