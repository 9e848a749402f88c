"""ctypes binding of ``libarcq_b200.so`` (the C ABI declared in ``include/arcq_b200.h``).

There is no fallback: if the library is missing or fails to load, importing
the ops raises with the build command.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libarcq_b200.so"

DT_F32, DT_F16, DT_BF16 = 0, 1, 2

# every symbol include/arcq_b200.h declares
EXPORTS = (
    "arcq_version", "arcq_last_error_string", "arcq_device_status", "arcq_debug_trace", "arcq_debug_set_option", "arcq_debug_get_option", "arcq_debug_last_gemm_kernel", "arcq_debug_wait_timeout", "arcq_act_quant", "arcq_gelu_act_quant", "arcq_packed_gemm", "arcq_packed_weight_gemm", "arcq_dense_weight_gemm", "arcq_packed_linear_static_scratch", "arcq_add_layernorm", "arcq_add_layernorm_act_quant", "arcq_attention", "arcq_attention_act_quant", "arcq_patchify", "arcq_assemble_tokens",
    "arcq_unpack_codes", "arcq_pack_codes", "arcq_dequant", "arcq_unpack_weight_f16", "arcq_dense_weight_gemm_prefetch",
)

_lib = None


class ArcqLibraryMissing(ImportError):
    pass


def load() -> ctypes.CDLL:
    """Load the shared library once and declare the argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ArcqLibraryMissing(
            f"{LIB_PATH} is not built. Build it with `python {PKG_DIR / 'build.py'}` "
            "(needs nvcc with sm_100a support); there is no CPU or PyTorch fallback for this path.")
    lib = ctypes.CDLL(str(LIB_PATH))
    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.arcq_version.restype = ci
    lib.arcq_last_error_string.restype = ctypes.c_char_p
    lib.arcq_device_status.restype = ci
    lib.arcq_debug_trace.argtypes = [vp]
    lib.arcq_debug_set_option.argtypes = [ctypes.c_char_p, ci]
    lib.arcq_debug_get_option.argtypes = [ctypes.c_char_p, ctypes.POINTER(ci)]
    lib.arcq_debug_last_gemm_kernel.argtypes = []
    lib.arcq_debug_wait_timeout.argtypes = [ctypes.c_uint, vp]
    lib.arcq_act_quant.argtypes = [vp, ci, i64, i64, vp, vp, ci, ci, vp, vp, vp, vp, vp, ci, vp]
    lib.arcq_gelu_act_quant.argtypes = lib.arcq_act_quant.argtypes
    lib.arcq_packed_gemm.argtypes = [vp] * 11 + [ci, ci, i64, i64, i64, vp, ci, vp]
    lib.arcq_packed_weight_gemm.argtypes = [vp] * 7 + [ci, ci, i64, i64, i64, vp, ci, vp]
    lib.arcq_dense_weight_gemm.argtypes = [vp, vp, vp, i64, i64, i64, vp, ci, vp]
    lib.arcq_packed_linear_static_scratch.argtypes = lib.arcq_packed_weight_gemm.argtypes
    lib.arcq_add_layernorm.argtypes = [vp, vp, vp, vp, ctypes.c_float, i64, i64, vp, vp, vp]
    lib.arcq_add_layernorm_act_quant.argtypes = [vp, vp, vp, vp, ctypes.c_float, i64, i64, vp, vp, ci, ci, vp, vp, vp, vp]
    lib.arcq_attention.argtypes = [vp, i64, i64, i64, ci, vp, vp]
    lib.arcq_attention_act_quant.argtypes = [vp, i64, i64, i64, ci, vp, vp, ci, ci, vp, vp]
    lib.arcq_patchify.argtypes = [vp, i64, i64, i64, i64, ci, vp, vp]
    lib.arcq_assemble_tokens.argtypes = [vp, vp, vp, i64, i64, i64, vp, vp]
    lib.arcq_unpack_codes.argtypes = [vp, i64, i64, ci, vp, vp]
    lib.arcq_pack_codes.argtypes = [vp, i64, i64, ci, vp, vp]
    lib.arcq_dequant.argtypes = [vp, vp, vp, vp, vp, ci, ci, i64, i64, vp, ci, vp]
    lib.arcq_unpack_weight_f16.argtypes = [vp, vp, vp, vp, vp, ci, ci, i64, i64, vp, vp]
    lib.arcq_dense_weight_gemm_prefetch.argtypes = [vp, vp, vp, i64, i64, i64, vp, ci, vp, vp, vp, vp, vp, ci, ci, i64, i64, vp, vp]
    for name in EXPORTS:
        getattr(lib, name)  # AttributeError here means header and library disagree
    _lib = lib
    return lib


def last_error() -> str:
    return load().arcq_last_error_string().decode("utf-8", "replace")


def set_option(name: str, value: int) -> None:
    """Override one tuning option of the library (see ``arcq_debug_set_option`` in the header)."""
    if load().arcq_debug_set_option(name.encode(), int(value)) != 0:
        raise ValueError(last_error())


def get_option(name: str) -> int:
    v = ctypes.c_int(0)
    if load().arcq_debug_get_option(name.encode(), ctypes.byref(v)) != 0:
        raise ValueError(last_error())
    return int(v.value)


class option:
    """``with option("ARCQ_ACT_QUANT_V1", 1): ...`` -- set a tuning option for a block, then restore it."""

    def __init__(self, name: str, value: int):
        self.name, self.value = name, value

    def __enter__(self):
        self.old = get_option(self.name)
        set_option(self.name, self.value)
        return self

    def __exit__(self, *exc):
        set_option(self.name, self.old)
        return False


GEMM_ONE_CTA_PACKED, GEMM_ONE_CTA_DENSE, GEMM_PAIR_PACKED, GEMM_PAIR_DENSE, GEMM_PAIR_DENSE_PREFETCH = 1, 2, 3, 4, 5


def last_gemm_kernel() -> int:
    """Which kernel form the last GEMM entry point called from this thread launched (see the header)."""
    return int(load().arcq_debug_last_gemm_kernel())
