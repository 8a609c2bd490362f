"""ctypes binding of ``libapnn_b200.so`` (the C ABI declared in ``include/apnn_b200.h``).

There is no fallback: if the shared object is missing or a call fails, an exception is
raised.  ``python -m apnn_tc_b200.build`` produces the library.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libapnn_b200.so")

# enums of include/apnn_b200.h
OUT_INT32, OUT_LOWBITS, OUT_THRESHOLDS, OUT_FLOAT = 0, 1, 2, 3
QUANT_CENTRED = 0x100   # flag in the `bits` argument of the first-layer int8 gathers
SIGN_NONE, SIGN_W, SIGN_X = 0, 1, 2
POOL_NONE, POOL_AVG2, POOL_MAX2 = 0, 1, 2
ALGO_AUTO, ALGO_BMMA, ALGO_IMMA, ALGO_TCGEN05, ALGO_TCGEN05_PAIR = 0, 1, 2, 3, 4
ALGOS = {"auto": ALGO_AUTO, "bmma": ALGO_BMMA, "imma": ALGO_IMMA, "tcgen05": ALGO_TCGEN05, "tcgen05_pair": ALGO_TCGEN05_PAIR}

# every symbol the header declares; the CPU test-suite checks the library exports them all
EXPORTS = (
    "apnn_status_string", "apnn_last_cuda_error", "apnn_version", "apnn_gemm", "apnn_gemm_ex",
    "apnn_gemm_workspace_bytes", "apnn_gemm_check", "apnn_expand_planes", "apnn_expand_planes_pair", "apnn_gemm_i8", "apnn_gemm_w8", "apnn_expand_planes_fp4", "apnn_gemm_fp4", "apnn_gemm_static_scratch", "apnn_conv2d", "apnn_conv2d_ex",
    "apnn_conv2d_workspace_bytes", "apnn_conv2d_check", "apnn_conv2d_i8", "apnn_bit_compress", "apnn_quantize_pack", "apnn_quantize_im2col", "apnn_create",
    "apnn_destroy", "apnn_gemm_host", "apnn_conv2d_host", "apnn_probe_peak", "apnn_quantize_im2col_i8", "apnn_quantize_window_rows_i8", "apnn_quantize_blocks_i8", "apnn_maxpool2x2_i8", "apnn_requantize_i32",
)


class Epilogue(ctypes.Structure):
    """``apnn_epilogue``; ``struct_size`` is filled in on construction (APNN_EPILOGUE_INIT)."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("out_mode", ctypes.c_int32),
        ("out_bits", ctypes.c_int32),
        ("signed_operand", ctypes.c_int32),
        ("pool", ctypes.c_int32),
        ("out_halo", ctypes.c_int32),
        ("in_halo", ctypes.c_int32),
        ("thresholds", ctypes.c_void_p),
        ("residual_in", ctypes.c_void_p),
        ("residual_out", ctypes.c_void_p),
        ("n_peer_out", ctypes.c_int32),
        ("out_i8", ctypes.c_int32),
        ("peer_out", ctypes.c_void_p * 7),
        ("residual_i16", ctypes.c_int32),
        ("affine_scale", ctypes.c_void_p),
        ("affine_bias", ctypes.c_void_p),
    ]

    def __init__(self, *args, **kw):
        super().__init__(*args, **kw)
        self.struct_size = ctypes.sizeof(Epilogue)


class ApnnError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(text)
        self.status = status


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m apnn_tc_b200.build` (there is no CPU fallback)")
    L = ctypes.CDLL(LIB_PATH)
    vp, i, sz, lg = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_long
    ep = ctypes.POINTER(Epilogue)
    L.apnn_status_string.restype = ctypes.c_char_p
    L.apnn_status_string.argtypes = [i]
    L.apnn_last_cuda_error.restype = ctypes.c_char_p
    L.apnn_version.restype = i
    L.apnn_gemm.argtypes = [vp, i, i, vp, vp, vp, i, i, i]
    L.apnn_gemm_ex.argtypes = [vp, i, i, i, vp, vp, vp, i, i, i, ep, vp, sz]
    L.apnn_gemm_workspace_bytes.restype = sz
    L.apnn_gemm_workspace_bytes.argtypes = [i, i, i, i, i, i]
    L.apnn_gemm_check.argtypes = [vp, vp, i, i, i]
    L.apnn_expand_planes.argtypes = [vp, vp, vp, lg, i, i, i]
    L.apnn_expand_planes_pair.argtypes = [vp, vp, vp, lg, i, i, vp, vp, lg, i, i, i]
    L.apnn_gemm_i8.argtypes = [vp, vp, vp, vp, i, i, i, i, i, ep, vp]
    L.apnn_gemm_w8.argtypes = [vp, vp, i, vp, vp, i, i, i, i, i, ep, vp]
    L.apnn_expand_planes_fp4.argtypes = [vp, vp, vp, lg, i, i, i]
    L.apnn_gemm_fp4.argtypes = [vp, vp, vp, vp, i, i, i, ep, vp]
    L.apnn_gemm_static_scratch.argtypes = [vp, i, i, vp, vp, vp, i, i, i, ep, vp]
    L.apnn_conv2d.argtypes = [vp, i, i, vp, vp, vp, i, i, i, i, i, i, i, ep]
    L.apnn_conv2d_ex.argtypes = [vp, i, i, i, vp, vp, vp, i, i, i, i, i, i, i, ep, vp, sz]
    L.apnn_conv2d_workspace_bytes.restype = sz
    L.apnn_conv2d_workspace_bytes.argtypes = [i, i, i, i, i, i, i]
    L.apnn_conv2d_check.argtypes = [vp, vp, i, i, i, i, i, i]
    L.apnn_conv2d_i8.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, i, i, ep, vp]
    L.apnn_bit_compress.argtypes = [vp, vp, vp, lg, i, i]
    L.apnn_quantize_pack.argtypes = [vp, vp, vp, lg, i, i]
    L.apnn_probe_peak.argtypes = [vp, i, i, vp, ctypes.POINTER(ctypes.c_double)]
    L.apnn_quantize_im2col.argtypes = [vp, vp, vp, i, i, i, i, i, i, i]
    L.apnn_quantize_im2col_i8.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, i]
    L.apnn_quantize_window_rows_i8.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, i]
    L.apnn_quantize_blocks_i8.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, i]
    L.apnn_maxpool2x2_i8.argtypes = [vp, vp, vp, i, i, i, i, i, i]
    L.apnn_requantize_i32.argtypes = [vp, vp, vp, ctypes.c_long, i, vp]
    L.apnn_create.argtypes = [ctypes.POINTER(vp), i]
    L.apnn_destroy.argtypes = [vp]
    L.apnn_gemm_host.argtypes = [vp, i, i, i, vp, vp, vp, i, i, i, ep]
    L.apnn_conv2d_host.argtypes = [vp, i, i, vp, vp, vp, i, i, i, i, i, i, i, ep]
    _lib = L
    return L


def check(status: int, what: str = "") -> None:
    if status != 0:
        L = lib()
        text = L.apnn_status_string(status).decode()
        if status == 5:
            text += ": " + L.apnn_last_cuda_error().decode()
        raise ApnnError(status, f"{what}: {text}" if what else text)
