"""B200-native (sm_100a) arbitrary-precision packed-bit GEMM and convolution: the hot path
of APNN-TC behind its own operator surface.

The compute lives in ``libapnn_b200.so`` (hand-written CUDA behind a C ABI, declared in
``include/apnn_b200.h``).  This package is the thin host-side mirror of the reference's
operator names over torch device tensors; torch is used for device memory, streams and
``torch.distributed`` only.
"""
from . import _cabi
from ._cabi import ApnnError, Epilogue  # noqa: F401
from .ops import (  # noqa: F401
    APConv_w1a2_pack, APConv_w1a2_pack_pool, APConv_w2a2_pack, APConv_w2a2_pack_pool, Bit_compression, HostHandle,
    apconv, apmm, conv_check, conv_workspace_bytes, apmm_w1a2, apmm_w1a2_decompose, apmm_w1a3, apmm_w1a4, apmm_w2a2, apmm_w2a2_decompose, expand_planes, expand_planes_fp4, gemm_fp4, gemm_i8, gemm_w8,
    gemm_check, gemm_workspace_bytes, images_quantization, make_epilogue,
)

__all__ = [n for n in dir() if not n.startswith("_")]
