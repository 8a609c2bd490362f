"""Host-side mirror of the reference's operator surface over torch device tensors.

Names and argument meaning follow the reference (paths inside the APNN-TC project):

* ``apmm_w1a2`` / ``apmm_w2a2`` / ``apmm_w1a4`` -- ``APNN-TC-lib/bmmaTensorCoreGemm/src/71,72,78_bmmaTensorCoreGemm.cu:80``
  (``(W, X, D, M_GLOBAL, N_GLOBAL, K_GLOBAL, wb, xb)``), plus ``apmm_w1a3``;
* ``apmm_w1a2_decompose`` / ``apmm_w2a2_decompose`` -- ``66_bmmaTensorCoreGemm.cuh:81``, ``73_...cuh:81``;
* ``APConv_w1a2_pack[_pool]`` / ``APConv_w2a2_pack[_pool]`` -- ``67_...cu:58``, ``68_...cu:58``, ``70_...cu:58``,
  ``69_...cuh:59`` (``(W, X, Output, Height, Width, CIN, COUT)``);
* ``Bit_compression`` / ``images_quantization`` -- ``APNN-TC-nn/src/kernel.cuh:46-77``, ``:129-161``.

Tensors are ``torch.int32`` words holding the reference's uint32 bit patterns, on a CUDA
device, in the reference's layouts (planes outermost).  Every call goes through the C ABI
on the current torch stream; nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _cabi
from ._cabi import Epilogue


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dev_words(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype not in (torch.int32, torch.uint32):
        raise ValueError(f"{name} must hold 32-bit words (torch.int32)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def make_epilogue(out_mode: str = "int32", out_bits: int = 0, signed: str = "none", pool: str = "none",
                  out_halo: int = 0, in_halo: int = 0, thresholds: Optional[torch.Tensor] = None,
                  residual_in: Optional[torch.Tensor] = None, residual_out: Optional[torch.Tensor] = None,
                  peer_out: Optional[list] = None, out_i8: bool = False, residual_i16: int = 0,
                  affine_scale: Optional[torch.Tensor] = None, affine_bias: Optional[torch.Tensor] = None) -> Epilogue:
    """Build the fused-epilogue descriptor.

    out_mode: "int32" | "lowbits" (the reference's ``val & (2^bits-1)``) | "thresholds" |
              "float" (float(value) * affine_scale[c] + affine_bias[c]; gemm_i8 / conv2d_i8 only)
    signed:   "none" | "w" | "x" -- which argument's bits mean -1/+1
    pool:     "none" | "avg" (reference: truncating (a+b+c+d)/4 before requantisation) | "max"
    residual_in / residual_out: dense int32 [rows, channels] added before / saved after the add
    peer_out: raw device addresses that also receive every output tile (tcgen05 pair GEMM only)
    """
    e = Epilogue()
    e.out_mode = {"int32": 0, "lowbits": 1, "thresholds": 2, "float": 3}[out_mode]
    e.out_bits = out_bits
    e.signed_operand = {"none": 0, "w": 1, "x": 2}[signed]
    e.pool = {"none": 0, "avg": 1, "max": 2}[pool]
    e.out_halo = out_halo
    e.in_halo = in_halo
    e.thresholds = thresholds.data_ptr() if thresholds is not None else None
    e.residual_in = residual_in.data_ptr() if residual_in is not None else None
    e.residual_out = residual_out.data_ptr() if residual_out is not None else None
    e.residual_i16 = int(residual_i16)   # bit 0: residual_in is int16, bit 1: residual_out is int16 (gemm_i8 / conv2d_i8)
    e.out_i8 = 1 if out_i8 else 0   # one byte per output element instead of packed planes (gemm_i8 / conv2d_i8)
    if peer_out:
        if len(peer_out) > 7:
            raise ValueError("at most 7 peer destinations")
        e.n_peer_out = len(peer_out)
        for i, ptr in enumerate(peer_out):   # raw device addresses (peer-mapped memory)
            e.peer_out[i] = int(ptr)
    e.affine_scale = affine_scale.data_ptr() if affine_scale is not None else None
    e.affine_bias = affine_bias.data_ptr() if affine_bias is not None else None
    e._keepalive = (thresholds, residual_in, residual_out, affine_scale, affine_bias)
    return e


def gemm_workspace_bytes(M: int, N: int, K: int, wbits: int = 1, xbits: int = 2, algo: str = "tcgen05") -> int:
    return int(_cabi.lib().apnn_gemm_workspace_bytes(_cabi.ALGOS[algo], wbits, xbits, M, N, K))


def gemm_check(workspace: torch.Tensor, M: int, N: int, K: int) -> None:
    """Synchronise and raise if the tcgen05 GEMM that last used ``workspace`` gave up on a wait."""
    _cabi.check(_cabi.lib().apnn_gemm_check(_stream_ptr(), workspace.data_ptr(), M, N, K), "apnn_gemm_check")


def expand_planes(planes: torch.Tensor, signed: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """planes [bits, rows, K/32] -> int8 [rows, K] (one byte per element) for ``gemm_i8``."""
    planes = _dev_words(planes, "planes")
    bits, rows, kw = planes.shape
    if out is None:
        out = torch.empty((rows, kw * 32), dtype=torch.uint8, device=planes.device)
    st = _cabi.lib().apnn_expand_planes(_stream_ptr(), planes.data_ptr(), out.data_ptr(), rows, kw * 32, bits,
                                        1 if signed else 0)
    _cabi.check(st, "apnn_expand_planes")
    return out


def gemm_i8(W8: torch.Tensor, X8: torch.Tensor, out: Optional[torch.Tensor] = None, *, w_signed: bool = False,
            x_signed: bool = False, epilogue: Optional[Epilogue] = None,
            status_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    """tcgen05 kind::i8 GEMM over operands produced by ``expand_planes``."""
    M, K = W8.shape
    N, K2 = X8.shape
    if K != K2:
        raise ValueError("operands disagree on K")
    packed = epilogue is not None and epilogue.out_mode in (1, 2)
    if out is None:
        shape = (epilogue.out_bits, M, N // 32) if packed else (M, N)
        is_float = epilogue is not None and epilogue.out_mode == 3
        out = torch.empty(shape, dtype=torch.float32 if is_float else torch.int32, device=W8.device)
    if status_flag is None:
        status_flag = torch.empty(1, dtype=torch.int32, device=W8.device)
    st = _cabi.lib().apnn_gemm_i8(_stream_ptr(), W8.data_ptr(), X8.data_ptr(), out.data_ptr(), M, N, K,
                                  1 if w_signed else 0, 1 if x_signed else 0,
                                  ctypes.byref(epilogue) if epilogue is not None else None, status_flag.data_ptr())
    _cabi.check(st, "apnn_gemm_i8")
    return out


def expand_planes_fp4(planes: torch.Tensor, signed: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """planes [bits <= 2, rows, K/32] -> e2m1 nibbles [rows, K/2] (two elements per byte) for ``gemm_fp4``."""
    planes = _dev_words(planes, "planes")
    bits, rows, kw = planes.shape
    if out is None:
        out = torch.empty((rows, kw * 16), dtype=torch.uint8, device=planes.device)
    st = _cabi.lib().apnn_expand_planes_fp4(_stream_ptr(), planes.data_ptr(), out.data_ptr(), rows, kw * 32, bits,
                                            1 if signed else 0)
    _cabi.check(st, "apnn_expand_planes_fp4")
    return out


def gemm_fp4(W4: torch.Tensor, X4: torch.Tensor, out: Optional[torch.Tensor] = None, *,
             epilogue: Optional[Epilogue] = None, status_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exact GEMM of operands of at most two bits on the 4-bit floating-point tensor path (kind::mxf4, unit
    scales): twice the int8 rate, sums exact in fp32.  Operands from ``expand_planes_fp4``."""
    M, kb = W4.shape
    N, kb2 = X4.shape
    if kb != kb2:
        raise ValueError("operands disagree on K")
    packed = epilogue is not None and epilogue.out_mode in (1, 2)
    if out is None:
        shape = (epilogue.out_bits, M, N // 32) if packed else (M, N)
        out = torch.empty(shape, dtype=torch.int32, device=W4.device)
    if status_flag is None:
        status_flag = torch.empty(1, dtype=torch.int32, device=W4.device)
    st = _cabi.lib().apnn_gemm_fp4(_stream_ptr(), W4.data_ptr(), X4.data_ptr(), out.data_ptr(), M, N, kb * 2,
                                   ctypes.byref(epilogue) if epilogue is not None else None, status_flag.data_ptr())
    _cabi.check(st, "apnn_gemm_fp4")
    return out


def gemm_w8(W8: torch.Tensor, X: torch.Tensor, out: Optional[torch.Tensor] = None, *, w_signed: bool = False,
            x_signed: bool = False, epilogue: Optional[Epilogue] = None,
            status_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    """GEMM of a layer with static weights: ``W8`` from ``expand_planes`` (made once), the activations ``X``
    as packed planes [xbits, N, K/32]; the CTA-pair kernel spreads the planes itself."""
    X = _dev_words(X, "X")
    M, K = W8.shape
    xbits, N, kw = X.shape
    if K != kw * 32:
        raise ValueError("operands disagree on K")
    packed = epilogue is not None and epilogue.out_mode in (1, 2)
    if out is None:
        shape = (epilogue.out_bits, M, N // 32) if packed else (M, N)
        out = torch.empty(shape, dtype=torch.int32, device=W8.device)
    if status_flag is None:
        status_flag = torch.empty(1, dtype=torch.int32, device=W8.device)
    st = _cabi.lib().apnn_gemm_w8(_stream_ptr(), W8.data_ptr(), xbits, X.data_ptr(), out.data_ptr(), M, N, K,
                                  1 if w_signed else 0, 1 if x_signed else 0,
                                  ctypes.byref(epilogue) if epilogue is not None else None, status_flag.data_ptr())
    _cabi.check(st, "apnn_gemm_w8")
    return out


def apmm(W: torch.Tensor, X: torch.Tensor, out: Optional[torch.Tensor] = None, *, epilogue: Optional[Epilogue] = None,
         algo: str = "auto", workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """D[m][n] = sum_wb sum_xb 2^(wb+xb) popcount(W[wb][m] & X[xb][n]).

    W: [wbits, M, K/32], X: [xbits, N, K/32].  Returns int32 [M, N], or packed
    [out_bits, M, N/32] when the epilogue requantises.
    """
    W = _dev_words(W, "W")
    X = _dev_words(X, "X")
    wbits, M, kw = W.shape
    xbits, N, kw2 = X.shape
    if kw != kw2:
        raise ValueError("W and X disagree on K")
    K = kw * 32
    packed = epilogue is not None and epilogue.out_mode != 0
    if out is None:
        if packed:
            out = torch.empty((epilogue.out_bits, M, N // 32), dtype=torch.int32, device=W.device)
        else:
            out = torch.empty((M, N), dtype=torch.int32, device=W.device)
    ws_ptr, ws_bytes = None, 0
    if workspace is not None:
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    st = _cabi.lib().apnn_gemm_ex(_stream_ptr(), _cabi.ALGOS[algo], wbits, xbits, W.data_ptr(), X.data_ptr(),
                                  out.data_ptr(), M, N, K, ctypes.byref(epilogue) if epilogue is not None else None,
                                  ws_ptr, ws_bytes)
    _cabi.check(st, "apnn_gemm_ex")
    return out


def _apmm_fixed(wb: int, xb: int):
    def fn(W, X, D=None, M_GLOBAL=None, N_GLOBAL=None, K_GLOBAL=None, wb_=wb, xb_=xb, **kw):
        if W.shape[0] != wb or X.shape[0] != xb:
            raise ValueError(f"expected {wb}-bit W and {xb}-bit X planes")
        for given, actual, nm in ((M_GLOBAL, W.shape[1], "M"), (N_GLOBAL, X.shape[1], "N"),
                                  (K_GLOBAL, W.shape[2] * 32, "K")):
            if given is not None and given != actual:
                raise ValueError(f"{nm}_GLOBAL={given} does not match the tensor ({actual})")
        return apmm(W, X, D, **kw)
    fn.__name__ = f"apmm_w{wb}a{xb}"
    fn.__doc__ = f"int32 GEMM for {wb}-bit W and {xb}-bit X; arguments as the reference kernel of the same name."
    return fn


apmm_w1a2 = _apmm_fixed(1, 2)
apmm_w1a3 = _apmm_fixed(1, 3)
apmm_w1a4 = _apmm_fixed(1, 4)
apmm_w2a2 = _apmm_fixed(2, 2)


def apmm_w1a2_decompose(W, X, D=None, **kw):
    """GEMM + low-2-bit requantisation packed along N (FC_new_global's kernel)."""
    return apmm(W, X, D, epilogue=make_epilogue("lowbits", 2), **kw)


def apmm_w2a2_decompose(W, X, D=None, **kw):
    return apmm(W, X, D, epilogue=make_epilogue("lowbits", 2), **kw)


def conv_workspace_bytes(B: int, H: int, W: int, CIN: int, COUT: int, R: int = 3) -> int:
    return int(_cabi.lib().apnn_conv2d_workspace_bytes(_cabi.ALGO_TCGEN05, B, H, W, CIN, COUT, R))


def conv_check(workspace: torch.Tensor, B: int, H: int, W: int, CIN: int, COUT: int, R: int = 3) -> None:
    """Synchronise and raise if the tcgen05 conv that last used ``workspace`` gave up on a wait."""
    _cabi.check(_cabi.lib().apnn_conv2d_check(_stream_ptr(), workspace.data_ptr(), B, H, W, CIN, COUT, R),
                "apnn_conv2d_check")


def apconv(Wt: torch.Tensor, X: torch.Tensor, out: Optional[torch.Tensor] = None, *, stride: int = 1,
           epilogue: Optional[Epilogue] = None, algo: str = "imma",
           workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Implicit-GEMM convolution over packed NHWC planes.

    X: [xbits, B, H+2p, W+2p, CIN/32] (halo stored), Wt: [wbits, COUT, R, R, CIN/32].
    Returns int32 [B, Ho, Wo, COUT] or packed [out_bits, B, Ho', Wo', COUT/32] (Ho', Wo'
    include pooling and the optional output ring, which is zero-filled here).
    """
    X = _dev_words(X, "X")
    Wt = _dev_words(Wt, "Wt")
    xbits, B, Hp, Wp, cw = X.shape
    wbits, COUT, R, R2, cw2 = Wt.shape
    if R != R2 or cw != cw2:
        raise ValueError("filter must be square and agree with X on CIN")
    p = (R - 1) // 2
    H, Wd = Hp - 2 * p, Wp - 2 * p
    Ho, Wo = (H - 1) // stride + 1, (Wd - 1) // stride + 1
    pool = epilogue.pool if epilogue is not None else 0
    halo = epilogue.out_halo if epilogue is not None else 0
    oh, ow = (Ho // 2, Wo // 2) if pool else (Ho, Wo)
    packed = epilogue is not None and epilogue.out_mode != 0
    if out is None:
        shape = (B, oh + 2 * halo, ow + 2 * halo)
        if packed:
            shape = (epilogue.out_bits,) + shape + (COUT // 32,)
        else:
            shape = shape + (COUT,)
        out = (torch.zeros if halo else torch.empty)(shape, dtype=torch.int32, device=X.device)
    ws_ptr, ws_bytes = None, 0
    if workspace is not None:
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    st = _cabi.lib().apnn_conv2d_ex(_stream_ptr(), _cabi.ALGOS[algo], wbits, xbits, Wt.data_ptr(), X.data_ptr(),
                                    out.data_ptr(), B, H, Wd, cw * 32, COUT, R, stride,
                                    ctypes.byref(epilogue) if epilogue is not None else None, ws_ptr, ws_bytes)
    _cabi.check(st, "apnn_conv2d_ex")
    return out


def _apconv_pack(wb: int, xb: int, pool: bool):
    def fn(W, X, Output=None, Height=None, Width=None, CIN=None, COUT=None):
        if W.shape[0] != wb or X.shape[0] != xb:
            raise ValueError(f"expected {wb}-bit W and {xb}-bit X planes")
        if W.dim() == 3:  # reference shape [wb][COUT][9*CIN/32]
            W = W.view(wb, W.shape[1], 3, 3, W.shape[2] // 9)
        if X.dim() == 4:  # reference shape [xb][H+2][W+2][CIN/32]: one image
            X = X.unsqueeze(1)
        return apconv(W, X, Output, epilogue=make_epilogue("lowbits", xb, pool="avg" if pool else "none"))
    fn.__name__ = f"APConv_w{wb}a{xb}_pack" + ("_pool" if pool else "")
    fn.__doc__ = "3x3 stride-1 conv over a pre-haloed image + low-bit requantisation packed along COUT" + \
                 (" after a truncating 2x2 average" if pool else "") + "; arguments as the reference kernel."
    return fn


APConv_w1a2_pack = _apconv_pack(1, 2, False)
APConv_w1a2_pack_pool = _apconv_pack(1, 2, True)
APConv_w2a2_pack = _apconv_pack(2, 2, False)
APConv_w2a2_pack_pool = _apconv_pack(2, 2, True)


def Bit_compression(qnt: torch.Tensor, bit: int = 2, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """levels [..., C] (one 32-bit word per element) -> planes [bit, ..., PAD128(C)/32]."""
    qnt = _dev_words(qnt, "qnt")
    C = qnt.shape[-1]
    rows = qnt.numel() // C
    cw = (C + 127) // 128 * 4
    if out is None:
        out = torch.empty((bit,) + tuple(qnt.shape[:-1]) + (cw,), dtype=torch.int32, device=qnt.device)
    st = _cabi.lib().apnn_bit_compress(_stream_ptr(), qnt.data_ptr(), out.data_ptr(), rows, C, bit)
    _cabi.check(st, "apnn_bit_compress")
    return out


def images_quantization(images: torch.Tensor, bit: int = 2, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float NHWC images -> planes [bit, N, H, W, PAD128(C)/32]: Quantize_val fused with Bit_compression."""
    if not images.is_cuda or images.dtype != torch.float32 or not images.is_contiguous():
        raise ValueError("images must be a contiguous float32 CUDA tensor")
    C = images.shape[-1]
    rows = images.numel() // C
    cw = (C + 127) // 128 * 4
    if out is None:
        out = torch.empty((bit,) + tuple(images.shape[:-1]) + (cw,), dtype=torch.int32, device=images.device)
    st = _cabi.lib().apnn_quantize_pack(_stream_ptr(), images.data_ptr(), out.data_ptr(), rows, C, bit)
    _cabi.check(st, "apnn_quantize_pack")
    return out


class HostHandle:
    """Host-buffer front end (``apnn_create`` / ``apnn_gemm_host``): operands and results are
    host arrays (numpy or pinned torch CPU tensors); copies happen inside the call."""

    def __init__(self, device: int = 0):
        self._h = ctypes.c_void_p()
        _cabi.check(_cabi.lib().apnn_create(ctypes.byref(self._h), device), "apnn_create")

    def close(self):
        if self._h:
            _cabi.lib().apnn_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _ptr(a):
        return a.data_ptr() if isinstance(a, torch.Tensor) else a.ctypes.data

    def gemm(self, W, X, D, wbits, xbits, M, N, K, algo="auto", epilogue: Optional[Epilogue] = None):
        st = _cabi.lib().apnn_gemm_host(self._h, _cabi.ALGOS[algo], wbits, xbits, self._ptr(W), self._ptr(X),
                                        self._ptr(D), M, N, K, ctypes.byref(epilogue) if epilogue is not None else None)
        _cabi.check(st, "apnn_gemm_host")
        return D

    def conv2d(self, Wt, X, Out, wbits, xbits, B, H, Wd, CIN, COUT, R=3, stride=1, epilogue: Optional[Epilogue] = None):
        st = _cabi.lib().apnn_conv2d_host(self._h, wbits, xbits, self._ptr(Wt), self._ptr(X), self._ptr(Out), B, H, Wd,
                                          CIN, COUT, R, stride, ctypes.byref(epilogue) if epilogue is not None else None)
        _cabi.check(st, "apnn_conv2d_host")
        return Out
