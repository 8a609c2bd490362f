"""ctypes front-end of the CPU oracle (``apnn_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, by the smoke entry and by
the benchmark's CPU-baseline / reference arm.  The product package never imports
this module and has no CPU fallback.

Every function takes and returns numpy arrays in the reference's layouts
(uint32 words, K or channel fastest, planes outermost); see the header of
``apnn_oracle.c`` for the layouts and for which results are pinned against the
reference's own host loops.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libapnn_oracle.so")
_lib = None

_u32p = ctypes.POINTER(ctypes.c_uint32)
_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)


def build(force: bool = False) -> str:
    """Compile ``apnn_oracle.c`` with gcc if the shared object is missing or stale."""
    src = os.path.join(_HERE, "apnn_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libapnn_oracle.so"])
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _u32(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data_as(_u32p)


def _i32(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_i32p)


def _opt_i32(a):
    if a is None:
        return None, None
    return _i32(a)


# ----------------------------------------------------------------------------- inputs
def rand_words(n: int, seed: int = 1) -> np.ndarray:
    """First ``n`` outputs of glibc ``rand()`` after ``srand(seed)`` (default seed = 1)."""
    out = np.empty(n, dtype=np.uint32)
    lib().apnn_oracle_rand_words(ctypes.c_uint32(seed), out.ctypes.data_as(_u32p), ctypes.c_long(n))
    return out


def fill_gemm(M, N, K, wbits, xbits, seed=1):
    """Operands of the reference GEMM programs: W[wb][M][K/32], X[xb][N][K/32]."""
    W = np.empty((wbits, M, K // 32), dtype=np.uint32)
    X = np.empty((xbits, N, K // 32), dtype=np.uint32)
    lib().apnn_oracle_fill_gemm(W.ctypes.data_as(_u32p), X.ctypes.data_as(_u32p), M, N, K, wbits, xbits,
                                ctypes.c_uint32(seed))
    return W, X


def fill_conv(H, Wd, CIN, COUT, xbits, wbits, seed=1):
    """Operands of the reference conv programs: X[xb][H+2][W+2][CIN/32] (halo ring
    random, as the reference leaves it) and Wt[wb][COUT][3][3][CIN/32]."""
    X = np.empty((xbits, 1, H + 2, Wd + 2, CIN // 32), dtype=np.uint32)
    Wt = np.empty((wbits, COUT, 3, 3, CIN // 32), dtype=np.uint32)
    lib().apnn_oracle_fill_conv(X.ctypes.data_as(_u32p), Wt.ctypes.data_as(_u32p), H, Wd, CIN, COUT, xbits, wbits,
                                ctypes.c_uint32(seed))
    return X, Wt


def value_planes(rng: np.random.Generator, rows: int, K: int, bits: int):
    """Seeded value-level operand: uniform levels in [0, 2^bits) split into planes,
    32 K-elements per word, lowest index in bit 31.  Returns (planes, levels)."""
    lv = rng.integers(0, 1 << bits, size=(rows, K), dtype=np.uint32)
    return pack_levels(lv, bits), lv


def pack_levels(lv: np.ndarray, bits: int) -> np.ndarray:
    """levels[..., K] -> planes[bits][..., K/32] (MSB-first), K a multiple of 32."""
    lv = np.ascontiguousarray(lv, dtype=np.uint32)
    K = lv.shape[-1]
    assert K % 32 == 0
    planes = []
    for b in range(bits):
        bitsarr = ((lv >> b) & 1).astype(np.uint8).reshape(*lv.shape[:-1], K // 32, 32)
        by = np.packbits(bitsarr, axis=-1, bitorder="big")  # [..., K/32, 4] big-endian bytes
        w = (by[..., 0].astype(np.uint32) << 24) | (by[..., 1].astype(np.uint32) << 16) | \
            (by[..., 2].astype(np.uint32) << 8) | by[..., 3].astype(np.uint32)
        planes.append(w)
    return np.stack(planes, axis=0)


def unpack_levels(planes: np.ndarray) -> np.ndarray:
    """planes[bits][..., K/32] -> levels[..., K] (inverse of pack_levels)."""
    bits = planes.shape[0]
    out = None
    for b in range(bits):
        w = planes[b]
        by = np.stack([(w >> 24) & 255, (w >> 16) & 255, (w >> 8) & 255, w & 255], axis=-1).astype(np.uint8)
        bb = np.unpackbits(by, axis=-1, bitorder="big").reshape(*w.shape[:-1], w.shape[-1] * 32).astype(np.uint32)
        out = (bb << b) if out is None else (out | (bb << b))
    return out


# ----------------------------------------------------------------------------- GEMM
def gemm_bitserial(W, X, rows=None):
    """The reference's compute_ref loop (bit by bit).  ``rows=(m0, m1)`` limits the
    output rows computed (the rest stay zero)."""
    W, pw = _u32(W)
    X, px = _u32(X)
    wbits, M, kw = W.shape
    xbits, N, _ = X.shape
    D = np.zeros((M, N), dtype=np.int32)
    m0, m1 = rows if rows is not None else (0, M)
    lib().apnn_oracle_gemm_bitserial_rows(pw, px, D.ctypes.data_as(_i32p), M, N, kw * 32, wbits, xbits, m0, m1)
    return D


def gemm_popc(W, X, threads: int = 1, rows=None):
    """Word-popcount form of the same accumulator, optionally threaded over rows."""
    W, pw = _u32(W)
    X, px = _u32(X)
    wbits, M, kw = W.shape
    xbits, N, _ = X.shape
    D = np.zeros((M, N), dtype=np.int32)
    pd = D.ctypes.data_as(_i32p)
    m0, m1 = rows if rows is not None else (0, M)
    fn = lib().apnn_oracle_gemm_popc_rows
    if threads <= 1:
        fn(pw, px, pd, M, N, kw * 32, wbits, xbits, m0, m1)
    else:
        edges = np.linspace(m0, m1, threads + 1).astype(int)
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(lambda i: fn(pw, px, pd, M, N, kw * 32, wbits, xbits, int(edges[i]), int(edges[i + 1])),
                        range(threads)))
    return D


def gemm_bitserial_threaded(W, X, threads: int, rows):
    """compute_ref's loop over a row range, split over ``threads`` host threads."""
    W, pw = _u32(W)
    X, px = _u32(X)
    wbits, M, kw = W.shape
    xbits, N, _ = X.shape
    D = np.zeros((M, N), dtype=np.int32)
    pd = D.ctypes.data_as(_i32p)
    m0, m1 = rows
    fn = lib().apnn_oracle_gemm_bitserial_rows
    edges = np.linspace(m0, m1, threads + 1).astype(int)
    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(lambda i: fn(pw, px, pd, M, N, kw * 32, wbits, xbits, int(edges[i]), int(edges[i + 1])),
                    range(threads)))
    return D


def row_sums(P):
    """S[r] = sum_b 2^b popcount(P[b][r][:])."""
    P, pp = _u32(P)
    bits, rows, kw = P.shape
    S = np.zeros(rows, dtype=np.int32)
    lib().apnn_oracle_row_sums(pp, S.ctypes.data_as(_i32p), rows, kw * 32, bits)
    return S


def gemm_pack(W, X, out_bits):
    """compute_ref_pack of the fused GEMM: low ``out_bits`` bits of the accumulator,
    packed along N -> [out_bits][M][N/32]."""
    W, pw = _u32(W)
    X, px = _u32(X)
    wbits, M, kw = W.shape
    xbits, N, _ = X.shape
    out = np.zeros((out_bits, M, N // 32), dtype=np.uint32)
    lib().apnn_oracle_gemm_pack(pw, px, out.ctypes.data_as(_u32p), M, N, kw * 32, wbits, xbits, out_bits)
    return out


# ----------------------------------------------------------------------------- conv
def _conv_dims(X, Wt):
    xbits, B, Hp, Wp, cw = X.shape
    wbits, COUT, R, _, _ = Wt.shape
    p = (R - 1) // 2
    return xbits, wbits, B, Hp - 2 * p, Wp - 2 * p, cw * 32, COUT, R


def conv_bitserial(Wt, X, stride=1):
    """Convolution accumulators, bit by bit: Out[B][Ho][Wo][COUT] int32."""
    X, px = _u32(X)
    Wt, pw = _u32(Wt)
    xbits, wbits, B, H, Wd, CIN, COUT, R = _conv_dims(X, Wt)
    Ho, Wo = (H - 1) // stride + 1, (Wd - 1) // stride + 1
    out = np.zeros((B, Ho, Wo, COUT), dtype=np.int32)
    lib().apnn_oracle_conv_bitserial(pw, px, out.ctypes.data_as(_i32p), B, H, Wd, CIN, COUT, R, stride, wbits, xbits)
    return out


def conv_popc(Wt, X, stride=1, threads: int = 1):
    """Word-popcount form of the convolution accumulators, threaded over channels."""
    X, px = _u32(X)
    Wt, pw = _u32(Wt)
    xbits, wbits, B, H, Wd, CIN, COUT, R = _conv_dims(X, Wt)
    Ho, Wo = (H - 1) // stride + 1, (Wd - 1) // stride + 1
    out = np.zeros((B, Ho, Wo, COUT), dtype=np.int32)
    po = out.ctypes.data_as(_i32p)
    fn = lib().apnn_oracle_conv_popc_range
    threads = max(1, min(threads, COUT))
    edges = np.linspace(0, COUT, threads + 1).astype(int)
    if threads == 1:
        fn(pw, px, po, B, H, Wd, CIN, COUT, R, stride, wbits, xbits, 0, COUT)
    else:
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(lambda i: fn(pw, px, po, B, H, Wd, CIN, COUT, R, stride, wbits, xbits,
                                     int(edges[i]), int(edges[i + 1])), range(threads)))
    return out


def conv_window_sums(X, R, stride=1):
    """S[B][Ho][Wo] = sum of activation values over each RxRxCIN window."""
    X, px = _u32(X)
    xbits, B, Hp, Wp, cw = X.shape
    p = (R - 1) // 2
    H, Wd = Hp - 2 * p, Wp - 2 * p
    Ho, Wo = (H - 1) // stride + 1, (Wd - 1) // stride + 1
    S = np.zeros((B, Ho, Wo), dtype=np.int32)
    lib().apnn_oracle_conv_window_sums(px, S.ctypes.data_as(_i32p), B, H, Wd, cw * 32, R, stride, xbits)
    return S


def conv_pack(Wt, X, out_bits, pool=False):
    """compute_ref_pack / compute_ref_pack_pool of the fused conv programs (one image,
    3x3, stride 1): low bits, optional 2x2 truncating average first, packed along COUT."""
    X, px = _u32(X)
    Wt, pw = _u32(Wt)
    xbits, wbits, B, H, Wd, CIN, COUT, R = _conv_dims(X, Wt)
    assert B == 1 and R == 3
    Ho, Wo = (H // 2, Wd // 2) if pool else (H, Wd)
    out = np.zeros((out_bits, 1, Ho, Wo, COUT // 32), dtype=np.uint32)
    lib().apnn_oracle_conv_pack(pw, px, out.ctypes.data_as(_u32p), H, Wd, CIN, COUT, wbits, xbits, out_bits,
                                1 if pool else 0)
    return out


# ----------------------------------------------------------------------------- epilogue
def signed_correct(acc, S, sign_axis):
    """v = 2*acc - S[row] (sign_axis 0) or 2*acc - S[col] (sign_axis 1), over [rows][C]."""
    V = np.array(acc, dtype=np.int32, copy=True)
    C = V.shape[-1]
    rows = V.size // C
    S, ps = _i32(np.asarray(S).reshape(-1))
    lib().apnn_oracle_signed_correct(V.ctypes.data_as(_i32p), ps, ctypes.c_long(rows), C, sign_axis)
    return V


def pool2x2(V, mode):
    """2x2 pooling over [B][H][W][C]; mode 1 = truncating average, 2 = maximum."""
    V, pv = _i32(V)
    B, H, Wd, C = V.shape
    out = np.zeros((B, H // 2, Wd // 2, C), dtype=np.int32)
    lib().apnn_oracle_pool2x2(pv, out.ctypes.data_as(_i32p), B, H, Wd, C, mode)
    return out


def levels(V, out_bits, mode, thresholds=None):
    """Per-element level: mode 1 low bits, mode 2 per-channel threshold count."""
    V, pv = _i32(V)
    C = V.shape[-1]
    rows = V.size // C
    T, pt = _opt_i32(thresholds)
    L = np.zeros(V.shape, dtype=np.int32)
    lib().apnn_oracle_levels(pv, L.ctypes.data_as(_i32p), ctypes.c_long(rows), C, out_bits, mode, pt)
    return L


def requant_pack(V, out_bits, mode, thresholds=None):
    """Requantise [..., C] and pack along C -> [out_bits][..., C/32]."""
    V, pv = _i32(V)
    C = V.shape[-1]
    rows = V.size // C
    T, pt = _opt_i32(thresholds)
    out = np.zeros((out_bits,) + V.shape[:-1] + (C // 32,), dtype=np.uint32)
    lib().apnn_oracle_requant_pack(pv, out.ctypes.data_as(_u32p), ctypes.c_long(rows), C, out_bits, mode, pt)
    return out


def fold_bn(scale, bias, mu, sigma, out_bits):
    """Batch-norm + clip/round quantiser folded to int32 thresholds [C][2^out_bits-1]."""
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    C = scale.shape[0]
    T = np.zeros((C, (1 << out_bits) - 1), dtype=np.int32)
    lib().apnn_oracle_fold_bn(scale.ctypes.data_as(_f32p), bias.ctypes.data_as(_f32p), ctypes.c_double(mu),
                              ctypes.c_double(sigma), C, out_bits, T.ctypes.data_as(_i32p))
    return T


# ----------------------------------------------------------------------------- packers
def quantize(x, bits):
    """Quantize_val: clip to [-10, 10], affine to 2^bits steps, round-to-nearest-even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    lv = np.zeros(x.shape, dtype=np.uint32)
    lib().apnn_oracle_quantize(x.ctypes.data_as(_f32p), lv.ctypes.data_as(_u32p), ctypes.c_long(x.size), bits)
    return lv


def bit_compress(lv, bits):
    """Bit_compression: levels[rows][C] -> planes[bits][rows][PAD128(C)/32]."""
    lv, pl = _u32(lv)
    C = lv.shape[-1]
    rows = lv.size // C
    cw = ((C + 127) // 128) * 4
    out = np.zeros((bits,) + lv.shape[:-1] + (cw,), dtype=np.uint32)
    lib().apnn_oracle_bit_compress(pl, out.ctypes.data_as(_u32p), ctypes.c_long(rows), C, bits)
    return out


def quantize_im2col(images, R, stride, bits):
    """First-layer re-layout: quantised RxRxC windows along the channel axis,
    planes[bits][B][Ho][Wo][PAD128(R*R*C)/32]."""
    images = np.ascontiguousarray(images, dtype=np.float32)
    B, H, Wd, C = images.shape
    Ho, Wo = (H - 1) // stride + 1, (Wd - 1) // stride + 1
    kw = (R * R * C + 127) // 128 * 4
    out = np.zeros((bits, B, Ho, Wo, kw), dtype=np.uint32)
    lib().apnn_oracle_quantize_im2col(images.ctypes.data_as(_f32p), out.ctypes.data_as(_u32p), B, H, Wd, C, R, stride,
                                      bits)
    return out


# ----------------------------------------------------------------------------- first / last layer (unpinned)
def centred_first_layer(Wt, levels8, real_channels: int, stride=1, threads: int = 1):
    """First layer at 8-bit precision ("parity unpinned": the reference's InConv128Layer,
    APNN-TC-nn/src/kernel.cuh:583-682, multiplies the float image by +-1 weights and accumulates in
    float, an order-dependent sum no test pins).  Defined here on exact integers: the image is
    quantised to 8 bits by ``quantize`` (clip to [-10, 10], 256 steps), re-centred to
    a = level - 128 so that zero means zero, padding contributes nothing (as the reference skips
    out-of-frame pixels), weights are -1/+1:

        value = sum w * a = (sum w * level) - 128 * (sum of w over the in-frame taps)

    both sums built from the pinned popcount convolution.  ``levels8``: uint [B, H, W, Cp] whose first
    ``real_channels`` channels are the image (the rest is storage padding and counts as zero);
    ``Wt``: 1-bit planes [1][COUT][R][R][Cp/32].  Returns int32 [B, Ho, Wo, COUT]."""
    R = Wt.shape[2]
    pad = (R - 1) // 2
    B, H, W, Cp = levels8.shape
    real = np.zeros((B, H, W, Cp), dtype=np.uint32)
    real[..., :real_channels] = 1
    xp = np.zeros((B, H + 2 * pad, W + 2 * pad, Cp), dtype=np.uint32)
    ip = np.zeros_like(xp)
    xp[:, pad:pad + H, pad:pad + W] = levels8
    ip[:, pad:pad + H, pad:pad + W] = real
    X8, X1 = pack_levels(xp, 8), pack_levels(ip, 1)
    first = signed_correct(conv_popc(Wt, X8, stride=stride, threads=threads), conv_window_sums(X8, R, stride), 0)
    second = signed_correct(conv_popc(Wt, X1, stride=stride, threads=threads), conv_window_sums(X1, R, stride), 0)
    return (first.astype(np.int64) - 128 * second.astype(np.int64)).astype(np.int32)


def affine_f32(V, scale, bias):
    """Output layer ("parity unpinned"; Out128Layer, APNN-TC-nn/src/kernel.cuh:397-447, whose
    (K - 2*popc) is the +-1 dot product V): float32(V) * scale[c] + bias[c], the multiply and the
    add each rounded to float32 (two IEEE operations, no fused multiply-add)."""
    prod = np.asarray(V).astype(np.float32) * np.asarray(scale, dtype=np.float32)
    return (prod + np.asarray(bias, dtype=np.float32)).astype(np.float32)
