"""Loader for ``oracle/_ref/libref_*.so``: the reference's own host-side functions
(init_matrices, compute_ref, compute_ref_pack, compute_ref_pack_pool), compiled
unmodified from the reference checkout by ``make -C oracle ref``.

TEST INFRASTRUCTURE ONLY.  Used to pin the C restatement in ``apnn_oracle.c`` and,
optionally, as the timed CPU baseline.  The functions are C++ (mangled names) and
take ``int4*`` operands, which are plain 16-byte-aligned word arrays.

Program numbers: 71 w1a2 GEMM, 72 w2a2 GEMM, 78 w1a4 GEMM, 66 w1a2 GEMM pack,
67 w1a2 conv pack, 68 w1a2 conv pool+pack, 70 w2a2 conv pack, 48 w2a2 conv int32.
All of them carry bit-width-generic host loops.
"""
from __future__ import annotations

import ctypes
import os
import threading

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF_DIR = os.path.join(_HERE, "_ref")
_libs = {}
_vp = ctypes.c_void_p

# mangled names (Itanium ABI): P4int4 = int4*, S0_ = same, Pi = int*, then the ints
_GEMM_INIT = "_Z13init_matricesP4int4S0_iiiii"        # (W, X, M, N, K, W_BIT, X_BIT)
_GEMM_REF = "_Z11compute_refP4int4S0_Piiiiii"          # (W, X, ref, M, N, K, W_BIT, X_BIT)
_GEMM_PACK = "_Z16compute_ref_packP4int4S0_Piiiiiii"   # (W, X, ref, M, N, K, W_BIT, X_BIT, OUT_BIT) in 66
_CONV_INIT = "_Z13init_matricesP4int4S0_iiiiii"        # (X, W, H, W, CIN, COUT, X_BIT, W_BIT)
_CONV_REF = "_Z11compute_refP4int4S0_Piiiiiii"         # (W, X, ref, H, W, CIN, COUT, W_BIT, X_BIT)
_CONV_PACK = "_Z16compute_ref_packP4int4S0_Piiiiiiii"  # (..., W_BIT, X_BIT, OUT_BIT)
_CONV_POOL = "_Z21compute_ref_pack_poolP4int4S0_Piiiiiiii"


def available(prog: int = 71) -> bool:
    return os.path.exists(os.path.join(_REF_DIR, f"libref_{prog}.so"))


def _lib(prog: int) -> ctypes.CDLL:
    if prog not in _libs:
        _libs[prog] = ctypes.CDLL(os.path.join(_REF_DIR, f"libref_{prog}.so"))
    return _libs[prog]


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


def _aligned(shape, dtype=np.uint32):
    n = int(np.prod(shape))
    raw = np.zeros(n * np.dtype(dtype).itemsize + 64, dtype=np.uint8)
    off = (-raw.ctypes.data) % 16
    return raw[off:off + n * np.dtype(dtype).itemsize].view(dtype).reshape(shape)


def _big_stack(fn):
    """Run ``fn`` on a thread with a 1 GiB stack: the pack oracles of the reference
    keep their int32 intermediates in variable-length arrays on the stack."""
    res = {}

    def run():
        res["v"] = fn()

    old = threading.stack_size(1 << 30)
    try:
        t = threading.Thread(target=run)
        t.start()
        t.join()
    finally:
        threading.stack_size(old)
    return res["v"]


def reset_rand():
    """srand(1): the state rand() has in a fresh process, which is what the reference runs with."""
    ctypes.CDLL(None).srand(1)


def gemm_init(prog, M, N, K, wbits, xbits):
    """init_matrices of a GEMM program after a rand() reset."""
    reset_rand()
    W = _aligned((wbits, M, K // 32))
    X = _aligned((xbits, N, K // 32))
    getattr(_lib(prog), _GEMM_INIT)(_ptr(W), _ptr(X), M, N, K, wbits, xbits)
    return W, X


def gemm_ref(prog, W, X):
    wbits, M, kw = W.shape
    xbits, N, _ = X.shape
    Wa, Xa = _aligned(W.shape), _aligned(X.shape)
    Wa[...] = W
    Xa[...] = X
    D = _aligned((M, N), np.int32)
    getattr(_lib(prog), _GEMM_REF)(_ptr(Wa), _ptr(Xa), _ptr(D), M, N, kw * 32, wbits, xbits)
    return np.array(D)


def gemm_ref_rows(prog, W, X, m0, m1):
    """compute_ref on the row slice [m0, m1) of a 1-bit-weight problem: the slice of W
    is itself a valid W operand, so the unmodified function can be threaded and sampled."""
    wbits, M, kw = W.shape
    assert wbits == 1
    xbits, N, _ = X.shape
    Ws = _aligned((1, m1 - m0, kw))
    Ws[...] = W[:, m0:m1]
    Xa = _aligned(X.shape)
    Xa[...] = X
    D = _aligned((m1 - m0, N), np.int32)
    getattr(_lib(prog), _GEMM_REF)(_ptr(Ws), _ptr(Xa), _ptr(D), m1 - m0, N, kw * 32, 1, xbits)
    return np.array(D)


def gemm_pack(W, X, out_bits):
    wbits, M, kw = W.shape
    xbits, N, _ = X.shape
    Wa, Xa = _aligned(W.shape), _aligned(X.shape)
    Wa[...] = W
    Xa[...] = X
    out = _aligned((out_bits, M, N // 32))
    fn = getattr(_lib(66), _GEMM_PACK)
    _big_stack(lambda: fn(_ptr(Wa), _ptr(Xa), _ptr(out), M, N, kw * 32, wbits, xbits, out_bits))
    return np.array(out)


def conv_init(prog, H, Wd, CIN, COUT, xbits, wbits):
    reset_rand()
    X = _aligned((xbits, 1, H + 2, Wd + 2, CIN // 32))
    Wt = _aligned((wbits, COUT, 3, 3, CIN // 32))
    getattr(_lib(prog), _CONV_INIT)(_ptr(X), _ptr(Wt), H, Wd, CIN, COUT, xbits, wbits)
    return X, Wt


def _conv_args(Wt, X):
    xbits, B, Hp, Wp, cw = X.shape
    wbits, COUT = Wt.shape[0], Wt.shape[1]
    assert B == 1
    Wa, Xa = _aligned(Wt.shape), _aligned(X.shape)
    Wa[...] = Wt
    Xa[...] = X
    return Wa, Xa, Hp - 2, Wp - 2, cw * 32, COUT, wbits, xbits


def conv_ref(prog, Wt, X):
    Wa, Xa, H, Wd, CIN, COUT, wbits, xbits = _conv_args(Wt, X)
    out = _aligned((1, H, Wd, COUT), np.int32)
    fn = getattr(_lib(prog), _CONV_REF)
    if prog in (48, 70):  # these two programs declare compute_ref(X, W, ..., X_BIT, W_BIT)
        fn(_ptr(Xa), _ptr(Wa), _ptr(out), H, Wd, CIN, COUT, xbits, wbits)
    else:                 # 67, 68: compute_ref(W, X, ..., W_BIT, X_BIT)
        fn(_ptr(Wa), _ptr(Xa), _ptr(out), H, Wd, CIN, COUT, wbits, xbits)
    return np.array(out)


def conv_pack(prog, Wt, X, out_bits, pool=False):
    Wa, Xa, H, Wd, CIN, COUT, wbits, xbits = _conv_args(Wt, X)
    Ho, Wo = (H // 2, Wd // 2) if pool else (H, Wd)
    out = _aligned((out_bits, 1, Ho, Wo, COUT // 32))
    fn = getattr(_lib(prog), _CONV_POOL if pool else _CONV_PACK)
    _big_stack(lambda: fn(_ptr(Wa), _ptr(Xa), _ptr(out), H, Wd, CIN, COUT, wbits, xbits, out_bits))
    return np.array(out)
