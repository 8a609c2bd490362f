"""Generates tests/golden/reference_host_loops.npz from the reference's own host functions.

Run where the reference checkout is present, after ``make -C oracle ref``:

    python tests/golden/make_golden.py

Inputs are the reference's init_matrices() stream (glibc rand(), default seed), outputs are
compute_ref / compute_ref_pack / compute_ref_pack_pool of the named reference program,
compiled unmodified.  Only outputs and an input checksum are stored; the test-suite
regenerates the inputs with the oracle's restatement of rand().
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref  # noqa: E402


def sha(*arrs):
    h = hashlib.sha256()
    for a in arrs:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main():
    out = {}
    # GEMM int32: program, wbits, xbits
    for prog, wb, xb in ((71, 1, 2), (72, 2, 2), (78, 1, 4), (71, 1, 3)):
        for n in (128, 256):
            # program 78 ships with its all-ones debugging fill enabled, so the random
            # operands always come from program 71's init_matrices (the loops are generic)
            W, X = ref.gemm_init(71, 64, n, n, wb, xb)
            D = ref.gemm_ref(prog, W, X)
            key = f"gemm_w{wb}a{xb}_64x{n}x{n}"
            out[key] = D
            out[key + "_insha"] = np.frombuffer(bytes.fromhex(sha(W, X)), dtype=np.uint8)
    # program 78 as shipped: all-ones operands, every output = 15 * K
    W, X = ref.gemm_init(78, 64, 128, 128, 1, 4)
    out["gemm_w1a4_allones_64x128x128"] = ref.gemm_ref(78, W, X)
    # the reference's own CPU-runnable case: w1a2 M=64 N=K=1024 -> checksum and corner
    W, X = ref.gemm_init(71, 64, 1024, 1024, 1, 2)
    D = ref.gemm_ref(71, W, X)
    out["gemm_w1a2_64x1024x1024_sum"] = np.array([D.astype(np.int64).sum(), D[0, 0]], dtype=np.int64)
    out["gemm_w1a2_64x1024x1024_sha"] = np.frombuffer(bytes.fromhex(sha(D)), dtype=np.uint8)
    # GEMM + low-bit pack (program 66's compute_ref_pack)
    for wb, xb in ((1, 2), (2, 2)):
        W, X = ref.gemm_init(71, 64, 128, 128, wb, xb)
        out[f"gemm_pack_w{wb}a{xb}_64x128x128"] = ref.gemm_pack(W, X, 2)
    # conv: program 67 (w1a2), 70 (w2a2): int32, pack, pool+pack on 8x8x128 -> 64
    for prog, wb, xb in ((67, 1, 2), (70, 2, 2), (67, 1, 4)):
        X, Wt = ref.conv_init(prog, 8, 8, 128, 64, xb, wb)
        key = f"conv_w{wb}a{xb}_8x8x128x64"
        out[key] = ref.conv_ref(prog, Wt, X)
        out[key + "_pack"] = ref.conv_pack(prog, Wt, X, 2)
        out[key + "_pool"] = ref.conv_pack(68, Wt, X, 2, pool=True)
        out[key + "_insha"] = np.frombuffer(bytes.fromhex(sha(X, Wt)), dtype=np.uint8)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_host_loops.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
