"""Times the reference's own GPU kernels on this GPU and checks them against the oracle.

Checker-side script, never imported by the product.  It runs the binaries that
``make -C oracle ref_gpu`` built from ``ref_gpu_bar.cu`` plus the unmodified reference programs
(APNN-TC-lib/bmmaTensorCoreGemm/src/71, 72, 78, 67, 70) on the reference's benchmark shapes
(README.md:135-142 and :160-167: M=64 with N=K=128..1024; 16x16 conv with C=O=128..1024) and on
M=N=K=8192, and prints one JSON object per shape:

    python oracle/ref_gpu_bar.py [gemm] [conv] [big]

``matches_oracle`` compares the kernel's whole output with the oracle on the same inputs (sampled
rows for 8192^3).  The reference's conv kernels take one image; a batch of 8 is timed the way
``Conv_new_global`` feeds it (APNN-TC-nn/src/kernel.cuh:287-288): the images stacked along H.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import oracle  # noqa: E402

_REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_THREADS = min(16, os.cpu_count() or 1)

GEMM_PROGRAMS = {"w1a2": ("bar_gemm_w1a2", 1, 2), "w2a2": ("bar_gemm_w2a2", 2, 2), "w1a4": ("bar_gemm_w1a4", 1, 4)}
CONV_PROGRAMS = {"w1a2": ("bar_conv_w1a2", 1, 2), "w2a2": ("bar_conv_w2a2", 2, 2)}


def _run(binary, args, W, X, out_words):
    with tempfile.TemporaryDirectory() as tmp:
        fin, fout = os.path.join(tmp, "in.bin"), os.path.join(tmp, "out.bin")
        with open(fin, "wb") as f:
            f.write(np.ascontiguousarray(W, dtype=np.uint32).tobytes())
            f.write(np.ascontiguousarray(X, dtype=np.uint32).tobytes())
        r = subprocess.run([os.path.join(_REF, binary)] + [str(a) for a in args] + [fin, fout],
                           capture_output=True, text=True, timeout=600)
        if r.returncode != 0:
            return {"error": (r.stderr or r.stdout).strip()[-300:]}, None
        rec = json.loads(r.stdout.strip().splitlines()[-1])
        out = np.fromfile(fout, dtype=np.uint32, count=out_words)
    return rec, out


def gemm_case(name, M, N, K, iters, sample_rows=None):
    binary, wb, xb = GEMM_PROGRAMS[name]
    rng = np.random.default_rng(M * 7 + N * 3 + K + wb * 100 + xb)
    W = rng.integers(0, 2**32, size=(wb, M, K // 32), dtype=np.uint64).astype(np.uint32)
    X = rng.integers(0, 2**32, size=(xb, N, K // 32), dtype=np.uint64).astype(np.uint32)
    rec, out = _run(binary, ["gemm", M, N, K, iters], W, X, M * N)
    rec.update({"case": f"gemm_{name}", "M": M, "N": N, "K": K})
    if out is not None:
        D = out.view(np.int32).reshape(M, N)
        if sample_rows is None:
            rec["matches_oracle"] = bool(np.array_equal(D, oracle.gemm_popc(W, X, threads=_THREADS)))
        else:
            ok = True
            for m0 in sample_rows:
                want = oracle.gemm_popc(W, X, threads=_THREADS, rows=(m0, m0 + _THREADS))
                ok = ok and np.array_equal(D[m0:m0 + _THREADS], want[m0:m0 + _THREADS])
            rec["matches_oracle"] = bool(ok)
            rec["checked"] = f"{len(sample_rows) * _THREADS} sampled rows"
    return rec


def conv_case(name, images, HW, C, iters):
    binary, wb, xb = CONV_PROGRAMS[name]
    H = images * HW   # the batch stacked along H, one halo ring around the stack
    rng = np.random.default_rng(C * 5 + images + wb * 100 + xb)
    X = rng.integers(0, 2**32, size=(xb, 1, H + 2, HW + 2, C // 32), dtype=np.uint64).astype(np.uint32)
    Wt = rng.integers(0, 2**32, size=(wb, C, 3, 3, C // 32), dtype=np.uint64).astype(np.uint32)
    rec, out = _run(binary, ["conv", H, HW, C, C, iters], Wt, X, 2 * H * HW * (C // 32))
    rec.update({"case": f"conv_{name}", "images_stacked": images, "H": HW, "W": HW, "C": C, "O": C})
    if out is not None:
        acc = oracle.conv_popc(Wt, X, threads=_THREADS)
        want = oracle.requant_pack(acc, 2, 1)
        rec["matches_oracle"] = bool(np.array_equal(out.reshape(want.shape), want))
    return rec


def main():
    what = set(sys.argv[1:]) or {"gemm", "conv", "big"}
    missing = [b for b, _, _ in list(GEMM_PROGRAMS.values()) + list(CONV_PROGRAMS.values())
               if not os.path.exists(os.path.join(_REF, b))]
    if missing:
        print(json.dumps({"unavailable": "reference timing binaries not built: " + ", ".join(missing)}))
        return
    if "gemm" in what:
        for name in GEMM_PROGRAMS:
            for n in range(128, 1025, 128):
                print(json.dumps(gemm_case(name, 64, n, n, 200)), flush=True)
    if "conv" in what:
        for name in CONV_PROGRAMS:
            for images in (1, 8):
                for c in range(128, 1025, 128):
                    print(json.dumps(conv_case(name, images, 16, c, 100)), flush=True)
    if "big" in what:
        for name in GEMM_PROGRAMS:
            print(json.dumps(gemm_case(name, 8192, 8192, 8192, 3, sample_rows=(0, 4000, 8192 - _THREADS))), flush=True)


if __name__ == "__main__":
    main()
