"""Timing sweeps over the reference's own benchmark shapes (run on a B200):

    python -m apnn_tc_b200.sweep gemm     # M=64, N=K=128..1024, w1a2/w1a3/w1a4/w2a2 (README.md:135-142)
    python -m apnn_tc_b200.sweep conv     # 16x16, C=O=128..1024, 3x3, batch 1 and 8 (README.md:160-167)
    python -m apnn_tc_b200.sweep big      # M=N=K=8192 for the four bit pairs and the three algorithms
    python -m apnn_tc_b200.sweep conv w=1 a=2 B=8 C=128      # one shape only (for ncu captures)
    python -m apnn_tc_b200.sweep layers [B=512] [mode=thresholds] [H=56] ...   # ResNet-18 layer shapes on
                                        # apnn_conv2d_i8 (pre-expanded operands) with each epilogue

Launch-bound shapes are timed by replaying a CUDA graph of many back-to-back launches (device time
per launch without host launch overhead) and, beside it, by plain back-to-back launches with one
event pair around the batch.  Between graph replays a buffer larger than L2 is rewritten.
TOPS = 2*M*N*K / t as the reference counts it; GB/s uses the algorithmic bytes (packed operands in,
int32 or packed result out).  One JSON object per line.
"""
from __future__ import annotations

import json
import sys

import torch

import apnn_tc_b200 as ap


def _words(shape, gen):
    return torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device="cuda", generator=gen)


_flush_buf = None


def flush_l2():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush_buf.fill_(1)


def time_call(fn, launches_per_graph=20, replays=10):
    """Returns (graph_us_per_launch, plain_us_per_launch)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    # plain back-to-back launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flush_l2()
    e0.record()
    for _ in range(launches_per_graph):
        fn()
    e1.record()
    torch.cuda.synchronize()
    plain = e0.elapsed_time(e1) * 1e3 / launches_per_graph
    # graph replay
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
        with torch.cuda.graph(g, stream=s):
            for _ in range(launches_per_graph):
                fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(replays):
        flush_l2()
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / launches_per_graph)
    return best, plain


def sweep_gemm():
    gen = torch.Generator(device="cuda").manual_seed(0xA9117C + 2)
    for wb, xb in ((1, 2), (1, 3), (1, 4), (2, 2)):
        for n in range(128, 1025, 128):
            M, N, K = 64, n, n
            if not _keep(w=wb, a=xb, N=n):
                continue
            W, X = _words((wb, M, K // 32), gen), _words((xb, N, K // 32), gen)
            D = torch.empty((M, N), dtype=torch.int32, device="cuda")
            gus, pus = time_call(lambda: ap.apmm(W, X, D, algo="imma"))
            byts = wb * M * K / 8 + xb * N * K / 8 + 4 * M * N
            print(json.dumps({"op": "gemm", "w": wb, "a": xb, "M": M, "N": N, "K": K, "graph_us": round(gus, 3),
                              "plain_us": round(pus, 3), "tops": round(2 * M * N * K / gus / 1e6, 2),
                              "algorithmic_bytes": int(byts), "gbps": round(byts / gus / 1e3, 1)}), flush=True)


def sweep_conv():
    gen = torch.Generator(device="cuda").manual_seed(0xA9117C + 3)
    for wb, xb in ((1, 2), (1, 4), (2, 2)):
        for B in (1, 8):
            for C in range(128, 1025, 128):
                H = Wd = 16
                if not _keep(w=wb, a=xb, B=B, C=C):
                    continue
                X = _words((xb, B, H + 2, Wd + 2, C // 32), gen)
                Wt = _words((wb, C, 3, 3, C // 32), gen)
                T = torch.sort(torch.randint(0, 9 * C * 3, (C, 3), dtype=torch.int32, device="cuda", generator=gen),
                               dim=1).values.contiguous()
                epi = ap.make_epilogue("thresholds", 2, signed="w" if wb == 1 else "none", thresholds=T)
                out = torch.empty((2, B, H, Wd, C // 32), dtype=torch.int32, device="cuda")
                ws = torch.empty(ap.conv_workspace_bytes(B, H, Wd, C, C, 3), dtype=torch.uint8, device="cuda")
                flops = 2.0 * B * H * Wd * C * 9 * C
                byts = xb * B * 18 * 18 * C / 8 + wb * 9 * C * C / 8 + 2 * B * 256 * C / 8 + 12 * C
                if wb == 1 and _keep(algo="tcgen05_i8"):
                    # the layer as a network chains it: filter expanded once, activations already int8
                    # rows (the previous layer's out_i8), so one launch per layer
                    import ctypes
                    from . import _cabi
                    from .ops import _stream_ptr
                    x8 = ap.expand_planes(X.reshape(xb, -1, C // 32))
                    w8 = ap.expand_planes(Wt.reshape(wb, C, -1), signed=True)
                    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
                    epi8 = ap.make_epilogue("thresholds", 2, thresholds=T)
                    L = _cabi.lib()
                    gus, pus = time_call(lambda: _cabi.check(L.apnn_conv2d_i8(
                        _stream_ptr(), w8.data_ptr(), x8.data_ptr(), out.data_ptr(), B, H, Wd, C, C, 3, 1, 1,
                        ctypes.byref(epi8), flag.data_ptr()), "conv2d_i8"))
                    print(json.dumps({"op": "conv3x3_bn_requant2", "w": wb, "a": xb, "B": B, "HW": 16, "C": C,
                                      "algo": "tcgen05_i8", "graph_us": round(gus, 3), "plain_us": round(pus, 3),
                                      "tops": round(flops / gus / 1e6, 2), "algorithmic_bytes": int(byts),
                                      "gbps": round(byts / gus / 1e3, 1)}), flush=True)
                for algo in ("imma", "tcgen05"):
                    if not _keep(algo=algo):
                        continue
                    gus, pus = time_call(lambda: ap.apconv(Wt, X, out, epilogue=epi, algo=algo, workspace=ws))
                    print(json.dumps({"op": "conv3x3_bn_requant2", "w": wb, "a": xb, "B": B, "HW": 16, "C": C,
                                      "algo": algo, "graph_us": round(gus, 3), "plain_us": round(pus, 3),
                                      "tops": round(flops / gus / 1e6, 2), "algorithmic_bytes": int(byts),
                                      "gbps": round(byts / gus / 1e3, 1)}), flush=True)


def sweep_big():
    gen = torch.Generator(device="cuda").manual_seed(0xA9117C + 4)
    M = N = K = 8192
    ws = torch.empty(ap.gemm_workspace_bytes(M, N, K), dtype=torch.uint8, device="cuda")
    D = torch.empty((M, N), dtype=torch.int32, device="cuda")
    for wb, xb in ((1, 2), (1, 3), (1, 4), (2, 2)):
        if not _keep(w=wb, a=xb):
            continue
        W, X = _words((wb, M, K // 32), gen), _words((xb, N, K // 32), gen)
        for algo in ("tcgen05", "imma", "bmma"):
            reps = 10 if algo == "tcgen05" else 3 if algo == "imma" else 1
            for _ in range(2):
                ap.apmm(W, X, D, algo=algo, workspace=ws)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                ap.apmm(W, X, D, algo=algo, workspace=ws)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            print(json.dumps({"op": "gemm", "w": wb, "a": xb, "M": M, "N": N, "K": K, "algo": algo,
                              "ms": round(ms, 4), "tops": round(2.0 * M * N * K / ms / 1e9, 1)}), flush=True)


def sweep_layers():
    """The 3x3 / 1x1 layer shapes of ResNet-18 at a large batch through ``apnn_conv2d_i8`` (int8 operands
    as the networks chain them), with int32, low-bit, threshold, threshold + int32 residual in/out and
    threshold -> int8 row ("i8rows") epilogues.  Plain back-to-back launches between one event pair (each call runs 50 us or more)."""
    import ctypes
    from . import _cabi
    from .ops import _stream_ptr
    L = _cabi.lib()
    B = int(FILTER.pop("B", 512))
    gen = torch.Generator(device="cuda").manual_seed(0xA9117C + 6)
    for (H, C, O, R) in ((56, 64, 64, 3), (56, 192, 64, 1), (56, 128, 128, 3), (28, 128, 128, 3), (14, 256, 256, 3),
                         (7, 512, 512, 3), (56, 256, 256, 3), (28, 512, 512, 3), (14, 512, 512, 3)):
        for mode, res in (("int32", False), ("lowbits", False), ("thresholds", False), ("thresholds", True),
                          ("i8rows", False)):
            if not _keep(H=H, C=C, mode=mode, res=int(res)):
                continue
            pad = (R - 1) // 2
            x8 = torch.randint(0, 4, (B, H + 2 * pad, H + 2 * pad, C), dtype=torch.uint8, device="cuda", generator=gen)
            w8 = (torch.randint(0, 2, (O, R, R, C), dtype=torch.int8, device="cuda", generator=gen) * 2 - 1)
            flag = torch.zeros(1, dtype=torch.int32, device="cuda")
            thr = torch.sort(torch.randint(-300, 300, (O, 3), dtype=torch.int32, device="cuda", generator=gen),
                             dim=1).values.contiguous()
            rin = torch.randint(-100, 100, (B * H * H, O), dtype=torch.int32, device="cuda", generator=gen) if res else None
            rout = torch.empty((B * H * H, O), dtype=torch.int32, device="cuda") if res else None
            if mode == "int32":
                out = torch.empty((B, H, H, O), dtype=torch.int32, device="cuda")
                epi = ap.make_epilogue("int32")
            elif mode == "i8rows":   # thresholds -> one byte per element, the form the networks chain
                out = torch.zeros((B, H + 2, H + 2, O), dtype=torch.uint8, device="cuda")
                epi = ap.make_epilogue("thresholds", 2, out_halo=1, thresholds=thr, out_i8=True)
            else:
                out = torch.zeros((2, B, H + 2, H + 2, O // 32), dtype=torch.int32, device="cuda")
                epi = ap.make_epilogue(mode, 2, out_halo=1, thresholds=thr if mode == "thresholds" else None,
                                       residual_in=rin, residual_out=rout)

            def call():
                _cabi.check(L.apnn_conv2d_i8(_stream_ptr(), w8.data_ptr(), x8.data_ptr(), out.data_ptr(), B, H, H, C, O, R, 1,
                                             1, ctypes.byref(epi), flag.data_ptr()), "conv")
            for _ in range(3):
                call()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                call()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 100.0
            print(json.dumps({"op": "conv2d_i8", "B": B, "HW": H, "C": C, "O": O, "R": R, "epilogue": mode,
                              "residual": res, "us": round(us, 1),
                              "tops": round(2.0 * B * H * H * O * R * R * C / us / 1e6, 1)}), flush=True)


FILTER = {}


def _keep(**kw):
    """True when the shape passes the command-line filter (e.g. ``C=128 B=8 w=1 a=2``)."""
    return all(str(kw[k]) == v for k, v in FILTER.items() if k in kw)


def main():
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    for tok in sys.argv[2:]:
        k, v = tok.split("=")
        FILTER[k] = v
    {"gemm": sweep_gemm, "conv": sweep_conv, "big": sweep_big, "layers": sweep_layers}[what]()


if __name__ == "__main__":
    main()
