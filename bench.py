#!/usr/bin/env python
"""Benchmark of the hot path: w1a2 arbitrary-precision GEMM, M = N = K = 8192, on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--algo tcgen05|imma|bmma]

One step = one pass of the GEMM over one batch of synthetic operands (uniform random bit
planes: 1-bit weights W[1][M][K/32], 2-bit activations X[2][N][K/32], int32 output D[M][N]).
With N > 1 GPUs (launched by torch.distributed.run) the problem is sharded along N: every
rank owns the same weights and its own 8192 activation rows, i.e. a slice D[:, n0:n1] of a
GEMM that is g times wider -- no data-path collective, weak scaling.

Prints ONE JSON line (rank 0).  Keys beyond the usual ones:
  roofline      tensor-pipe roofline of the dominant kernel (tc5_gemm_pair_kernel), timed with its
                own CUDA events inside the timed steps; peak = the tcgen05 kind::i8 issue-loop
                peak measured in this run (MEASURED_PEAKS.json's bf16 figure is quoted beside it)
  cpu_baseline  the reference's own bit-serial compute_ref (compiled unmodified into
                oracle/_ref) on a bounded sample of rows of the same problem
  e2e           the same metric through the host-buffer C-ABI call (pinned host operands,
                H2D + GEMM + D2H of the int32 result inside the timed region)
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N = K = 8192
WBITS, XBITS = 1, 2
METRIC = "w1a2_gemm_effective_tops"
UNIT = "TOPS"  # 2*M*N*K / t, counted once whatever the plane count (the reference's formula)
N_OPERAND_SETS = 4


def workload_config(n_gpus: int, algo: str) -> dict:
    return {
        "workload": "gemm_w1a2_M8192_N8192_K8192_int32out",
        "M": M, "N_per_gpu": N, "K": K, "wbits": WBITS, "xbits": XBITS,
        "sharding": "replicated W, N-sharded X (g x 8192 rows), no collective" if n_gpus > 1 else "single GPU",
        "algo": algo,
        "l2": "4 rotating operand sets; each step rewrites 128 MiB of int8 workspace and 256 MiB of output (> 126 MB L2)",
    }


# ----------------------------------------------------------------------------- reference arm
def run_reference(args) -> None:
    """The reference's CPU implementation of this path: compute_ref of its w1a2 GEMM program,
    compiled unmodified (oracle/_ref), all host threads, on a bounded sample of rows."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import oracle
    from oracle import ref
    threads = os.cpu_count() or 1
    rows_per_thread = 4
    rows = threads * rows_per_thread
    rng = np.random.default_rng(0xA9117C + 1)
    W = rng.integers(0, 2**32, size=(WBITS, M, K // 32), dtype=np.uint32)
    X = rng.integers(0, 2**32, size=(XBITS, N, K // 32), dtype=np.uint32)
    kind = "reference" if ref.available(71) else "port"

    def one_step():
        from concurrent.futures import ThreadPoolExecutor
        if kind == "reference":
            fn = lambda i: ref.gemm_ref_rows(71, W, X, i * rows_per_thread, (i + 1) * rows_per_thread)
        else:
            fn = lambda i: oracle.gemm_bitserial(W, X, rows=(i * rows_per_thread, (i + 1) * rows_per_thread))[
                i * rows_per_thread:(i + 1) * rows_per_thread]
        with ThreadPoolExecutor(threads) as ex:
            return list(ex.map(fn, range(threads)))

    for _ in range(min(args.warmup, 1)):
        one_step()
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        out = one_step()
    dt = (time.perf_counter() - t0) / steps
    # spot-check the sample against the popcount form of the oracle
    chk = oracle.gemm_popc(W, X, rows=(0, rows_per_thread))[:rows_per_thread]
    if not np.array_equal(np.asarray(out[0]), chk):
        raise SystemExit("reference arm: bit-serial sample disagrees with the popcount form")
    tops = 2.0 * rows * N * K / dt / 1e12
    sample = f"{rows} of {M} output rows per step ({rows_per_thread} per thread), full N and K"
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32 bit-serial", "data": "synthetic",
        "config": workload_config(args.gpus, "cpu:compute_ref"),
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- helpers
class ClockSampler:
    """Polls SM clock, power and clock-event reasons through NVML on a host thread while the
    timed region runs (read-only queries; no setting is changed)."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, gpu_index: int, period_s: float = 0.002):
        self.samples = []
        self.stop_flag = threading.Event()
        self.thread = None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = None
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(gpu_index).uuid)
            except Exception:
                pass
            h = None
            if uuid:
                try:
                    h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
                except Exception:
                    h = None
            if h is None:
                h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self.stop_flag.is_set():
                    try:
                        mhz = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                        pw = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                        try:
                            rs = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                        except Exception:
                            rs = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                        self.samples.append((time.perf_counter(), float(mhz), pw, int(rs)))
                    except Exception:
                        pass
                    time.sleep(period_s)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception as exc:  # NVML missing: report it rather than guess
            self.error = repr(exc)

    def stop(self, t_begin: float, t_end: float) -> dict:
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + getattr(self, "error", "")]}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        inside = [x for x in self.samples if t_begin <= x[0] <= t_end]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples inside the timed region"]}
        mhz = sorted(x[1] for x in inside)
        reasons = set()
        for x in inside:
            for bit, nm in self.REASONS.items():
                if x[3] & bit:
                    reasons.add(nm)
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons),
                "samples": len(inside), "power_w_max": max(x[2] for x in inside)}


def measured_peaks() -> dict:
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


def probe_peak(torch, cabi, kind: int, iters: int) -> float:
    """Peak of one contraction instruction in ops/s (issue loop with resident operands)."""
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops = ctypes.c_double()
    L = cabi.lib()
    s = torch.cuda.current_stream().cuda_stream
    cabi.check(L.apnn_probe_peak(s, kind, max(1, iters // 10), flag.data_ptr(), ctypes.byref(ops)), "probe")
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    cabi.check(L.apnn_probe_peak(s, kind, iters, flag.data_ptr(), ctypes.byref(ops)), "probe")
    e1.record()
    torch.cuda.synchronize()
    if int(flag.item()) != 0:
        return float("nan")
    return ops.value / (e0.elapsed_time(e1) * 1e-3)


# ----------------------------------------------------------------------------- our arm
def run_ours(args) -> None:
    import numpy as np
    import torch
    import apnn_tc_b200 as ap
    from apnn_tc_b200 import _cabi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        torch.cuda.set_device(0)
    dev = torch.device("cuda", torch.cuda.current_device())
    algo = args.algo

    # ---- synthetic operands, resident in HBM before the timed region
    g = torch.Generator(device=dev).manual_seed(0xA9117C + 1 + rank)
    gw = torch.Generator(device=dev).manual_seed(0xA9117C + 1)  # weights are the same on every rank
    Ws = [torch.randint(-2**31, 2**31 - 1, (WBITS, M, K // 32), dtype=torch.int32, device=dev, generator=gw)
          for _ in range(N_OPERAND_SETS)]
    Xs = [torch.randint(-2**31, 2**31 - 1, (XBITS, N, K // 32), dtype=torch.int32, device=dev, generator=g)
          for _ in range(N_OPERAND_SETS)]
    D = torch.empty((M, N), dtype=torch.int32, device=dev)
    W8 = torch.empty((M, K), dtype=torch.uint8, device=dev)
    X8 = torch.empty((N, K), dtype=torch.uint8, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    ws = torch.empty(ap.gemm_workspace_bytes(M, N, K), dtype=torch.uint8, device=dev)

    def step(i: int, ev=None):
        W, X = Ws[i % N_OPERAND_SETS], Xs[i % N_OPERAND_SETS]
        if algo == "tcgen05":
            # the same two launches apnn_gemm_ex(APNN_ALGO_TCGEN05) makes, issued one by one
            # so the GEMM kernel can be bracketed by its own events
            _cabi.check(_cabi.lib().apnn_expand_planes_pair(torch.cuda.current_stream().cuda_stream, W.data_ptr(),
                                                             W8.data_ptr(), M, WBITS, 0, X.data_ptr(), X8.data_ptr(), N,
                                                             XBITS, 0, K), "apnn_expand_planes_pair")
            if ev is not None:
                ev[0].record()
            ap.gemm_i8(W8, X8, D, status_flag=flag)
            if ev is not None:
                ev[1].record()
        else:
            if ev is not None:
                ev[0].record()
            ap.apmm(W, X, D, algo=algo)
            if ev is not None:
                ev[1].record()

    launches_per_step = 2 if algo == "tcgen05" else 1
    gathered = None
    if args.allgather != "none" and dist is not None:
        from apnn_tc_b200 import shard
        if args.allgather == "nccl":
            gathered = torch.empty((world, M, N), dtype=torch.int32, device=dev)
            base_step = step

            def step(i: int, ev=None):  # noqa: F811 -- the GEMM followed by an NCCL all-gather of the slices
                base_step(i, ev)
                shard.allgather_columns(D, out=gathered)
        else:
            # fused: the GEMM epilogue stores every tile into all ranks' buffers (peer stores over NVLink)
            sg = shard.SymmetricGather(M, N, dev)
            gathered = sg.buffer
            D = sg.local_slot()
            fused_epi = ap.make_epilogue("int32", peer_out=sg.peer_destinations())

            def step(i: int, ev=None):  # noqa: F811
                W, X = Ws[i % N_OPERAND_SETS], Xs[i % N_OPERAND_SETS]
                _cabi.check(_cabi.lib().apnn_expand_planes_pair(torch.cuda.current_stream().cuda_stream, W.data_ptr(),
                                                                 W8.data_ptr(), M, WBITS, 0, X.data_ptr(), X8.data_ptr(),
                                                                 N, XBITS, 0, K), "apnn_expand_planes_pair")
                if ev is not None:
                    ev[0].record()
                ap.gemm_i8(W8, X8, D, status_flag=flag, epilogue=fused_epi)
                if ev is not None:
                    ev[1].record()
                sg.barrier()   # every rank's tiles have landed before the next step overwrites them

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if int(flag.item()) != 0:
        raise SystemExit("tcgen05 kernel reported an expired wait during warm-up")

    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    for i in range(2):  # keep the device busy while the sampler thread starts
        step(i)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    wall0 = time.perf_counter()
    t0.record()
    for i in range(args.steps):
        step(i, kev[i])
    t1.record()
    torch.cuda.synchronize()
    wall1 = time.perf_counter()
    if dist is not None:
        dist.barrier()
    elapsed_ms = t0.elapsed_time(t1)
    kernel_ms = sum(a.elapsed_time(b) for a, b in kev) / args.steps
    if int(flag.item()) != 0:
        raise SystemExit("tcgen05 kernel reported an expired wait")
    if dist is not None:
        t = torch.tensor([elapsed_ms, kernel_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, kernel_ms = float(t[0]), float(t[1])
    clocks = sampler.stop(wall0, wall1) if sampler is not None else None

    # ---- quick correctness guard on the last step's output (a few rows against the oracle)
    if rank == 0:
        import oracle
        last = (args.steps - 1) % N_OPERAND_SETS
        rows = np.array([0, 4097, M - 1])
        Wh = Ws[last].cpu().numpy().view(np.uint32)
        Xh = Xs[last].cpu().numpy().view(np.uint32)
        want = oracle.gemm_popc(np.ascontiguousarray(Wh[:, rows]), Xh, threads=min(8, os.cpu_count() or 1))
        got = D[torch.from_numpy(rows).to(dev)].cpu().numpy()
        if not np.array_equal(got, want):
            raise SystemExit("bench output does not match the oracle")

    if gathered is not None:
        # every rank: the gathered buffer must equal an NCCL all-gather of the ranks' own slices
        ref = torch.empty((world, M, N), dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(ref.view(world * M, N), D.contiguous())
        torch.cuda.synchronize()
        if not torch.equal(ref, gathered):
            raise SystemExit(f"rank {rank}: gathered output differs from the all-gather of the slices")
        del ref

    if args.profile:
        if rank == 0:
            ms = elapsed_ms / args.steps
            print(json.dumps({"profile_run": True, "ms_per_step": ms, "kernel_ms": kernel_ms,
                              "config": workload_config(world, algo)}), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- end-to-end through the host-buffer C-ABI call (pinned host operands, D2H of the result)
    e2e = None
    e2e_steps = max(2, min(args.steps, 5))
    hW = torch.empty((WBITS, M, K // 32), dtype=torch.int32).pin_memory()
    hX = torch.empty((XBITS, N, K // 32), dtype=torch.int32).pin_memory()
    hW.copy_(Ws[0].cpu())
    hX.copy_(Xs[0].cpu())
    hD = torch.empty((M, N), dtype=torch.int32).pin_memory()
    handle = ap.HostHandle(torch.cuda.current_device())
    handle.gemm(hW, hX, hD, WBITS, XBITS, M, N, K, algo=algo)  # warm-up: arena allocation
    handle.gemm(hW, hX, hD, WBITS, XBITS, M, N, K, algo=algo)
    if dist is not None:
        dist.barrier()
    tt0 = time.perf_counter()
    for _ in range(e2e_steps):
        handle.gemm(hW, hX, hD, WBITS, XBITS, M, N, K, algo=algo)  # synchronises before returning
    e2e_s = (time.perf_counter() - tt0) / e2e_steps
    handle.close()
    if dist is not None:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t[0])
    if rank == 0 and not torch.equal(hD, ap.apmm(Ws[0], Xs[0], algo="imma").cpu()):
        raise SystemExit("host-buffer path disagrees with the device path")
    flops_step = 2.0 * M * N * K
    e2e = {"value": world * flops_step / e2e_s / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": hW.numel() * 4 + hX.numel() * 4, "d2h_bytes_per_step": hD.numel() * 4,
           "steps": e2e_steps, "timer": "host wall clock around the synchronous C-ABI call, max over ranks"}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel
    peaks = measured_peaks()
    kind = {"tcgen05": 0, "imma": 1, "bmma": 2}[algo]
    peak_ops = probe_peak(torch, _cabi, kind, 20000 if kind == 0 else 4000)
    ops_launch = flops_step * (WBITS * XBITS if algo == "bmma" else 1)  # bit-ops for the b1 path
    achieved = ops_launch / (kernel_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": {"tcgen05": "tc5_gemm_pair_kernel (cta_group::2)", "imma": "plane_core_kernel<u8>",
                                      "bmma": "plane_core_kernel<b1>"}[algo],
        "achieved": achieved, "peak": peak_ops / 1e12, "unit": "TOP/s" if algo != "bmma" else "Tbitop/s",
        "frac": achieved / (peak_ops / 1e12),
        "peak_source": "issue-loop peak of this instruction measured in this run (apnn_probe_peak)",
        "bf16_tflops_measured": peaks.get("bf16_tflops"), "bf16_tflops_sustained": peaks.get("bf16_tflops_sustained"),
        "frac_of_2x_bf16_burst": achieved / (2 * peaks["bf16_tflops"]) if peaks.get("bf16_tflops") else None,
        "kernel_ms": kernel_ms, "algorithmic_ops_per_launch": ops_launch,
        "traffic": 578794000 if algo == "tcgen05" else None,
        "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum per launch, ncu capture of `bench.py --profile` at full size",
        "algorithmic_bytes_per_launch": M * K + N * K + 4 * M * N,
    }

    # ---- CPU baseline: the reference's compute_ref on a bounded sample of rows
    from oracle import ref
    import oracle
    threads = os.cpu_count() or 1
    rpt = 2
    Wh = Ws[0].cpu().numpy().view(np.uint32)
    Xh = Xs[0].cpu().numpy().view(np.uint32)
    kind_cpu = "reference" if ref.available(71) else "port"
    from concurrent.futures import ThreadPoolExecutor
    if kind_cpu == "reference":
        fn = lambda i: ref.gemm_ref_rows(71, Wh, Xh, i * rpt, (i + 1) * rpt)
    else:
        fn = lambda i: oracle.gemm_bitserial(Wh, Xh, rows=(i * rpt, (i + 1) * rpt))[i * rpt:(i + 1) * rpt]
    c0 = time.perf_counter()
    with ThreadPoolExecutor(threads) as ex:
        cpu_out = list(ex.map(fn, range(threads)))
    cdt = time.perf_counter() - c0
    if not np.array_equal(np.concatenate(cpu_out), ap.apmm(Ws[0], Xs[0], algo="imma")[: threads * rpt].cpu().numpy()):
        raise SystemExit("CPU baseline and GPU disagree on the sampled rows")
    cpu_baseline = {"value": 2.0 * threads * rpt * N * K / cdt / 1e12, "unit": UNIT, "cores": threads,
                    "kind": kind_cpu,
                    "sample": f"{threads * rpt} of {M} output rows ({rpt} per thread), full N and K, bit-serial compute_ref"}

    # beside the CPU loops: the reference's own GPU kernel for this pair, compiled unmodified for
    # sm_100a into oracle/_ref (part of the same baseline leg; absent -> omitted)
    bar = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "bar_gemm_w1a2")
    if world == 1 and os.path.exists(bar) and (WBITS, XBITS) == (1, 2):
        try:
            import subprocess
            torch.cuda.synchronize()
            r = subprocess.run([bar, "gemm", str(M), str(N), str(K), "3"], capture_output=True, text=True, timeout=120)
            rec = json.loads(r.stdout.strip().splitlines()[-1])
            cpu_baseline["reference_gpu_kernel"] = {
                "kernel": rec["kernel"], "value": rec["tops"], "unit": UNIT, "ms_per_launch": rec["us_per_launch"] / 1e3,
                "note": "APNN-TC-lib/bmmaTensorCoreGemm/src/71_bmmaTensorCoreGemm.cu built for sm_100a, its own launch "
                        "configuration, same shape, on this GPU"}
        except Exception as exc:   # the bar is optional
            cpu_baseline["reference_gpu_kernel"] = {"unavailable": str(exc)[:120]}

    ms_per_step = elapsed_ms / args.steps
    line = {
        "metric": METRIC, "value": world * flops_step / (ms_per_step * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8 operands, int32 accumulate (exact)", "data": "synthetic",
        "config": dict(workload_config(world, algo), collective=("all_gather of the int32 output slices, "
                       f"{(world - 1) * M * N * 4} B inbound per rank per step, mode " + args.allgather if gathered is not None
                       else "none")),
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- network workloads
NET_BATCH = {"resnet18": 1024, "vgg_variant": 1024, "alexnet": 128}


def run_net(args) -> None:
    """images/s of a whole w1a2 network (the AlexNet / VGG-variant / ResNet-18 model lists of APNN-TC-nn):
    global batch sharded over the ranks
    (no collective), one CUDA-graph replay of the layer sequence per step."""
    import numpy as np
    import torch
    from apnn_tc_b200 import nets

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        torch.cuda.set_device(0)
    dev = torch.device("cuda", torch.cuda.current_device())
    gb = args.batch or NET_BATCH[args.workload]
    batch = gb // world
    spec = nets.MODELS[args.workload]()
    net = nets.Network(spec, batch, device=dev, use_tcgen05=(args.algo == "tcgen05"))
    g = torch.Generator(device=dev).manual_seed(0xA9117C + 5 + rank)
    images = (torch.rand((batch, spec.image_hw, spec.image_hw, 3), device=dev, generator=g) * 20 - 10).contiguous()
    net.capture(images)
    for _ in range(args.warmup):
        net.replay()
    net.check()
    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    net.replay()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    wall0 = time.perf_counter()
    t0.record()
    for _ in range(args.steps):
        net.replay()
    t1.record()
    torch.cuda.synchronize()
    wall1 = time.perf_counter()
    if dist is not None:
        dist.barrier()
    net.check()
    ms = t0.elapsed_time(t1) / args.steps
    # end to end: pinned host images in, logits out, through the same layer sequence
    himg = images.cpu().pin_memory()
    hlog = torch.empty(net.out[spec.layers[-1].name].shape, dtype=torch.int32).pin_memory()
    e2e_steps = max(2, min(args.steps, 5))
    torch.cuda.synchronize()
    c0 = time.perf_counter()
    for _ in range(e2e_steps):
        images.copy_(himg, non_blocking=True)
        net.replay()
        hlog.copy_(net.out[spec.layers[-1].name], non_blocking=True)
        torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - c0) / e2e_steps
    if dist is not None:
        t = torch.tensor([ms, e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    clocks = sampler.stop(wall0, wall1) if sampler is not None else None
    if rank == 0:
        line = {
            "metric": f"{args.workload}_w1a2_images_per_s", "value": batch * world / (ms * 1e-3), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "u8 operands, int32 accumulate (exact)",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}_w1a2_224x224x3", "global_batch": batch * world,
                       "per_gpu_batch": batch, "algo": args.algo, "sharding": "batch-sharded, no collective",
                       "l2": "activations of one step exceed L2 at this batch"},
            "e2e": {"value": batch * world / e2e_s, "unit": "images/s", "h2d_bytes_per_step": himg.numel() * 4,
                    "d2h_bytes_per_step": hlog.numel() * 4, "steps": e2e_steps},
            "gpu_launches": net.launches_per_forward * args.steps, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main() -> None:
    ap_ = argparse.ArgumentParser()
    ap_.add_argument("--gpus", type=int, default=1)
    ap_.add_argument("--steps", type=int, default=200)
    ap_.add_argument("--warmup", type=int, default=5)
    ap_.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap_.add_argument("--algo", default="tcgen05", choices=["tcgen05", "imma", "bmma"])
    ap_.add_argument("--allgather", default="none", choices=["none", "nccl", "fused"],
                     help="N > 1 only: gather the int32 output slices on every rank inside every timed step, by an "
                          "NCCL all-gather after the GEMM or fused into the GEMM epilogue as peer stores")
    ap_.add_argument("--profile", action="store_true",
                     help="timed steps only (no e2e, probe or CPU baseline): the command ncu captures")
    ap_.add_argument("--workload", default="gemm", choices=["gemm", "resnet18", "vgg_variant", "alexnet"],
                     help="gemm (default, the headline line) or a whole w1a2 network (images/s)")
    ap_.add_argument("--batch", type=int, default=0, help="global batch of a network workload")
    args = ap_.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload != "gemm":
        if args.steps == 200:
            args.steps = 20
        run_net(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
