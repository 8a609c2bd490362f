#!/usr/bin/env python
"""Benchmark of the hot path on B200: w1a2 arbitrary-precision GEMM, M = N = K = 8192 (headline), plus
the other workloads of the metric in the same JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--algo tcgen05|imma|bmma]

Headline step = one GEMM over one batch of synthetic operands resident in HBM as packed bit planes
(1-bit weights W[1][M][K/32], 2-bit activations X[2][N][K/32], int32 output D[M][N]).  The weights are a
static operand: their tensor-core image is made once before the timed region; every step converts a fresh
activation batch and runs the GEMM.  Operands of at most two bits are exact e2m1 values, so the default
path is tcgen05.mma kind::mxf4 with unit scale factors (sums of small integers in fp32: exact, checked
against the oracle after the timed region); --path int8 times the kind::i8 kernel, whose numbers the line
also carries as int8_path.  With N > 1 GPUs (torch.distributed.run) the problem is sharded along N: every
rank owns the same weights and its own 8192 activation rows -- no data-path collective, weak scaling.

Prints ONE JSON line (rank 0).  Keys beyond the usual ones:
  roofline      tensor-pipe roofline of the dominant kernel (tc5_gemm_pair_kernel), timed with its own
                CUDA events inside the timed steps; peak = the issue-loop peak of the same tcgen05.mma kind
                measured in this run (MEASURED_PEAKS.json's bf16 figure is quoted beside it)
  int8_path     the same step on the kind::i8 kernel (one byte per level), with its own roofline fraction
  cpu_baseline  the reference's own bit-serial compute_ref (compiled unmodified into oracle/_ref) on a
                bounded sample of rows of the same problem
  e2e           the same metric through the host-buffer C-ABI call (pinned host operands, H2D + GEMM +
                D2H of the int32 result inside the timed region)
  sustained     the headline step repeated for at least two seconds, with the clocks sampled across it
  resnet18      ResNet-18 w1a2 images/s at global batch 1024, batch-sharded over the ranks (every N)
  allgather     N > 1: the N-sharded GEMM with its output gathered on every rank inside the step, fused
                into the epilogue as peer stores (int32 slices and the 2-bit packed output) and by NCCL
  pairs_8192, m64_sweep, conv_c3   N = 1: the other bit pairs at 8192^3, the M = 64 sweep and the
                batch-8 16x16 convolution sweep (graph-replayed launches)
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
RESNET_GLOBAL_BATCH = 1024
# dram__bytes_read.sum + dram__bytes_write.sum per launch of tc5_gemm_pair_kernel at 8192^3, from the ncu captures
# summarised in profiles/ (kind::i8: before its tiles left by bulk tensor stores)
TRAFFIC_8192 = {"int8": (578794000, "profiles/tc5_gemm_pair_kernel_gemm_w1a2_8192.md"),
                "fp4": (384500000, "profiles/tc5_gemm_pair_kernel_mxf4_gemm_w1a2_8192.md")}


def workload_config(n_gpus: int) -> dict:
    """The same dictionary for both arms (ours and --impl reference)."""
    return {
        "workload": "gemm_w1a2_M8192_N8192_K8192_int32out",
        "M": M, "N_per_gpu": N, "K": K, "wbits": WBITS, "xbits": XBITS,
        "sharding": "replicated W, N-sharded X (g x 8192 rows), no collective" if n_gpus > 1 else "single GPU",
        "l2": "4 rotating activation sets; each step rewrites the activations' tensor-core image (32 MiB e2m1 or 64 MiB int8) "
              "and 256 MiB of output (> 126 MB L2)",
        "collective": "none",
    }


# ----------------------------------------------------------------------------- reference arm
def run_reference(args) -> None:
    """The reference's CPU implementation of this path: compute_ref of its w1a2 GEMM program,
    compiled unmodified (oracle/_ref), all host threads, on a bounded sample of rows per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import oracle
    from oracle import ref
    threads = os.cpu_count() or 1
    rows_per_thread = 1
    rows = threads * rows_per_thread
    rng = np.random.default_rng(0xA9117C + 1)
    W = rng.integers(0, 2**32, size=(WBITS, M, K // 32), dtype=np.uint32)
    X = rng.integers(0, 2**32, size=(XBITS, N, K // 32), dtype=np.uint32)
    kind = "reference" if ref.available(71) else "port"
    from concurrent.futures import ThreadPoolExecutor

    def one_step():
        if kind == "reference":
            fn = lambda i: ref.gemm_ref_rows(71, W, X, i * rows_per_thread, (i + 1) * rows_per_thread)
        else:
            fn = lambda i: oracle.gemm_bitserial(W, X, rows=(i * rows_per_thread, (i + 1) * rows_per_thread))[
                i * rows_per_thread:(i + 1) * rows_per_thread]
        with ThreadPoolExecutor(threads) as ex:
            return list(ex.map(fn, range(threads)))

    for _ in range(args.warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = one_step()
    dt = (time.perf_counter() - t0) / args.steps
    # spot-check the sample against the popcount form of the oracle
    chk = oracle.gemm_popc(W, X, rows=(0, rows_per_thread))[:rows_per_thread]
    if not np.array_equal(np.asarray(out[0]), chk):
        raise SystemExit("reference arm: bit-serial sample disagrees with the popcount form")
    tops = 2.0 * rows * N * K / dt / 1e12
    sample = (f"{rows} of {M} output rows per step ({rows_per_thread} per thread), full N and K; one host's CPU "
              f"whatever --gpus says")
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32 bit-serial", "data": "synthetic",
        "config": workload_config(args.gpus), "algo": "cpu:compute_ref",
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

    def window(self, t_begin: float, t_end: float) -> dict:
        """Summary of the samples taken inside [t_begin, t_end] (the sampler keeps running)."""
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + getattr(self, "error", "")]}
        inside = [x for x in list(self.samples) if t_begin <= x[0] <= t_end]
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

    def stop(self) -> None:
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)


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


_FLUSH = None


def flush_l2(torch):
    """Rewrites a 256 MiB buffer (twice the L2) so the next measurement starts cold."""
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _FLUSH.fill_(1)


def graph_time_us(torch, fn, launches: int = 20, replays: int = 5) -> float:
    """Device time per call of fn when `launches` calls are replayed from one CUDA graph (no host launch
    overhead), L2 flushed before each replay; best of `replays`."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for _ in range(launches):
                fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(replays):
        flush_l2(torch)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / launches)
    return best


def words(torch, shape, gen):
    return torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device="cuda", generator=gen)


# ----------------------------------------------------------------------------- the headline GEMM
class GemmPipeline:
    """The 8192^3 step on device-resident operands.  The weights are a layer's static operand: their tensor-core
    image is made once before the timed region; every step converts that step's activation planes and runs
    the GEMM, both on the current stream.  (Running the conversion of step i+1 on a second stream beside
    GEMM i was measured: the persistent GEMM's statically scheduled tiles on the SMs that also host the
    conversion blocks become stragglers, which cancels what the overlap hides.)

    path "fp4" (both operands of at most two bits): e2m1 nibble images, tcgen05.mma kind::mxf4 with unit
    scale factors -- exact, twice the int8 rate.  path "int8": one byte per level, kind::i8.  path
    "planes": ONE launch, apnn_gemm_w8 spreads the activation planes inside the GEMM kernel (no activation
    image in HBM; slower)."""

    def __init__(self, torch, ap, cabi, dev, rank, wbits=WBITS, xbits=XBITS, algo="tcgen05", epilogue=None, D=None,
                 path=None):
        self.torch, self.ap, self.cabi, self.algo = torch, ap, cabi, algo
        if path is None:
            path = "fp4" if (wbits <= 2 and xbits <= 2) else "int8"
        if path == "planes" and xbits > 4:
            path = "int8"
        self.path = path if algo == "tcgen05" else algo
        self.wbits, self.xbits = wbits, xbits
        g = torch.Generator(device=dev).manual_seed(0xA9117C + 1 + rank)
        gw = torch.Generator(device=dev).manual_seed(0xA9117C + 1)  # weights are the same on every rank
        self.W = words(torch, (wbits, M, K // 32), gw)
        self.Xs = [words(torch, (xbits, N, K // 32), g) for _ in range(N_OPERAND_SETS)]
        self.D = D if D is not None else torch.empty((M, N), dtype=torch.int32, device=dev)
        self.epilogue = epilogue
        self.flag = torch.zeros(1, dtype=torch.int32, device=dev)
        self.L = cabi.lib()
        if self.path == "fp4":
            self.Wt = ap.expand_planes_fp4(self.W)
            self.Xt = torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
        elif self.path in ("int8", "planes"):
            self.Wt = ap.expand_planes(self.W)
            if self.path == "int8":
                self.Xt = torch.empty((N, K), dtype=torch.uint8, device=dev)
        self.launches_per_step = 2 if self.path in ("fp4", "int8") else 1
        torch.cuda.synchronize()

    def step(self, i: int, ev=None):
        X = self.Xs[i % N_OPERAND_SETS]
        if self.path == "fp4":
            self.ap.expand_planes_fp4(X, out=self.Xt)
        elif self.path == "int8":
            self.ap.expand_planes(X, out=self.Xt)
        if ev is not None:
            ev[0].record()
        if self.path == "fp4":
            self.ap.gemm_fp4(self.Wt, self.Xt, self.D, status_flag=self.flag, epilogue=self.epilogue)
        elif self.path == "int8":
            self.ap.gemm_i8(self.Wt, self.Xt, self.D, status_flag=self.flag, epilogue=self.epilogue)
        elif self.path == "planes":
            self.ap.gemm_w8(self.Wt, X, self.D, status_flag=self.flag, epilogue=self.epilogue)
        else:
            self.ap.apmm(self.W, X, self.D, algo=self.algo)
        if ev is not None:
            ev[1].record()

    def begin(self, t0):
        t0.record()

    def end(self, t1):
        t1.record()


def timed_gemm_steps(torch, dist, pipe, steps, warmup, sampler=None):
    for i in range(warmup):
        pipe.step(i)
    torch.cuda.synchronize()
    if int(pipe.flag.item()) != 0:
        raise SystemExit("tcgen05 kernel reported an expired wait during warm-up")
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    wall0 = time.perf_counter()
    # An untimed millisecond of device spinning ahead of the first event: the host queues the steps meanwhile, so a
    # scheduling hiccup of this process (two launches and two event records per 0.2 ms step) does not idle the GPU
    # inside the timed region.
    torch.cuda._sleep(2_000_000)
    pipe.begin(t0)
    for i in range(steps):
        pipe.step(i, kev[i])
    pipe.end(t1)
    torch.cuda.synchronize()
    wall1 = time.perf_counter()
    if dist is not None:
        dist.barrier()
    if int(pipe.flag.item()) != 0:
        raise SystemExit("tcgen05 kernel reported an expired wait")
    elapsed_ms = t0.elapsed_time(t1)
    kernel_ms = sum(a.elapsed_time(b) for a, b in kev) / steps
    clocks = sampler.window(wall0, wall1) if sampler is not None else None
    return elapsed_ms, kernel_ms, clocks


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

    def max_over_ranks(*vals):
        if dist is None:
            return vals
        t = torch.tensor(list(vals), dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return tuple(float(x) for x in t)

    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    pipe = GemmPipeline(torch, ap, _cabi, dev, rank, algo=algo, path=args.path or None)
    for i in range(2):  # keep the device busy while the sampler thread starts
        pipe.step(i)
    elapsed_ms, kernel_ms, clocks = timed_gemm_steps(torch, dist, pipe, args.steps, args.warmup, sampler)
    elapsed_ms, kernel_ms = max_over_ranks(elapsed_ms, kernel_ms)
    flops_step = 2.0 * M * N * K
    ms_per_step = elapsed_ms / args.steps

    # ---- correctness guard on the last step's output (a few rows against the oracle)
    if rank == 0:
        import oracle
        last = (args.steps - 1) % N_OPERAND_SETS
        rows = np.array([0, 4097, M - 1])
        Wh = pipe.W.cpu().numpy().view(np.uint32)
        Xh = pipe.Xs[last].cpu().numpy().view(np.uint32)
        want = oracle.gemm_popc(np.ascontiguousarray(Wh[:, rows]), Xh, threads=min(8, os.cpu_count() or 1))
        got = pipe.D[torch.from_numpy(rows).to(dev)].cpu().numpy()
        if not np.array_equal(got, want):
            raise SystemExit("bench output does not match the oracle")

    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "ms_per_step": ms_per_step, "kernel_ms": kernel_ms,
                              "config": workload_config(world)}), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- sustained: the same step for at least two seconds, clocks sampled across the whole region
    sustained = None
    if algo == "tcgen05":
        n_sus = max(args.steps, int(2.2e3 / ms_per_step))
        s_ms, s_kernel_ms, s_clocks = timed_gemm_steps(torch, dist, pipe, n_sus, 1, sampler)
        s_ms, s_kernel_ms = max_over_ranks(s_ms, s_kernel_ms)
        sustained = {
            "seconds": s_ms / 1e3, "steps": n_sus, "ms_per_step": s_ms / n_sus,
            "tops": world * flops_step / (s_ms / n_sus * 1e-3) / 1e12, "kernel_ms": s_kernel_ms,
            "kernel_tops": flops_step / (s_kernel_ms * 1e-3) / 1e12, "clocks": s_clocks,
            "ms_x_mhz": (s_ms / n_sus) * s_clocks["sm_mhz"] if s_clocks and s_clocks.get("sm_mhz") else None,
            "note": "the headline region lasts milliseconds at boost clocks; this one runs long enough for the power "
                    "limit to set the clock",
        }

    # ---- the same step on the int8 path (kind::i8), for comparison with the 4-bit floating-point headline
    int8_block = None
    if algo == "tcgen05" and pipe.path == "fp4" and not args.profile:
        p8 = GemmPipeline(torch, ap, _cabi, dev, rank, algo=algo, path="int8")
        e8, k8, _ = timed_gemm_steps(torch, dist, p8, args.steps, args.warmup, None)
        e8, k8 = max_over_ranks(e8, k8)
        # all 2^26 outputs of one operand set, e2m1 path against int8 path (same synthetic weights, this rank's activations)
        p8.Xs[0].copy_(pipe.Xs[0])
        pipe.step(0)
        p8.step(0)
        torch.cuda.synchronize()
        same = bool(torch.equal(pipe.D, p8.D))
        if not same:
            raise SystemExit("the e2m1 path and the int8 path disagree")
        int8_block = {"ms_per_step": e8 / args.steps, "tops": world * flops_step / (e8 / args.steps * 1e-3) / 1e12,
                      "kernel_ms": k8, "kernel_tops": flops_step / (k8 * 1e-3) / 1e12,
                      "kernel": "tc5_gemm_pair_kernel (cta_group::2, kind::i8)",
                      "e2m1_output_equal_on_all_elements": same}
        del p8
        torch.cuda.empty_cache()

    # ---- end-to-end through the host-buffer C-ABI call (pinned host operands, D2H of the result)
    e2e_steps = max(2, min(args.steps, 5))
    hW = torch.empty((WBITS, M, K // 32), dtype=torch.int32).pin_memory()
    hX = torch.empty((XBITS, N, K // 32), dtype=torch.int32).pin_memory()
    hW.copy_(pipe.W.cpu())
    hX.copy_(pipe.Xs[0].cpu())
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
    (e2e_s,) = max_over_ranks(e2e_s)
    if rank == 0 and not torch.equal(hD, ap.apmm(pipe.W, pipe.Xs[0], algo="imma").cpu()):
        raise SystemExit("host-buffer path disagrees with the device path")
    e2e = {"value": world * flops_step / e2e_s / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": hW.numel() * 4 + hX.numel() * 4, "d2h_bytes_per_step": hD.numel() * 4,
           "steps": e2e_steps, "timer": "host wall clock around the synchronous C-ABI call, max over ranks",
           "bound": "PCIe: every rank of a node moves its 256 MiB result through the same host"}
    del hW, hX, hD

    # ---- the other workloads of the metric
    Wkeep, Xkeep = pipe.W, pipe.Xs[0]
    step_path, launches_per_step = pipe.path, pipe.launches_per_step
    del pipe
    torch.cuda.empty_cache()
    resnet = resnet_block(torch, dist, dev, world, rank, args)
    gather = allgather_block(torch, dist, ap, _cabi, dev, world, rank, args) if world > 1 else None
    pairs = sweep = conv = None
    if world == 1 and algo == "tcgen05" and not args.quick:
        pairs = pairs_block(torch, ap, _cabi, dev, max(5, args.steps // 2))
        sweep = m64_sweep_block(torch, ap)
        conv = conv_c3_block(torch, ap, _cabi)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel
    peaks = measured_peaks()
    kind = {"tcgen05": 5 if step_path == "fp4" else 0, "imma": 1, "bmma": 2}[algo]
    peak_ops = probe_peak(torch, _cabi, kind, 20000 if kind in (0, 5) else 4000)
    peak_i8 = probe_peak(torch, _cabi, 0, 20000) if kind == 5 else peak_ops
    ops_launch = flops_step * (WBITS * XBITS if algo == "bmma" else 1)  # bit-ops for the b1 path
    achieved = ops_launch / (kernel_ms * 1e-3) / 1e12
    full_shape_one_gpu = world == 1 and algo == "tcgen05" and step_path in TRAFFIC_8192
    operand_bytes = (M * K + N * K) // 2 if step_path == "fp4" else M * K + N * K
    roofline = {
        "bound": "tensor", "kernel": {"tcgen05": "tc5_gemm_pair_kernel (cta_group::2, kind::mxf4: e2m1 operands, unit scales)"
                                      if step_path == "fp4" else "tc5_gemm_pair_kernel (cta_group::2, kind::i8)",
                                      "imma": "plane_core_kernel<u8>", "bmma": "plane_core_kernel<b1>"}[algo],
        "achieved": achieved, "peak": peak_ops / 1e12, "unit": "TOP/s" if algo != "bmma" else "Tbitop/s",
        "frac": achieved / (peak_ops / 1e12),
        "peak_source": "issue-loop peak of this instruction measured in this run (apnn_probe_peak)",
        "bf16_tflops_measured": peaks.get("bf16_tflops"), "bf16_tflops_sustained": peaks.get("bf16_tflops_sustained"),
        "frac_of_2x_bf16_burst": achieved / (2 * peaks["bf16_tflops"]) if peaks.get("bf16_tflops") else None,
        "kernel_ms": kernel_ms, "algorithmic_ops_per_launch": ops_launch,
        "traffic": TRAFFIC_8192[step_path][0] if full_shape_one_gpu else None,
        "traffic_source": ("constant from an earlier capture, not measured in this run: dram__bytes_read.sum + "
                           "dram__bytes_write.sum per launch, " + TRAFFIC_8192[step_path][1])
        if full_shape_one_gpu else None,
        "algorithmic_bytes_per_launch": operand_bytes + 4 * M * N,
    }
    if int8_block is not None:
        int8_block["kernel_frac_of_i8_probe_peak"] = int8_block["kernel_tops"] / (peak_i8 / 1e12)
        int8_block["i8_probe_peak_tops"] = peak_i8 / 1e12
    if sustained is not None:
        sustained["kernel_frac_of_probe_peak"] = sustained["kernel_tops"] / (peak_ops / 1e12)

    # ---- CPU baseline: the reference's compute_ref on a bounded sample of rows
    from oracle import ref
    import oracle
    threads = os.cpu_count() or 1
    rpt = 2
    Wh = Wkeep.cpu().numpy().view(np.uint32)
    Xh = Xkeep.cpu().numpy().view(np.uint32)
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
    if not np.array_equal(np.concatenate(cpu_out), ap.apmm(Wkeep, Xkeep, algo="imma")[: threads * rpt].cpu().numpy()):
        raise SystemExit("CPU baseline and GPU disagree on the sampled rows")
    cpu_baseline = {"value": 2.0 * threads * rpt * N * K / cdt / 1e12, "unit": UNIT, "cores": threads,
                    "kind": kind_cpu,
                    "sample": f"{threads * rpt} of {M} output rows ({rpt} per thread), full N and K, bit-serial compute_ref"}

    # beside the CPU loops: the reference's own GPU kernel for this pair, compiled unmodified for
    # sm_100a into oracle/_ref (part of the same baseline leg; absent -> omitted)
    bar = os.path.join(ROOT, "oracle", "_ref", "bar_gemm_w1a2")
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

    if sampler is not None:
        sampler.stop()
    line = {
        "metric": METRIC, "value": world * flops_step / (ms_per_step * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": {"fp4": "e2m1 operands holding the integer levels, fp32 accumulate (sums of small integers: exact), int32 out",
                                                     "int8": "u8/s8 operands, int32 accumulate (exact)",
                                                     "planes": "u8/s8 operands, int32 accumulate (exact)"}.get(step_path, "int32 (exact)"),
        "data": "synthetic", "config": workload_config(world), "algo": algo, "path": step_path,
        "step": {"fp4": "activation planes -> e2m1 nibbles, then the tcgen05 kind::mxf4 GEMM",
                 "int8": "activation planes -> int8 rows, then the tcgen05 kind::i8 GEMM",
                 "planes": "one launch: tcgen05 kind::i8 GEMM reading the packed activation planes (bits spread inside the kernel)"
                 }.get(step_path, "one launch of the warp-level kernel")
                + "; the static weights' tensor-core image is made once before the timed region",
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        "sustained": sustained, "int8_path": int8_block, "resnet18": resnet, "allgather": gather,
        "pairs_8192": pairs, "m64_sweep": sweep, "conv_c3": conv,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- other blocks of the line
def resnet_block(torch, dist, dev, world, rank, args):
    """ResNet-18 w1a2, 224x224x3, global batch 1024 sharded over the ranks (no collective): one CUDA-graph
    replay of the forward per step, max over ranks; end to end with pinned host images in and logits out."""
    from apnn_tc_b200 import nets
    batch = RESNET_GLOBAL_BATCH // world
    steps = max(10, min(args.steps, 50))
    spec = nets.resnet18_spec()
    net = nets.Network(spec, batch, device=dev)
    g = torch.Generator(device=dev).manual_seed(0xA9117C + 5 + rank)
    images = (torch.rand((batch, spec.image_hw, spec.image_hw, 3), device=dev, generator=g) * 20 - 10).contiguous()
    net.capture(images)
    for _ in range(max(3, args.warmup)):
        net.replay()
    net.check()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t0.record()
    for _ in range(steps):
        net.replay()
    t1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    net.check()
    ms = t0.elapsed_time(t1) / steps
    logits = net.out[spec.layers[-1].name]
    himg = images.cpu().pin_memory()
    hlog = torch.empty(logits.shape, dtype=logits.dtype).pin_memory()
    e2e_steps = 5
    torch.cuda.synchronize()
    c0 = time.perf_counter()
    for _ in range(e2e_steps):
        images.copy_(himg, non_blocking=True)
        net.replay()
        hlog.copy_(logits, non_blocking=True)
        torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - c0) / e2e_steps
    if dist is not None:
        t = torch.tensor([ms, e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    out = {
        "metric": "resnet18_w1a2_images_per_s", "images_per_s": batch * world / (ms * 1e-3), "ms_per_step": ms,
        "steps": steps, "global_batch": batch * world, "per_gpu_batch": batch, "scaling": "strong",
        "sharding": "batch-sharded, no collective", "launches_per_forward": net.launches_per_forward,
        "e2e_images_per_s": batch * world / e2e_s, "h2d_bytes_per_step": himg.numel() * 4,
        "d2h_bytes_per_step": hlog.numel() * hlog.element_size(),
        "l2": "activations of one forward exceed L2 at every per-GPU batch used here",
    }
    del net, images, himg, hlog
    torch.cuda.empty_cache()
    return out


def allgather_block(torch, dist, ap, cabi, dev, world, rank, args):
    """N > 1: the N-sharded 8192^3 GEMM with its output gathered on every rank inside each step.  Fused: the
    GEMM epilogue stores every tile into all ranks' [g][M][N/g] buffers (plain peer stores over NVLink), for the
    int32 slices and for the 2-bit packed output; NCCL: all_gather_into_tensor after the GEMM.  Every fused
    result is checked against an NCCL all-gather of the ranks' slices."""
    from apnn_tc_b200 import shard
    steps = max(5, min(args.steps, 20))
    out = {"ranks": world}

    def timed(pipe, after_step):
        def one(i, ev=None):
            pipe.step(i, ev)
            after_step()
        for i in range(3):
            one(i)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        torch.cuda._sleep(2_000_000)   # untimed: lets the host queue ahead of the device (see timed_gemm_steps)
        pipe.begin(t0)
        for i in range(steps):
            one(i)
        pipe.end(t1)
        torch.cuda.synchronize()
        dist.barrier()
        if int(pipe.flag.item()) != 0:
            raise SystemExit("tcgen05 kernel reported an expired wait")
        t = torch.tensor([t0.elapsed_time(t1) / steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def check(gathered, local):
        ref = torch.empty_like(gathered)
        dist.all_gather_into_tensor(ref.view(world * gathered.shape[1], -1), local.contiguous().view(gathered.shape[1], -1))
        torch.cuda.synchronize()
        if not torch.equal(ref, gathered):
            raise SystemExit(f"rank {rank}: gathered output differs from the all-gather of the slices")

    # int32 slices, fused
    sg = shard.SymmetricGather(M, N, dev)
    pipe = GemmPipeline(torch, ap, cabi, dev, rank, D=sg.local_slot(),
                        epilogue=ap.make_epilogue("int32", peer_out=sg.peer_destinations()))
    ms = timed(pipe, sg.barrier)   # every rank's tiles have landed before the next step overwrites them
    check(sg.buffer, sg.local_slot())
    egress = (world - 1) * M * N * 4
    out["fused_int32"] = {"path": pipe.path, "ms_per_step": ms, "bytes_leaving_each_gpu": egress, "egress_gb_s": egress / (ms * 1e-3) / 1e9,
                          "tops": world * 2.0 * M * N * K / (ms * 1e-3) / 1e12, "verified_against_nccl": True}
    # int32 slices, NCCL after the GEMM
    gathered = torch.empty((world, M, N), dtype=torch.int32, device=dev)
    pipe2 = GemmPipeline(torch, ap, cabi, dev, rank)
    ms = timed(pipe2, lambda: shard.allgather_columns(pipe2.D, out=gathered))
    out["nccl_int32"] = {"ms_per_step": ms, "bytes_leaving_each_gpu": egress, "egress_gb_s": egress / (ms * 1e-3) / 1e9,
                         "tops": world * 2.0 * M * N * K / (ms * 1e-3) / 1e12}
    del pipe, pipe2, gathered, sg
    torch.cuda.empty_cache()
    # the 2-bit packed output [2][M][N/32] (low bits, the reference's fused decompose kernels), fused
    sgp = shard.SymmetricGather(2 * M, N // 32, dev)
    # (int8 kernel: its 256-wide tiles give every row 32 contiguous bytes of packed words, one store per destination;
    # the 224-wide tiles of the e2m1 kernel would scatter 4-byte words over NVLink)
    pipe3 = GemmPipeline(torch, ap, cabi, dev, rank, D=sgp.local_slot(), path="int8",
                         epilogue=ap.make_epilogue("lowbits", 2, peer_out=sgp.peer_destinations()))
    ms = timed(pipe3, sgp.barrier)
    check(sgp.buffer, sgp.local_slot())
    egress = (world - 1) * 2 * M * (N // 32) * 4
    out["fused_packed_2bit"] = {"path": "int8", "ms_per_step": ms, "bytes_leaving_each_gpu": egress,
                                "egress_gb_s": egress / (ms * 1e-3) / 1e9,
                                "tops": world * 2.0 * M * N * K / (ms * 1e-3) / 1e12, "verified_against_nccl": True}
    out["link"] = "NVLink 5 through NVSwitch; 770 GB/s per direction measured peer copy on this pool (900 nominal)"
    out["steps"] = steps
    del pipe3, sgp
    torch.cuda.empty_cache()
    return out


def pairs_block(torch, ap, cabi, dev, steps):
    """The other bit pairs of the sweep at 8192^3: w2a2 on the 4-bit floating-point path like w1a2, w1a3 and
    w1a4 on the int8 path (one byte per level whatever its width); kernel time by events, effective TOPS."""
    out = {}
    for wb, xb in ((1, 3), (1, 4), (2, 2)):
        pipe = GemmPipeline(torch, ap, cabi, dev, 0, wbits=wb, xbits=xb)
        ms, kms, _ = timed_gemm_steps(torch, None, pipe, steps, 3)
        out[f"w{wb}a{xb}"] = {"path": pipe.path, "ms_per_step": ms / steps, "tops": 2.0 * M * N * K / (ms / steps * 1e-3) / 1e12,
                              "kernel_ms": kms, "kernel_tops": 2.0 * M * N * K / (kms * 1e-3) / 1e12}
        del pipe
        torch.cuda.empty_cache()
    return out


def m64_sweep_block(torch, ap):
    """M = 64, N = K = 128..1024 for the four bit pairs (the reference's GEMM sweep): microseconds per launch
    from a graph of 20 launches (L2 flushed before each replay), against the HBM time of the algorithmic bytes."""
    gen = torch.Generator(device="cuda").manual_seed(0xA9117C + 2)
    hbm = (measured_peaks().get("hbm_gbs") or 6545.0) * 1e9
    out = {"unit": "us per launch (graph replay)", "hbm_gbs_measured": hbm / 1e9, "rows": []}
    for wb, xb in ((1, 2), (1, 3), (1, 4), (2, 2)):
        for n in range(128, 1025, 128):
            W, X = words(torch, (wb, 64, n // 32), gen), words(torch, (xb, n, n // 32), gen)
            D = torch.empty((64, n), dtype=torch.int32, device="cuda")
            us = graph_time_us(torch, lambda: ap.apmm(W, X, D, algo="imma"))
            byts = wb * 64 * n // 8 + xb * n * n // 8 + 4 * 64 * n
            out["rows"].append({"pair": f"w{wb}a{xb}", "n": n, "us": round(us, 2), "tops": round(2 * 64 * n * n / us / 1e6, 2),
                                "algorithmic_bytes": byts, "hbm_frac": round(byts / (us * 1e-6) / hbm, 4)})
    return out


def conv_c3_block(torch, ap, cabi):
    """Batch 8, 16x16, C = O = 128..1024, 3x3, BN thresholds -> 2-bit output: one launch as a network chains it
    (int8 rows in, filter expanded once), and from packed planes through apnn_conv2d_ex (expand + conv)."""
    from apnn_tc_b200.ops import _stream_ptr
    gen = torch.Generator(device="cuda").manual_seed(0xA9117C + 3)
    L = cabi.lib()
    peak = probe_peak(torch, cabi, 0, 20000) / 1e12
    out = {"unit": "us per launch (graph replay)", "tensor_peak_tops": peak, "rows": []}
    B, H = 8, 16
    for wb, xb in ((1, 2), (1, 4), (2, 2)):
        for C in range(128, 1025, 128):
            X = words(torch, (xb, B, H + 2, H + 2, C // 32), gen)
            Wt = words(torch, (wb, C, 3, 3, C // 32), gen)
            T = torch.sort(torch.randint(0, 9 * C * 3, (C, 3), dtype=torch.int32, device="cuda", generator=gen),
                           dim=1).values.contiguous()
            flops = 2.0 * B * H * H * C * 9 * C
            x8 = ap.expand_planes(X.reshape(xb, -1, C // 32))
            w8 = ap.expand_planes(Wt.reshape(wb, C, -1), signed=(wb == 1))
            flag = torch.zeros(1, dtype=torch.int32, device="cuda")
            o8 = torch.zeros((B, H, H, C), dtype=torch.uint8, device="cuda")
            epi8 = ap.make_epilogue("thresholds", 2, thresholds=T, out_i8=True)
            us_chain = graph_time_us(torch, lambda: cabi.check(L.apnn_conv2d_i8(
                _stream_ptr(), w8.data_ptr(), x8.data_ptr(), o8.data_ptr(), B, H, H, C, C, 3, 1, 1 if wb == 1 else 0,
                ctypes.byref(epi8), flag.data_ptr()), "conv"))
            ws = torch.empty(ap.conv_workspace_bytes(B, H, H, C, C, 3), dtype=torch.uint8, device="cuda")
            outp = torch.empty((2, B, H, H, C // 32), dtype=torch.int32, device="cuda")
            epi = ap.make_epilogue("thresholds", 2, signed="w" if wb == 1 else "none", thresholds=T)
            us_planes = graph_time_us(torch, lambda: ap.apconv(Wt, X, outp, epilogue=epi, algo="tcgen05", workspace=ws))
            out["rows"].append({"pair": f"w{wb}a{xb}", "C": C, "us_chained": round(us_chain, 2),
                                "tops_chained": round(flops / us_chain / 1e6, 1),
                                "tensor_frac_chained": round(flops / us_chain / 1e6 / peak, 3),
                                "us_from_planes": round(us_planes, 2), "tops_from_planes": round(flops / us_planes / 1e6, 1)})
    return out


# ----------------------------------------------------------------------------- single kernels (profiling cases)
def kernel_cases(torch, ap, cabi):
    """name -> (kernel it exercises, set-up returning (call, algorithmic bytes, algorithmic ops)).  Small enough for
    an ncu capture (inputs above the 126 MB L2 where the kernel is memory-bound, a few hundred MB at most)."""
    from apnn_tc_b200.ops import _stream_ptr
    L = cabi.lib()
    gen = torch.Generator(device="cuda").manual_seed(0xA9117C + 9)

    def gemm(M_, N_, K_, algo, wb=1, xb=2):
        def setup():
            W, X = words(torch, (wb, M_, K_ // 32), gen), words(torch, (xb, N_, K_ // 32), gen)
            D = torch.empty((M_, N_), dtype=torch.int32, device="cuda")
            ws = torch.empty(ap.gemm_workspace_bytes(M_, N_, K_), dtype=torch.uint8, device="cuda") if algo == "tcgen05" else None
            return (lambda: ap.apmm(W, X, D, algo=algo, workspace=ws)), wb * M_ * K_ // 8 + xb * N_ * K_ // 8 + 4 * M_ * N_, 2.0 * M_ * N_ * K_
        return setup

    def pack(from_float):
        def setup():
            rows, C = 65536, 512
            src = (torch.rand((rows, C), device="cuda", generator=gen) * 20 - 10) if from_float else \
                torch.randint(0, 4, (rows, C), dtype=torch.int32, device="cuda", generator=gen)
            out = torch.empty((2, rows, C // 32), dtype=torch.int32, device="cuda")
            fn = (lambda: ap.images_quantization(src, 2, out)) if from_float else (lambda: ap.Bit_compression(src, 2, out))
            return fn, 4 * rows * C + 2 * rows * C // 8, 0.0
        return setup

    def expand():
        P = words(torch, (2, 8192, 8192 // 32), gen)
        out = torch.empty((8192, 8192), dtype=torch.uint8, device="cuda")
        return (lambda: ap.expand_planes(P, out=out)), 2 * 8192 * 8192 // 8 + 8192 * 8192, 0.0

    def expand_fp4():
        # 16384 rows so that the output (64 MiB) and the L2 flush between calls keep the case above L2
        P = words(torch, (2, 16384, 8192 // 32), gen)
        out = torch.empty((16384, 8192 // 2), dtype=torch.uint8, device="cuda")
        return (lambda: ap.expand_planes_fp4(P, out=out)), 2 * 16384 * 8192 // 8 + 16384 * 8192 // 2, 0.0

    def gemm_fp4(M_, N_, K_):
        def setup():
            W4 = ap.expand_planes_fp4(words(torch, (1, M_, K_ // 32), gen), signed=True)
            X4 = ap.expand_planes_fp4(words(torch, (2, N_, K_ // 32), gen))
            D = torch.empty((M_, N_), dtype=torch.int32, device="cuda")
            flag = torch.zeros(1, dtype=torch.int32, device="cuda")
            return (lambda: ap.gemm_fp4(W4, X4, D, status_flag=flag)), (M_ * K_ + N_ * K_) // 2 + 4 * M_ * N_, 2.0 * M_ * N_ * K_
        return setup

    def window_rows():
        B_ = 128
        img = (torch.rand((B_, 224, 224, 3), device="cuda", generator=gen) * 20 - 10).contiguous()
        kp = 192
        out = torch.empty((B_ * 56 * 56, kp), dtype=torch.uint8, device="cuda")
        fn = lambda: cabi.check(L.apnn_quantize_window_rows_i8(_stream_ptr(), img.data_ptr(), out.data_ptr(), B_, 224, 224, 3, 7, 4,
                                                               8 | cabi.QUANT_CENTRED, kp), "gather")
        return fn, img.numel() * 4 + out.numel(), 0.0

    def maxpool():
        B_, H_, C_ = 64, 112, 128
        x = torch.randint(0, 4, (B_, H_, H_, C_), dtype=torch.uint8, device="cuda", generator=gen)
        out = torch.empty((B_, H_ // 2, H_ // 2, C_), dtype=torch.uint8, device="cuda")
        fn = lambda: cabi.check(L.apnn_maxpool2x2_i8(_stream_ptr(), x.data_ptr(), out.data_ptr(), B_, H_, H_, C_, 0, 0), "maxpool")
        return fn, x.numel() + out.numel(), 0.0

    def requantize():
        rows, N_ = 16384, 4096
        acc = torch.randint(-3000, 3000, (rows, N_), dtype=torch.int32, device="cuda", generator=gen)
        T = torch.sort(torch.randint(-2000, 2000, (N_, 3), dtype=torch.int32, device="cuda", generator=gen), dim=1).values.contiguous()
        out = torch.empty((rows, N_), dtype=torch.uint8, device="cuda")
        epi = ap.make_epilogue("thresholds", 2, thresholds=T, out_i8=True)
        fn = lambda: cabi.check(L.apnn_requantize_i32(_stream_ptr(), acc.data_ptr(), out.data_ptr(), rows, N_, ctypes.byref(epi)), "requantize")
        return fn, 4 * rows * N_ + rows * N_, 0.0

    def conv(B_, H_, CIN, COUT, R=3):
        def setup():
            pad = (R - 1) // 2
            x8 = torch.zeros((B_, H_ + 2 * pad, H_ + 2 * pad, CIN), dtype=torch.uint8, device="cuda")
            x8[:, pad:pad + H_, pad:pad + H_] = torch.randint(0, 4, (B_, H_, H_, CIN), dtype=torch.uint8, device="cuda", generator=gen)
            w8 = (torch.randint(0, 2, (COUT, R * R * CIN), dtype=torch.int8, device="cuda", generator=gen) * 2 - 1).contiguous()
            T = torch.sort(torch.randint(-300, 300, (COUT, 3), dtype=torch.int32, device="cuda", generator=gen), dim=1).values.contiguous()
            out = torch.zeros((B_, H_ + 2, H_ + 2, COUT), dtype=torch.uint8, device="cuda")
            flag = torch.zeros(1, dtype=torch.int32, device="cuda")
            epi = ap.make_epilogue("thresholds", 2, thresholds=T, out_i8=True, out_halo=1)
            fn = lambda: cabi.check(L.apnn_conv2d_i8(_stream_ptr(), w8.data_ptr(), x8.data_ptr(), out.data_ptr(), B_, H_, H_, CIN, COUT,
                                                     R, 1, 1, ctypes.byref(epi), flag.data_ptr()), "conv")
            return fn, x8.numel() + w8.numel() + B_ * H_ * H_ * COUT, 2.0 * B_ * H_ * H_ * COUT * R * R * CIN
        return setup

    return {
        "gemm_u8_m64": ("plane_core_kernel<u8> (GEMM, small tile class)", gemm(64, 1024, 1024, "imma")),
        "gemm_u8_2048": ("plane_core_kernel<u8> (GEMM)", gemm(2048, 2048, 2048, "imma")),
        "gemm_b1_m64": ("plane_core_kernel<b1> (GEMM, small tile class)", gemm(64, 1024, 1024, "bmma")),
        "gemm_b1_2048": ("plane_core_kernel<b1> (GEMM)", gemm(2048, 2048, 2048, "bmma")),
        "pair_gemm_4096": ("expand_planes_kernel + tc5_gemm_pair_kernel", gemm(4096, 4096, 4096, "tcgen05")),
        "pack_planes": ("pack_planes_kernel<levels>", pack(False)),
        "quantize_pack": ("pack_planes_kernel<float>", pack(True)),
        "expand_planes": ("expand_planes_kernel", expand),
        "expand_planes_fp4": ("expand_nibbles_kernel", expand_fp4),
        "pair_gemm_fp4_4096": ("tc5_gemm_pair_kernel<MX> (kind::mxf4)", gemm_fp4(4096, 4096, 4096)),
        "window_rows": ("quantize_window_rows_i8_kernel (ResNet-18 first layer, 128 images, centred 8-bit)", window_rows),
        "maxpool": ("maxpool2x2_i8_kernel", maxpool),
        "requantize": ("requantize_i32_kernel", requantize),
        "conv_c3_1024": ("tc5_gemm_kernel<256,128,split-K> (batch 8, 16x16, 1024 -> 1024)", conv(8, 16, 1024, 1024)),
        "conv_l1": ("tc5_gemm_kernel<64,64> flat (128 images, 56x56, 64 -> 64)", conv(128, 56, 64, 64)),
        "conv_l4": ("tc5_gemm_kernel<256,128> boxes (128 images, 7x7, 512 -> 512)", conv(128, 7, 512, 512)),
        "pair_conv": ("tc5_conv_pair_kernel<3> (64 images, 28x28, 512 -> 512)", conv(64, 28, 512, 512)),
    }


def run_case(args) -> None:
    """One kernel on one fixed small problem: `--steps` launches after three warm-up launches, device time per launch by
    CUDA events.  The command the ncu captures under profiles/ run."""
    import torch
    import apnn_tc_b200 as ap
    from apnn_tc_b200 import _cabi
    torch.cuda.set_device(0)
    cases = kernel_cases(torch, ap, _cabi)
    if args.case not in cases:
        raise SystemExit("--case is one of: " + ", ".join(sorted(cases)))
    kernel, setup = cases[args.case]
    fn, byts, ops = setup()
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0.0
    for _ in range(args.steps):
        flush_l2(torch)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    us = total * 1e3 / args.steps
    hbm = (measured_peaks().get("hbm_gbs") or 6545.0)
    print(json.dumps({"case": args.case, "kernel": kernel, "us_per_call": round(us, 2), "steps": args.steps,
                      "algorithmic_bytes": int(byts), "gb_s": round(byts / us / 1e3, 1), "hbm_frac_of_measured": round(byts / us / 1e3 / hbm, 3),
                      "algorithmic_ops": ops, "tops": round(ops / us / 1e6, 1) if ops else None,
                      "l2": "256 MiB rewritten before every launch"}), flush=True)


# ----------------------------------------------------------------------------- network workloads
NET_BATCH = {"resnet18": 1024, "vgg_variant": 1024, "alexnet": 128}


def run_net(args) -> None:
    """images/s of a whole w1a2 network (the AlexNet / VGG-variant / ResNet-18 model lists of APNN-TC-nn):
    global batch sharded over the ranks (no collective), one CUDA-graph replay of the layer sequence per step."""
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
    logits = net.out[spec.layers[-1].name]
    himg = images.cpu().pin_memory()
    hlog = torch.empty(logits.shape, dtype=logits.dtype).pin_memory()
    e2e_steps = max(2, min(args.steps, 5))
    torch.cuda.synchronize()
    c0 = time.perf_counter()
    for _ in range(e2e_steps):
        images.copy_(himg, non_blocking=True)
        net.replay()
        hlog.copy_(logits, non_blocking=True)
        torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - c0) / e2e_steps
    if dist is not None:
        t = torch.tensor([ms, e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    clocks = sampler.window(wall0, wall1) if sampler is not None else None
    if sampler is not None:
        sampler.stop()
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
                    "d2h_bytes_per_step": hlog.numel() * hlog.element_size(), "steps": e2e_steps},
            "gpu_launches": net.launches_per_forward * args.steps, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main() -> None:
    ap_ = argparse.ArgumentParser()
    ap_.add_argument("--gpus", type=int, default=1)
    ap_.add_argument("--steps", type=int, default=20)
    ap_.add_argument("--warmup", type=int, default=5)
    ap_.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap_.add_argument("--algo", default="tcgen05", choices=["tcgen05", "imma", "bmma"])
    ap_.add_argument("--profile", action="store_true",
                     help="timed GEMM steps only (no e2e, probe, CPU baseline or other blocks): the command ncu captures")
    ap_.add_argument("--path", default="", choices=["", "fp4", "int8", "planes"],
                     help="tensor path of the headline step: fp4 (default for w1a2: e2m1 operands, kind::mxf4, exact), int8 "
                          "(kind::i8), planes (one launch, apnn_gemm_w8 spreads the activation planes in the GEMM kernel)")
    ap_.add_argument("--quick", action="store_true", help="skip the N = 1 sweep blocks (pairs_8192, m64_sweep, conv_c3)")
    ap_.add_argument("--workload", default="gemm", choices=["gemm", "resnet18", "vgg_variant", "alexnet"],
                     help="gemm (default: the headline line with every block) or one whole w1a2 network (images/s)")
    ap_.add_argument("--batch", type=int, default=0, help="global batch of a network workload")
    ap_.add_argument("--case", default="", help="time one kernel on a fixed small problem (see kernel_cases) and exit")
    args = ap_.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload != "gemm":
        run_net(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
