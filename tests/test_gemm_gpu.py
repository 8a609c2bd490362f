"""GPU parity of the GEMM path against the CPU oracle, through the C ABI.  Bit-exact."""
import os

import numpy as np
import pytest
import torch

import oracle
from gpu_util import to_dev, to_host

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_host_loops.npz"))
PAIRS = [(1, 2), (1, 3), (1, 4), (2, 2)]


def run_gemm(W, X, **kw):
    import apnn_tc_b200 as ap
    out = ap.apmm(to_dev(W), to_dev(X), **kw)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("algo", ["imma", "bmma"])
@pytest.mark.parametrize("wb,xb", PAIRS)
def test_reference_inputs_small(cuda_device, wb, xb, algo):
    """The reference's own operands (default-seed rand stream), M=64, N=K=128/256, against
    the committed outputs of the reference's compute_ref."""
    for n in (128, 256):
        W, X = oracle.fill_gemm(64, n, n, wb, xb)
        D = to_host(run_gemm(W, X, algo=algo), np.int32)
        assert np.array_equal(D, GOLD[f"gemm_w{wb}a{xb}_64x{n}x{n}"])


@pytest.mark.parametrize("algo", ["imma", "bmma"])
def test_config1_w1a2_64x1024x1024(cuda_device, algo):
    W, X = oracle.fill_gemm(64, 1024, 1024, 1, 2)
    D = to_host(run_gemm(W, X, algo=algo), np.int32)
    assert int(D.astype(np.int64).sum()) == 49072252 and int(D[0, 0]) == 722
    assert np.array_equal(D, oracle.gemm_popc(W, X, threads=4))


@pytest.mark.parametrize("wb,xb", PAIRS + [(2, 1), (4, 1), (1, 1)])
def test_m64_sweep(cuda_device, wb, xb):
    """M=64, N=K in 128..1024 (the reference's sweep), value-level seeded operands."""
    rng = np.random.default_rng(0xA9117C + 2)
    for n in range(128, 1025, 128):
        W, _ = oracle.value_planes(rng, 64, n, wb)
        X, _ = oracle.value_planes(rng, n, n, xb)
        D = to_host(run_gemm(W, X, algo="imma"), np.int32)
        assert np.array_equal(D, oracle.gemm_popc(W, X, threads=4)), (wb, xb, n)


@pytest.mark.parametrize("algo", ["imma", "bmma"])
@pytest.mark.parametrize("M,N,K", [(1, 1, 128), (5, 3, 128), (64, 40, 384), (130, 257, 640), (300, 520, 1152),
                                   (128, 128, 8192)])
def test_ragged_shapes(cuda_device, M, N, K, algo):
    rng = np.random.default_rng(M * 1000 + N)
    W, wl = oracle.value_planes(rng, M, K, 1)
    X, xl = oracle.value_planes(rng, N, K, 2)
    D = to_host(run_gemm(W, X, algo=algo), np.int32)
    assert np.array_equal(D, wl.astype(np.int64) @ xl.astype(np.int64).T)


def test_big_tile_all_pairs(cuda_device):
    """Shapes large enough to select the 128x128 tile class."""
    rng = np.random.default_rng(99)
    for wb, xb in PAIRS + [(2, 1), (3, 1), (4, 1), (1, 1)]:
        W, wl = oracle.value_planes(rng, 1100, 512, wb)
        X, xl = oracle.value_planes(rng, 1300, 512, xb)
        D = to_host(run_gemm(W, X, algo="imma"), np.int32)
        assert np.array_equal(D, wl.astype(np.int64) @ xl.astype(np.int64).T), (wb, xb)


def test_extreme_values(cuda_device):
    """All-ones operands (the reference's known-answer fill): D = (2^w-1)(2^x-1) K."""
    for wb, xb in PAIRS:
        K = 1024
        W = np.full((wb, 64, K // 32), 0xFFFFFFFF, dtype=np.uint32)
        X = np.full((xb, 96, K // 32), 0xFFFFFFFF, dtype=np.uint32)
        D = to_host(run_gemm(W, X, algo="imma"), np.int32)
        assert (D == ((1 << wb) - 1) * ((1 << xb) - 1) * K).all()
        D0 = to_host(run_gemm(np.zeros_like(W), X, algo="imma"), np.int32)
        assert not D0.any()


@pytest.mark.parametrize("wb,xb", [(1, 2), (2, 2)])
def test_lowbit_pack_against_reference_golden(cuda_device, wb, xb):
    import apnn_tc_b200 as ap
    W, X = oracle.fill_gemm(64, 128, 128, wb, xb)
    fn = ap.apmm_w1a2_decompose if wb == 1 else ap.apmm_w2a2_decompose
    P = to_host(fn(to_dev(W), to_dev(X)))
    assert np.array_equal(P, GOLD[f"gemm_pack_w{wb}a{xb}_64x128x128"])


@pytest.mark.parametrize("algo", ["imma", "bmma"])
@pytest.mark.parametrize("signed", ["none", "w", "x"])
@pytest.mark.parametrize("mode", ["int32", "lowbits", "thresholds"])
def test_fused_epilogues(cuda_device, mode, signed, algo):
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(17)
    M, N, K = 200, 352, 768
    wb, xb = (1, 2) if signed != "x" else (2, 1)
    W, wl = oracle.value_planes(rng, M, K, wb)
    X, xl = oracle.value_planes(rng, N, K, xb)
    acc = oracle.gemm_popc(W, X, threads=4)
    if signed == "w":
        v = oracle.signed_correct(acc, oracle.row_sums(X), 1)
        assert np.array_equal(v, (2 * wl.astype(np.int64) - 1) @ xl.astype(np.int64).T)
    elif signed == "x":
        v = oracle.signed_correct(acc, oracle.row_sums(W), 0)
    else:
        v = acc
    T = None
    if mode == "thresholds":
        scale = rng.uniform(0.5, 1.5, N).astype(np.float32)
        bias = rng.uniform(-1, 1, N).astype(np.float32)
        T = oracle.fold_bn(scale, bias, float(v.mean()), float(v.std()) / 4, 2)
    epi = ap.make_epilogue(mode, 2 if mode != "int32" else 0, signed=signed,
                           thresholds=to_dev(T) if T is not None else None)
    out = ap.apmm(to_dev(W), to_dev(X), epilogue=epi, algo=algo)
    if mode == "int32":
        assert np.array_equal(to_host(out, np.int32), v)
    else:
        want = oracle.requant_pack(v, 2, 1 if mode == "lowbits" else 2, T)
        assert np.array_equal(to_host(out), want)
        if mode == "thresholds":
            assert len(np.unique(oracle.levels(v, 2, 2, T))) == 4  # all four levels occur


def test_three_bit_requant(cuda_device):
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(23)
    W, _ = oracle.value_planes(rng, 64, 256, 1)
    X, _ = oracle.value_planes(rng, 128, 256, 3)
    acc = oracle.gemm_popc(W, X)
    out = ap.apmm(to_dev(W), to_dev(X), epilogue=ap.make_epilogue("lowbits", 3))
    assert np.array_equal(to_host(out), oracle.requant_pack(acc, 3, 1))


def test_host_buffer_front_end(cuda_device):
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(31)
    M, N, K = 64, 1024, 1024
    W, _ = oracle.value_planes(rng, M, K, 1)
    X, _ = oracle.value_planes(rng, N, K, 2)
    h = ap.HostHandle(0)
    D = np.zeros((M, N), dtype=np.int32)
    h.gemm(W, X, D, 1, 2, M, N, K, algo="imma")
    assert np.array_equal(D, oracle.gemm_popc(W, X, threads=4))
    P = np.zeros((2, M, N // 32), dtype=np.uint32)
    h.gemm(W, X, P, 1, 2, M, N, K, algo="imma", epilogue=ap.make_epilogue("lowbits", 2))
    assert np.array_equal(P, oracle.requant_pack(D, 2, 1))
    h.close()


def test_errors_raise(cuda_device):
    import apnn_tc_b200 as ap
    W = torch.zeros((1, 64, 3), dtype=torch.int32, device="cuda")  # K = 96
    X = torch.zeros((2, 64, 3), dtype=torch.int32, device="cuda")
    with pytest.raises(ap.ApnnError):
        ap.apmm(W, X)
    with pytest.raises(ValueError):
        ap.apmm(W.cpu(), X)


# ------------------------------------------------------------------ tcgen05 kind::i8 path
def run_tc5(W, X, epilogue=None):
    import apnn_tc_b200 as ap
    wb, M, kw = W.shape
    xb, N, _ = X.shape
    ws = torch.empty(ap.gemm_workspace_bytes(M, N, kw * 32), dtype=torch.uint8, device="cuda")
    out = ap.apmm(to_dev(W), to_dev(X), algo="tcgen05", workspace=ws, epilogue=epilogue)
    ap.gemm_check(ws, M, N, kw * 32)  # synchronises; raises if a bounded wait expired
    return out


@pytest.mark.parametrize("wb,xb", PAIRS + [(2, 1), (4, 1)])
def test_tcgen05_all_pairs(cuda_device, wb, xb):
    rng = np.random.default_rng(wb * 10 + xb)
    W, wl = oracle.value_planes(rng, 384, 1024, wb)
    X, xl = oracle.value_planes(rng, 768, 1024, xb)
    D = to_host(run_tc5(W, X), np.int32)
    assert np.array_equal(D, wl.astype(np.int64) @ xl.astype(np.int64).T)


@pytest.mark.parametrize("M,N,K", [(1, 1, 128), (64, 1024, 1024), (130, 257, 640), (1000, 1000, 2048), (128, 256, 8192)])
def test_tcgen05_ragged_shapes(cuda_device, M, N, K):
    rng = np.random.default_rng(M + N + K)
    W, wl = oracle.value_planes(rng, M, K, 1)
    X, xl = oracle.value_planes(rng, N, K, 2)
    D = to_host(run_tc5(W, X), np.int32)
    assert np.array_equal(D, wl.astype(np.int64) @ xl.astype(np.int64).T)


def test_tcgen05_many_tiles_per_cta(cuda_device):
    """More tiles than SMs: every CTA walks several tiles and both TMEM accumulators."""
    rng = np.random.default_rng(77)
    W, _ = oracle.value_planes(rng, 2560, 512, 1)
    X, _ = oracle.value_planes(rng, 4096 + 96, 512, 2)
    D = to_host(run_tc5(W, X), np.int32)
    assert np.array_equal(D, oracle.gemm_popc(W, X, threads=8))


def test_tcgen05_reference_inputs_config1(cuda_device):
    W, X = oracle.fill_gemm(64, 1024, 1024, 1, 2)
    D = to_host(run_tc5(W, X), np.int32)
    assert int(D.astype(np.int64).sum()) == 49072252 and int(D[0, 0]) == 722


@pytest.mark.parametrize("signed", ["none", "w", "x"])
@pytest.mark.parametrize("mode", ["int32", "lowbits", "thresholds"])
def test_tcgen05_fused_epilogues(cuda_device, mode, signed):
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(19)
    M, N, K = 200, 352, 768
    wb, xb = (1, 2) if signed != "x" else (2, 1)
    W, _ = oracle.value_planes(rng, M, K, wb)
    X, _ = oracle.value_planes(rng, N, K, xb)
    acc = oracle.gemm_popc(W, X, threads=4)
    v = acc
    if signed == "w":
        v = oracle.signed_correct(acc, oracle.row_sums(X), 1)
    elif signed == "x":
        v = oracle.signed_correct(acc, oracle.row_sums(W), 0)
    T = None
    if mode == "thresholds":
        scale = rng.uniform(0.5, 1.5, N).astype(np.float32)
        bias = rng.uniform(-1, 1, N).astype(np.float32)
        T = oracle.fold_bn(scale, bias, float(v.mean()), float(v.std()) / 4, 2)
    epi = ap.make_epilogue(mode, 2 if mode != "int32" else 0, signed=signed,
                           thresholds=to_dev(T) if T is not None else None)
    out = run_tc5(W, X, epi)
    if mode == "int32":
        assert np.array_equal(to_host(out, np.int32), v)
    else:
        assert np.array_equal(to_host(out), oracle.requant_pack(v, 2, 1 if mode == "lowbits" else 2, T))


def test_large_shape_properties(cuda_device):
    """M=N=K=8192 (the compute-bound configuration): the three contraction paths agree
    bit for bit, sampled rows equal the oracle, and the result is linear in the planes
    (D(w1a2) = D(plane0) + 2 D(plane1))."""
    import apnn_tc_b200 as ap
    M = N = K = 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    W = torch.randint(-2**31, 2**31 - 1, (1, M, K // 32), dtype=torch.int32, device="cuda", generator=g)
    X = torch.randint(-2**31, 2**31 - 1, (2, N, K // 32), dtype=torch.int32, device="cuda", generator=g)
    ws = torch.empty(ap.gemm_workspace_bytes(M, N, K), dtype=torch.uint8, device="cuda")
    D = ap.apmm(W, X, algo="tcgen05", workspace=ws)
    ap.gemm_check(ws, M, N, K)
    assert torch.equal(D, ap.apmm(W, X, algo="imma"))
    rows = np.array([0, 1, 127, 128, 4095, 4096, 8191])
    want = oracle.gemm_popc(np.ascontiguousarray(to_host(W)[:, rows]), to_host(X), threads=8)
    assert np.array_equal(to_host(D[torch.from_numpy(rows).cuda()], np.int32), want)
    D0 = ap.apmm(W, X[0:1].contiguous(), algo="tcgen05", workspace=ws)
    D1 = ap.apmm(W, X[1:2].contiguous(), algo="tcgen05", workspace=ws)
    assert torch.equal(D, D0 + 2 * D1)
    del D0, D1
    assert torch.equal(D, ap.apmm(W, X, algo="bmma"))
    # the workspace route took the 4-bit floating-point path (two-bit operands); the int8 pair kernel explicitly
    flag = torch.ones(1, dtype=torch.int32, device="cuda")
    D8 = ap.gemm_i8(ap.expand_planes(W), ap.expand_planes(X), status_flag=flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0 and torch.equal(D, D8)


@pytest.mark.parametrize("algo", ["imma", "bmma", "tcgen05"])
def test_gemm_residual(cuda_device, algo):
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(83)
    M, N, K = 150, 288, 512
    W, _ = oracle.value_planes(rng, M, K, 2)
    X, _ = oracle.value_planes(rng, N, K, 1)
    v = oracle.signed_correct(oracle.gemm_popc(W, X, threads=4), oracle.row_sums(W), 0)
    res = rng.integers(-300, 300, size=v.shape).astype(np.int32)
    v = v + res
    res_out = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    epi = ap.make_epilogue("lowbits", 2, signed="x", residual_in=to_dev(res), residual_out=res_out)
    if algo == "tcgen05":
        out = run_tc5(W, X, epi)
    else:
        out = ap.apmm(to_dev(W), to_dev(X), epilogue=epi, algo=algo)
    assert np.array_equal(to_host(res_out, np.int32), v)
    assert np.array_equal(to_host(out), oracle.requant_pack(v, 2, 1))


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (300, 260, 384), (130, 257, 640)])
@pytest.mark.parametrize("mode", ["int32", "lowbits"])
def test_tcgen05_peer_destinations(cuda_device, M, N, K, mode):
    """Every output tile also lands in the extra destinations (the fused all-gather's store path);
    here the extra destinations are two more local buffers."""
    import apnn_tc_b200 as ap
    if mode == "lowbits" and N % 32:
        pytest.skip("packed outputs need N % 32 == 0")
    rng = np.random.default_rng(M + 3 * N + K)
    W, _ = oracle.value_planes(rng, M, K, 1)
    X, _ = oracle.value_planes(rng, N, K, 2)
    acc = oracle.gemm_popc(W, X, threads=4)
    if mode == "int32":
        want = acc
        extra = [torch.full((M, N), -7, dtype=torch.int32, device="cuda") for _ in range(2)]
        epi = ap.make_epilogue("int32", peer_out=[t.data_ptr() for t in extra])
    else:
        want = oracle.requant_pack(acc, 2, 1)
        extra = [torch.full(want.shape, -7, dtype=torch.int32, device="cuda") for _ in range(2)]
        epi = ap.make_epilogue("lowbits", 2, peer_out=[t.data_ptr() for t in extra])
    out = run_tc5(W, X, epi)
    host = np.int32 if mode == "int32" else np.uint32
    assert np.array_equal(to_host(out, host), want)
    for t in extra:
        assert np.array_equal(to_host(t, host), want)


def test_peer_destinations_refused_off_the_pair_kernel(cuda_device):
    import apnn_tc_b200 as ap
    W = torch.zeros((1, 64, 4), dtype=torch.int32, device="cuda")
    X = torch.zeros((2, 64, 4), dtype=torch.int32, device="cuda")
    extra = torch.zeros((64, 64), dtype=torch.int32, device="cuda")
    with pytest.raises(ap.ApnnError):
        ap.apmm(W, X, algo="imma", epilogue=ap.make_epilogue("int32", peer_out=[extra.data_ptr()]))


@pytest.mark.parametrize("wb,xb", [(4, 4), (1, 8), (2, 8), (3, 3), (8, 8)])
def test_tcgen05_wider_pairs(cuda_device, wb, xb):
    """Bit pairs beyond the warp-level instantiations (the reference's w4a4 / w1a8 / w2a8 programs,
    LIB/83, 77, 76) run on the int8 path: any level of up to 8 bits is one byte."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(wb * 16 + xb)
    W, wl = oracle.value_planes(rng, 200, 1024, wb)
    X, xl = oracle.value_planes(rng, 328, 1024, xb)
    want = wl.astype(np.int64) @ xl.astype(np.int64).T
    assert np.array_equal(to_host(run_tc5(W, X), np.int32), want)
    assert np.array_equal(oracle.gemm_popc(W, X, threads=4), want)
    # AUTO picks the int8 path when given a workspace; without one the pair is refused
    ws = torch.empty(ap.gemm_workspace_bytes(200, 328, 1024), dtype=torch.uint8, device="cuda")
    assert np.array_equal(to_host(ap.apmm(to_dev(W), to_dev(X), algo="auto", workspace=ws), np.int32), want)
    with pytest.raises(ap.ApnnError):
        ap.apmm(to_dev(W), to_dev(X), algo="imma")


@pytest.mark.parametrize("M,N,K", [(128, 512, 25088), (200, 256, 4096), (64, 128, 8192)])
def test_tcgen05_split_k_and_requantize(cuda_device, M, N, K):
    """Few tiles, long K: apnn_gemm_i8 splits K over the SMs (atomic adds into the zeroed int32
    output); apnn_requantize_i32 then applies the thresholds."""
    import ctypes
    import apnn_tc_b200 as ap
    from apnn_tc_b200 import _cabi
    from gpu_util import spread_bytes
    rng = np.random.default_rng(M + N + K)
    W, wl = oracle.value_planes(rng, M, K, 2)
    X, xl = oracle.value_planes(rng, N, K, 1)
    want = (wl.astype(np.int64) @ (2 * xl.astype(np.int64) - 1).T).astype(np.int32)     # +-1 second operand
    a8 = ap.expand_planes(to_dev(W))
    b8 = ap.expand_planes(to_dev(X), signed=True)
    D = torch.full((M, N), 12345, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    epi = ap.make_epilogue("int32")
    _cabi.check(_cabi.lib().apnn_gemm_i8(s, a8.data_ptr(), b8.data_ptr(), D.data_ptr(), M, N, K, 0, 1, ctypes.byref(epi),
                                         flag.data_ptr()), "gemm_i8")
    assert int(flag.item()) == 0
    assert np.array_equal(D.cpu().numpy(), want)
    T = oracle.fold_bn(np.ones(N, np.float32), np.zeros(N, np.float32), float(want.mean()), float(want.std()) / 4, 2)
    q = ap.make_epilogue("thresholds", 2, thresholds=to_dev(T), out_i8=True)
    out8 = torch.zeros((M, N), dtype=torch.uint8, device="cuda")
    _cabi.check(_cabi.lib().apnn_requantize_i32(s, D.data_ptr(), out8.data_ptr(), M, N, ctypes.byref(q)), "requantize")
    assert np.array_equal(out8.cpu().numpy(), spread_bytes(oracle.levels(want, 2, 2, T).astype(np.uint8)))
    q2 = ap.make_epilogue("thresholds", 2, thresholds=to_dev(T))
    outp = torch.zeros((2, M, N // 32), dtype=torch.int32, device="cuda")
    _cabi.check(_cabi.lib().apnn_requantize_i32(s, D.data_ptr(), outp.data_ptr(), M, N, ctypes.byref(q2)), "requantize")
    assert np.array_equal(to_host(outp), oracle.requant_pack(want, 2, 2, T))
    q3 = ap.make_epilogue("lowbits", 3)
    outl = torch.zeros((3, M, N // 32), dtype=torch.int32, device="cuda")
    _cabi.check(_cabi.lib().apnn_requantize_i32(s, D.data_ptr(), outl.data_ptr(), M, N, ctypes.byref(q3)), "requantize")
    assert np.array_equal(to_host(outl), oracle.requant_pack(want, 3, 1))


@pytest.mark.parametrize("xb", [2, 3])
@pytest.mark.parametrize("M,N", [(2304, 2304), (2300, 2336)])
@pytest.mark.parametrize("mode", ["thresholds", "lowbits", "int32"])
def test_tcgen05_pair_kernel_epilogues(cuda_device, M, N, mode, xb):
    """81 pair tiles and K = 1024: the GEMM runs on CTA pairs (cta_group::2) -- with two-bit activations as
    e2m1 operands on the 4-bit floating-point path, with three-bit ones on the int8 path.  Its +-1 weights,
    threshold / low-bit requantisation and residual in / out against the oracle, on a tile-aligned
    and a ragged shape."""
    import apnn_tc_b200 as ap
    K = 1024
    rng = np.random.default_rng(M + N)
    W, _ = oracle.value_planes(rng, M, K, 1)
    X, _ = oracle.value_planes(rng, N, K, xb)
    v = oracle.signed_correct(oracle.gemm_popc(W, X, threads=8), oracle.row_sums(X), 1)
    res = rng.integers(-400, 400, size=v.shape).astype(np.int32)
    v = v + res
    T = None
    if mode == "thresholds":
        scale = rng.uniform(0.5, 1.5, N).astype(np.float32)
        bias = rng.uniform(-1, 1, N).astype(np.float32)
        T = oracle.fold_bn(scale, bias, float(v.mean()), float(v.std()) / 4, 2)
    res_out = torch.full((M, N), -1, dtype=torch.int32, device="cuda")
    epi = ap.make_epilogue(mode, 2 if mode != "int32" else 0, signed="w", thresholds=to_dev(T) if T is not None else None,
                           residual_in=to_dev(res), residual_out=res_out)
    out = run_tc5(W, X, epi)
    assert np.array_equal(to_host(res_out, np.int32), v)
    if mode == "int32":
        assert np.array_equal(to_host(out, np.int32), v)
    else:
        assert np.array_equal(to_host(out), oracle.requant_pack(v, 2, 1 if mode == "lowbits" else 2, T))
        if mode == "thresholds":
            assert len(np.unique(oracle.levels(v, 2, 2, T))) == 4
    # the same without residuals, explicitly on the pair kernel
    ws = torch.empty(ap.gemm_workspace_bytes(M, N, K), dtype=torch.uint8, device="cuda")
    epi2 = ap.make_epilogue(mode, 2 if mode != "int32" else 0, signed="w", thresholds=to_dev(T) if T is not None else None)
    out2 = ap.apmm(to_dev(W), to_dev(X), algo="tcgen05_pair", workspace=ws, epilogue=epi2)
    ap.gemm_check(ws, M, N, K)
    v0 = v - res
    if mode == "int32":
        assert np.array_equal(to_host(out2, np.int32), v0)
    else:
        assert np.array_equal(to_host(out2), oracle.requant_pack(v0, 2, 1 if mode == "lowbits" else 2, T))


@pytest.mark.parametrize("M,N,K", [(130, 544, 4096), (128, 512, 25088), (64, 1024, 2048), (300, 4096, 1152), (128, 128, 8192)])
def test_tcgen05_cluster_split_k_epilogues(cuda_device, M, N, K):
    """Few tiles and a long K: the GEMM runs as clusters whose CTAs each sum a share of K and exchange
    partial tiles through distributed shared memory before the ordinary epilogue.  int32, packed
    thresholds, int8 rows and residual in / out (int32 and int16), against the oracle."""
    import ctypes
    import apnn_tc_b200 as ap
    from apnn_tc_b200 import _cabi
    from gpu_util import spread_bytes
    rng = np.random.default_rng(M + N + K)
    W, wl = oracle.value_planes(rng, M, K, 2)
    X, xl = oracle.value_planes(rng, N, K, 1)
    v = (wl.astype(np.int64) @ (2 * xl.astype(np.int64) - 1).T).astype(np.int32)     # +-1 second operand
    a8 = ap.expand_planes(to_dev(W))
    b8 = ap.expand_planes(to_dev(X), signed=True)
    L = _cabi.lib()
    s = torch.cuda.current_stream().cuda_stream
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")

    def run(out, epi):
        _cabi.check(L.apnn_gemm_i8(s, a8.data_ptr(), b8.data_ptr(), out.data_ptr(), M, N, K, 0, 1, ctypes.byref(epi),
                                   flag.data_ptr()), "gemm_i8")
        torch.cuda.synchronize()
        assert int(flag.item()) == 0
        return out

    D = run(torch.full((M, N), 12345, dtype=torch.int32, device="cuda"), ap.make_epilogue("int32"))
    assert np.array_equal(D.cpu().numpy(), v)
    scale = rng.uniform(0.5, 1.5, N).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    T = oracle.fold_bn(scale, bias, float(v.mean()), float(v.std()) / 4, 2)
    P = run(torch.zeros((2, M, N // 32), dtype=torch.int32, device="cuda"), ap.make_epilogue("thresholds", 2, thresholds=to_dev(T)))
    assert np.array_equal(to_host(P), oracle.requant_pack(v, 2, 2, T))
    O8 = run(torch.zeros((M, N), dtype=torch.uint8, device="cuda"),
             ap.make_epilogue("thresholds", 2, thresholds=to_dev(T), out_i8=True))
    assert np.array_equal(O8.cpu().numpy(), spread_bytes(oracle.levels(v, 2, 2, T).astype(np.uint8)))
    res = rng.integers(-2000, 2000, size=v.shape).astype(np.int32)
    v2 = v + res
    for widths in (0, 3):
        rin = torch.from_numpy(res.astype(np.int16) if widths & 1 else res).cuda()
        rout = torch.zeros((M, N), dtype=torch.int16 if widths & 2 else torch.int32, device="cuda")
        epi = ap.make_epilogue("lowbits", 3, residual_in=rin, residual_out=rout, residual_i16=widths)
        P3 = run(torch.zeros((3, M, N // 32), dtype=torch.int32, device="cuda"), epi)
        want_res = np.clip(v2, -32768, 32767) if widths & 2 else v2
        assert np.array_equal(rout.cpu().numpy().astype(np.int32), want_res)
        assert np.array_equal(to_host(P3), oracle.requant_pack(v2, 3, 1))


@pytest.mark.parametrize("xb,x_signed", [(1, False), (1, True), (2, False), (3, False), (4, False)])
@pytest.mark.parametrize("M,N,K", [(100, 70, 128), (2304, 2304, 1152), (2300, 2336, 1024), (256, 512, 3200)])
def test_tcgen05_activation_planes_in_kernel(cuda_device, M, N, K, xb, x_signed):
    """apnn_gemm_w8: weights as int8 rows made once, activations straight from their packed planes -- the
    CTA-pair kernel's own warps spread the bits into its stages.  One K block, K blocks that are no
    multiple of the register prefetch depth, more tiles than SM pairs (two tiles per pair for some),
    ragged M and N, every activation width and a -1/+1 activation plane, against the oracle."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(M + N + K + 7 * xb)
    wb = 2 if x_signed else 1
    W, wl = oracle.value_planes(rng, M, K, wb)
    X, xl = oracle.value_planes(rng, N, K, xb)
    wv = wl.astype(np.int64) if x_signed else 2 * wl.astype(np.int64) - 1   # +-1 weights unless the activations are
    xv = 2 * xl.astype(np.int64) - 1 if x_signed else xl.astype(np.int64)
    want = (wv @ xv.T).astype(np.int32)
    w8 = ap.expand_planes(to_dev(W), signed=not x_signed)
    flag = torch.ones(1, dtype=torch.int32, device="cuda")
    out = ap.gemm_w8(w8, to_dev(X), w_signed=not x_signed, x_signed=x_signed, status_flag=flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    assert np.array_equal(to_host(out, np.int32), want)
    if N % 32 == 0 and not x_signed:
        scale = rng.uniform(0.5, 1.5, N).astype(np.float32)
        bias = rng.uniform(-1, 1, N).astype(np.float32)
        T = oracle.fold_bn(scale, bias, float(want.mean()), float(want.std()) / 4, 2)
        epi = ap.make_epilogue("thresholds", 2, thresholds=to_dev(T))
        packed = ap.gemm_w8(w8, to_dev(X), w_signed=True, epilogue=epi, status_flag=flag)
        torch.cuda.synchronize()
        assert int(flag.item()) == 0
        assert np.array_equal(to_host(packed), oracle.requant_pack(want, 2, 2, T))


@pytest.mark.parametrize("wb,xb,signed", [(1, 2, "w"), (2, 2, "none"), (1, 1, "x"), (2, 1, "none"), (1, 2, "none")])
@pytest.mark.parametrize("M,N,K", [(100, 70, 256), (300, 520, 1024), (2300, 2340, 768), (2304, 2464, 1024)])
def test_fp4_path_against_oracle(cuda_device, M, N, K, wb, xb, signed):
    """Operands of at most two bits as e2m1 values on tcgen05.mma kind::mxf4 with unit scale factors
    (apnn_expand_planes_fp4 + apnn_gemm_fp4): one tile, ragged tiles, more 256 x 224 tiles than SM pairs,
    unsigned and -1/+1 operands on either side, int32 and thresholded packed outputs, against the oracle."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(M + N + K + 5 * wb + xb)
    W, wl = oracle.value_planes(rng, M, K, wb)
    X, xl = oracle.value_planes(rng, N, K, xb)
    acc = oracle.gemm_popc(W, X, threads=8)
    if signed == "w":
        want = oracle.signed_correct(acc, oracle.row_sums(X), 1)
    elif signed == "x":
        want = oracle.signed_correct(acc, oracle.row_sums(W), 0)
    else:
        want = acc
    w4 = ap.expand_planes_fp4(to_dev(W), signed=signed == "w")
    x4 = ap.expand_planes_fp4(to_dev(X), signed=signed == "x")
    flag = torch.ones(1, dtype=torch.int32, device="cuda")
    out = ap.gemm_fp4(w4, x4, status_flag=flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    assert np.array_equal(to_host(out, np.int32), want)
    if N % 32 == 0:
        scale = rng.uniform(0.5, 1.5, N).astype(np.float32)
        bias = rng.uniform(-1, 1, N).astype(np.float32)
        T = oracle.fold_bn(scale, bias, float(want.mean()), float(want.std()) / 4, 2)
        res = rng.integers(-300, 300, size=want.shape).astype(np.int32)
        res_out = torch.full((M, N), -1, dtype=torch.int32, device="cuda")
        epi = ap.make_epilogue("thresholds", 2, thresholds=to_dev(T), residual_in=to_dev(res), residual_out=res_out)
        packed = ap.gemm_fp4(w4, x4, epilogue=epi, status_flag=flag)
        torch.cuda.synchronize()
        assert int(flag.item()) == 0
        assert np.array_equal(to_host(res_out, np.int32), want + res)
        assert np.array_equal(to_host(packed), oracle.requant_pack(want + res, 2, 2, T))


@pytest.mark.parametrize("extreme", [False, True])
def test_fp4_path_long_k_sums_stay_exact(cuda_device, extreme):
    """K = 262144: sums reach 3 * K = 786432 (all-ones planes) -- fp32 accumulation of these integers is exact
    below 2^24.  Against a float64 matrix product of the levels (exact at this size)."""
    import apnn_tc_b200 as ap
    M, N, K = 256, 448, 262144
    rng = np.random.default_rng(11 + int(extreme))
    W, wl = oracle.value_planes(rng, M, K, 2)
    X, xl = oracle.value_planes(rng, N, K, 2)
    if extreme:
        W[:] = 0xFFFFFFFF
        X[:] = 0xFFFFFFFF
        wl[:] = 3
        xl[:] = 3
    want = (wl.astype(np.float64) @ xl.astype(np.float64).T).astype(np.int64)
    assert want.max() < 2 ** 24
    flag = torch.ones(1, dtype=torch.int32, device="cuda")
    out = ap.gemm_fp4(ap.expand_planes_fp4(to_dev(W)), ap.expand_planes_fp4(to_dev(X)), status_flag=flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    assert np.array_equal(to_host(out, np.int32).astype(np.int64), want)


@pytest.mark.parametrize("bits,signed", [(1, False), (1, True), (2, False)])
def test_fp4_nibble_image(cuda_device, bits, signed):
    """apnn_expand_planes_fp4 writes what the header says: two e2m1 codes per byte, the element whose bit sits
    at position p of a 32-k plane word in nibble p >> 2 of output word p & 3, levels 0..3 as 0 / 1 / 2 / 3 and
    a signed plane as -1 / +1."""
    import apnn_tc_b200 as ap
    rows, K = 37, 512
    rng = np.random.default_rng(40 + bits + int(signed))
    P, lv = oracle.value_planes(rng, rows, K, bits)
    img = ap.expand_planes_fp4(to_dev(P), signed=signed).cpu().numpy()          # [rows, K/2] bytes
    assert img.shape == (rows, K // 2)
    e2m1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6])
    words = img.reshape(rows, K // 32, 4, 4).astype(np.uint32)                      # [row][group][word q][byte]
    w32 = words[..., 0] | (words[..., 1] << 8) | (words[..., 2] << 16) | (words[..., 3] << 24)
    got = np.zeros((rows, K // 32, 32))
    for q in range(4):
        for i in range(8):
            got[:, :, 4 * i + q] = e2m1[(w32[:, :, q] >> (4 * i)) & 15]             # bit position p = 4*i + q
    # element j of a 32-k group sits in bit 31 - j of the plane word (the packed layout of the reference)
    want = lv.reshape(rows, K // 32, 32)[:, :, ::-1].astype(np.float64)
    if signed:
        want = 2 * want - 1
    assert np.array_equal(got, want)
