"""GPU parity of the implicit-GEMM convolution against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest
import torch

import oracle
from gpu_util import spread_bytes, to_dev, to_host

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_host_loops.npz"))


@pytest.mark.parametrize("wb,xb", [(1, 2), (2, 2), (1, 4)])
def test_reference_inputs(cuda_device, wb, xb):
    """The reference's conv operands (random halo ring included) on 8x8x128 -> 64 against the
    committed outputs of its compute_ref / compute_ref_pack / compute_ref_pack_pool."""
    import apnn_tc_b200 as ap
    X, Wt = oracle.fill_conv(8, 8, 128, 64, xb, wb)
    key = f"conv_w{wb}a{xb}_8x8x128x64"
    acc = to_host(ap.apconv(to_dev(Wt), to_dev(X)), np.int32)
    assert np.array_equal(acc, GOLD[key])
    pk = to_host(ap.apconv(to_dev(Wt), to_dev(X), epilogue=ap.make_epilogue("lowbits", 2)))
    assert np.array_equal(pk, GOLD[key + "_pack"])
    pl = to_host(ap.apconv(to_dev(Wt), to_dev(X), epilogue=ap.make_epilogue("lowbits", 2, pool="avg")))
    assert np.array_equal(pl, GOLD[key + "_pool"])


def test_reference_named_wrappers(cuda_device):
    import apnn_tc_b200 as ap
    X, Wt = oracle.fill_conv(8, 8, 128, 64, 2, 1)
    # reference shapes: X[xb][H+2][W+2][CIN/32], W[wb][COUT][9*CIN/32]
    out = ap.APConv_w1a2_pack(to_dev(Wt.reshape(1, 64, -1)), to_dev(X[:, 0]))
    assert np.array_equal(to_host(out), GOLD["conv_w1a2_8x8x128x64_pack"])
    out = ap.APConv_w1a2_pack_pool(to_dev(Wt.reshape(1, 64, -1)), to_dev(X[:, 0]))
    assert np.array_equal(to_host(out), GOLD["conv_w1a2_8x8x128x64_pool"])


def make_conv(rng, B, H, Wd, CIN, COUT, R, wb, xb):
    p = (R - 1) // 2
    xl = rng.integers(0, 1 << xb, size=(B, H + 2 * p, Wd + 2 * p, CIN), dtype=np.uint32)
    if p:
        xl[:, 0] = xl[:, -1] = 0
        xl[:, :, 0] = xl[:, :, -1] = 0
    wl = rng.integers(0, 1 << wb, size=(COUT, R, R, CIN), dtype=np.uint32)
    return oracle.pack_levels(xl, xb), oracle.pack_levels(wl, wb)


@pytest.mark.parametrize("wb,xb", [(1, 2), (1, 4), (2, 2), (1, 3)])
@pytest.mark.parametrize("C", [128, 256, 384, 512, 640, 768, 896, 1024])
def test_config3_batch8_16x16(cuda_device, wb, xb, C):
    """The convolution sweep as configured: batch 8, 16x16, C = O in 128..1024 step 128, 3x3, stride 1,
    pad 1, BN thresholds (scale U[0.5,1.5], bias U[-1,1]) -> 2-bit packed output, with +-1 weights for
    the 1-bit filters; int32 accumulators and packed outputs, on the warp-level and the tcgen05 path,
    against one oracle evaluation."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(0xA9117C + 3)
    X, Wt = make_conv(rng, 8, 16, 16, C, C, 3, wb, xb)
    acc = oracle.conv_popc(Wt, X, threads=8)
    signed = "w" if wb == 1 else "none"
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, 3), 0) if wb == 1 else acc
    scale = rng.uniform(0.5, 1.5, C).astype(np.float32)
    bias = rng.uniform(-1, 1, C).astype(np.float32)
    T = oracle.fold_bn(scale, bias, float(v.mean()), float(v.std()) / 4, 2)
    want = oracle.requant_pack(v, 2, 2, T)
    epi = ap.make_epilogue("thresholds", 2, signed=signed, thresholds=to_dev(T))
    assert np.array_equal(to_host(ap.apconv(to_dev(Wt), to_dev(X)), np.int32), acc)
    assert np.array_equal(to_host(ap.apconv(to_dev(Wt), to_dev(X), epilogue=epi)), want)
    assert np.array_equal(to_host(run_tc5_conv(Wt, X), np.int32), acc)
    assert np.array_equal(to_host(run_tc5_conv(Wt, X, epi)), want)


@pytest.mark.parametrize("R,stride", [(3, 1), (3, 2), (1, 1), (1, 2)])
@pytest.mark.parametrize("pool", ["none", "avg", "max"])
def test_filters_strides_pools(cuda_device, R, stride, pool):
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(R * 10 + stride)
    B, H, Wd, CIN, COUT = 3, 12, 20, 256, 96
    X, Wt = make_conv(rng, B, H, Wd, CIN, COUT, R, 1, 2)
    acc = oracle.conv_popc(Wt, X, stride=stride, threads=4)
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, R, stride), 0)
    if pool != "none":
        v = oracle.pool2x2(v, 1 if pool == "avg" else 2)
    out = ap.apconv(to_dev(Wt), to_dev(X), stride=stride, epilogue=ap.make_epilogue("int32", signed="w", pool=pool))
    assert np.array_equal(to_host(out, np.int32), v)
    T = oracle.fold_bn(np.ones(COUT, np.float32), np.zeros(COUT, np.float32), float(v.mean()), float(v.std()) / 4, 2)
    out = ap.apconv(to_dev(Wt), to_dev(X), stride=stride,
                    epilogue=ap.make_epilogue("thresholds", 2, signed="w", pool=pool, thresholds=to_dev(T)))
    assert np.array_equal(to_host(out), oracle.requant_pack(v, 2, 2, T))


def test_output_halo_chains_into_next_conv(cuda_device):
    """A conv that writes its packed output inside a zero ring feeds the next conv directly."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(41)
    B, H, Wd, C = 2, 8, 8, 128
    X, W1 = make_conv(rng, B, H, Wd, C, C, 3, 1, 2)
    _, W2 = make_conv(rng, B, H, Wd, C, 64, 3, 1, 2)
    acc1 = oracle.conv_popc(W1, X)
    l1 = oracle.levels(acc1, 2, 1)
    mid = ap.apconv(to_dev(W1), to_dev(X), epilogue=ap.make_epilogue("lowbits", 2, out_halo=1))
    assert mid.shape == (2, B, H + 2, Wd + 2, C // 32)
    padded = np.zeros((B, H + 2, Wd + 2, C), dtype=np.uint32)
    padded[:, 1:-1, 1:-1] = l1
    assert np.array_equal(to_host(mid), oracle.pack_levels(padded, 2))
    acc2 = to_host(ap.apconv(to_dev(W2), mid), np.int32)
    assert np.array_equal(acc2, oracle.conv_popc(W2, oracle.pack_levels(padded, 2)))


def test_conv_host_front_end(cuda_device):
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(43)
    X, Wt = make_conv(rng, 2, 8, 8, 128, 64, 3, 1, 2)
    out = np.zeros((2, 2, 8, 8, 2), dtype=np.uint32)
    h = ap.HostHandle(0)
    h.conv2d(Wt, X, out, 1, 2, 2, 8, 8, 128, 64, epilogue=ap.make_epilogue("lowbits", 2))
    h.close()
    assert np.array_equal(out, oracle.requant_pack(oracle.conv_popc(Wt, X), 2, 1))


# ------------------------------------------------------------------ tcgen05 implicit-GEMM path
def run_tc5_conv(Wt, X, epilogue=None, stride=1):
    import apnn_tc_b200 as ap
    xb, B, Hp, Wp, cw = X.shape
    wb, COUT, R = Wt.shape[0], Wt.shape[1], Wt.shape[2]
    p = (R - 1) // 2
    H, Wd, CIN = Hp - 2 * p, Wp - 2 * p, cw * 32
    ws = torch.empty(ap.conv_workspace_bytes(B, H, Wd, CIN, COUT, R), dtype=torch.uint8, device="cuda")
    out = ap.apconv(to_dev(Wt), to_dev(X), stride=stride, epilogue=epilogue, algo="tcgen05", workspace=ws)
    ap.conv_check(ws, B, H, Wd, CIN, COUT, R)  # synchronises; raises if a bounded wait expired
    return out


@pytest.mark.parametrize("wb,xb", [(1, 2), (2, 2), (1, 4)])
def test_tcgen05_reference_inputs(cuda_device, wb, xb):
    import apnn_tc_b200 as ap
    X, Wt = oracle.fill_conv(8, 8, 128, 64, xb, wb)
    key = f"conv_w{wb}a{xb}_8x8x128x64"
    assert np.array_equal(to_host(run_tc5_conv(Wt, X), np.int32), GOLD[key])
    assert np.array_equal(to_host(run_tc5_conv(Wt, X, ap.make_epilogue("lowbits", 2))), GOLD[key + "_pack"])
    assert np.array_equal(to_host(run_tc5_conv(Wt, X, ap.make_epilogue("lowbits", 2, pool="avg"))), GOLD[key + "_pool"])


@pytest.mark.parametrize("B,H,Wd", [(3, 12, 20), (5, 8, 8), (2, 56, 56), (1, 4, 4), (2, 6, 130)])
@pytest.mark.parametrize("R", [3, 1])
@pytest.mark.parametrize("pool", ["none", "avg", "max"])
def test_tcgen05_shapes_filters_pools(cuda_device, B, H, Wd, R, pool):
    """Boxes that do not divide the image, images smaller than a tile, ragged batch."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(B * 100 + H + R)
    CIN, COUT = 128, 96
    X, Wt = make_conv(rng, B, H, Wd, CIN, COUT, R, 1, 2)
    acc = oracle.conv_popc(Wt, X, threads=4)
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, R, 1), 0)
    if pool != "none":
        v = oracle.pool2x2(v, 1 if pool == "avg" else 2)
    out = run_tc5_conv(Wt, X, ap.make_epilogue("int32", signed="w", pool=pool))
    assert np.array_equal(to_host(out, np.int32), v)
    T = oracle.fold_bn(np.ones(COUT, np.float32), np.zeros(COUT, np.float32), float(v.mean()), float(v.std()) / 4, 2)
    out = run_tc5_conv(Wt, X, ap.make_epilogue("thresholds", 2, signed="w", pool=pool, out_halo=1, thresholds=to_dev(T)))
    want = oracle.requant_pack(v, 2, 2, T)
    got = to_host(out)
    assert got.shape[2] == want.shape[2] + 2 and got.shape[3] == want.shape[3] + 2
    assert np.array_equal(got[:, :, 1:-1, 1:-1], want)
    assert not got[:, :, 0].any() and not got[:, :, -1].any() and not got[:, :, :, 0].any() and not got[:, :, :, -1].any()


def test_tcgen05_many_tiles_and_auto(cuda_device):
    """More tiles than SMs (both TMEM accumulators, several tiles per CTA) and the AUTO choice."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(57)
    B, H, Wd, CIN, COUT = 16, 32, 32, 256, 512
    X, Wt = make_conv(rng, B, H, Wd, CIN, COUT, 3, 2, 2)
    want = oracle.conv_popc(Wt, X, threads=8)
    assert np.array_equal(to_host(run_tc5_conv(Wt, X), np.int32), want)
    ws = torch.empty(ap.conv_workspace_bytes(B, H, Wd, CIN, COUT, 3), dtype=torch.uint8, device="cuda")
    out = ap.apconv(to_dev(Wt), to_dev(X), algo="auto", workspace=ws)
    assert np.array_equal(to_host(out, np.int32), want)


# ------------------------------------------------------------------ wider filters, residuals
@pytest.mark.parametrize("R,stride", [(5, 1), (7, 2), (7, 4), (11, 4), (5, 3)])
def test_wide_filters_and_strides(cuda_device, R, stride):
    """First-layer shapes of the model lists (11x11 s4, 7x7 s4, 5x5) on the warp-level kernel."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(R * 7 + stride)
    X, Wt = make_conv(rng, 2, 24, 20, 128, 64, R, 1, 2)
    acc = oracle.conv_popc(Wt, X, stride=stride, threads=4)
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, R, stride), 0)
    out = ap.apconv(to_dev(Wt), to_dev(X), stride=stride, epilogue=ap.make_epilogue("int32", signed="w"))
    assert np.array_equal(to_host(out, np.int32), v)
    if stride in (1, 2):
        got = run_tc5_conv(Wt, X, ap.make_epilogue("int32", signed="w"), stride=stride)
        assert np.array_equal(to_host(got, np.int32), v)


@pytest.mark.parametrize("algo", ["imma", "tcgen05"])
@pytest.mark.parametrize("pool", ["none", "max"])
def test_residual_in_and_out(cuda_device, algo, pool):
    """value = conv + residual_in; residual_out receives it; the requantised output uses it."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(71)
    B, H, Wd, CIN, COUT = 3, 12, 8, 128, 160
    X, Wt = make_conv(rng, B, H, Wd, CIN, COUT, 3, 1, 2)
    acc = oracle.conv_popc(Wt, X, threads=4)
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, 3), 0)
    if pool != "none":
        v = oracle.pool2x2(v, 2)
    res = rng.integers(-500, 500, size=v.shape).astype(np.int32)
    v = v + res
    T = oracle.fold_bn(np.ones(COUT, np.float32), np.zeros(COUT, np.float32), float(v.mean()), float(v.std()) / 4, 2)
    res_out = torch.zeros(v.shape, dtype=torch.int32, device="cuda")
    epi = ap.make_epilogue("thresholds", 2, signed="w", pool=pool, out_halo=1, thresholds=to_dev(T),
                           residual_in=to_dev(res), residual_out=res_out)
    if algo == "tcgen05":
        out = run_tc5_conv(Wt, X, epi)
    else:
        out = ap.apconv(to_dev(Wt), to_dev(X), epilogue=epi)
    assert np.array_equal(to_host(res_out, np.int32), v)
    assert np.array_equal(to_host(out)[:, :, 1:-1, 1:-1], oracle.requant_pack(v, 2, 2, T))


@pytest.mark.parametrize("B,H,Wd", [(2, 16, 16), (3, 14, 10), (1, 56, 56), (5, 7, 7)])
@pytest.mark.parametrize("R", [3, 1])
@pytest.mark.parametrize("pool", ["none", "max"])
def test_tcgen05_stride2(cuda_device, B, H, Wd, R, pool):
    """Stride-2 convolution on the tcgen05 path (TMA boxes that pick every second pixel)."""
    import apnn_tc_b200 as ap
    Ho, Wo = (H - 1) // 2 + 1, (Wd - 1) // 2 + 1
    if pool != "none" and (Ho % 2 or Wo % 2):
        pytest.skip("pooling needs even output")
    rng = np.random.default_rng(B * 31 + H + R)
    X, Wt = make_conv(rng, B, H, Wd, 256, 64, R, 1, 2)
    acc = oracle.conv_popc(Wt, X, stride=2, threads=4)
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, R, 2), 0)
    if pool != "none":
        v = oracle.pool2x2(v, 2)
    out = run_tc5_conv(Wt, X, ap.make_epilogue("int32", signed="w", pool=pool), stride=2)
    assert np.array_equal(to_host(out, np.int32), v)


# ------------------------------------------------------------------ 64-channel maps, resident filter
@pytest.mark.parametrize("CIN,COUT", [(64, 64), (64, 128), (192, 64), (128, 64)])
@pytest.mark.parametrize("R,stride,pool", [(3, 1, "none"), (3, 1, "max"), (1, 1, "none"), (3, 2, "none")])
def test_tcgen05_64_channel_maps(cuda_device, CIN, COUT, R, stride, pool):
    """Feature maps whose channel count is a multiple of 64 only (64-byte swizzle rows) and
    64-column tiles, with thresholds, residual in / out and an output ring."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(CIN + COUT + R + stride)
    B, H, Wd = 3, 12, 16
    X, Wt = make_conv(rng, B, H, Wd, CIN, COUT, R, 1, 2)
    acc = oracle.conv_popc(Wt, X, stride=stride, threads=4)
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, R, stride), 0)
    if pool != "none":
        v = oracle.pool2x2(v, 2)
    out = run_tc5_conv(Wt, X, ap.make_epilogue("int32", signed="w", pool=pool), stride=stride)
    assert np.array_equal(to_host(out, np.int32), v)
    res = rng.integers(-300, 300, size=v.shape).astype(np.int32)
    v2 = v + res
    T = oracle.fold_bn(np.ones(COUT, np.float32), np.zeros(COUT, np.float32), float(v2.mean()), float(v2.std()) / 4, 2)
    res_out = torch.zeros(v2.shape, dtype=torch.int32, device="cuda")
    epi = ap.make_epilogue("thresholds", 2, signed="w", pool=pool, out_halo=1, thresholds=to_dev(T),
                           residual_in=to_dev(res), residual_out=res_out)
    got = to_host(run_tc5_conv(Wt, X, epi, stride=stride))
    assert np.array_equal(to_host(res_out, np.int32), v2)
    assert np.array_equal(got[:, :, 1:-1, 1:-1], oracle.requant_pack(v2, 2, 2, T))


@pytest.mark.parametrize("CIN,COUT,R", [(64, 64, 3), (128, 128, 3), (128, 128, 1), (256, 64, 1)])
def test_tcgen05_resident_filter(cuda_device, CIN, COUT, R):
    """Enough row tiles per SM that the kernel keeps the whole filter in shared memory and
    streams activation tiles only (one tile column, >= 4 tiles per SM)."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(CIN * 3 + COUT + R)
    B, H, Wd = 25, 56, 56       # 28 pixel boxes per image: 700 row tiles, more than 4 per SM
    X, Wt = make_conv(rng, B, H, Wd, CIN, COUT, R, 1, 2)
    acc = oracle.conv_popc(Wt, X, threads=8)
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, R, 1), 0)
    T = oracle.fold_bn(np.ones(COUT, np.float32), np.zeros(COUT, np.float32), float(v.mean()), float(v.std()) / 4, 2)
    out = run_tc5_conv(Wt, X, ap.make_epilogue("thresholds", 2, signed="w", thresholds=to_dev(T)))
    assert np.array_equal(to_host(out), oracle.requant_pack(v, 2, 2, T))


@pytest.mark.parametrize("CIN,COUT,pool", [(64, 64, "none"), (128, 192, "max"), (256, 128, "none")])
def test_tcgen05_int8_row_output_chains(cuda_device, CIN, COUT, pool):
    """out_i8: the quantised output leaves the epilogue as one byte per element inside its ring,
    and is the next convolution's operand as it stands (no packed planes, no expand pass)."""
    import ctypes
    import apnn_tc_b200 as ap
    from apnn_tc_b200 import _cabi
    rng = np.random.default_rng(CIN + COUT)
    B, H, Wd = 3, 12, 16
    X, Wt = make_conv(rng, B, H, Wd, CIN, COUT, 3, 1, 2)
    acc = oracle.conv_popc(Wt, X, threads=4)
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, 3), 0)
    if pool != "none":
        v = oracle.pool2x2(v, 2)
    T = oracle.fold_bn(np.ones(COUT, np.float32), np.zeros(COUT, np.float32), float(v.mean()), float(v.std()) / 4, 2)
    lv = oracle.levels(v, 2, 2, T)                                  # [B, Ho, Wo, COUT]
    Ho, Wo = lv.shape[1], lv.shape[2]
    x8 = ap.expand_planes(to_dev(X).reshape(2, -1, CIN // 32))
    w8 = ap.expand_planes(to_dev(Wt).reshape(1, COUT, -1), signed=True)
    out = torch.zeros((B, Ho + 2, Wo + 2, COUT), dtype=torch.uint8, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    epi = ap.make_epilogue("thresholds", 2, pool=pool, out_halo=1, thresholds=to_dev(T), out_i8=True)
    s = torch.cuda.current_stream().cuda_stream
    _cabi.check(_cabi.lib().apnn_conv2d_i8(s, w8.data_ptr(), x8.data_ptr(), out.data_ptr(), B, H, Wd, CIN, COUT, 3, 1, 1,
                                           ctypes.byref(epi), flag.data_ptr()), "conv")
    got = out.cpu().numpy()
    assert int(flag.item()) == 0
    assert np.array_equal(got[:, 1:-1, 1:-1], spread_bytes(lv.astype(np.uint8)))
    assert not got[:, 0].any() and not got[:, -1].any() and not got[:, :, 0].any() and not got[:, :, -1].any()
    # second convolution straight from those bytes
    rng2 = np.random.default_rng(5)
    wl2 = rng2.integers(0, 2, size=(64, 3, 3, COUT), dtype=np.uint32)
    W2 = oracle.pack_levels(wl2, 1)
    w8b = ap.expand_planes(to_dev(W2).reshape(1, 64, -1), signed=True)
    out2 = torch.zeros((B, Ho, Wo, 64), dtype=torch.int32, device="cuda")
    epi2 = ap.make_epilogue("int32")
    _cabi.check(_cabi.lib().apnn_conv2d_i8(s, w8b.data_ptr(), out.data_ptr(), out2.data_ptr(), B, Ho, Wo, COUT, 64, 3, 1, 1,
                                           ctypes.byref(epi2), flag.data_ptr()), "conv2")
    xp = np.zeros((B, Ho + 2, Wo + 2, COUT), dtype=np.uint32)
    xp[:, 1:-1, 1:-1] = lv
    X2 = oracle.pack_levels(xp, 2)
    want2 = oracle.signed_correct(oracle.conv_popc(W2, X2, threads=4), oracle.conv_window_sums(X2, 3), 0)
    assert np.array_equal(out2.cpu().numpy(), want2)


@pytest.mark.parametrize("B,H,Wd,CIN,COUT,R,ring,bits", [(300, 14, 14, 128, 256, 3, 1, 2), (90, 28, 28, 128, 256, 3, 1, 2),
                                                         (400, 14, 14, 256, 256, 1, 0, 2), (40, 28, 28, 128, 512, 3, 2, 1),
                                                         (301, 13, 15, 256, 256, 3, 1, 2)])
def test_tcgen05_pair_flat_conv(cuda_device, B, H, Wd, CIN, COUT, R, ring, bits):
    """Wide layers (CIN % 128 == 0, COUT % 256 == 0, thresholds -> int8 rows, at least one tile per SM pair)
    run the flat convolution on CTA pairs: same bytes as the oracle's levels, ring left untouched."""
    import ctypes
    import apnn_tc_b200 as ap
    from apnn_tc_b200 import _cabi
    rng = np.random.default_rng(B + H + CIN + COUT + R)
    pad = (R - 1) // 2
    X, Wt = make_conv(rng, B, H, Wd, CIN, COUT, R, 1, 2)           # X carries a ring of pad pixels
    acc = oracle.conv_popc(Wt, X, threads=8)
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, R), 0)
    scale = rng.uniform(0.5, 1.5, COUT).astype(np.float32)
    bias = rng.uniform(-1, 1, COUT).astype(np.float32)
    T = oracle.fold_bn(scale, bias, float(v.mean()), float(v.std()) / 4, bits)
    lv = oracle.levels(v, bits, 2, T)                               # [B, H, Wd, COUT]
    x8 = ap.expand_planes(to_dev(X).reshape(2, -1, CIN // 32)).reshape(B, H + 2 * pad, Wd + 2 * pad, CIN)
    if ring > pad:   # a wider stored ring than the filter needs
        wide = torch.zeros((B, H + 2 * ring, Wd + 2 * ring, CIN), dtype=torch.uint8, device="cuda")
        wide[:, ring - pad:ring - pad + H + 2 * pad, ring - pad:ring - pad + Wd + 2 * pad] = x8
        x8 = wide
    in_halo = max(ring, pad)
    w8 = ap.expand_planes(to_dev(Wt).reshape(1, COUT, -1), signed=True)
    out = torch.full((B, H + 2, Wd + 2, COUT), 0x77, dtype=torch.uint8, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    epi = ap.make_epilogue("thresholds", bits, out_halo=1, thresholds=to_dev(T), out_i8=True)
    epi.in_halo = in_halo
    s = torch.cuda.current_stream().cuda_stream
    _cabi.check(_cabi.lib().apnn_conv2d_i8(s, w8.data_ptr(), x8.data_ptr(), out.data_ptr(), B, H, Wd, CIN, COUT, R, 1, 1,
                                           ctypes.byref(epi), flag.data_ptr()), "conv")
    got = out.cpu().numpy()
    assert int(flag.item()) == 0
    assert np.array_equal(got[:, 1:-1, 1:-1], spread_bytes(lv.astype(np.uint8)))
    assert (got[:, 0] == 0x77).all() and (got[:, -1] == 0x77).all() and (got[:, :, 0] == 0x77).all() and (got[:, :, -1] == 0x77).all()


@pytest.mark.parametrize("widths", [1, 2, 3])
@pytest.mark.parametrize("CIN,COUT", [(64, 64), (128, 160)])
def test_tcgen05_int16_residuals(cuda_device, widths, CIN, COUT):
    """residual_i16: bit 0 = residual_in is int16, bit 1 = residual_out is int16; same values as int32."""
    import ctypes
    import apnn_tc_b200 as ap
    from apnn_tc_b200 import _cabi
    rng = np.random.default_rng(widths + CIN)
    B, H, Wd = 3, 12, 16
    X, Wt = make_conv(rng, B, H, Wd, CIN, COUT, 3, 1, 2)
    v = oracle.signed_correct(oracle.conv_popc(Wt, X, threads=4), oracle.conv_window_sums(X, 3), 0)
    res = rng.integers(-3000, 3000, size=v.shape).astype(np.int32)
    v = v + res
    T = oracle.fold_bn(np.ones(COUT, np.float32), np.zeros(COUT, np.float32), float(v.mean()), float(v.std()) / 4, 2)
    x8 = ap.expand_planes(to_dev(X).reshape(2, -1, CIN // 32))
    w8 = ap.expand_planes(to_dev(Wt).reshape(1, COUT, -1), signed=True)
    rin = torch.from_numpy(res.astype(np.int16) if widths & 1 else res).cuda()
    rout = torch.zeros(v.shape, dtype=torch.int16 if widths & 2 else torch.int32, device="cuda")
    out = torch.zeros((2, B, H + 2, Wd + 2, COUT // 32), dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    epi = ap.make_epilogue("thresholds", 2, out_halo=1, thresholds=to_dev(T), residual_in=rin, residual_out=rout,
                           residual_i16=widths)
    _cabi.check(_cabi.lib().apnn_conv2d_i8(torch.cuda.current_stream().cuda_stream, w8.data_ptr(), x8.data_ptr(),
                                           out.data_ptr(), B, H, Wd, CIN, COUT, 3, 1, 1, ctypes.byref(epi), flag.data_ptr()),
                "conv")
    assert int(flag.item()) == 0
    assert np.array_equal(rout.cpu().numpy().astype(np.int32), v)
    assert np.array_equal(to_host(out)[:, :, 1:-1, 1:-1], oracle.requant_pack(v, 2, 2, T))


@pytest.mark.parametrize("wb,xb", [(4, 4), (2, 8)])
def test_tcgen05_wider_pairs_conv(cuda_device, wb, xb):
    rng = np.random.default_rng(wb + xb)
    X, Wt = make_conv(rng, 2, 10, 12, 128, 64, 3, wb, xb)
    assert np.array_equal(to_host(run_tc5_conv(Wt, X), np.int32), oracle.conv_popc(Wt, X, threads=4))


@pytest.mark.parametrize("R,ring", [(1, 1), (3, 2), (1, 3)])
def test_tcgen05_flat_conv_with_wider_input_ring(cuda_device, R, ring):
    """The stored ring of the input may be wider than the filter needs (a 1x1 convolution reading a map
    whose other consumer is a 3x3 one): in_halo tells the kernel, which offsets its reads."""
    import ctypes
    import apnn_tc_b200 as ap
    from apnn_tc_b200 import _cabi
    rng = np.random.default_rng(R * 10 + ring)
    B, H, Wd, CIN, COUT = 3, 10, 14, 128, 96
    pad = (R - 1) // 2
    xl = np.zeros((B, H + 2 * ring, Wd + 2 * ring, CIN), dtype=np.uint32)
    xl[:, ring:ring + H, ring:ring + Wd] = rng.integers(0, 4, size=(B, H, Wd, CIN), dtype=np.uint32)
    wl = rng.integers(0, 2, size=(COUT, R, R, CIN), dtype=np.uint32)
    # oracle on the exactly-padded image
    xe = xl[:, ring - pad:ring + H + pad, ring - pad:ring + Wd + pad]
    X, Wt = oracle.pack_levels(np.ascontiguousarray(xe), 2), oracle.pack_levels(wl, 1)
    want = oracle.signed_correct(oracle.conv_popc(Wt, X, threads=4), oracle.conv_window_sums(X, R), 0)
    x8 = ap.expand_planes(to_dev(oracle.pack_levels(xl, 2)).reshape(2, -1, CIN // 32))
    w8 = ap.expand_planes(to_dev(Wt).reshape(1, COUT, -1), signed=True)
    out = torch.zeros((B, H, Wd, COUT), dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    epi = ap.make_epilogue("int32", in_halo=ring)
    _cabi.check(_cabi.lib().apnn_conv2d_i8(torch.cuda.current_stream().cuda_stream, w8.data_ptr(), x8.data_ptr(),
                                           out.data_ptr(), B, H, Wd, CIN, COUT, R, 1, 1, ctypes.byref(epi), flag.data_ptr()),
                "conv")
    assert int(flag.item()) == 0
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("R,B,H,Wd,COUT", [(5, 2, 10, 40, 160), (5, 2, 12, 20, 320), (7, 2, 9, 30, 160), (7, 2, 8, 16, 288),
                                           (9, 2, 12, 12, 160), (9, 2, 10, 34, 288), (11, 2, 12, 14, 160),
                                           (11, 2, 11, 40, 192), (7, 8, 24, 40, 512), (9, 8, 24, 40, 512)])
def test_tcgen05_wide_filters_stride1(cuda_device, R, B, H, Wd, COUT):
    """Stride-1 convolutions with 5x5 ... 11x11 filters on the tcgen05 path: one input box per
    (tile, channel block) while it has at most 256 rows, one box per filter row beyond that, and the
    pixel-box formulation where neither fits in shared memory (11x11; 9x9 with 256-column tiles)."""
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(R * 100 + Wd)
    X, Wt = make_conv(rng, B, H, Wd, 128, COUT, R, 1, 2)
    acc = oracle.conv_popc(Wt, X, threads=8)
    v = oracle.signed_correct(acc, oracle.conv_window_sums(X, R), 0)
    got = run_tc5_conv(Wt, X, ap.make_epilogue("int32", signed="w"))
    assert np.array_equal(to_host(got, np.int32), v)
    T = oracle.fold_bn(np.ones(COUT, np.float32), np.zeros(COUT, np.float32), float(v.mean()), float(v.std()) / 4, 2)
    got = run_tc5_conv(Wt, X, ap.make_epilogue("thresholds", 2, signed="w", thresholds=to_dev(T)))
    assert np.array_equal(to_host(got), oracle.requant_pack(v, 2, 2, T))


def test_tcgen05_pair_split_plans_forced():
    """Split-K over clusters of CTA pairs (two pairs = four CTAs sharing a pair of tile rows) is not a plan the
    library picks on its own (it measured slower than the single-CTA split); APNN_PAIR_SPLIT=1 forces it, read
    once per process, so the check runs in a child process: the batch-8 16x16 convolution of 512 channels and a
    skinny GEMM against the oracle."""
    import subprocess
    import sys
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    code = r'''
import sys, os, ctypes
import numpy as np, torch
sys.path.insert(0, os.getcwd()); sys.path.insert(0, os.path.join(os.getcwd(), "tests"))
import oracle, apnn_tc_b200 as ap
from apnn_tc_b200 import _cabi
from test_conv_gpu import make_conv, run_tc5_conv
from gpu_util import to_dev, to_host, spread_bytes
rng = np.random.default_rng(7)
X, Wt = make_conv(rng, 8, 16, 16, 512, 512, 3, 1, 2)
acc = oracle.conv_popc(Wt, X, threads=8)
v = oracle.signed_correct(acc, oracle.conv_window_sums(X, 3), 0)
T = oracle.fold_bn(np.ones(512, np.float32), np.zeros(512, np.float32), float(v.mean()), float(v.std()) / 4, 2)
got = run_tc5_conv(Wt, X, ap.make_epilogue("thresholds", 2, signed="w", thresholds=to_dev(T)))
assert np.array_equal(to_host(got), oracle.requant_pack(v, 2, 2, T)), "conv"
M, N, K = 256, 512, 8192
W, wl = oracle.value_planes(rng, M, K, 2); Xg, xl = oracle.value_planes(rng, N, K, 1)
want = (wl.astype(np.int64) @ (2 * xl.astype(np.int64) - 1).T).astype(np.int32)
a8 = ap.expand_planes(to_dev(W)); b8 = ap.expand_planes(to_dev(Xg), signed=True)
D = torch.zeros((M, N), dtype=torch.int32, device="cuda"); flag = torch.zeros(1, dtype=torch.int32, device="cuda")
epi = ap.make_epilogue("int32")
_cabi.check(_cabi.lib().apnn_gemm_i8(torch.cuda.current_stream().cuda_stream, a8.data_ptr(), b8.data_ptr(), D.data_ptr(), M, N, K, 0, 1, ctypes.byref(epi), flag.data_ptr()), "gemm")
torch.cuda.synchronize()
assert int(flag.item()) == 0 and np.array_equal(D.cpu().numpy(), want), "gemm"
print("pair split ok")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=dict(os.environ, APNN_PAIR_SPLIT="1"), capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0 and "pair split ok" in r.stdout, r.stdout + r.stderr
