"""CPU tests of the oracle: pinned against the golden vectors generated from the reference's
own host functions (tests/golden/make_golden.py) and, where oracle/_ref is built, against
those functions directly."""
import ctypes
import hashlib
import os

import numpy as np
import pytest

import oracle
from oracle import ref

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_host_loops.npz"))


def sha(*arrs):
    h = hashlib.sha256()
    for a in arrs:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest(), dtype=np.uint8)


def test_rand_stream_matches_glibc():
    w = oracle.rand_words(2000)
    assert w[0] == 0x6B8B4567  # first word of the reference's operands
    libc = ctypes.CDLL(None)
    libc.srand(1)
    assert [libc.rand() for _ in range(2000)] == [int(x) for x in w]
    assert (w >> 31).max() == 0  # rand() is 31-bit: bit 31 of every operand word is 0


@pytest.mark.parametrize("wb,xb", [(1, 2), (2, 2), (1, 4), (1, 3)])
@pytest.mark.parametrize("n", [128, 256])
def test_gemm_against_golden(wb, xb, n):
    W, X = oracle.fill_gemm(64, n, n, wb, xb)
    key = f"gemm_w{wb}a{xb}_64x{n}x{n}"
    assert np.array_equal(sha(W, X), GOLD[key + "_insha"])
    D = oracle.gemm_bitserial(W, X)
    assert np.array_equal(D, GOLD[key])
    assert np.array_equal(oracle.gemm_popc(W, X, threads=2), D)


def test_w1a4_all_ones_known_answer():
    # program 78 ships with all-ones operands: every output is (1+2+4+8) * K
    W = np.full((1, 64, 4), 0xFFFFFFFF, dtype=np.uint32)
    X = np.full((4, 128, 4), 0xFFFFFFFF, dtype=np.uint32)
    D = oracle.gemm_bitserial(W, X)
    assert np.array_equal(D, GOLD["gemm_w1a4_allones_64x128x128"]) and (D == 15 * 128).all()


def test_gemm_config1_checksum():
    # w1a2, M=64, N=K=1024 on the reference's default-seed inputs
    W, X = oracle.fill_gemm(64, 1024, 1024, 1, 2)
    D = oracle.gemm_popc(W, X, threads=4)
    assert int(D.astype(np.int64).sum()) == int(GOLD["gemm_w1a2_64x1024x1024_sum"][0]) == 49072252
    assert int(D[0, 0]) == int(GOLD["gemm_w1a2_64x1024x1024_sum"][1]) == 722
    assert np.array_equal(sha(D), GOLD["gemm_w1a2_64x1024x1024_sha"])
    # bit-serial loop on a row sample equals the popcount form
    assert np.array_equal(oracle.gemm_bitserial(W, X, rows=(8, 12))[8:12], D[8:12])


@pytest.mark.parametrize("wb,xb", [(1, 2), (2, 2)])
def test_gemm_pack_against_golden(wb, xb):
    W, X = oracle.fill_gemm(64, 128, 128, wb, xb)
    assert np.array_equal(oracle.gemm_pack(W, X, 2), GOLD[f"gemm_pack_w{wb}a{xb}_64x128x128"])
    # composed form: accumulators -> low bits -> pack
    D = oracle.gemm_popc(W, X)
    assert np.array_equal(oracle.requant_pack(D, 2, 1), GOLD[f"gemm_pack_w{wb}a{xb}_64x128x128"])


@pytest.mark.parametrize("wb,xb", [(1, 2), (2, 2), (1, 4)])
def test_conv_against_golden(wb, xb):
    X, Wt = oracle.fill_conv(8, 8, 128, 64, xb, wb)
    key = f"conv_w{wb}a{xb}_8x8x128x64"
    assert np.array_equal(sha(X, Wt), GOLD[key + "_insha"])
    acc = oracle.conv_bitserial(Wt, X)
    assert np.array_equal(acc, GOLD[key])
    assert np.array_equal(oracle.conv_popc(Wt, X, threads=2), acc)
    assert np.array_equal(oracle.conv_pack(Wt, X, 2), GOLD[key + "_pack"])
    assert np.array_equal(oracle.conv_pack(Wt, X, 2, pool=True), GOLD[key + "_pool"])
    # composed: pool (truncating average) then low bits then pack
    pooled = oracle.pool2x2(acc, 1)
    assert np.array_equal(oracle.requant_pack(pooled, 2, 1), GOLD[key + "_pool"])


@pytest.mark.skipif(not ref.available(71), reason="oracle/_ref not built (needs the reference checkout)")
def test_against_compiled_reference():
    Wr, Xr = ref.gemm_init(72, 64, 384, 256, 2, 2)
    W, X = oracle.fill_gemm(64, 384, 256, 2, 2)
    assert np.array_equal(W, Wr) and np.array_equal(X, Xr)
    assert np.array_equal(oracle.gemm_bitserial(W, X), ref.gemm_ref(72, W, X))
    Xc, Wc = oracle.fill_conv(4, 8, 256, 32, 2, 1)
    assert np.array_equal(oracle.conv_bitserial(Wc, Xc), ref.conv_ref(67, Wc, Xc))
    assert np.array_equal(oracle.conv_pack(Wc, Xc, 2, pool=True), ref.conv_pack(68, Wc, Xc, 2, pool=True))


def test_value_level_semantics():
    """acc equals the integer dot product of the levels the planes encode."""
    rng = np.random.default_rng(7)
    Wp, wl = oracle.value_planes(rng, 16, 256, 2)
    Xp, xl = oracle.value_planes(rng, 24, 256, 3)
    D = oracle.gemm_bitserial(Wp, Xp)
    assert np.array_equal(D, wl.astype(np.int64) @ xl.astype(np.int64).T)
    assert np.array_equal(oracle.unpack_levels(Wp), wl)
    # +-1 reading of a 1-bit operand: sum (2w-1) x = 2 acc - S_x
    W1, w1 = oracle.value_planes(rng, 16, 256, 1)
    acc = oracle.gemm_popc(W1, Xp)
    v = oracle.signed_correct(acc, oracle.row_sums(Xp), 1)
    assert np.array_equal(v, (2 * w1.astype(np.int64) - 1) @ xl.astype(np.int64).T)


def test_conv_extensions_match_dense_definition():
    """Batch, stride 2 and 1x1 filters against a plain numpy correlation of the levels."""
    rng = np.random.default_rng(11)
    for R, stride in ((3, 1), (3, 2), (1, 1), (1, 2)):
        B, H, Wd, CIN, COUT, p = 2, 6, 4, 128, 32, (R - 1) // 2
        xl = rng.integers(0, 4, size=(B, H + 2 * p, Wd + 2 * p, CIN), dtype=np.uint32)
        if p:
            xl[:, 0] = xl[:, -1] = 0
            xl[:, :, 0] = xl[:, :, -1] = 0
        wl = rng.integers(0, 2, size=(COUT, R, R, CIN), dtype=np.uint32)
        X, Wt = oracle.pack_levels(xl, 2), oracle.pack_levels(wl, 1)
        got = oracle.conv_bitserial(Wt, X, stride=stride)
        Ho, Wo = (H - 1) // stride + 1, (Wd - 1) // stride + 1
        want = np.zeros((B, Ho, Wo, COUT), dtype=np.int64)
        for ho in range(Ho):
            for wo in range(Wo):
                win = xl[:, ho * stride:ho * stride + R, wo * stride:wo * stride + R, :].astype(np.int64)
                want[:, ho, wo, :] = np.einsum("bijc,oijc->bo", win, wl.astype(np.int64))
        assert np.array_equal(got, want)
        assert np.array_equal(oracle.conv_popc(Wt, X, stride=stride, threads=2), got)
        S = oracle.conv_window_sums(X, R, stride)
        assert np.array_equal(S, np.stack([[[xl[b, ho * stride:ho * stride + R, wo * stride:wo * stride + R].sum()
                                             for wo in range(Wo)] for ho in range(Ho)] for b in range(B)]))


def test_threshold_requant_and_fold_bn():
    rng = np.random.default_rng(3)
    C = 64
    scale = rng.uniform(0.5, 1.5, C).astype(np.float32)
    bias = rng.uniform(-1, 1, C).astype(np.float32)
    mu, sigma = 500.0, 40.0
    T = oracle.fold_bn(scale, bias, mu, sigma, 2)
    assert T.shape == (C, 3) and (np.diff(T, axis=1) >= 0).all()
    V = rng.integers(200, 800, size=(10, C)).astype(np.int32)
    L = oracle.levels(V, 2, 2, T)
    # same thing through the float definition, away from the decision edges
    y = scale * (V - mu) / sigma + bias
    q = np.clip(y, -10, 10)
    lv = np.minimum(np.rint((q + 10) * 4 / 20), 3)
    edge = np.abs(((q + 10) * 4 / 20) % 1 - 0.5) < 1e-3
    assert np.array_equal(L[~edge], lv[~edge].astype(np.int32))
    packed = oracle.requant_pack(V, 2, 2, T)
    assert np.array_equal(oracle.unpack_levels(packed).astype(np.int32), L)


def test_packers():
    rng = np.random.default_rng(5)
    x = rng.uniform(-12, 12, size=(9, 3)).astype(np.float32)
    lv = oracle.quantize(x, 2)
    assert lv.max() <= 3 and lv.min() >= 0
    planes = oracle.bit_compress(lv, 2)
    assert planes.shape == (2, 9, 4)
    back = oracle.unpack_levels(planes)
    assert np.array_equal(back[:, :3], lv) and not back[:, 3:].any()
    lv2 = rng.integers(0, 16, size=(5, 160), dtype=np.uint32)
    assert np.array_equal(oracle.unpack_levels(oracle.bit_compress(lv2, 4))[:, :160], lv2)
    assert np.array_equal(oracle.bit_compress(lv2[:, :128], 4), oracle.pack_levels(lv2[:, :128], 4))


def test_network_value_bounds_decide_int16_residuals():
    """nets.value_bounds: ResNet-18 w1a2 residual values stay below 2^15 (so they may be stored as
    int16); with 4-bit activations the deep blocks do not, and stay int32."""
    from apnn_tc_b200 import nets
    spec = nets.resnet18_spec(n_classes=10)
    params = nets.make_params(spec, image_hw=32)
    b = nets.value_bounds(spec, params)
    assert b["Conv1"] == 128 * 7 * 7 * 3          # the 8-bit, re-centred first layer: |a| <= 128
    assert b["L1B1C2"] == 3 * 9 * 64 + b["Conv1"]
    assert max(v for k, v in b.items() if k.endswith("C2")) == b["L4B2C2"] == 28416
    spec4 = nets.resnet18_spec(n_classes=10)
    spec4.a_bit = 4
    b4 = nets.value_bounds(spec4, nets.make_params(spec4, image_hw=32))
    assert b4["L4B2C2"] > 32767 and b4["L1B1C2"] <= 32767


def test_eight_bit_quantiser_needs_no_division(tmp_path):
    """oracle/check_quantise8.c: for every float t in [0, 20], rint((t * 256) / 20) == rint(t * 12.8f) -- the form
    the GPU packers use for the 8-bit first layer is the reference quantiser's, exhaustively."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("gcc not on PATH")
    src = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "check_quantise8.c")
    exe = str(tmp_path / "check_quantise8")
    subprocess.check_call([gcc, "-O2", "-mfma", "-ffp-contract=off", "-o", exe, src, "-lm"])
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout
    assert "checked=1101004801 mismatches=0" in r.stdout
