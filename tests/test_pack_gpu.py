"""GPU parity of the layer-boundary packers against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import spread_bytes, to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,C,bits", [(7, 3, 2), (64, 128, 2), (33, 160, 4), (1000, 64, 3), (5, 1, 1), (4096, 512, 2),
                                         (3, 130, 8)])
def test_bit_compression(cuda_device, rows, C, bits):
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(rows + C)
    lv = rng.integers(0, 1 << bits, size=(rows, C), dtype=np.uint32)
    got = to_host(ap.Bit_compression(to_dev(lv), bits))
    assert np.array_equal(got, oracle.bit_compress(lv, bits))


@pytest.mark.parametrize("shape,bits", [((2, 5, 7, 3), 2), ((4, 8, 8, 128), 2), ((1, 3, 3, 200), 4)])
def test_images_quantization(cuda_device, shape, bits):
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(sum(shape))
    x = rng.uniform(-12, 12, size=shape).astype(np.float32)
    # exact grid points and half-way points exercise round-to-nearest-even
    flat = x.reshape(-1)
    step = 20.0 / (1 << bits)
    flat[: min(64, flat.size)] = (-10 + step * (np.arange(min(64, flat.size)) % ((1 << bits) * 2 + 1)) / 2).astype(np.float32)
    got = to_host(ap.images_quantization(torch.from_numpy(x).cuda(), bits))
    assert np.array_equal(got, oracle.bit_compress(oracle.quantize(x, bits), bits))


@pytest.mark.parametrize("B,H,Wd,C,R,stride,bits", [(2, 9, 7, 3, 3, 2, 2), (3, 32, 32, 3, 7, 4, 2), (2, 20, 24, 3, 11, 4, 2),
                                                    (1, 8, 8, 5, 5, 1, 4), (2, 6, 6, 40, 3, 1, 2),
                                                    (1, 224, 224, 3, 7, 4, 2), (1, 16, 12, 3, 3, 1, 8),
                                                    (1, 12, 1500, 3, 11, 4, 2)])
def test_quantize_im2col(cuda_device, B, H, Wd, C, R, stride, bits):
    """First-layer re-layout: quantised RxRxC windows gathered along the channel axis."""
    import ctypes
    from apnn_tc_b200 import _cabi
    rng = np.random.default_rng(B + H + R)
    x = rng.uniform(-12, 12, size=(B, H, Wd, C)).astype(np.float32)
    want = oracle.quantize_im2col(x, R, stride, bits)
    out = torch.full(want.shape, -1, dtype=torch.int32, device="cuda")
    xd = torch.from_numpy(x).cuda()
    st = _cabi.lib().apnn_quantize_im2col(torch.cuda.current_stream().cuda_stream, xd.data_ptr(), out.data_ptr(), B, H, Wd,
                                          C, R, stride, bits)
    _cabi.check(st, "apnn_quantize_im2col")
    assert np.array_equal(to_host(out), want)


@pytest.mark.parametrize("bits,rows,K", [(1, 5, 64), (2, 37, 128), (4, 9, 320), (3, 3, 192)])
def test_expand_planes_byte_layout(cuda_device, bits, rows, K):
    import apnn_tc_b200 as ap
    rng = np.random.default_rng(bits + rows + K)
    planes, lv = oracle.value_planes(rng, rows, K, bits)
    got = ap.expand_planes(torch.from_numpy(planes.view(np.int32)).cuda()).cpu().numpy()
    assert np.array_equal(got, spread_bytes(lv.astype(np.uint8)))


@pytest.mark.parametrize("B,H,Wd,C,R,stride,bits,kp", [(2, 9, 7, 3, 3, 2, 2, 64), (3, 32, 32, 3, 7, 4, 2, 192),
                                                       (2, 20, 24, 3, 11, 4, 2, 384), (1, 8, 8, 5, 5, 1, 4, 128),
                                                       (1, 224, 224, 3, 7, 4, 2, 192), (2, 6, 6, 40, 3, 1, 2, 384)])
def test_quantize_im2col_i8(cuda_device, B, H, Wd, C, R, stride, bits, kp):
    """First layer straight to int8 rows: the oracle's gathered levels in the operand byte order."""
    from apnn_tc_b200 import _cabi
    rng = np.random.default_rng(B + H + R + kp)
    x = rng.uniform(-12, 12, size=(B, H, Wd, C)).astype(np.float32)
    # the points where the level changes (ties round to even) and their float neighbours
    step = 20.0 / (1 << bits)
    edges = (-10 + step * (np.arange(1 << bits) + 0.5)).astype(np.float32)
    probe = np.concatenate([edges, np.nextafter(edges, np.float32(-20)), np.nextafter(edges, np.float32(20)),
                            np.array([-10, 10, -10.5, 10.5, 0], np.float32)])
    flat = x.reshape(-1)
    flat[: min(probe.size, flat.size)] = probe[: flat.size]
    lv = oracle.unpack_levels(oracle.quantize_im2col(x, R, stride, bits))     # [B, Ho, Wo, PAD128(R*R*C)]
    want = np.zeros(lv.shape[:3] + (kp,), dtype=np.uint8)
    n = min(kp, lv.shape[-1])
    want[..., :n] = lv[..., :n]
    assert not lv[..., n:].any()
    want = spread_bytes(want)
    out = torch.full(want.shape, 0x55, dtype=torch.uint8, device="cuda")
    xd = torch.from_numpy(x).cuda()
    st = _cabi.lib().apnn_quantize_im2col_i8(torch.cuda.current_stream().cuda_stream, xd.data_ptr(), out.data_ptr(), B, H,
                                             Wd, C, R, stride, bits, kp)
    _cabi.check(st, "apnn_quantize_im2col_i8")
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("B,H,Wd,C,R,stride,bits,kp", [(2, 10, 8, 3, 3, 2, 2, 64), (3, 32, 32, 3, 7, 4, 2, 192),
                                                       (2, 20, 24, 3, 11, 4, 2, 448), (1, 8, 8, 4, 5, 1, 4, 128),
                                                       (1, 224, 224, 3, 7, 4, 2, 192), (2, 224, 224, 3, 11, 4, 2, 448),
                                                       (1, 224, 224, 3, 3, 2, 2, 64), (2, 6, 6, 40, 3, 1, 3, 384)])
def test_quantize_window_rows_i8(cuda_device, B, H, Wd, C, R, stride, bits, kp):
    """First layer as R segments per pixel: segment i of pixel (ho, wo) = the oracle's levels of the R*C
    elements of image row ho*stride - pad + i from column wo*stride - pad on, zero outside the image."""
    from apnn_tc_b200 import _cabi
    rng = np.random.default_rng(B + H + R + kp)
    x = rng.uniform(-12, 12, size=(B, H, Wd, C)).astype(np.float32)
    step = 20.0 / (1 << bits)
    edges = (-10 + step * (np.arange(1 << bits) + 0.5)).astype(np.float32)
    probe = np.concatenate([edges, np.nextafter(edges, np.float32(-20)), np.nextafter(edges, np.float32(20)),
                            np.array([-10, 10, -10.5, 10.5, 0], np.float32)])
    flat = x.reshape(-1)
    flat[: min(probe.size, flat.size)] = probe[: flat.size]
    pad, seg = (R - 1) // 2, (R * C + 3) // 4 * 4
    Ho, Wo = (H - 1) // stride + 1, (Wd - 1) // stride + 1
    lv = oracle.quantize(x, bits).astype(np.uint8).reshape(B, H, Wd * C)
    # every image row with pad*C zero bytes on the left and enough on the right, pad zero rows above and below
    padded = np.zeros((B, H + 2 * pad, pad * C + Wd * C + pad * C + 4), dtype=np.uint8)
    padded[:, pad:pad + H, pad * C:pad * C + Wd * C] = lv
    want = np.zeros((B, Ho, Wo, kp), dtype=np.uint8)
    for i in range(R):
        for wo in range(Wo):
            a = wo * stride * C
            want[:, :, wo, i * seg:i * seg + R * C] = padded[:, i:i + (Ho - 1) * stride + 1:stride, a:a + R * C]
    out = torch.full(want.shape, 0x55, dtype=torch.uint8, device="cuda")
    xd = torch.from_numpy(x).cuda()
    st = _cabi.lib().apnn_quantize_window_rows_i8(torch.cuda.current_stream().cuda_stream, xd.data_ptr(), out.data_ptr(),
                                                  B, H, Wd, C, R, stride, bits, kp)
    _cabi.check(st, "apnn_quantize_window_rows_i8")
    assert np.array_equal(out.cpu().numpy(), want)


def test_quantize_window_rows_i8_refuses_what_it_does_not_cover(cuda_device):
    from apnn_tc_b200 import _cabi
    x = torch.zeros((1, 8, 7, 3), dtype=torch.float32, device="cuda")     # W*C = 21: not whole quads
    out = torch.zeros((1, 8, 7, 64), dtype=torch.uint8, device="cuda")
    st = _cabi.lib().apnn_quantize_window_rows_i8(torch.cuda.current_stream().cuda_stream, x.data_ptr(), out.data_ptr(),
                                                  1, 8, 7, 3, 3, 1, 2, 64)
    assert st == 2   # APNN_ERR_UNSUPPORTED


@pytest.mark.parametrize("B,H,Wd,C,ih,oh", [(2, 8, 12, 64, 0, 1), (3, 6, 6, 128, 1, 0), (1, 56, 56, 16, 0, 0)])
def test_maxpool2x2_i8(cuda_device, B, H, Wd, C, ih, oh):
    from apnn_tc_b200 import _cabi
    rng = np.random.default_rng(B + H + C)
    x = rng.integers(0, 256, size=(B, H + 2 * ih, Wd + 2 * ih, C), dtype=np.uint8)
    core = x[:, ih:ih + H, ih:ih + Wd]
    want = core.reshape(B, H // 2, 2, Wd // 2, 2, C).max(axis=(2, 4))
    out = torch.full((B, H // 2 + 2 * oh, Wd // 2 + 2 * oh, C), 7, dtype=torch.uint8, device="cuda")
    xd = torch.from_numpy(x).cuda()
    _cabi.check(_cabi.lib().apnn_maxpool2x2_i8(torch.cuda.current_stream().cuda_stream, xd.data_ptr(), out.data_ptr(), B, H, Wd,
                                               C, ih, oh), "apnn_maxpool2x2_i8")
    got = out.cpu().numpy()
    assert np.array_equal(got[:, oh:oh + H // 2, oh:oh + Wd // 2], want)
    if oh:
        assert (got[:, 0] == 7).all() and (got[:, :, 0] == 7).all()   # the ring is not written


@pytest.mark.parametrize("B,H,Wd,C,stride,bits,centred,halo,cpad", [(2, 32, 32, 3, 4, 8, True, 1, 64), (1, 224, 224, 3, 4, 8, True, 1, 64),
                                                                    (3, 8, 12, 4, 2, 2, False, 2, 16), (2, 12, 8, 2, 2, 4, False, 0, 32),
                                                                    (1, 16, 16, 1, 4, 8, True, 1, 16)])
def test_quantize_blocks_i8(cuda_device, B, H, Wd, C, stride, bits, centred, halo, cpad):
    """The image as stride x stride pixel blocks: byte (di*stride + dj)*C + c of block (hb, wb) = the oracle's level
    of pixel (stride*hb + di, stride*wb + dj), channel c (minus 128 in the centred 8-bit form), zero bytes after
    stride*stride*C, the ring of halo blocks untouched."""
    from apnn_tc_b200 import _cabi
    rng = np.random.default_rng(B + H + stride + cpad)
    x = rng.uniform(-12, 12, size=(B, H, Wd, C)).astype(np.float32)
    lv = oracle.quantize(x, bits).astype(np.uint8)
    if centred:
        lv = lv ^ np.uint8(0x80)
    Hb, Wb = H // stride, Wd // stride
    blocks = lv.reshape(B, Hb, stride, Wb, stride, C).transpose(0, 1, 3, 2, 4, 5).reshape(B, Hb, Wb, stride * stride * C)
    want = np.full((B, Hb + 2 * halo, Wb + 2 * halo, cpad), 0x55, dtype=np.uint8)
    want[:, halo:halo + Hb, halo:halo + Wb, :] = 0
    want[:, halo:halo + Hb, halo:halo + Wb, : stride * stride * C] = blocks
    out = torch.full(want.shape, 0x55, dtype=torch.uint8, device="cuda")
    xd = torch.from_numpy(x).cuda()
    st = _cabi.lib().apnn_quantize_blocks_i8(torch.cuda.current_stream().cuda_stream, xd.data_ptr(), out.data_ptr(), B, H, Wd, C,
                                             stride, bits | (_cabi.QUANT_CENTRED if centred else 0), halo, cpad)
    _cabi.check(st, "apnn_quantize_blocks_i8")
    assert np.array_equal(out.cpu().numpy(), want)


def test_quantize_blocks_i8_refuses_what_it_does_not_cover(cuda_device):
    from apnn_tc_b200 import _cabi
    x = torch.zeros((1, 8, 8, 3), dtype=torch.float32, device="cuda")
    out = torch.zeros((1, 6, 6, 64), dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    L = _cabi.lib()
    assert L.apnn_quantize_blocks_i8(s, x.data_ptr(), out.data_ptr(), 1, 8, 8, 3, 2, 8, 1, 64) == 2    # stride * C = 6: no whole quads
    assert L.apnn_quantize_blocks_i8(s, x.data_ptr(), out.data_ptr(), 1, 8, 8, 3, 4, 8, 1, 32) == 2    # 48 level bytes > cpad
    assert L.apnn_quantize_blocks_i8(s, x.data_ptr(), out.data_ptr(), 1, 7, 8, 3, 4, 8, 1, 64) == 2    # H not a multiple of stride
