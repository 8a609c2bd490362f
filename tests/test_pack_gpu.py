"""GPU parity of the layer-boundary packers against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import to_dev, to_host

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
