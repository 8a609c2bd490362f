"""GPU parity of the model runners (AlexNet, VGG-variant, ResNet-18 layer lists) against the CPU
restatement in net_reference.py, on reduced image sizes so the oracle finishes in seconds."""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import to_host
from net_reference import forward_reference

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("use_tcgen05", [False, True])
@pytest.mark.parametrize("model,hw,batch", [("resnet18", 32, 3), ("alexnet", 64, 2), ("vgg_variant", 32, 2)])
def test_model_logits_match_reference(cuda_device, model, hw, batch, use_tcgen05):
    from apnn_tc_b200 import nets
    spec = nets.MODELS[model](n_classes=200)
    if not use_tcgen05:
        spec.first_bits = 0      # the 8-bit first layer exists on the tcgen05 path; float logits run on both
    params = nets.make_params(spec, image_hw=hw, narrow=use_tcgen05)
    rng = np.random.default_rng(123)
    images = rng.uniform(-10, 10, size=(batch, hw, hw, 3)).astype(np.float32)
    want, levels, values = forward_reference(spec, params, images)
    net = nets.Network(spec, batch, params, image_hw=hw, use_tcgen05=use_tcgen05)
    logits = net.forward(torch.from_numpy(images).cuda())
    net.check()
    assert logits.dtype == torch.float32 and np.array_equal(logits.cpu().numpy(), want)   # bit-exact floats
    # every hidden layer too: packed planes (inside their ring) and saved residuals
    for ls in spec.layers:
        if ls.kind == "conv" and ls.quantise:
            # packed planes or int8 rows, ring removed
            assert np.array_equal(net.levels_of(ls.name).cpu().numpy(), levels[ls.name]), ls.name
        if ls.name in net.res:
            got = net.res[ls.name].cpu().numpy().astype(np.int32)        # int32, or int16 where the values provably fit
            assert np.array_equal(got.reshape(values[ls.name].shape), values[ls.name]), ls.name
    # the quantiser is exercised: more than one level occurs in the last hidden layer
    assert len(np.unique(levels[spec.layers[-2].name])) > 1


@pytest.mark.parametrize("model", ["alexnet", "resnet18", "vgg_variant"])
def test_full_size_models_match_reference(cuda_device, model):
    """The model lists as the benchmark configurations state them -- 224x224x3 images, 1000 classes
    (APNN-TC-nn/src/alexnet.cu:43-81, resnet18.cu:40-142, vgg.cu:49-127) -- on the tcgen05 path:
    logits, every hidden layer and every saved residual bit for bit against the CPU restatement."""
    from apnn_tc_b200 import nets
    spec = nets.MODELS[model](n_classes=1000)
    params = nets.make_params(spec, narrow=True)
    rng = np.random.default_rng(224)
    batch = 2
    images = rng.uniform(-10, 10, size=(batch, 224, 224, 3)).astype(np.float32)
    want, levels, values = forward_reference(spec, params, images)
    net = nets.Network(spec, batch, params, use_tcgen05=True)
    logits = net.forward(torch.from_numpy(images).cuda())
    net.check()
    for ls in spec.layers:
        if ls.kind == "conv" and ls.quantise:
            assert np.array_equal(net.levels_of(ls.name).cpu().numpy(), levels[ls.name]), ls.name
        if ls.name in net.res:
            got = net.res[ls.name].cpu().numpy().astype(np.int32)
            assert np.array_equal(got.reshape(values[ls.name].shape), values[ls.name]), ls.name
    assert logits.dtype == torch.float32 and np.array_equal(logits.cpu().numpy(), want)
    assert len(np.unique(levels[spec.layers[-2].name])) > 1
    assert len(np.unique(levels[spec.layers[0].name])) == 4        # the 8-bit first layer uses every output level


def test_quantised_first_layer_and_integer_logits(cuda_device):
    """first_bits = 0 / float_logits = False: the image quantised to a_bit like a hidden map and int32 logits."""
    from apnn_tc_b200 import nets
    spec = nets.resnet18_spec(n_classes=200)
    spec.first_bits, spec.float_logits = 0, False
    params = nets.make_params(spec, image_hw=64)
    images = np.random.default_rng(5).uniform(-10, 10, size=(3, 64, 64, 3)).astype(np.float32)
    want, levels, _ = forward_reference(spec, params, images)
    net = nets.Network(spec, 3, params, image_hw=64)
    logits = net.forward(torch.from_numpy(images).cuda())
    net.check()
    assert logits.dtype == torch.int32 and np.array_equal(logits.cpu().numpy(), want)
    assert np.array_equal(net.levels_of("Conv1").cpu().numpy(), levels["Conv1"])


@pytest.mark.parametrize("model,batch", [("alexnet", 128), ("resnet18", 128), ("resnet18", 1024), ("vgg_variant", 128)])
def test_benchmark_batches_match_reference(cuda_device, model, batch):
    """The batches the benchmark runs (AlexNet 128; ResNet-18 1024 on one GPU and 128 per GPU on eight;
    the VGG-variant) select other kernels than a batch of 2 does (CTA-pair convolutions, resident
    filters, split-K): the batch is filled with copies of 8 distinct images, whose reference logits
    every copy must reproduce (images are independent), through eager launches and a graph replay."""
    from apnn_tc_b200 import nets
    spec = nets.MODELS[model](n_classes=1000)
    params = nets.make_params(spec, narrow=True)
    rng = np.random.default_rng(batch)
    distinct = rng.uniform(-10, 10, size=(8, 224, 224, 3)).astype(np.float32)
    want, _, _ = forward_reference(spec, params, distinct)
    net = nets.Network(spec, batch, params, use_tcgen05=True)
    images = torch.from_numpy(distinct).cuda().repeat(batch // 8, 1, 1, 1).contiguous()
    logits = net.forward(images).clone()
    net.check()
    expect = torch.from_numpy(want).cuda().repeat(batch // 8, 1)
    assert torch.equal(logits, expect)
    net.capture(images)
    assert torch.equal(net.replay(), expect)
    net.check()


def test_graph_replay_matches_eager(cuda_device):
    from apnn_tc_b200 import nets
    spec = nets.resnet18_spec(n_classes=100)
    net = nets.Network(spec, 4, image_hw=32)
    g = torch.Generator(device="cuda").manual_seed(9)
    images = (torch.rand((4, 32, 32, 3), device="cuda", generator=g) * 20 - 10).contiguous()
    eager = net.forward(images).clone()
    net.capture(images)
    images.copy_((torch.rand((4, 32, 32, 3), device="cuda", generator=g) * 20 - 10))
    second = net.forward(images).clone()
    replayed = net.replay().clone()
    net.check()
    assert torch.equal(replayed, second) and not torch.equal(eager, second)
