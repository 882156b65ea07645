"""ResNet-50 v1.5 int8 on the GPU against the same quantized network on the CPU oracle: every
layer is integer arithmetic, so the int8 logits must match bit for bit."""
import numpy as np
import pytest
import torch

from glow_b200 import ops, resnet

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def net():
    layers = resnet.architecture(num_classes=100)
    w = resnet.float_weights(layers)
    g = torch.Generator().manual_seed(7)
    calib = torch.randn((4, 3, 64, 64), generator=g)
    _, ranges = resnet.float_forward(layers, w, calib, DEV)
    q = resnet.quantize_network(layers, w, ranges)
    return layers, w, q


def test_resnet50_int8_bit_exact_against_oracle(oracle, net):
    layers, w, q = net
    model = resnet.ResNet50Int8(layers, q, DEV)
    g = torch.Generator().manual_seed(11)
    x = torch.randn((2, 3, 64, 64), generator=g)
    logits = model.forward(x.to(DEV))
    torch.cuda.synchronize()
    assert int(model.status.item()) == 0
    want = resnet.run_oracle(oracle, layers, q, x.numpy())
    np.testing.assert_array_equal(model.logits_q.cpu().numpy(), want)
    assert len(np.unique(want)) > 20
    # and the quantized network still tracks the fp32 one (quantisation error only)
    ref, _ = resnet.float_forward(layers, w, x, DEV)
    err = (logits - ref).abs().max() / (ref.max() - ref.min())
    assert float(err) < 0.25
    assert model.launches > 100


def test_every_conv_takes_the_tensor_core_path(net):
    """All 53 convolutions of the network are group-1 and land on the contraction kernel
    (im2col or direct); their results equal the direct kernel's on a real activation."""
    layers, w, q = net
    rng = np.random.default_rng(3)
    for name in ("conv1", "s1b0_b", "s2b0_sc", "s4b2_c"):
        c = q["conv"][name]
        spec = c["spec"]
        x = torch.from_numpy(rng.integers(-128, 128, (2, 20, 20, spec["cin"]), dtype=np.int8)).to(DEV)
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
        pp = [to(a) for a in c["params"]]
        args = (x, to(c["filter"]), to(c["bias"]), (spec["k"],) * 2, (spec["stride"],) * 2, (spec["pad"],) * 4, 1, (1, 1),
                c["out_offset"], c["in_offset"], to(c["filter_offsets"]), to(c["bias_offsets"]), pp[:3], pp[3:],
                1 if spec["relu"] else 0, None)
        assert not c["filter_offsets"].any()  # symmetric filters
        a = ops.channelwise_quantized_conv2d(*args, flags=ops.FC_WEIGHT_OFFSETS_ZERO)
        b = ops.channelwise_quantized_conv2d(*args, flags=ops.FC_FORCE_ANY_SHAPE_KERNEL)
        assert torch.equal(a, b)
