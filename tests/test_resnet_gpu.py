"""ResNet-50 v1.5 int8 on the GPU against the same quantized network on the CPU oracle: every
layer is integer arithmetic, so the int8 logits must match bit for bit."""
import numpy as np
import pytest
import torch

from glow_b200 import ops, resnet

pytestmark = pytest.mark.gpu
DEV = "cuda"


def run_oracle(oracle, layers, q, x_nchw):
    """The same quantized network through the CPU oracle (numpy in, int8 logits out)."""
    tqp = q["tqp"]
    x = oracle.element_quantize_i8(np.ascontiguousarray(np.transpose(x_nchw, (0, 2, 3, 1))), *tqp["input"])

    def conv(name, t):
        c = q["conv"][name]
        spec = c["spec"]
        k, s, p = (spec["k"],) * 2, (spec["stride"],) * 2, (spec["pad"],) * 4
        ohw = ops.conv_out_hw(t.shape[1:3], k, s, p)
        return oracle.conv2d_i8_i32(t, c["filter"], c["bias"], ohw, k, s, p, 1, (1, 1), c["out_offset"], c["in_offset"],
                                    c["filter_offsets"], c["bias_offsets"], c["params"][:3], c["params"][3:],
                                    1 if spec["relu"] else 0, None)

    for l in layers:
        if l[0] == "conv":
            x = conv(l[1]["name"], x)
        elif l[0] == "maxpool":
            x = oracle.max_pool_i8(x, ops.conv_out_hw(x.shape[1:3], (3, 3), (2, 2), (1, 1, 1, 1)), (3, 3), (2, 2), (1, 1, 1, 1),
                                   tqp["conv1"][1])
        elif l[0] == "block":
            y = x
            for c in l[2]:
                y = conv(c["name"], y)
            sc = conv(l[3]["name"], x) if l[3] else x
            a = q["add"][l[1]]
            out_off = tqp[a["out"]][1]
            x = oracle.element_add_i8(y, sc, out_off, tqp[a["lhs"]][1], tqp[a["rhs"]][1], a["lhs_triple"], a["rhs_triple"])
            x = oracle.element_maxsplat_i8(x, out_off)
        elif l[0] == "avgpool":
            src = q["avgpool_in"]
            hw = x.shape[1]
            tr = ops.quantize_scale_offset_32to8(np.float32(tqp[src][0]) / np.float32(tqp["avgpool"][0]) / np.float32(hw * hw))
            x = oracle.avg_pool_i8(x, (1, 1), (hw, hw), (1, 1), (0, 0, 0, 0), True, tqp["avgpool"][1], tqp[src][1], tr)
        elif l[0] == "fc":
            f = q["fc"]
            x = oracle.rowwise_quantized_fc_i8_i32(x.reshape(x.shape[0], -1), f["w"], f["bias"], f["w_offsets"], f["params"][:3],
                                                   f["params"][3:], tqp["fc"][1], tqp[f["in_name"]][1], 0)
    return x


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
    want = run_oracle(oracle, layers, q, x.numpy())
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
    for name in ("conv1", "s1b0_b", "s2b0_b", "s3b0_b", "s2b0_sc", "s4b2_c"):
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



def test_programmatic_launches_do_not_change_results(net):
    """The library's kernels start beside their predecessors' tails (programmatic dependent launch)
    and touch global memory only after them: the whole network gives the same bytes with the
    switch off, on, and replayed from a CUDA graph captured with it on."""
    layers, w, q = net
    model = resnet.ResNet50Int8(layers, q, DEV)
    x = torch.randn((3, 3, 96, 96), generator=torch.Generator().manual_seed(5)).to(DEV)
    with ops.programmatic_launch(False):
        model.forward(x)
        plain = model.logits_q.clone()
    with ops.programmatic_launch(True):
        for _ in range(3):
            model.forward(x)
            assert torch.equal(model.logits_q, plain)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            model.forward(x)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                model.forward(x)
                captured = model.logits_q
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(captured, plain)
    assert int(model.status.item()) == 0
