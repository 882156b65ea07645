"""ResNet-50 v1.5, fully int8 (channelwise-quantized convolutions), on the glow_b200 kernels:
the third benchmark configuration.

    fp32 NCHW input -> Quantize + Transpose (NHWC) -> conv 7x7/2 + Relu -> MaxPool 3x3/2
    -> 16 bottleneck blocks (1x1, 3x3 [stride here: v1.5], 1x1, shortcut 1x1 where shapes change,
       ElementAdd, Relu) -> AvgPool 7x7 -> rowwise-quantized FC -> Dequantize

Weights are random He-normal (batch-norm folded away), quantized per output channel with the
symmetric schema; activations use the asymmetric int8 schema with ranges taken from a
calibration pass of the fp32 network over seeded N(0,1) images -- the flow Glow's own
quantization procedure follows (profile, then quantizeFunction with enableChannelwise,
lib/Quantization/Quantization.cpp:762-844).  Relu after a convolution is fused into it
(CPUBackend::supportsFusedActivation, lib/Backends/CPU/CPUBackend.cpp:86-112); Relu after the
residual add is the max-with-constant the CPU backend lowers it to.

Harness code: builds the network description and drives glow_b200.ops (the tests run the same
description through the CPU checker).
"""
import math

import numpy as np
import torch

from . import ops

STAGES = [(64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)]  # (bottleneck width, blocks, stride of the first)


def _conv_spec(name, cin, cout, k, stride, pad, relu):
    return dict(name=name, cin=cin, cout=cout, k=k, stride=stride, pad=pad, relu=relu)


def architecture(num_classes=1000):
    """The layer list: ('conv', spec) / ('maxpool',) / ('block', [convs...], shortcut or None) ..."""
    layers = [("conv", _conv_spec("conv1", 3, 64, 7, 2, 3, True)), ("maxpool",)]
    cin = 64
    for si, (width, blocks, stride) in enumerate(STAGES):
        for b in range(blocks):
            s = stride if b == 0 else 1
            cout = width * 4
            pre = "s%db%d" % (si + 1, b)
            convs = [_conv_spec(pre + "_a", cin, width, 1, 1, 0, True),
                     _conv_spec(pre + "_b", width, width, 3, s, 1, True),
                     _conv_spec(pre + "_c", width, cout, 1, 1, 0, False)]
            short = _conv_spec(pre + "_sc", cin, cout, 1, s, 0, False) if (s != 1 or cin != cout) else None
            layers.append(("block", pre, convs, short))
            cin = cout
    layers.append(("avgpool",))
    layers.append(("fc", dict(name="fc", cin=cin, cout=num_classes)))
    return layers


def float_weights(layers, seed=0x610B200):
    """He-normal filters [outC, kH, kW, inC] and small biases, fp32 numpy."""
    rng = np.random.default_rng(seed)
    w = {}

    def conv(spec):
        fan_in = spec["k"] * spec["k"] * spec["cin"]
        w[spec["name"]] = ((rng.standard_normal((spec["cout"], spec["k"], spec["k"], spec["cin"])) *
                            math.sqrt(2.0 / fan_in)).astype(np.float32),
                           (rng.standard_normal(spec["cout"]) * 0.02).astype(np.float32))

    for l in layers:
        if l[0] == "conv":
            conv(l[1])
        elif l[0] == "block":
            for c in l[2]:
                conv(c)
            if l[3]:
                conv(l[3])
        elif l[0] == "fc":
            spec = l[1]
            w["fc"] = ((rng.standard_normal((spec["cout"], spec["cin"])) * math.sqrt(1.0 / spec["cin"])).astype(np.float32),
                       (rng.standard_normal(spec["cout"]) * 0.02).astype(np.float32))
    return w


def float_forward(layers, w, x_nchw, device):
    """fp32 forward (torch) that records (min, max) of every tensor that gets a quantized type."""
    import torch.nn.functional as F
    ranges = {}

    def rec(name, t):
        lo, hi = float(t.min()), float(t.max())
        old = ranges.get(name)
        ranges[name] = (min(lo, old[0]), max(hi, old[1])) if old else (lo, hi)

    def conv(spec, t):
        f, b = w[spec["name"]]
        wt = torch.from_numpy(f).to(device).permute(0, 3, 1, 2).contiguous()
        y = F.conv2d(t, wt, torch.from_numpy(b).to(device), stride=spec["stride"], padding=spec["pad"])
        if spec["relu"]:
            y = torch.relu(y)
        rec(spec["name"], y)
        return y

    t = x_nchw.to(device)
    rec("input", t)
    for l in layers:
        if l[0] == "conv":
            t = conv(l[1], t)
        elif l[0] == "maxpool":
            t = F.max_pool2d(t, 3, 2, 1)
        elif l[0] == "block":
            y = t
            for c in l[2]:
                y = conv(c, y)
            sc = conv(l[3], t) if l[3] else t
            t = torch.relu(y + sc)
            rec(l[1] + "_out", t)
        elif l[0] == "avgpool":
            t = F.avg_pool2d(t, t.shape[-1])
            rec("avgpool", t)
        elif l[0] == "fc":
            f, b = w["fc"]
            t = t.flatten(1) @ torch.from_numpy(f).to(device).T + torch.from_numpy(b).to(device)
            rec("fc", t)
    return t, ranges


def quantize_network(layers, w, ranges):
    """Quantized constants and integer requantisation parameters of every layer (numpy)."""
    tqp = {k: ops.choose_quantization_params(v[0], v[1], ops.ASYMMETRIC) for k, v in ranges.items()}
    q = {"tqp": tqp, "conv": {}, "add": {}}

    def conv(spec, in_name):
        in_scale, in_off = tqp[in_name]
        out_scale, out_off = tqp[spec["name"]]
        c = ops.channelwise_conv_prepare(w[spec["name"]][0], w[spec["name"]][1], in_scale, ops.SYMMETRIC)
        c["params"] = ops.rowwise_requant_params(c["filter_scales"], in_scale, c["bias_scales"], out_scale)
        c.update(in_offset=in_off, out_offset=out_off, spec=spec)
        q["conv"][spec["name"]] = c

    cur = "input"
    for l in layers:
        if l[0] == "conv":
            conv(l[1], cur)
            cur = l[1]["name"]
        elif l[0] == "block":
            x_in = cur
            for c in l[2]:
                conv(c, cur)
                cur = c["name"]
            if l[3]:
                conv(l[3], x_in)
                sc = l[3]["name"]
            else:
                sc = x_in
            out = l[1] + "_out"
            # ElementAdd into the block output's type: each side rescaled on its own
            # (LLVMIRGen.cpp:1716-1771), then Relu = max with the output offset
            q["add"][l[1]] = dict(lhs=cur, rhs=sc, out=out,
                                  lhs_triple=ops.quantize_scale_offset_32to8(np.float32(tqp[cur][0]) / np.float32(tqp[out][0])),
                                  rhs_triple=ops.quantize_scale_offset_32to8(np.float32(tqp[sc][0]) / np.float32(tqp[out][0])))
            cur = out
        elif l[0] == "avgpool":
            # libjit_avg_pool_i8 with countIncludePads: scale = in/out/(kernel area) (LLVMIRGen.cpp:3003-3046)
            q["avgpool_in"] = cur
            cur = "avgpool"
        elif l[0] == "fc":
            f, b = w["fc"]
            wq, ws, wo = ops.tensor_rowwise_quantize_i8(f, ops.ASYMMETRIC)
            w_tensor_scale, _ = ops.choose_quantization_params(float(f.min()), float(f.max()), ops.ASYMMETRIC)
            bias_scale = float(np.float32(tqp[cur][0]) * np.float32(w_tensor_scale))
            q["fc"] = dict(w=wq, w_offsets=wo, bias=ops.quantize_bias_i32(b, bias_scale, 0),
                           params=ops.rowwise_requant_params(ws, tqp[cur][0], np.float32(bias_scale), tqp["fc"][0]),
                           in_name=cur)
    return q


class ResNet50Int8:
    """The quantized network resident on one GPU."""

    def __init__(self, layers, q, device="cuda"):
        self.layers, self.q, self.dev = layers, q, torch.device(device)
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.dev)
        self.conv = {}
        for name, c in q["conv"].items():
            f = to(c["filter"])
            self.conv[name] = dict(filter=f, bias=to(c["bias"]), fo=to(c["filter_offsets"]), bo=to(c["bias_offsets"]),
                                   params=[to(a) for a in c["params"]],
                                   row_sums=ops.i8_row_sums(f.view(f.shape[0], -1)), c=c)
        fc = q["fc"]
        self.fc = dict(w=to(fc["w"]), w_off=to(fc["w_offsets"]), bias=to(fc["bias"]), params=[to(a) for a in fc["params"]])
        self.fc["row_sums"] = ops.i8_row_sums(self.fc["w"])
        self.status = ops.new_status(self.dev)
        self.ws = None
        self.launches = 0

    def _workspace(self, nbytes):
        if self.ws is None or self.ws.numel() < nbytes:
            self.ws = torch.empty(int(nbytes * 1.1) + 256, dtype=torch.uint8, device=self.dev)
        return self.ws

    def _conv(self, name, x):
        d = self.conv[name]
        c, spec = d["c"], d["c"]["spec"]
        k, s, p = (spec["k"],) * 2, (spec["stride"],) * 2, (spec["pad"],) * 4
        n, h, w_, cin = x.shape
        oh, ow = ops.conv_out_hw((h, w_), k, s, p)
        need = n * oh * ow * ((spec["k"] ** 2 * cin + 15) // 16 * 16) + spec["cout"] * ((spec["k"] ** 2 * cin + 15) // 16 * 16) + \
            ops.i8_gemm_workspace_bytes(n * oh * ow, 16, spec["cout"]) + 4096
        self.launches += 2
        return ops.channelwise_quantized_conv2d(x, d["filter"], d["bias"], k, s, p, 1, (1, 1), c["out_offset"], c["in_offset"],
                                                d["fo"], d["bo"], d["params"][:3], d["params"][3:],
                                                1 if spec["relu"] else 0, None, filter_row_sums=d["row_sums"],
                                                flags=ops.FC_WEIGHT_OFFSETS_ZERO, workspace=self._workspace(need),
                                                status=self.status)

    def forward(self, x_nchw):
        """x_nchw: fp32 [N,3,H,W] on the device -> fp32 logits [N, classes]."""
        tqp = self.q["tqp"]
        self.launches = 0
        # Quantize, then Transpose: the order Glow's optimizer leaves (it sinks a Transpose below the
        # Quantize that consumes it, GraphOptimizer.cpp:1076-1086) -- the layout change moves bytes, not floats
        x = ops.quantize_transpose_i8(x_nchw, (0, 2, 3, 1), *tqp["input"])   # one kernel for the pair
        self.launches += 1
        for l in self.layers:
            if l[0] == "conv":
                x = self._conv(l[1]["name"], x)
            elif l[0] == "maxpool":
                x = ops.max_pool_i8(x, (3, 3), (2, 2), (1, 1, 1, 1), tqp["conv1"][1])
                self.launches += 1
            elif l[0] == "block":
                y = x
                for c in l[2]:
                    y = self._conv(c["name"], y)
                sc = self._conv(l[3]["name"], x) if l[3] else x
                a = self.q["add"][l[1]]
                out_off = tqp[a["out"]][1]
                x = ops.element_add_maxsplat_i8(y, sc, out_off, tqp[a["lhs"]][1], tqp[a["rhs"]][1], a["lhs_triple"],
                                                a["rhs_triple"], out_off)
                self.launches += 1
            elif l[0] == "avgpool":
                src = self.q["avgpool_in"]
                hw = x.shape[1]
                tr = ops.quantize_scale_offset_32to8(np.float32(tqp[src][0]) / np.float32(tqp["avgpool"][0]) / np.float32(hw * hw))
                x = ops.avg_pool_i8(x, (hw, hw), (1, 1), (0, 0, 0, 0), True, tqp["avgpool"][1], tqp[src][1], tr)
                self.launches += 1
            elif l[0] == "fc":
                f = self.fc
                x2 = x.reshape(x.shape[0], -1)
                y = ops.rowwise_quantized_fc(x2, f["w"], f["bias"], f["w_off"], f["params"][:3], f["params"][3:], tqp["fc"][1],
                                             tqp[self.q["fc"]["in_name"]][1], 0, weights_row_sums=f["row_sums"],
                                             workspace=self._workspace(ops.i8_gemm_workspace_bytes(x2.shape[0], x2.shape[1], f["w"].shape[0])),
                                             status=self.status)
                self.logits_q = y
                x = ops.element_dequantize_i8(y, *tqp["fc"])
                self.launches += 3
        return x


def conv_ops_per_image(layers, hw=224):
    """2 * MACs of every convolution and the FC for one hw x hw image (from the layer list)."""
    total, size = 0, hw
    cur = size

    def conv(spec, s_in):
        s_out = (s_in + 2 * spec["pad"] - spec["k"]) // spec["stride"] + 1
        return 2 * s_out * s_out * spec["cout"] * spec["k"] * spec["k"] * spec["cin"], s_out

    for l in layers:
        if l[0] == "conv":
            o, cur = conv(l[1], cur)
            total += o
        elif l[0] == "maxpool":
            cur = (cur + 2 - 3) // 2 + 1
        elif l[0] == "block":
            s_in = cur
            for c in l[2]:
                o, cur = conv(c, cur)
                total += o
            if l[3]:
                total += conv(l[3], s_in)[0]
        elif l[0] == "fc":
            total += 2 * l[1]["cin"] * l[1]["cout"]
    return total
