"""Synthetic `.espdl` networks with the topologies of the benchmark configurations.

The trained model-zoo files cannot travel with this repository and the exporter (esp-ppq) is a separate
project, so the benchmark and the tests build their networks here: same graph structure, node attributes and
tensor conventions as the exported files (NHWC activations, filters declared [KH,KW,Cin,Cout] with target "c"
byte order [Cout][KH][KW][Cin], int32 bias at exponent e_in + e_w[c], per-channel power-of-two filter
exponents, ONNX pad order [t,l,b,r]), random int8 weights from a seeded generator.

Weight amplitudes are scaled per output channel so that the requantised activations use the int8 range without
saturating everywhere (the configurations ask for random weights, not for a particular amplitude).
"""
import numpy as np

from . import espdl_file

# MobileNetV2-1.0 inverted-residual settings: expansion t, output channels c, repeats n, first stride s
MBV2_SETTINGS = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]


class _Net:
    def __init__(self, name, seed, e_act=(-8, -4), e_w=(-9, -5)):
        self.g = espdl_file.GraphBuilder(name, {"target": "c"})
        self.rng = np.random.default_rng(seed)
        self.e_act, self.e_w = e_act, e_w
        self.exp = {}     # tensor name -> exponent
        self.shape = {}   # tensor name -> NHWC shape (batch 1)
        self.rms = {}     # tensor name -> estimated rms of the quantised values
        self.count = 0

    def fresh(self, prefix):
        self.count += 1
        return f"{prefix}_{self.count}"

    def tensor(self, name, shape, exponent, rms):
        self.exp[name], self.shape[name], self.rms[name] = exponent, list(shape), rms
        self.g.add_value_info(name, np.int8, shape, exponent)

    def pick_exponent(self, e_acc, need, allowed):
        """Output exponent from `allowed` = (lo, hi) such that every shift e_out - e_acc[c] is >= 1 and as many channels
        as possible get a weight amplitude need * 2^shift inside [3, 127]; ties are broken at random."""
        scored = []
        for e in range(allowed[0], allowed[1] + 1):
            shift = e - e_acc
            if shift.min() < 1:
                continue
            amp = need * 2.0 ** shift
            scored.append((float(((amp >= 3) & (amp <= 127)).mean()), e))
        if not scored:
            return int(e_acc.max() + 1)
        top = max(s for s, _ in scored)
        good = [e for s, e in scored if s >= top - 0.1]
        return int(good[int(self.rng.integers(0, len(good)))])

    def conv(self, x, cout, k, stride=1, group=1, relu=True, e_out=None, bias=True, name=None):
        n, h, w, cin = self.shape[x]
        depthwise = group != 1
        pad = k // 2
        oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        e_in = self.exp[x]
        ew = self.rng.integers(self.e_w[0], self.e_w[1] + 1, size=cout)
        taps = k * k * (1 if depthwise else cin)
        target = 28.0  # wanted rms of the requantised output, in codes
        need = target * np.sqrt(3.0) / (self.rms[x] * np.sqrt(taps))  # weight amplitude wanted at shift 0
        if e_out is None:
            e_out = self.pick_exponent(ew + e_in, need, self.e_act)
        shift = e_out - ew - e_in
        # amplitude so that the requantised output has rms ~ target: rms_acc = rms_in * (wmax/sqrt(3)) * sqrt(taps)
        wmax = np.clip(np.round(need * (2.0 ** shift)), 1, 127).astype(np.int64)
        if depthwise:
            wt = np.stack([self.rng.integers(-wmax[c], wmax[c] + 1, size=(k, k)) for c in range(cout)], axis=-1).astype(np.int8)  # [KH][KW][C]
            declared = (k, k, cin, 1)
        else:
            wt = np.stack([self.rng.integers(-wmax[c], wmax[c] + 1, size=(k, k, cin)) for c in range(cout)]).astype(np.int8)  # [Cout][KH][KW][Cin]
            declared = (k, k, cin, cout)
        node = name or self.fresh("conv")
        wname, bname, out = node + ".weight", node + ".bias", node + "_out"
        # the payload keeps the target-"c" byte order; only the declared dims are [KH,KW,Cin,Cout]
        self.g.add_initializer(wname, wt.reshape(declared), list(ew))
        inputs = [x, wname]
        if bias:
            acc_rms = self.rms[x] * (wmax / np.sqrt(3.0)) * np.sqrt(taps)
            b = np.round(self.rng.uniform(-0.5, 0.5, size=cout) * acc_rms).astype(np.int32)
            self.g.add_initializer(bname, b, list(ew + e_in))
            inputs.append(bname)
        self.g.add_node("Conv", node, inputs, [out], activation="Relu" if relu else "Linear", dilations=[1, 1], group=int(group),
                        kernel_shape=[k, k], pads=[pad, pad, pad, pad], quant_type="S8", strides=[stride, stride])
        est = np.minimum(target, self.rms[x] * (wmax / np.sqrt(3.0)) * np.sqrt(taps) / (2.0 ** shift)).mean()
        self.tensor(out, (n, oh, ow, cout), e_out, float(est / np.sqrt(2.0) if relu else est))
        return out

    def requantize(self, x, e_out):
        node = self.fresh("requantize")
        out = node + "_out"
        self.g.add_node("RequantizeLinear", node, [x], [out], quant_type="S8")
        self.tensor(out, self.shape[x], e_out, self.rms[x] * 2.0 ** (self.exp[x] - e_out))
        return out

    def add(self, a, b, e_out):
        if self.exp[a] != e_out:
            a = self.requantize(a, e_out)
        if self.exp[b] != e_out:
            b = self.requantize(b, e_out)
        node = self.fresh("add")
        out = node + "_out"
        self.g.add_node("Add", node, [a, b], [out], quant_type="S8")
        self.tensor(out, self.shape[a], e_out, float(np.hypot(self.rms[a], self.rms[b])))
        return out


def mobilenet_v2(seed=5, input_hw=224, num_classes=1000, width=1.0, e_act=(-8, -4), e_w=(-9, -5)):
    """MobileNetV2 classifier graph: 3x3 s2 stem, 17 inverted-residual blocks, 1x1 conv to 1280,
    GlobalAveragePool, Transpose + Flatten, Gemm.  Returns the GraphBuilder (batch 1; the batch is chosen when
    the model is built).  Same node mix as the exported classifier: 52 Conv, 10 Add, GlobalAveragePool,
    Transpose, Flatten, Gemm, plus a RequantizeLinear wherever a residual's exponents differ."""
    net = _Net("mobilenet_v2", seed, e_act, e_w)
    g = net.g
    e0 = int(net.rng.integers(e_act[0], e_act[1] + 1))
    g.add_input("input", np.int8, [1, input_hw, input_hw, 3], e0)
    net.exp["input"], net.shape["input"], net.rms["input"] = e0, [1, input_hw, input_hw, 3], 74.0

    def ch(c):
        return max(8, int(c * width + 4) // 8 * 8)

    x = net.conv("input", ch(32), 3, stride=2, relu=True, name="features.0")
    cin = ch(32)
    block = 1
    residuals = 0
    for t, c, n, s in MBV2_SETTINGS:
        for i in range(n):
            stride = s if i == 0 else 1
            inp = x
            hidden = cin * t
            y = x
            if t != 1:
                y = net.conv(y, hidden, 1, relu=True, name=f"features.{block}.expand")
            y = net.conv(y, hidden, 3, stride=stride, group=hidden, relu=True, name=f"features.{block}.dw")
            use_res = stride == 1 and cin == ch(c)
            # most projections are exported at the residual's exponent; some differ and get a RequantizeLinear
            e_proj = None
            if use_res:
                e_proj = net.exp[inp] if residuals % 3 else None
            y = net.conv(y, ch(c), 1, relu=False, e_out=e_proj, name=f"features.{block}.project")
            if use_res:
                residuals += 1
                y = net.add(inp, y, max(net.exp[inp], net.exp[y]))
            x, cin = y, ch(c)
            block += 1
    x = net.conv(x, 1280, 1, relu=True, name=f"features.{block}")
    n, h, w, c = net.shape[x]
    e_gap = int(net.rng.integers(e_act[0], e_act[1] + 1))
    g.add_node("GlobalAveragePool", "gap", [x], ["gap_out"], quant_type="S8")
    net.tensor("gap_out", (1, 1, 1, c), e_gap, 0.45 * net.rms[x] * 2.0 ** (net.exp[x] - e_gap))
    g.add_node("Transpose", "transpose", ["gap_out"], ["transpose_out"], perm=[0, 3, 1, 2], quant_type="S8")
    net.tensor("transpose_out", (1, c, 1, 1), e_gap, net.rms["gap_out"])
    g.add_node("Flatten", "flatten", ["transpose_out"], ["flatten_out"], axis=1, quant_type="S8")
    net.tensor("flatten_out", (1, c), e_gap, net.rms["gap_out"])
    # classifier: Gemm with weights declared [1,1,K,N], payload [N][K]
    ew = net.rng.integers(e_w[0], e_w[1] + 1, size=num_classes)
    rms_in = max(net.rms["flatten_out"], 1.0)
    need = 28.0 * np.sqrt(3.0) / (rms_in * np.sqrt(c))
    e_out = net.pick_exponent(ew + e_gap, need, (-8, 0))
    shift = e_out - ew - e_gap
    wmax = np.clip(np.round(need * (2.0 ** shift)), 1, 127).astype(np.int64)
    wt = np.stack([net.rng.integers(-wmax[o], wmax[o] + 1, size=c) for o in range(num_classes)]).astype(np.int8)
    g.add_initializer("classifier.weight", wt.reshape(1, 1, c, num_classes), list(ew))
    g.add_initializer("classifier.bias", net.rng.integers(-(1 << 12), (1 << 12) + 1, size=num_classes).astype(np.int32), list(ew + e_gap))
    g.add_node("Gemm", "classifier", ["flatten_out", "classifier.weight", "classifier.bias"], ["logits"], activation="Linear",
               alpha=1.0, beta=1.0, quant_type="S8", transB=0)
    g.add_output("logits", np.int8, [1, num_classes], e_out)
    return g


def inverted_residual_block(seed=4, hw=112, cin=32, expand=6, e_act=(-8, -4), e_w=(-9, -5)):
    """One MobileNetV2 inverted-residual block as its own model: 1x1 expand (ReLU), 3x3 depthwise stride 1 (ReLU),
    1x1 project (linear), residual Add."""
    net = _Net("inverted_residual", seed, e_act, e_w)
    g = net.g
    e0 = -5
    g.add_input("input", np.int8, [1, hw, hw, cin], e0)
    net.exp["input"], net.shape["input"], net.rms["input"] = e0, [1, hw, hw, cin], 74.0
    y = net.conv("input", cin * expand, 1, relu=True, name="expand")
    y = net.conv(y, cin * expand, 3, group=cin * expand, relu=True, name="dw")
    y = net.conv(y, cin, 1, relu=False, e_out=e0, name="project")
    out = net.add("input", y, e0)
    g.outputs.append((out, np.int8, net.shape[out], [e0]))
    g.value_info = [v for v in g.value_info if v[0] != out]
    return g


# ------------------------------------------------------------------------------------------ YOLO11n-style detector
class _DetNet(_Net):
    """Helpers for the detector graph on top of _Net: 8-bit LUT activations, pools, resize, concat / split, the
    shape-only nodes and the attention block's MatMul / Mul / Softmax / QuantizeLinear chain."""

    def swish(self, x):
        """Swish as the exported graphs carry it: a node with a 256-entry int8 table built with the reference's own
        formula, sat(round(x * sigmoid(x) * 2^-e_out)) over the input codes (dl_module_swish.hpp:62-76); the table is
        indexed with (uint8)q ^ 0x80, i.e. entry i belongs to code i - 128."""
        e_in = self.exp[x]
        e_out = e_in
        q = np.arange(-128, 128, dtype=np.float32)
        v = q * np.float32(2.0 ** e_in)
        y = (v / (np.float32(1.0) + np.exp(-v, dtype=np.float32))) * np.float32(2.0 ** -e_out)
        table = np.clip(np.floor(y.astype(np.float64) + 0.5), -128, 127).astype(np.int8)
        node = self.fresh("swish")
        out = node + "_out"
        self.g.add_initializer(node + ".lut", table, [e_out])
        self.g.add_node("Swish", node, [x], [out], quant_type="S8", lut=node + ".lut")
        self.tensor(out, self.shape[x], e_out, 0.6 * self.rms[x])
        return out

    def cbs(self, x, cout, k, stride=1, name=None):
        """Conv (linear) + Swish: the detector's basic unit."""
        return self.swish(self.conv(x, cout, k, stride=stride, relu=False, name=name))

    def maxpool(self, x, k):
        node = self.fresh("maxpool")
        out = node + "_out"
        p = k // 2
        self.g.add_node("MaxPool", node, [x], [out], kernel_shape=[k, k], pads=[p, p, p, p], strides=[1, 1], quant_type="S8")
        self.tensor(out, self.shape[x], self.exp[x], 1.3 * self.rms[x])
        return out

    def resize2(self, x):
        node = self.fresh("resize")
        out = node + "_out"
        n, h, w, c = self.shape[x]
        self.g.add_initializer(node + ".roi", np.zeros(0, dtype=np.float32))
        self.g.add_initializer(node + ".scales", np.array([1.0, 1.0, 2.0, 2.0], dtype=np.float32))  # ONNX order: N, C, H, W
        self.g.add_node("Resize", node, [x, node + ".roi", node + ".scales"], [out], mode="nearest", coordinate_transformation_mode="asymmetric",
                        nearest_mode="floor", quant_type="S8")
        self.tensor(out, (n, 2 * h, 2 * w, c), self.exp[x], self.rms[x])
        return out

    def concat(self, xs, axis=3):
        e = max(self.exp[x] for x in xs)  # a pure copy: every input is brought to one exponent first
        xs = [x if self.exp[x] == e else self.requantize(x, e) for x in xs]
        node = self.fresh("concat")
        out = node + "_out"
        shape = list(self.shape[xs[0]])
        shape[axis] = sum(self.shape[x][axis] for x in xs)
        self.g.add_node("Concat", node, xs, [out], axis=axis, quant_type="S8")
        self.tensor(out, shape, e, float(np.mean([self.rms[x] for x in xs])))
        return out

    def split(self, x, sizes, axis=3):
        node = self.fresh("split")
        outs = [f"{node}_out{i}" for i in range(len(sizes))]
        self.g.add_initializer(node + ".split", np.array(sizes, dtype=np.int64))
        self.g.add_node("Split", node, [x, node + ".split"], outs, axis=axis, num_outputs=len(sizes), quant_type="S8")
        for o, s in zip(outs, sizes):
            shape = list(self.shape[x])
            shape[axis] = s
            self.tensor(o, shape, self.exp[x], self.rms[x])
        return outs

    def reshape(self, x, shape):
        """`shape` starts with 0 (keep the batch extent, whatever it is at run time)."""
        node = self.fresh("reshape")
        out = node + "_out"
        self.g.add_initializer(node + ".shape", np.array(shape, dtype=np.int64))
        self.g.add_node("Reshape", node, [x, node + ".shape"], [out], quant_type="S8")
        self.tensor(out, [self.shape[x][0]] + list(shape[1:]), self.exp[x], self.rms[x])
        return out

    def transpose(self, x, perm):
        node = self.fresh("transpose")
        out = node + "_out"
        self.g.add_node("Transpose", node, [x], [out], perm=list(perm), quant_type="S8")
        self.tensor(out, [self.shape[x][p] for p in perm], self.exp[x], self.rms[x])
        return out

    def matmul(self, a, b, rms_target=28.0):
        """MatMul of two activations; b is declared [.., K, N] and holds its values as [N][K] (see MatMul in the host
        layer: that is how the reference's generic C kernel reads the second operand)."""
        node = self.fresh("matmul")
        out = node + "_out"
        k = self.shape[a][-1]
        acc = self.rms[a] * self.rms[b] * np.sqrt(k)
        e_acc = self.exp[a] + self.exp[b]
        shift = max(1, int(np.round(np.log2(max(acc / rms_target, 1.0)))))
        e_out = e_acc + shift
        self.g.add_node("MatMul", node, [a, b], [out], quant_type="S8", activation="Linear")
        self.tensor(out, list(self.shape[a][:-1]) + [self.shape[b][-1]], e_out, float(min(acc / 2.0 ** shift, 60.0)))
        return out

    def mul_scalar(self, x, code, e_scalar, e_out):
        node = self.fresh("mul")
        out = node + "_out"
        self.g.add_initializer(node + ".scale", np.array([code], dtype=np.int8), [e_scalar])
        self.g.add_node("Mul", node, [x, node + ".scale"], [out], quant_type="S8")
        self.tensor(out, self.shape[x], e_out, self.rms[x] * code * 2.0 ** (self.exp[x] + e_scalar - e_out))
        return out

    def softmax_q(self, x, e_out=-7):
        """Softmax (float32 out, as the reference's int8 Softmax produces) followed by QuantizeLinear back to int8."""
        node = self.fresh("softmax")
        f = node + "_out"
        self.g.add_node("Softmax", node, [x], [f], axis=-1, quant_type="S8")
        self.g.add_value_info(f, np.float32, self.shape[x], None)
        self.exp[f], self.shape[f], self.rms[f] = 0, list(self.shape[x]), 0.1
        qn = self.fresh("quantize")
        out = qn + "_out"
        self.g.add_node("QuantizeLinear", qn, [f], [out], quant_type="S8")
        self.tensor(out, self.shape[x], e_out, 12.0)
        return out

    def c3k2(self, x, cout, hidden):
        """cv1 (1x1) -> split in two -> a bottleneck of two 3x3 convs with a shortcut on the second half -> concat of
        the three pieces -> cv2 (1x1)."""
        y = self.cbs(x, 2 * hidden, 1)
        a, b = self.split(y, [hidden, hidden])
        z = self.cbs(self.cbs(b, hidden, 3), hidden, 3)
        z = self.add(b, z, max(self.exp[b], self.exp[z]))
        return self.cbs(self.concat([a, b, z]), cout, 1)

    def sppf(self, x, cout):
        c = self.shape[x][3] // 2
        y0 = self.cbs(x, c, 1)
        y1 = self.maxpool(y0, 5)
        y2 = self.maxpool(y1, 5)
        y3 = self.maxpool(y2, 5)
        return self.cbs(self.concat([y0, y1, y2, y3]), cout, 1)

    def c2psa(self, x, heads=2, key_dim=32):
        """cv1 -> split -> [attention + feed-forward, both with shortcuts] on one half -> concat -> cv2."""
        n, h, w, c = self.shape[x]
        half = c // 2
        head_dim = half // heads
        y = self.cbs(x, c, 1)
        a, b = self.split(y, [half, half])
        per_head = 2 * key_dim + head_dim
        qkv = self.conv(b, heads * per_head, 1, relu=False)
        t = self.transpose(self.reshape(qkv, [0, h * w, heads, per_head]), (0, 2, 1, 3))      # [N, heads, HW, per_head]
        q, k, v = self.split(t, [key_dim, key_dim, head_dim], axis=3)
        kt = self.reshape(k, [0, heads, key_dim, h * w])          # same bytes: the second operand is read as [N][K]
        logits = self.matmul(q, kt)
        # Scale factor of the logits: random weights give nearly flat logits, and a flat softmax over hundreds of tokens
        # quantises to all zeros.  The scalar (code 91, its exponent chosen here) brings the real-valued spread to
        # about four units, so that the quantised attention has a few large entries per row, as a trained one has.
        real = self.rms[logits] * 2.0 ** self.exp[logits]
        e_s = int(np.round(np.log2(16.0 / max(real * 91.0, 1e-9))))      # the estimate of `real` runs about 4x high
        e_l = int(np.round(np.log2(16.0 / 28.0)))
        logits = self.mul_scalar(logits, 91, e_s, e_l)
        attn = self.softmax_q(logits)
        vt = self.reshape(self.transpose(v, (0, 1, 3, 2)), [0, heads, h * w, head_dim])   # values stored [head_dim][HW]
        o = self.matmul(attn, vt)
        o = self.reshape(self.transpose(o, (0, 2, 1, 3)), [0, h, w, half])
        o = self.conv(o, half, 1, relu=False)
        b = self.add(b, o, max(self.exp[b], self.exp[o]))
        f = self.conv(self.cbs(b, 2 * half, 1), half, 1, relu=False)
        b = self.add(b, f, max(self.exp[b], self.exp[f]))
        return self.cbs(self.concat([a, b]), c, 1)


def yolo11n_style(seed=6, input_hw=640, num_classes=80, e_act=(-8, -4), e_w=(-9, -5)):
    """A YOLO11n-shaped detector: Conv + Swish (8-bit LUT) units, C3k2 blocks (Split / Add / Concat), SPPF (three
    5x5 max-pools), a C2PSA attention block (int8 MatMul for QK^T and for the value product, LUT-exp Softmax followed by
    QuantizeLinear), a top-down / bottom-up neck (nearest Resize x2 + Concat, stride-2 convs) and three detection heads
    with a box and a class branch each.  Channel widths are those of the "n" scale (16 ... 256).  Six outputs."""
    net = _DetNet("yolo11n_style", seed, e_act, e_w)
    g = net.g
    e0 = -7
    g.add_input("input", np.int8, [1, input_hw, input_hw, 3], e0)
    net.exp["input"], net.shape["input"], net.rms["input"] = e0, [1, input_hw, input_hw, 3], 74.0
    x = net.cbs("input", 16, 3, stride=2, name="model.0")
    x = net.cbs(x, 32, 3, stride=2, name="model.1")
    x = net.c3k2(x, 64, 16)
    x = net.cbs(x, 64, 3, stride=2, name="model.3")
    p3 = net.c3k2(x, 128, 32)
    x = net.cbs(p3, 128, 3, stride=2, name="model.5")
    p4 = net.c3k2(x, 128, 64)
    x = net.cbs(p4, 256, 3, stride=2, name="model.7")
    x = net.c3k2(x, 256, 128)
    x = net.sppf(x, 256)
    p5 = net.c2psa(x)
    # neck
    n4 = net.c3k2(net.concat([net.resize2(p5), p4]), 128, 64)
    n3 = net.c3k2(net.concat([net.resize2(n4), p3]), 64, 32)
    m4 = net.c3k2(net.concat([net.cbs(n3, 64, 3, stride=2), n4]), 128, 64)
    m5 = net.c3k2(net.concat([net.cbs(m4, 128, 3, stride=2), p5]), 256, 128)
    # heads
    for i, f in enumerate((n3, m4, m5)):
        box = net.conv(net.cbs(net.cbs(f, 64, 3), 64, 3), 64, 1, relu=False, name=f"head{i}.box")
        cls = net.conv(net.cbs(net.cbs(f, num_classes, 3), num_classes, 3), num_classes, 1, relu=False, name=f"head{i}.cls")
        for t in (box, cls):
            g.outputs.append((t, np.int8, net.shape[t], [net.exp[t]]))
            g.value_info = [v for v in g.value_info if v[0] != t]
    return g


# ------------------------------------------------------------------------------------------------ topology files
_NP_OF_ELEM = {1: np.float32, 3: np.int8, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_}


def from_topology(topo, seed=6, target_rms=28.0):
    """Builds a network from a topology description: the node list, tensor shapes, element types and activation exponents
    of an exported graph, without its weights (a dict as written by tests/golden/make_golden.py::write_topology, e.g. the
    249-node YOLO11n detector at 640x640).  Every Conv gets seeded random int8 weights with per-channel power-of-two
    exponents drawn from about four neighbouring values, amplitudes chosen so that the requantised output uses the int8
    range at the output exponent the graph prescribes, and an int32 bias at exponent e_in + e_w[c]; every Swish node gets
    the 256-entry table of the reference's formula for its input / output exponents (dl_module_swish.hpp:62-76); the
    small structural constants (Reshape / Split / Resize operands, the Mul scalar) are taken from the description.
    Filters are stored in the order of target "c".  Returns the GraphBuilder."""
    rng = np.random.default_rng(seed)
    g = espdl_file.GraphBuilder("from_topology", {"target": "c"})
    info = {v["name"]: v for v in topo["value_info"] + topo["inputs"] + topo["outputs"]}
    params = topo["parameters"]
    exp = {n: (v["exponents"][0] if v["exponents"] else 0) for n, v in info.items()}
    ms = {}      # tensor name -> estimated mean square of the codes
    for v in topo["inputs"]:
        g.add_input(v["name"], _NP_OF_ELEM[v["elem_type"]], v["shape"], exp[v["name"]])
        ms[v["name"]] = 74.0 ** 2
    for v in topo["value_info"]:
        if v["shape"] is None or v["name"] in params:
            continue
        g.add_value_info(v["name"], _NP_OF_ELEM[v["elem_type"]], v["shape"], exp[v["name"]] if v["exponents"] else None)
    for v in topo["outputs"]:
        g.add_output(v["name"], _NP_OF_ELEM[v["elem_type"]], v["shape"], exp[v["name"]])
    done = set()

    def constant(name):
        if name in done or name not in params:
            return
        p = params[name]
        if "values" not in p:
            raise ValueError(f"parameter {name} has no values in the topology description")
        arr = np.array(p["values"], dtype=_NP_OF_ELEM[p["data_type"]]).reshape(p["dims"] if p["dims"] else ())
        g.add_initializer(name, arr, p.get("exponents") or None)
        done.add(name)

    for node in topo["nodes"]:
        op, ins, outs, attrs = node["op_type"], [i for i in node["inputs"]], node["outputs"], dict(node["attrs"])
        x = ins[0]
        if op == "Conv":
            wname = ins[1]
            kh, kw, cin_g, cout_decl = params[wname]["dims"]
            group = int(attrs.get("group", 1))
            depthwise = group != 1
            cout = info[outs[0]]["shape"][-1]
            taps = kh * kw * (1 if depthwise else cin_g)
            e_in, e_out = exp[x], exp[outs[0]]
            need = target_rms * np.sqrt(3.0) / (np.sqrt(ms[x]) * np.sqrt(taps))   # weight amplitude wanted at shift 0
            good = [s for s in range(1, 25) if 3 <= need * 2.0 ** s <= 127] or [max(1, int(np.round(np.log2(20.0 / need))))]
            base = good[len(good) // 2 - (1 if len(good) > 3 else 0)] if len(good) > 1 else good[0]
            choices = [s for s in good if base - 1 <= s <= base + 2] or good
            shift = rng.choice(choices, size=cout)
            ew = e_out - e_in - shift
            wmax = np.clip(np.round(need * 2.0 ** shift), 1, 127).astype(np.int64)
            if depthwise:
                wt = np.stack([rng.integers(-wmax[c], wmax[c] + 1, size=(kh, kw)) for c in range(cout)], axis=-1).astype(np.int8)
            else:
                wt = np.stack([rng.integers(-wmax[c], wmax[c] + 1, size=(kh, kw, cin_g)) for c in range(cout)]).astype(np.int8)
            g.add_initializer(wname, wt.reshape(params[wname]["dims"]), [int(e) for e in ew])
            acc_rms = np.sqrt(ms[x]) * (wmax / np.sqrt(3.0)) * np.sqrt(taps)
            if len(ins) > 2 and ins[2]:
                b = np.round(rng.uniform(-0.5, 0.5, size=cout) * acc_rms).astype(np.int32)
                g.add_initializer(ins[2], b, [int(e) for e in ew + e_in])
            out_rms = np.minimum(acc_rms / 2.0 ** shift, 70.0).mean()
            ms[outs[0]] = float(out_rms ** 2) * (0.5 if attrs.get("activation") == "Relu" else 1.0)
        elif op == "Swish":
            e_in, e_out = exp[x], exp[outs[0]]
            q = np.arange(-128, 128, dtype=np.float32)
            v = q * np.float32(2.0 ** e_in)
            with np.errstate(over="ignore"):   # exp overflows to inf for very negative inputs: x / inf = -0, as in C
                y = (v / (np.float32(1.0) + np.exp(-v, dtype=np.float32))) * np.float32(2.0 ** -e_out)
            table = np.clip(np.floor(y.astype(np.float64) + 0.5), -128, 127).astype(np.int8)
            g.add_initializer(attrs["lut"], table, [e_out])
            sample = np.clip(np.round(rng.standard_normal(4096) * np.sqrt(ms[x])), -128, 127).astype(np.int64)
            ms[outs[0]] = float(np.mean(table[sample + 128].astype(np.float64) ** 2)) + 1.0
        elif "lut" in attrs:
            raise ValueError(f"{op}: only Swish tables can be regenerated")
        else:
            for name in ins[1:]:
                if name:
                    constant(name)
            if op in ("Add", "Sub"):
                ms[outs[0]] = min(ms[ins[0]] + ms[ins[1]], 100.0 ** 2)
            elif op == "Concat":
                ms[outs[0]] = float(np.mean([ms[i] for i in ins]))
            elif op in ("RequantizeLinear",):
                ms[outs[0]] = min(ms[x] * 4.0 ** (exp[x] - exp[outs[0]]), 100.0 ** 2)
            elif op == "MaxPool":
                ms[outs[0]] = ms[x] * 1.7
            elif op == "MatMul":
                k = info[x]["shape"][-1]
                shift = exp[outs[0]] - exp[ins[0]] - exp[ins[1]]
                ms[outs[0]] = float(np.clip(ms[ins[0]] * ms[ins[1]] * k / 4.0 ** shift, 1.0, 100.0 ** 2))
            elif op == "Mul":
                c = params[ins[1]]
                scale = c["values"][0] * 2.0 ** (c["exponents"][0] if c.get("exponents") else 0)
                ms[outs[0]] = float(np.clip(ms[x] * (scale * 2.0 ** (exp[x] - exp[outs[0]])) ** 2, 1.0, 100.0 ** 2))
            elif op == "Softmax":
                ms[outs[0]] = 1.0
            elif op == "QuantizeLinear":
                n_tok = info[x]["shape"][-1]
                ms[outs[0]] = float(np.clip((2.0 ** -exp[outs[0]] / n_tok) ** 2 * 4.0, 1.0, 100.0 ** 2))
            else:   # Split, Reshape, Transpose, Resize, Slice, ...: the values move, their statistics stay
                for o in outs:
                    ms[o] = ms[x]
        for o in outs:
            ms.setdefault(o, ms.get(x, 400.0))
        g.add_node(op, node["name"], ins, outs, **attrs)
    return g


def yolo11n_640(topology_path, seed=6):
    """The YOLO11n detector at 640x640 as the reference ships it (249 nodes: 87 Conv, 77 Swish tables, 19 RequantizeLinear,
    17 Concat, 14 Add, 10 Split, 8 Transpose, 7 Reshape, 3 MaxPool, 2 MatMul, 2 Resize, Mul, Softmax, QuantizeLinear) with
    seeded random weights; `topology_path` is the JSON description of that graph."""
    import json
    with open(topology_path) as f:
        return from_topology(json.load(f), seed=seed)
