"""Synthetic topologies of the benchmark configurations, as engine-independent
primitive lists (constants are numpy arrays until `realise` uploads them).

ResNet-50 v1, int8: random-init s8 weights uniform in [-127, 127], i32 biases
uniform in [-4096, 4096], per-output-channel f32 scales uniform in
[2^-14, 2^-10], u8 224x224x3 inputs uniform in [0, 255]; bottleneck 1x1 / 3x3 /
1x1 convolutions with the residual sum + ReLU fused into the expanding 1x1
(fused_conv_eltwise), 3x3/2 max pooling, global average pooling, a 2048 -> 1000
fully_connected and softmax.  No trained weights or dataset images are involved.
"""
import numpy as np

from . import cldnn as cl


class Spec:
    """A topology before upload: primitives in order, numpy constants by id."""

    def __init__(self):
        self.prims = []
        self.consts = {}
        self.input_id = None
        self.input_layout = None
        self.outputs = []

    def const(self, id, arr):
        self.consts[id] = arr
        self.prims.append(cl.primitive("data", id, array=arr))
        return id

    def add(self, prim):
        self.prims.append(prim)
        return prim.id

    def realise(self, eng):
        """Upload the constants and return (topology, memories kept alive)."""
        topo, keep = cl.topology(), []
        for p in self.prims:
            if p.kind == "data":
                m = cl.memory.from_numpy(eng, p.args["array"])
                keep.append(m)
                topo.add(cl.data(p.id, m))
            else:
                topo.add(p)
        return topo, keep


def _conv_consts(spec, rng, name, cin, cout, k, scale_lo, scale_hi, w_range=127, float_bias=False):
    w = rng.integers(-w_range, w_range + 1, size=(cout, cin, k, k), dtype=np.int64).astype(np.int8)
    spec.const(name + "_w", w)
    if float_bias:
        spec.const(name + "_b", rng.uniform(-8.0, 8.0, size=cout).astype(np.float32))
    else:
        spec.const(name + "_b", rng.integers(-4096, 4097, size=cout, dtype=np.int64).astype(np.int32))
    spec.const(name + "_q", rng.uniform(scale_lo, scale_hi, size=cout).astype(np.float32))


def resnet50_int8(batch, seed=2019, image=224, scale_lo=2.0 ** -14, scale_hi=2.0 ** -10, classes=1000, widths=(64, 128, 256, 512),
                  blocks=(3, 4, 6, 3), stem=64):
    rng = np.random.default_rng(seed)
    s = Spec()
    dt = cl.data_types
    s.input_id = "input"
    s.input_layout = cl.layout(dt.u8, cl.format.bfyx, cl.tensor(batch, 3, image, image))
    s.add(cl.input_layout("input", s.input_layout))
    _conv_consts(s, rng, "conv1", 3, stem, 7, scale_lo, scale_hi)
    s.add(cl.convolution("conv1", "input", "conv1_w", "conv1_b", "conv1_q", output_data_type=dt.u8, stride=(2, 2), input_offset=(-3, -3),
                         with_activation=True))
    s.add(cl.pooling("pool1", "conv1", cl.pooling_mode.max, size=(3, 3), stride=(2, 2)))
    x, cin = "pool1", stem
    n_stage = len(widths)
    for si, (w, nb) in enumerate(zip(widths, blocks)):
        for b in range(nb):
            name = "s%d_b%d" % (si + 2, b)
            stride = 2 if (b == 0 and si > 0) else 1
            last = si == n_stage - 1 and b == nb - 1
            _conv_consts(s, rng, name + "_a", cin, w, 1, scale_lo, scale_hi)
            s.add(cl.convolution(name + "_a", x, name + "_a_w", name + "_a_b", name + "_a_q", output_data_type=dt.u8, stride=(stride, stride),
                                 with_activation=True))
            _conv_consts(s, rng, name + "_b", w, w, 3, scale_lo, scale_hi)
            s.add(cl.convolution(name + "_b", name + "_a", name + "_b_w", name + "_b_b", name + "_b_q", output_data_type=dt.u8,
                                 input_offset=(-1, -1), with_activation=True))
            if b == 0:
                _conv_consts(s, rng, name + "_proj", cin, 4 * w, 1, scale_lo, scale_hi)
                s.add(cl.convolution(name + "_proj", x, name + "_proj_w", name + "_proj_b", name + "_proj_q", output_data_type=dt.i8,
                                     stride=(stride, stride)))
                shortcut = name + "_proj"
            else:
                shortcut = x
            _conv_consts(s, rng, name + "_c", w, 4 * w, 1, scale_lo, scale_hi)
            s.add(cl.fused_conv_eltwise(name + "_c", name + "_b", shortcut, name + "_c_w", name + "_c_b", name + "_c_q",
                                        eltw_activation=True, output_data_type=dt.i8 if last else dt.u8))
            x, cin = name + "_c", 4 * w
    s.add(cl.pooling("pool5", x, cl.pooling_mode.average, global_pooling=True))
    rngf = np.random.default_rng(seed + 1)
    s.const("fc_w", rngf.integers(-127, 128, size=(classes, cin, 1, 1), dtype=np.int64).astype(np.int8))
    s.const("fc_b", rngf.uniform(-8.0, 8.0, size=classes).astype(np.float32))
    s.const("fc_q", rngf.uniform(scale_lo, scale_hi, size=classes).astype(np.float32))
    s.const("fc_c", rngf.uniform(0.03, 0.06, size=classes).astype(np.float32))
    s.add(cl.fully_connected("fc", "pool5", "fc_w", "fc_b", "fc_q", "fc_c"))
    s.add(cl.reorder("fc_f32", "fc", cl.format.bfyx, dt.f32))
    s.add(cl.softmax("prob", "fc_f32"))
    s.outputs = ["prob", "fc"]
    return s


# MobileNet-v2: (expansion, output features, repeats, stride of the first repeat)
MOBILENET_V2_BLOCKS = ((1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1))


def mobilenet_v2_int8(batch, seed=2, image=224, blocks=MOBILENET_V2_BLOCKS, stem=32, head=1280, classes=1000):
    """int8 MobileNet-v2: 3x3/2 stem, inverted-residual blocks (1x1 expansion, 3x3 depthwise, linear 1x1 projection, residual
    sum where the shapes allow), 1x1 head, global average pooling, fully_connected, softmax.  s8 weights with per-feature
    scales sized so the dequantised values spread over ReLU6's range; ReLU6 is an `activation` primitive (clamp 0..6) after
    each convolution, which the optimising build folds in front of the requantisation (O_QF = 255 / 6 onto u8), as the
    reference's activation fusing does."""
    rng = np.random.default_rng(seed)
    s = Spec()
    dt = cl.data_types
    s.input_id = "input"
    s.input_layout = cl.layout(dt.u8, cl.format.bfyx, cl.tensor(batch, 3, image, image))
    s.add(cl.input_layout("input", s.input_layout))

    def conv(name, x, cin, cout, k, stride, groups=1, relu6=True, in_scale=42.5):
        fan = (cin // groups) * k * k
        s.const(name + "_w", rng.integers(-127, 128, size=(cout, cin // groups, k, k), dtype=np.int64).astype(np.int8))
        s.const(name + "_b", rng.integers(-2048, 2049, size=cout, dtype=np.int64).astype(np.int32))
        # accumulators spread over ~ sqrt(fan) * 73 * (input scale): bring them to a few units
        sigma = np.sqrt(fan) * 73.0 * (74.0 if in_scale is None else 60.0)
        s.const(name + "_q", (rng.uniform(1.0, 3.0, size=cout) / sigma).astype(np.float32))
        pad = -(k // 2)
        s.add(cl.convolution(name, x, name + "_w", name + "_b", name + "_q", output_data_type=dt.u8 if relu6 else dt.i8, stride=(stride, stride),
                             input_offset=(pad, pad), groups=groups, output_quantization_factor=42.5 if relu6 else 16.0))
        if relu6:
            s.add(cl.activation(name + "_relu6", name, cl.activation_func.clamp, 0.0, 6.0))
            return name + "_relu6"
        return name

    x = conv("stem", "input", 3, stem, 3, 2, in_scale=None)
    cin = stem
    for bi, (t, c, n, st) in enumerate(blocks):
        for r in range(n):
            name = "b%d_%d" % (bi, r)
            stride = st if r == 0 else 1
            inp = x
            h = cin * t
            y = conv(name + "_exp", x, cin, h, 1, 1) if t != 1 else x
            y = conv(name + "_dw", y, h, h, 3, stride, groups=h)
            y = conv(name + "_proj", y, h, c, 1, 1, relu6=False)
            if stride == 1 and cin == c and inp != "stem_relu6" and not inp.endswith("_relu6"):
                s.add(cl.eltwise(name + "_sum", y, inp, cl.eltwise_mode.sum))
                y = name + "_sum"
            x, cin = y, c
    x = conv("head", x, cin, head, 1, 1)
    s.add(cl.pooling("pool", x, cl.pooling_mode.average, global_pooling=True))
    s.const("fc_w", rng.integers(-127, 128, size=(classes, head, 1, 1), dtype=np.int64).astype(np.int8))
    s.const("fc_b", rng.uniform(-8.0, 8.0, size=classes).astype(np.float32))
    s.const("fc_q", (rng.uniform(1.0, 3.0, size=classes) / (np.sqrt(head) * 73.0 * 60.0)).astype(np.float32))
    s.const("fc_c", rng.uniform(8.0, 16.0, size=classes).astype(np.float32))
    s.add(cl.fully_connected("fc", "pool", "fc_w", "fc_b", "fc_q", "fc_c"))
    s.add(cl.reorder("fc_f32", "fc", cl.format.bfyx, dt.f32))
    s.add(cl.softmax("prob", "fc_f32"))
    s.outputs = ["prob", "fc"]
    return s


# VGG16 (configuration D): 13 3x3 pad-1 convolutions in five stages, 2x2 max pooling after each stage.
VGG16_STAGES = ((64, 2), (128, 2), (256, 3), (512, 3), (512, 3))


def vgg16_fp16(batch, seed=16, image=224, stages=VGG16_STAGES, classes=1000, fc_width=4096):
    """fp16 VGG16: weights N(0, sqrt(2 / fan_in)), inputs N(0, 1) supplied by the caller; convolution + ReLU, max pooling,
    three fully_connected layers and softmax."""
    rng = np.random.default_rng(seed)
    s = Spec()
    dt = cl.data_types
    s.input_id = "input"
    s.input_layout = cl.layout(dt.f16, cl.format.bfyx, cl.tensor(batch, 3, image, image))
    s.add(cl.input_layout("input", s.input_layout))
    x, cin, size = "input", 3, image
    for si, (w, n) in enumerate(stages):
        for li in range(n):
            name = "conv%d_%d" % (si + 1, li + 1)
            s.const(name + "_w", (rng.standard_normal((w, cin, 3, 3)) * np.sqrt(2.0 / (cin * 9))).astype(np.float16))
            s.const(name + "_b", (rng.standard_normal(w) * 0.05).astype(np.float16))
            s.add(cl.convolution(name, x, name + "_w", name + "_b", input_offset=(-1, -1), with_activation=True))
            x, cin = name, w
        s.add(cl.pooling("pool%d" % (si + 1), x, cl.pooling_mode.max, size=(2, 2), stride=(2, 2)))
        x, size = "pool%d" % (si + 1), size // 2
    fan = cin * size * size
    for i, (wout, act) in enumerate(((fc_width, True), (fc_width, True), (classes, False))):
        name = "fc%d" % (i + 6)
        shape = (wout, cin, size, size) if i == 0 else (wout, fan, 1, 1)
        s.const(name + "_w", (rng.standard_normal(shape) * np.sqrt(2.0 / fan)).astype(np.float16))
        s.const(name + "_b", (rng.standard_normal(wout) * 0.05).astype(np.float16))
        s.add(cl.fully_connected(name, x, name + "_w", name + "_b", with_activation=act))
        x, fan = name, wout
    s.add(cl.softmax("prob", x))
    s.outputs = ["prob", x]
    return s


def vgg16_conv_layers(image=224, stages=VGG16_STAGES):
    """(name, input features, output features, map size) of the 13 convolutions: the per-layer sweep."""
    out, cin, size = [], 3, image
    for si, (w, n) in enumerate(stages):
        for li in range(n):
            out.append(("conv%d_%d" % (si + 1, li + 1), cin, w, size))
            cin = w
        size //= 2
    return out


# AlexNet (one-tower weights with the original two-group layers): (features, filter, stride, pad, groups, lrn + pool after)
ALEXNET_CONVS = ((96, 11, 4, 0, 1, True), (256, 5, 1, 2, 2, True), (384, 3, 1, 1, 1, False), (384, 3, 1, 1, 2, False), (256, 3, 1, 1, 2, False))


def alexnet_fp16(batch, seed=12, image=227, convs=ALEXNET_CONVS, classes=1000, fc_width=4096, w_std=0.01):
    """fp16 AlexNet: 11x11 stride-4 first convolution, grouped conv2 / conv4 / conv5, LRN (5, k=1, alpha=1e-4, beta=0.75) and
    3x3 stride-2 max pooling after conv1 and conv2, max pooling after conv5, three fully_connected layers, softmax.
    Weights N(0, w_std), small positive biases so the ReLUs stay alive, inputs N(0, 1) supplied by the caller."""
    rng = np.random.default_rng(seed)
    s = Spec()
    dt = cl.data_types
    s.input_id = "input"
    s.input_layout = cl.layout(dt.f16, cl.format.bfyx, cl.tensor(batch, 3, image, image))
    s.add(cl.input_layout("input", s.input_layout))
    x, cin, size = "input", 3, image
    for i, (w, k, stride, pad, groups, norm) in enumerate(convs):
        name = "conv%d" % (i + 1)
        s.const(name + "_w", (rng.standard_normal((w, cin // groups, k, k)) * w_std).astype(np.float16))
        s.const(name + "_b", (rng.standard_normal(w) * 0.02 + 0.1).astype(np.float16))
        s.add(cl.convolution(name, x, name + "_w", name + "_b", stride=(stride, stride), input_offset=(-pad, -pad), with_activation=True, groups=groups))
        x, cin, size = name, w, (size + 2 * pad - k) // stride + 1
        if norm:
            s.add(cl.lrn("norm%d" % (i + 1), x, size=5, k=1.0, alpha=1e-4, beta=0.75))
            x = "norm%d" % (i + 1)
        if norm or i == len(convs) - 1:
            s.add(cl.pooling("pool%d" % (i + 1), x, cl.pooling_mode.max, size=(3, 3), stride=(2, 2)))
            x, size = "pool%d" % (i + 1), (size - 3) // 2 + 1
    fan = cin * size * size
    for i, (wout, act) in enumerate(((fc_width, True), (fc_width, True), (classes, False))):
        name = "fc%d" % (i + 6)
        shape = (wout, cin, size, size) if i == 0 else (wout, fan, 1, 1)
        s.const(name + "_w", (rng.standard_normal(shape) * w_std).astype(np.float16))
        s.const(name + "_b", (rng.standard_normal(wout) * 0.02 + 0.1).astype(np.float16))
        s.add(cl.fully_connected(name, x, name + "_w", name + "_b", with_activation=act))
        x, fan = name, wout
    s.add(cl.softmax("prob", x))
    s.outputs = ["prob", x]
    return s


def alexnet_int8(batch, seed=13, image=227, convs=ALEXNET_CONVS, classes=1000, fc_width=4096):
    """int8 AlexNet: the fp16 topology without its LRN layers (the reference's LRN kernels take fp16 / fp32 only): u8 image,
    11x11 stride-4 first convolution, two-group conv2 / conv4 / conv5, 3x3 stride-2 max pooling, three quantised
    fully_connected layers (f32 bias after the dequantisation, per-output calibration), softmax.  s8 weights uniform in
    [-127, 127], i32 convolution biases, per-feature scales sized so the dequantised values spread over a few units, ReLU,
    then a uniform requantisation onto u8."""
    rng = np.random.default_rng(seed)
    s = Spec()
    dt = cl.data_types
    s.input_id = "input"
    s.input_layout = cl.layout(dt.u8, cl.format.bfyx, cl.tensor(batch, 3, image, image))
    s.add(cl.input_layout("input", s.input_layout))
    x, cin, size = "input", 3, image
    in_sigma = 74.0                                                    # a u8 image; later layers see requantised ReLU outputs
    for i, (w, k, stride, pad, groups, pool) in enumerate(convs):
        name = "conv%d" % (i + 1)
        fan = (cin // groups) * k * k
        s.const(name + "_w", rng.integers(-127, 128, size=(w, cin // groups, k, k), dtype=np.int64).astype(np.int8))
        s.const(name + "_b", rng.integers(-2048, 2049, size=w, dtype=np.int64).astype(np.int32))
        s.const(name + "_q", (rng.uniform(1.0, 3.0, size=w) / (np.sqrt(fan) * 73.0 * in_sigma)).astype(np.float32))
        s.add(cl.convolution(name, x, name + "_w", name + "_b", name + "_q", output_data_type=dt.u8, stride=(stride, stride), input_offset=(-pad, -pad),
                             with_activation=True, groups=groups, output_quantization_factor=24.0))
        x, cin, size, in_sigma = name, w, (size + 2 * pad - k) // stride + 1, 40.0
        if pool or i == len(convs) - 1:
            s.add(cl.pooling("pool%d" % (i + 1), x, cl.pooling_mode.max, size=(3, 3), stride=(2, 2)))
            x, size = "pool%d" % (i + 1), (size - 3) // 2 + 1
    fan = cin * size * size
    for i, (wout, act) in enumerate(((fc_width, True), (fc_width, True), (classes, False))):
        name = "fc%d" % (i + 6)
        shape = (wout, cin, size, size) if i == 0 else (wout, fan, 1, 1)
        s.const(name + "_w", rng.integers(-127, 128, size=shape, dtype=np.int64).astype(np.int8))
        s.const(name + "_b", rng.uniform(-1.0, 1.0, size=wout).astype(np.float32))
        s.const(name + "_q", (rng.uniform(1.0, 3.0, size=wout) / (np.sqrt(fan) * 73.0 * 40.0)).astype(np.float32))
        s.const(name + "_c", rng.uniform(6.0, 12.0, size=wout).astype(np.float32))
        s.add(cl.fully_connected(name, x, name + "_w", name + "_b", name + "_q", name + "_c", with_activation=act))
        x, fan = name, wout
    s.add(cl.reorder("fc8_f32", x, cl.format.bfyx, dt.f32))
    s.add(cl.softmax("prob", "fc8_f32"))
    s.outputs = ["prob", x]
    return s


def conv_ops(spec):
    """Multiply-add operations x2 of every convolution / fully_connected of a spec, per image (padding taps counted)."""
    shapes, total = {}, 0
    lay = spec.input_layout
    shapes[spec.input_id] = (lay.size.feature, lay.size.y, lay.size.x)
    per_layer = []
    for p in spec.prims:
        a = p.args
        if p.kind == "data" or p.kind == "input_layout":
            continue
        c, h, w = shapes[a["input"]]
        if p.kind in ("convolution", "fused_conv_eltwise"):
            wt = spec.consts[a["weights"]]
            k, _, kh, kw = wt.shape
            ho = (h - 2 * a["input_offset"][1] - ((kh - 1) * a["dilation"][1] + 1)) // a["stride"][1] + 1
            wo = (w - 2 * a["input_offset"][0] - ((kw - 1) * a["dilation"][0] + 1)) // a["stride"][0] + 1
            ops = 2 * k * ho * wo * (c // a.get("groups", 1)) * kh * kw
            shapes[p.id] = (k, ho, wo)
            per_layer.append((p.id, p.kind, ops, (c, k, h, kh, a["stride"][0])))
            total += ops
        elif p.kind == "fully_connected":
            wt = spec.consts[a["weights"]]
            ops = 2 * wt.shape[0] * c * h * w
            shapes[p.id] = (wt.shape[0], 1, 1)
            per_layer.append((p.id, p.kind, ops, (c, wt.shape[0], 1, 1, 1)))
            total += ops
        elif p.kind == "pooling":
            if a["global_pooling"]:
                shapes[p.id] = (c, 1, 1)
            else:
                from . import cldnn as _c  # noqa: F401
                ext_y = max(a["size"][1], a["stride"][1]); ext_x = max(a["size"][0], a["stride"][0])
                ho = min((h - 2 * a["input_offset"][1] - ext_y + a["stride"][1] - 1) // a["stride"][1] + 1, (h - a["input_offset"][1] - 1) // a["stride"][1] + 1)
                wo = min((w - 2 * a["input_offset"][0] - ext_x + a["stride"][0] - 1) // a["stride"][0] + 1, (w - a["input_offset"][0] - 1) // a["stride"][0] + 1)
                shapes[p.id] = (c, ho, wo)
        else:
            shapes[p.id] = (c, h, w)
    return total, per_layer


def primitive_inputs(spec):
    """{primitive id: [ids of its activation inputs]} of a spec, in the spec's own (unfused) terms."""
    out = {}
    for p in spec.prims:
        if p.kind in ("data", "input_layout"):
            continue
        out[p.id] = [p.args[k] for k in ("input", "input2") if k in p.args and p.args[k]]
    return out


def weight_bytes(spec):
    """{primitive id: bytes of its constants (weights, bias, scales)} as the caller provides them."""
    out = {}
    for p in spec.prims:
        if p.kind in ("data", "input_layout"):
            continue
        n = 0
        for k, v in p.args.items():
            if isinstance(v, str) and v in spec.consts and k not in ("input", "input2"):
                n += spec.consts[v].nbytes
        out[p.id] = n
    return out
