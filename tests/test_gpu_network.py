"""Whole topologies through the host layer (topology -> program -> network) on the GPU, against the same topology run
primitive by primitive on the CPU oracle.  Integer outputs must be bit-exact."""
import numpy as np
import pytest

import oracle_net
from cldnn_b200 import abi, topologies
from cldnn_b200 import cldnn as cl

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    return cl.engine(0)


def _run(eng, spec, x, **opts):
    topo, keep = spec.realise(eng)
    net = cl.network(eng, topo, cl.build_options(outputs=spec.outputs, **opts))
    net.set_input_data(spec.input_id, cl.memory.from_numpy(eng, x))
    net.execute()
    return net, {o: net.get_output(o).to_numpy() for o in spec.outputs}


def _input(spec, seed=99):
    lay = spec.input_layout
    return np.random.default_rng(seed).integers(0, 256, size=(lay.size.batch, lay.size.feature, lay.size.y, lay.size.x)).astype(np.uint8)


def _compare(spec, want, got):
    for k in spec.outputs:
        if want[k].dtype.kind in "iu":
            assert np.array_equal(want[k], got[k]), "%s: %d mismatches" % (k, int((want[k] != got[k]).sum()))
        else:
            np.testing.assert_allclose(got[k], want[k], rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("optimize", [False, True])
def test_small_residual_network_bit_exact(eng, optimize):
    spec = topologies.resnet50_int8(3, seed=5, image=64, widths=(32, 64), blocks=(2, 2), stem=32, classes=40)
    x = _input(spec)
    stats = {}
    want = oracle_net.run(spec, {spec.input_id: x}, stats=stats)
    assert stats["fc:out_of_range"] == 0
    net, got = _run(eng, spec, x, optimize_data=optimize)
    _compare(spec, want, got)
    info = net.primitives_info()
    convs = [r for r in info if r["type"] in ("convolution", "fused_conv_eltwise", "fully_connected")]
    if optimize:
        # the layout optimiser moved the 8-bit path to byxf_af32 and every convolution onto the tensor-core kernel
        assert all(r["kernel"] in ("conv_i8_tc", "conv_i8_first") and r["format"] == "byxf_af32" for r in convs)
        assert convs[0]["kernel"] == "conv_i8_first"          # the image is consumed in its planar layout, no input reorder
        assert any(r["kernel"] == "pooling_i8_byxf" for r in info)
        # prepare_conv_eltw_read_write_opt: an identity-shortcut block writes its result over the shortcut's buffer; a projection
        # shortcut (s8 against the u8 result) or the last block (s8 result over a u8 shortcut) cannot
        assert {r["id"] for r in info if r["in_place"]} == {"s2_b1_c"}
    else:
        # optimize_data(false): reference-order kernels in the caller's layout, like the reference's own tests
        assert all(r["kernel"] in ("conv_ref", "fc_ref") and r["format"] == "bfyx" for r in convs)
    # repeated execution replays the captured graph and gives the same bits
    net.execute()
    assert np.array_equal(net.get_output("fc").to_numpy(), got["fc"])


def test_resnet50_int8_batch2_bit_exact(eng):
    """The headline workload: ResNet-50 v1 int8, full size (224x224), here at batch 2 so the CPU oracle finishes in seconds."""
    spec = topologies.resnet50_int8(2)
    x = _input(spec, seed=7)
    stats = {}
    want = oracle_net.run(spec, {spec.input_id: x}, stats=stats)
    assert stats["fc:out_of_range"] == 0
    layers = [v for v in stats.values() if isinstance(v, dict)]
    assert np.mean([v["saturated"] for v in layers]) < 0.2            # the comparison is not on saturated constants
    net, got = _run(eng, spec, x, optimize_data=True)
    _compare(spec, want, got)
    assert (want["fc"] != 0).mean() > 0.5
    assert net.stats()["launches_per_execute"] >= 53


def test_batch_independence_of_the_sharded_path(eng):
    """Images are independent units: running a batch in two halves gives the bits of the whole batch (the property the
    multi-GPU data-parallel split relies on)."""
    spec4 = topologies.resnet50_int8(4, seed=3, image=64, widths=(32, 64), blocks=(1, 1), stem=32, classes=24)
    spec2 = topologies.resnet50_int8(2, seed=3, image=64, widths=(32, 64), blocks=(1, 1), stem=32, classes=24)
    x = _input(spec4, seed=1)
    _, whole = _run(eng, spec4, x, optimize_data=True)
    _, lo = _run(eng, spec2, x[:2], optimize_data=True)
    _, hi = _run(eng, spec2, x[2:], optimize_data=True)
    assert np.array_equal(whole["fc"], np.concatenate([lo["fc"], hi["fc"]]))


def test_conv_quantized_kat_through_the_topology_api(eng):
    """ConvQuantizedTest_u8_to_u8 of the reference (tests/test_cases/convolution_gpu_test.cpp:4133-4166), written the way
    the reference writes it: input_layout + data + convolution, optimize_data(false), exact integer equality."""
    from golden import kat_conv_quantized
    feats = kat_conv_quantized.CASES["u8_to_u8"]["features"]
    n = len(feats)
    inp = np.array([f[0] for f in feats], dtype=np.uint8).reshape(1, n, 1, 4)
    w = np.zeros((n, n, 1, 3), dtype=np.int8)
    for i, f in enumerate(feats):
        w[i, i, 0, :] = f[1]
    input_mem = cl.memory.from_numpy(eng, inp)
    topo = cl.topology(
        cl.input_layout("input", input_mem.get_layout()),
        cl.data("weights", cl.memory.from_numpy(eng, w)),
        cl.data("biases", cl.memory.from_numpy(eng, np.array([f[2] for f in feats], dtype=np.int32))),
        cl.data("quantization", cl.memory.from_numpy(eng, np.array([f[3] for f in feats], dtype=np.float32))),
        cl.convolution("conv", "input", "weights", "biases", "quantization", output_data_type=cl.data_types.u8, with_activation=True))
    net = cl.network(eng, topo, cl.build_options(optimize_data=False))
    net.set_input_data("input", input_mem)
    net.execute()
    out = net.get_output("conv")
    lay = out.get_layout()
    assert (lay.format, lay.size.y, lay.size.x, lay.size.feature, lay.size.batch) == (cl.format.bfyx, 1, 2, n, 1)
    expected = np.clip(np.array([f[4] for f in feats]), 0, 255)
    assert np.array_equal(out.to_numpy()[0, :, 0, :].astype(np.int64), expected)


def test_activation_and_eltwise_fusing_passes(eng):
    """conv -> eltwise(sum) -> relu collapses into one fused_conv_eltwise under optimize_data (prepare_primitive_fusing +
    prepare_conv_eltw_fusing) and computes what the unfused graph computes when nothing saturates."""
    rng = np.random.default_rng(0)
    x = rng.integers(0, 8, size=(2, 32, 6, 6)).astype(np.uint8)
    w = rng.integers(-3, 4, size=(32, 32, 3, 3)).astype(np.int8)
    other = rng.integers(0, 16, size=(2, 32, 6, 6)).astype(np.uint8)
    def build(e):
        xm, om = cl.memory.from_numpy(e, x), cl.memory.from_numpy(e, other)
        topo = cl.topology(
            cl.input_layout("input", xm.get_layout()), cl.input_layout("other", om.get_layout()),
            cl.data("w", cl.memory.from_numpy(e, w)), cl.data("q", cl.memory.from_numpy(e, np.full(32, 0.25, dtype=np.float32))),
            cl.convolution("conv", "input", "w", "", "q", output_data_type=cl.data_types.i8, input_offset=(-1, -1)),
            cl.eltwise("sum", "conv", "other", cl.eltwise_mode.sum, quantized=True),
            cl.activation("relu", "sum", cl.activation_func.relu))
        return topo, xm, om
    outs = {}
    for optimize in (False, True):
        topo, xm, om = build(eng)
        net = cl.network(eng, topo, cl.build_options(optimize_data=optimize))
        net.set_input_data("input", xm); net.set_input_data("other", om)
        net.execute()
        outs[optimize] = net.get_output("relu").to_numpy()
        kinds = [r["type"] for r in net.primitives_info() if r["kernel"]]
        if optimize:
            assert "fused_conv_eltwise" in kinds and "eltwise" not in kinds and "activation" not in kinds
        else:
            assert kinds.count("convolution") == 1 and "eltwise" in kinds and "activation" in kinds
    assert np.array_equal(outs[False], outs[True])


def test_errors_surface_as_status_codes(eng):
    xm = cl.memory.from_numpy(eng, np.zeros((1, 8, 4, 4), dtype=np.uint8))
    bad = cl.topology(cl.input_layout("input", xm.get_layout()),
                      cl.data("w", cl.memory.from_numpy(eng, np.zeros((8, 4, 3, 3), dtype=np.int8))),      # 4 input features, tensor has 8
                      cl.convolution("conv", "input", "w"))
    with pytest.raises(cl.error) as e:
        cl.network(eng, bad)
    assert e.value.status == abi.DIMENSION_MISMATCH
    with pytest.raises(cl.error) as e:
        cl.network(eng, cl.topology(cl.input_layout("input", xm.get_layout()), cl.softmax("s", "nowhere")))
    assert e.value.status == abi.INVALID_ARG


@pytest.mark.parametrize("optimize", [False, True])
def test_small_vgg_fp16_network(eng, optimize):
    """fp16 VGG-style network (convolution + ReLU, max pooling, fully_connected, softmax) against the oracle, within the
    fp16 tolerance of 1e-2 relative to each output's scale; with optimize_data every convolution runs on conv_f16_tc."""
    spec = topologies.vgg16_fp16(2, seed=3, image=32, stages=((32, 1), (32, 2), (64, 1)), classes=10, fc_width=64)
    lay = spec.input_layout
    x = np.random.default_rng(7).standard_normal((lay.size.batch, lay.size.feature, lay.size.y, lay.size.x)).astype(np.float16)
    want = oracle_net.run(spec, {spec.input_id: x})
    net, got = _run(eng, spec, x, optimize_data=optimize)
    for k in spec.outputs:
        w, g = want[k].astype(np.float32), got[k].astype(np.float32)
        scale = float(np.abs(w).max())
        assert np.abs(g - w).max() <= 1e-2 * scale, "%s: max abs error %.4g on scale %.4g" % (k, float(np.abs(g - w).max()), scale)
    convs = [r for r in net.primitives_info() if r["type"] == "convolution"]
    assert len(convs) == 4
    fcs = [r for r in net.primitives_info() if r["type"] == "fully_connected"]
    if optimize:
        # the image layer is gathered in place from the planar input, the rest (inner products included) are tensor-core GEMMs
        assert [r["kernel"] for r in convs] == ["conv_first_tc"] + ["conv_f16_tc"] * 3, [r["kernel"] for r in convs]
        assert all(r["kernel"] == "conv_f16_tc" for r in fcs), [r["kernel"] for r in fcs]
    else:
        assert all(r["kernel"] == "conv_ref" for r in convs)
        assert all(r["kernel"] == "fc_ref" for r in fcs)


@pytest.mark.parametrize("optimize", [False, True])
def test_small_alexnet_fp16_network(eng, optimize):
    """fp16 AlexNet-style network: 11x11 stride-4 first convolution, two-group convolutions, LRN, 3x3 stride-2 max
    pooling, three fully_connected layers (the first over a 3x3 map), softmax; 1e-2 relative to each output's scale."""
    spec = topologies.alexnet_fp16(3, seed=5, image=99, convs=((32, 11, 4, 0, 1, True), (64, 5, 1, 2, 2, True), (96, 3, 1, 1, 1, False),
                                                                (96, 3, 1, 1, 2, False), (64, 3, 1, 1, 2, False)),
                                   classes=10, fc_width=64, w_std=0.05)
    lay = spec.input_layout
    x = np.random.default_rng(8).standard_normal((lay.size.batch, lay.size.feature, lay.size.y, lay.size.x)).astype(np.float16)
    want = oracle_net.run(spec, {spec.input_id: x})
    net, got = _run(eng, spec, x, optimize_data=optimize)
    for k in spec.outputs:
        w, g = want[k].astype(np.float32), got[k].astype(np.float32)
        scale = float(np.abs(w).max())
        assert scale > 0 and np.abs(g - w).max() <= 1e-2 * scale, "%s: max abs error %.4g on scale %.4g" % (k, float(np.abs(g - w).max()), scale)
    info = net.primitives_info()
    convs = [r for r in info if r["type"] == "convolution"]
    fcs = [r for r in info if r["type"] == "fully_connected"]
    assert len(convs) == 5 and len(fcs) == 3
    if optimize:
        assert [r["kernel"] for r in convs] == ["conv_first_tc"] + ["conv_f16_tc"] * 4, [r["kernel"] for r in convs]
        assert all(r["kernel"] == "conv_f16_tc" for r in fcs), [r["kernel"] for r in fcs]
        # LRN and pooling stay in the feature-innermost layout: no reorder between the first convolution and the last pooling
        assert sum(1 for r in info if r["type"] == "reorder" and r["kernel"]) <= 2, [(r["id"], r["kernel"]) for r in info if r["type"] == "reorder"]


@pytest.mark.parametrize("optimize", [False, True])
def test_small_alexnet_int8_network_bit_exact(eng, optimize):
    """int8 AlexNet-style network (no LRN: the reference's LRN is floating-point only): 11x11 stride-4 first convolution read
    from the planar image, two-group convolutions, quantised inner products (the first over a 2x2 map), unsigned outputs."""
    spec = topologies.alexnet_int8(3, seed=6, image=99, convs=((32, 11, 4, 0, 1, True), (64, 5, 1, 2, 2, True), (96, 3, 1, 1, 1, False),
                                                                (96, 3, 1, 1, 2, False), (64, 3, 1, 1, 2, False)), classes=10, fc_width=64)
    x = _input(spec)
    want = oracle_net.run(spec, {spec.input_id: x})
    net, got = _run(eng, spec, x, optimize_data=optimize)
    _compare(spec, want, got)
    assert len(np.unique(got["fc8"])) > 3
    info = net.primitives_info()
    convs = [r for r in info if r["type"] == "convolution"]
    fcs = [r for r in info if r["type"] == "fully_connected"]
    if optimize:
        assert [r["kernel"] for r in convs] == ["conv_first_tc"] + ["conv_i8_tc"] * 4, [r["kernel"] for r in convs]
        assert all(r["kernel"] == "conv_i8_tc" for r in fcs), [r["kernel"] for r in fcs]


@pytest.mark.parametrize("optimize", [False, True])
def test_small_mobilenet_v2_int8_network_bit_exact(eng, optimize):
    """Inverted-residual blocks: 1x1 expansion and projection on the tensor cores, 3x3 depthwise on conv_i8_dw, ReLU6 as a
    clamp activation, quantised residual sums.  The optimising build folds each ReLU6 into its convolution, in front of
    the requantisation (the reference's activation fusing), and is compared with the oracle run the same way; the plain
    build keeps the activations separate, on the 8-bit values, like the oracle's primitive-by-primitive run."""
    spec = topologies.mobilenet_v2_int8(3, seed=4, image=48, blocks=((1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 2, 1)), stem=32, head=64, classes=20)
    x = _input(spec)
    stats = {}
    want = oracle_net.run(spec, {spec.input_id: x}, stats=stats, fuse_activations=optimize)
    assert stats["fc:out_of_range"] == 0
    net, got = _run(eng, spec, x, optimize_data=optimize)
    _compare(spec, want, got)
    info = net.primitives_info()
    convs = [r for r in info if r["type"] == "convolution"]
    if optimize:
        assert any(r["kernel"] == "conv_i8_dw" for r in convs)
        assert all(r["kernel"] in ("conv_i8_tc", "conv_i8_first", "conv_i8_dw") for r in convs), [(r["id"], r["kernel"]) for r in convs]
        assert not any(r["type"] == "activation" for r in info if r["kernel"])          # every ReLU6 was folded
        assert len(np.unique(got["fc"])) > 8


def test_grouped_convolutions_run_dense_on_block_diagonal_weights(eng):
    """AlexNet-style split layers (2 groups, 48 / 96 input features per group) through the host layer: the optimising build
    packs the group filters block-diagonally and runs the dense tensor-core kernel; bit-exact against the grouped oracle."""
    rng = np.random.default_rng(12)
    s = topologies.Spec()
    dt = cl.data_types
    s.input_id = "input"
    s.input_layout = cl.layout(dt.u8, cl.format.bfyx, cl.tensor(3, 96, 13, 13))
    s.add(cl.input_layout("input", s.input_layout))
    def conv(name, x, cin, cout, k, groups, out_dt, scale=2.0):
        s.const(name + "_w", rng.integers(-127, 128, size=(cout, cin // groups, k, k), dtype=np.int64).astype(np.int8))
        s.const(name + "_b", rng.integers(-4096, 4097, size=cout, dtype=np.int64).astype(np.int32))
        s.const(name + "_q", (rng.uniform(1.0, 3.0, size=cout) / (np.sqrt(cin // groups * k * k) * 73.0 * scale)).astype(np.float32))
        s.add(cl.convolution(name, x, name + "_w", name + "_b", name + "_q", output_data_type=out_dt, input_offset=(-(k // 2), -(k // 2)),
                             groups=groups, with_activation=True))
        return name
    x = conv("c2", "input", 96, 256, 5, 2, dt.u8, scale=3.0)
    x = conv("c3", x, 256, 384, 3, 1, dt.u8)
    x = conv("c4", x, 384, 384, 3, 2, dt.u8)
    x = conv("c5", x, 384, 256, 3, 4, dt.i8)
    s.outputs = [x]
    xin = _input(s)
    want = oracle_net.run(s, {s.input_id: xin})
    for optimize in (False, True):
        net, got = _run(eng, s, xin, optimize_data=optimize)
        _compare(s, want, got)
        convs = [r for r in net.primitives_info() if r["type"] == "convolution"]
        if optimize:
            assert all(r["kernel"] == "conv_i8_tc" for r in convs), [(r["id"], r["kernel"]) for r in convs]
    assert len(np.unique(want["c5"])) > 8


@pytest.mark.parametrize("optimize", [False, True])
@pytest.mark.parametrize("axis", ["f", "y", "b"])
def test_concatenation_of_convolution_branches(eng, optimize, axis):
    """Two quantised branches of different width joined by `concatenation` (src/gpu/concatenation_gpu.cpp: one copy per
    input at its offset) and consumed by a further convolution; along features the joined tensor has 48 + 80 features,
    so in the feature-innermost padded layout the second slice starts inside a 32-feature group."""
    rng = np.random.default_rng(21)
    s = topologies.Spec()
    dt = cl.data_types
    s.input_id = "input"
    s.input_layout = cl.layout(dt.u8, cl.format.bfyx, cl.tensor(2, 32, 10, 9))
    s.add(cl.input_layout("input", s.input_layout))

    def conv(name, x, cin, cout, k, out_dt=dt.u8):
        s.const(name + "_w", rng.integers(-127, 128, size=(cout, cin, k, k), dtype=np.int64).astype(np.int8))
        s.const(name + "_b", rng.integers(-4096, 4097, size=cout, dtype=np.int64).astype(np.int32))
        s.const(name + "_q", (rng.uniform(1.0, 3.0, size=cout) / (np.sqrt(cin * k * k) * 73.0 * 2.0)).astype(np.float32))
        s.add(cl.convolution(name, x, name + "_w", name + "_b", name + "_q", output_data_type=out_dt, input_offset=(-(k // 2), -(k // 2)), with_activation=True))
        return name
    same = axis != "f"
    a = conv("left", "input", 32, 48, 1)
    b = conv("right", "input", 32, 48 if same else 80, 3)
    ax = {"b": cl.concatenation_axis.along_b, "f": cl.concatenation_axis.along_f, "y": cl.concatenation_axis.along_y}[axis]
    s.add(cl.concatenation("joined", [a, b], ax))
    conv("head", "joined", 48 if same else 128, 64, 1, dt.i8)
    s.outputs = ["joined", "head"]
    x = _input(s)
    want = oracle_net.run(s, {s.input_id: x})
    net, got = _run(eng, s, x, optimize_data=optimize)
    _compare(s, want, got)
    assert want["joined"].shape[{"b": 0, "f": 1, "y": 2}[axis]] == (4 if axis == "b" else (128 if axis == "f" else 18))
    assert len(np.unique(want["head"])) > 16


def _single_fp16_conv(batch, cin, cout, size, seed=31):
    rng = np.random.default_rng(seed)
    s = topologies.Spec()
    dt = cl.data_types
    s.input_id = "input"
    s.input_layout = cl.layout(dt.f16, cl.format.bfyx, cl.tensor(batch, cin, size, size))
    s.add(cl.input_layout("input", s.input_layout))
    s.const("w", (rng.standard_normal((cout, cin, 3, 3)) * np.sqrt(2.0 / (cin * 9))).astype(np.float16))
    s.const("b", (rng.standard_normal(cout) * 0.05).astype(np.float16))
    s.add(cl.convolution("conv", "input", "w", "b", input_offset=(-1, -1), with_activation=True))
    s.outputs = ["conv"]
    x = rng.standard_normal((batch, cin, size, size)).astype(np.float16)
    return s, x


def _winograd_close(got, want):
    """Winograd F(2x2, 3x3) against the direct-form oracle: 1e-2 relative to each value, an absolute 1e-3 of the output scale
    for the small ones (measured: at most 6.7e-4 of the scale, the final rounding to fp16 at the top of the range)."""
    w, g = want.astype(np.float32), got.astype(np.float32)
    scale = float(np.abs(w).max())
    err = np.abs(g - w)
    bad = err > np.maximum(1e-2 * np.abs(w), 1e-3 * scale)
    assert not bad.any(), "%d of %d values; worst %.4g on scale %.4g" % (int(bad.sum()), w.size, float(err.max()), scale)
    return float(err.max() / scale)


def test_winograd_is_a_selectable_alternative_of_the_fp16_convolution(eng):
    """The gate modelled on should_use_winograd_2x3_s1 (src/layout_optimizer.cpp:34-53) admits this layer, so
    conv_f16_winograd is a candidate of the primitive: forced, it runs inside a network and agrees with the oracle; a layer the
    gate refuses (48 features) never gets it."""
    s, x = _single_fp16_conv(4, 64, 64, 16)
    want = oracle_net.run(s, {s.input_id: x})
    net, got = _run(eng, s, x, optimize_data=True, force_kernel="conv=conv_f16_winograd")
    info = {r["id"]: r for r in net.primitives_info()}
    assert info["conv"]["kernel"] == "conv_f16_winograd"
    _winograd_close(got["conv"], want["conv"])
    s2, x2 = _single_fp16_conv(4, 48, 64, 16)
    with pytest.raises(cl.error):
        _run(eng, s2, x2, optimize_data=True, force_kernel="conv=conv_f16_winograd")


def test_tuner_times_winograd_against_the_direct_form_on_a_vgg_layer(eng):
    """VGG16's 512 -> 512 layer on a 14x14 map at batch 32, tile shapes and form chosen by on-device timing: whichever of the
    two wins is recorded as the primitive's kernel, and the result agrees with the oracle (first and last image)."""
    s, x = _single_fp16_conv(32, 512, 512, 14)
    net, got = _run(eng, s, x, optimize_data=True, tuning=cl.tuning_mode.tuning_tune_and_cache)
    info = {r["id"]: r for r in net.primitives_info()}
    assert info["conv"]["kernel"] in ("conv_f16_tc", "conv_f16_winograd")
    small, _ = _single_fp16_conv(2, 512, 512, 14)
    want = oracle_net.run(small, {small.input_id: x[[0, 31]]})
    if info["conv"]["kernel"] == "conv_f16_winograd":
        _winograd_close(got["conv"][[0, 31]], want["conv"])
    else:
        w, g = want["conv"].astype(np.float32), got["conv"][[0, 31]].astype(np.float32)
        assert np.abs(g - w).max() <= 1e-2 * float(np.abs(w).max())
