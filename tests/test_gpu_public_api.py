"""clDNN's own public API, unchanged, in front of the B200 engine.

tests/_ref_api/ref_api_driver is compiled from tests/api_cpp/ref_api_driver.cpp against the reference's unmodified
header-only C++ API (api/CPP/*.hpp, api_extension/CPP/fused_conv_eltwise.hpp) and linked to cldnn_b200/libclDNN64.so, which
exports the C entry points those headers call (api/C/cldnn.h:537-805).  The tests describe a topology once, hand it to the
driver as a script (cldnn::engine / memory / topology / network do the work) and to the CPU oracle, and compare:
the reference's ConvQuantizedTest vectors (tests/test_cases/convolution_gpu_test.cpp:3971-4197) exactly, a ResNet bottleneck
with fused_conv_eltwise bit for bit, with optimize_data off and on.
"""
import os
import subprocess

import numpy as np
import pytest

import oracle_net
from cldnn_b200 import cldnn as cl
from cldnn_b200 import topologies

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "tests", "_ref_api", "ref_api_driver")

DT = {np.dtype(np.uint8): "u8", np.dtype(np.int8): "i8", np.dtype(np.int32): "i32", np.dtype(np.float32): "f32", np.dtype(np.float16): "f16"}
DT_OF_CODE = {cl.data_types.u8: "u8", cl.data_types.i8: "i8", cl.data_types.i32: "i32", cl.data_types.f32: "f32", cl.data_types.f16: "f16"}
NP_OF_NAME = {"u8": np.uint8, "i8": np.int8, "i32": np.int32, "f32": np.float32, "f16": np.float16}


def _need_driver():
    if not os.path.exists(DRIVER):
        pytest.fail("tests/_ref_api/ref_api_driver is missing: build it with `make -C tests/api_cpp REF=<clDNN tree>` "
                    "(the build entry point does so where the tree is present)")


def _mem_line(kind, name, arr, d):
    a = np.ascontiguousarray(arr)
    if a.ndim == 1:
        b, f, y, x = 1, 1, 1, a.shape[0]                  # a per-feature vector: tensor(1, 1, n, 1)
    else:
        b, f, y, x = a.shape
    a.tofile(os.path.join(d, name + ".bin"))
    return "%s %s %s %d %d %d %d %s.bin" % (kind, name, DT[a.dtype], b, f, x, y, name)


def _o(s):
    return s if s else "-"


def spec_to_script(spec, x, d, optimize, outputs, attach_input=False):
    """The topology of `spec` as a driver script; constants and the input go to files in directory `d`."""
    lines = []
    for name, arr in spec.consts.items():
        lines.append(_mem_line("mem", name, arr, d))
    lines.append(_mem_line("attach" if attach_input else "mem", "input_values", x, d))
    for p in spec.prims:
        a, k = p.args, p.kind
        if k == "data":
            lines.append("data %s %s" % (p.id, p.id))
        elif k == "input_layout":
            lines.append("input_layout %s input_values" % p.id)
        elif k == "convolution":
            assert a.get("groups", 1) == 1 and not a["output_calibration_factors"]
            lines.append("convolution %s %s %s %s %s %s %d %d %d %d %d %d %d" % (
                p.id, a["input"], a["weights"], _o(a["bias"]), _o(a["weights_quantization_factors"]), DT_OF_CODE.get(a["output_data_type"], "-"),
                a["stride"][0], a["stride"][1], a["input_offset"][0], a["input_offset"][1], a["dilation"][0], a["dilation"][1], int(a["with_activation"])))
        elif k == "fused_conv_eltwise":
            lines.append("fused_conv_eltwise %s %s %s %s %s %s %s %d %d %d %d %d %d" % (
                p.id, a["input"], a["input2"], a["weights"], _o(a["bias"]), _o(a["weights_quantization_factors"]), DT_OF_CODE[a["output_data_type"]],
                a["stride"][0], a["stride"][1], a["input_offset"][0], a["input_offset"][1], int(a["with_activation"]), int(a["eltw_activation"])))
        elif k == "pooling":
            assert not a["global_pooling"]
            lines.append("pooling %s %s %s %d %d %d %d %d %d" % (p.id, a["input"], "max" if a["mode"] == cl.pooling_mode.max else "average", a["size"][0], a["size"][1],
                                                              a["stride"][0], a["stride"][1], a["input_offset"][0], a["input_offset"][1]))
        elif k == "fully_connected":
            lines.append("fully_connected %s %s %s %s %s %s %d" % (p.id, a["input"], a["weights"], _o(a["bias"]), _o(a["weights_quantization_factors"]),
                                                                 _o(a["output_calibration_factors"]), int(a["with_activation"])))
        elif k == "softmax":
            lines.append("softmax %s %s" % (p.id, a["input"]))
        elif k == "reorder":
            lines.append("reorder %s %s %s %s" % (p.id, a["input"], cl.format.names[a["out_format"]], DT_OF_CODE[a["out_data_type"]]))
        elif k == "concatenation":
            lines.append("concatenation %s %s %s" % (p.id, "bfxy"[a["axis"]], " ".join(a["inputs"])))
        else:
            raise AssertionError("no script form for " + k)
    lines.append("option optimize_data %d" % int(optimize))
    lines.append("option outputs " + " ".join(outputs))
    lines += ["build", "set_input %s input_values" % spec.input_id, "execute"]
    for o in outputs:
        lines += ["info " + o, "save %s out_%s.bin" % (o, o)]
    path = os.path.join(d, "script.txt")
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    return path


def run_driver(script):
    r = subprocess.run([DRIVER, script], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, "driver failed:\n" + r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def read_output(d, name, like):
    return np.fromfile(os.path.join(d, "out_%s.bin" % name), dtype=like.dtype).reshape(like.shape)


@pytest.mark.parametrize("case", ["u8_to_u8", "i8_to_u8", "u8_to_i8", "i8_to_float"])
def test_conv_quantized_vectors_through_the_reference_cpp_api(tmp_path, case):
    _need_driver()
    from golden import kat_conv_quantized
    kc = kat_conv_quantized.CASES[case]
    feats = kc["features"]
    n = len(feats)
    in_dt, out_dt = np.dtype(kc["in_dtype"]), np.dtype(kc["out_dtype"])
    s = topologies.Spec()
    s.input_id = "input"
    s.input_layout = cl.layout(cl.data_types.u8 if in_dt == np.uint8 else cl.data_types.i8, cl.format.bfyx, cl.tensor(1, n, 4, 1))
    s.add(cl.input_layout("input", s.input_layout))
    w = np.zeros((n, n, 1, 3), dtype=np.int8)
    for i, f in enumerate(feats):
        w[i, i, 0, :] = f[1]
    s.const("weights", w)
    s.const("biases", np.array([f[2] for f in feats], dtype=np.int32))
    s.const("quantization", np.array([f[3] for f in feats], dtype=np.float32))
    odt = {np.dtype(np.uint8): cl.data_types.u8, np.dtype(np.int8): cl.data_types.i8, np.dtype(np.float32): cl.data_types.f32}[out_dt]
    s.add(cl.convolution("conv", "input", "weights", "biases", "quantization", output_data_type=odt, with_activation=True))
    x = np.array([f[0] for f in feats], dtype=in_dt).reshape(1, n, 1, 4)
    d = str(tmp_path)
    out = run_driver(spec_to_script(s, x, d, optimize=False, outputs=["conv"]))
    assert "format 2, b 1 f %d y 1 x 2" % n in out                       # bfyx, the shape the reference's test asserts
    got = np.fromfile(os.path.join(d, "out_conv.bin"), dtype=out_dt).reshape(n, 2)
    pre = np.array([f[4] for f in feats], dtype=np.float64)
    if out_dt.kind in "iu":
        info = np.iinfo(out_dt)
        assert np.array_equal(got.astype(np.int64), np.clip(np.maximum(pre, 0), info.min, info.max).astype(np.int64))
    else:
        np.testing.assert_allclose(got, np.maximum(pre, 0), atol=1e-3)


def _bottleneck(batch=3, cin=64, width=32, size=14, seed=17):
    """One ResNet bottleneck in the caller's terms: 1x1 -> 3x3 -> (1x1 fused with the residual sum + ReLU) beside a 1x1
    projection, then 2x2 max pooling; u8 activations, s8 weights, i32 bias, per-feature scales."""
    rng = np.random.default_rng(seed)
    s = topologies.Spec()
    dt = cl.data_types
    s.input_id = "input"
    s.input_layout = cl.layout(dt.u8, cl.format.bfyx, cl.tensor(batch, cin, size, size))
    s.add(cl.input_layout("input", s.input_layout))

    def consts(name, ci, co, k):
        s.const(name + "_w", rng.integers(-127, 128, size=(co, ci, k, k), dtype=np.int64).astype(np.int8))
        s.const(name + "_b", rng.integers(-4096, 4097, size=co, dtype=np.int64).astype(np.int32))
        s.const(name + "_q", (rng.uniform(1.0, 3.0, size=co) / (np.sqrt(ci * k * k) * 73.0 * 74.0) * 40.0).astype(np.float32))
    consts("a", cin, width, 1)
    s.add(cl.convolution("a", "input", "a_w", "a_b", "a_q", output_data_type=dt.u8, with_activation=True))
    consts("b", width, width, 3)
    s.add(cl.convolution("b", "a", "b_w", "b_b", "b_q", output_data_type=dt.u8, input_offset=(-1, -1), with_activation=True))
    consts("proj", cin, 4 * width, 1)
    s.add(cl.convolution("proj", "input", "proj_w", "proj_b", "proj_q", output_data_type=dt.i8))
    consts("c", width, 4 * width, 1)
    s.add(cl.fused_conv_eltwise("c", "b", "proj", "c_w", "c_b", "c_q", eltw_activation=True, output_data_type=dt.u8))
    s.add(cl.pooling("pool", "c", cl.pooling_mode.max, size=(2, 2), stride=(2, 2)))
    s.outputs = ["c", "pool"]
    x = rng.integers(0, 256, size=(batch, cin, size, size), dtype=np.int64).astype(np.uint8)
    return s, x


@pytest.mark.parametrize("optimize", [False, True])
@pytest.mark.parametrize("attach", [False, True])
def test_bottleneck_with_fused_conv_eltwise_through_the_reference_cpp_api(tmp_path, optimize, attach):
    _need_driver()
    s, x = _bottleneck()
    want = oracle_net.run(s, {s.input_id: x})
    d = str(tmp_path)
    out = run_driver(spec_to_script(s, x, d, optimize=optimize, outputs=s.outputs, attach_input=attach))
    for o in s.outputs:
        got = read_output(d, o, want[o])
        assert np.array_equal(got, want[o]), "%s: %d of %d values differ" % (o, int((got != want[o]).sum()), got.size)
    assert len(np.unique(want["c"])) > 32
    if optimize:
        assert "kernel: conv_i8_tc" in out                               # the optimising build put the block on the tensor-core kernel
    else:
        assert "kernel: conv_ref" in out


def test_unsupported_primitives_and_bad_topologies_come_back_as_errors(tmp_path):
    """A dimension mismatch surfaces as the reference's exception type with the library's message; nothing is emulated."""
    _need_driver()
    s, x = _bottleneck()
    s.consts["b_w"] = s.consts["b_w"][:, :16]                              # 16 input features where the tensor has 32
    d = str(tmp_path)
    script = spec_to_script(s, x, d, optimize=False, outputs=["c"])
    text = open(script).read().replace("\nbuild\n", "\nexpect_build_error\n").split("set_input")[0]
    with open(script, "w") as f:
        f.write(text)
    out = run_driver(script)
    assert "build refused" in out and "do not match input features" in out
