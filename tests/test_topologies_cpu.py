"""The synthetic topologies of the benchmark configurations: operation counts against the architectures' published
multiply-add counts, and shape bookkeeping (no GPU needed)."""
import numpy as np

from cldnn_b200 import topologies


def _gop(spec):
    total, per_layer = topologies.conv_ops(spec)
    return total / 1e9, per_layer


def test_resnet50_operation_count():
    gop, per_layer = _gop(topologies.resnet50_int8(1))
    assert abs(gop - 7.716) < 0.01                      # 3.856 GMAC of convolutions + the 2048 -> 1000 inner product
    convs = [l for l in per_layer if l[1] in ("convolution", "fused_conv_eltwise")]
    assert len(convs) == 53
    assert sum(1 for l in per_layer if l[1] == "fused_conv_eltwise") == 16


def test_vgg16_operation_count():
    gop, per_layer = _gop(topologies.vgg16_fp16(1))
    assert abs(gop - 30.94) < 0.05                      # 15.35 GMAC of convolutions + 0.12 GMAC of inner products
    layers = topologies.vgg16_conv_layers()
    assert len(layers) == 13 and layers[0][1:] == (3, 64, 224) and layers[-1][1:] == (512, 512, 14)
    sweep_gop = sum(2.0 * 32 * size * size * cout * cin * 9 for _, cin, cout, size in layers) / 1e9
    assert abs(sweep_gop - 982.2) < 0.5                 # the batch-32 sweep of the 13 convolutions


def test_alexnet_operation_count_and_groups():
    for make in (topologies.alexnet_fp16, topologies.alexnet_int8):
        spec = make(1)
        gop, per_layer = _gop(spec)
        assert abs(gop - 1.449) < 0.01                  # 0.666 GMAC of (grouped) convolutions + 0.0586 GMAC of inner products
        groups = [p.args.get("groups", 1) for p in spec.prims if p.kind == "convolution"]
        assert groups == [1, 2, 1, 2, 2]
        fcs = [spec.consts[p.args["weights"]].shape for p in spec.prims if p.kind == "fully_connected"]
        assert fcs == [(4096, 256, 6, 6), (4096, 4096, 1, 1), (1000, 4096, 1, 1)]
    assert not any(p.kind == "lrn" for p in topologies.alexnet_int8(1).prims)
    assert sum(1 for p in topologies.alexnet_fp16(1).prims if p.kind == "lrn") == 2


def test_mobilenet_v2_operation_count():
    gop, per_layer = _gop(topologies.mobilenet_v2_int8(1))
    assert abs(gop - 0.6015) < 0.005                    # ~0.30 GMAC
    spec = topologies.mobilenet_v2_int8(1)
    dw = [p for p in spec.prims if p.kind == "convolution" and p.args.get("groups", 1) > 4]
    assert len(dw) == 17 and all(spec.consts[p.args["weights"]].shape[1] == 1 for p in dw)


def test_tuning_cache_reader_is_a_real_json_reader(tmp_path):
    """The cache file has the reference's schema ({ "<compute units>": { "<hash>": ["kernel", index] } },
    kernel_selector/core/auto_tuner.cpp:72-118).  Reformatting, other devices' sections in front of the wanted one, braces
    inside strings and escapes must not lose entries; malformed input is an error, not an empty cache."""
    import ctypes as C
    from cldnn_b200 import abi
    from cldnn_b200 import cldnn as cl
    lib = cl.load_library()
    lib.cldnn_host_last_error.restype = C.c_char_p if hasattr(lib, "cldnn_host_last_error") else None
    n = C.c_size_t()

    def check(text, units=148):
        p = tmp_path / "cache.json"
        p.write_text(text)
        return lib.cldnn_host_tuning_cache_check(str(p).encode(), units, C.byref(n)), n.value

    shipped = open(__import__("os").path.join(__import__("os").path.dirname(cl.__file__), "cache", "tuning_cache.json")).read()
    st, count = check(shipped)
    assert st == 0 and count > 100
    tricky = '{"72":{"aa":["conv_ref",0]},\n\t"148" : { "k}1" : [ "conv_{i8}_tc" , 7 ],"k\\"2":["a\\u0041b",\n 3 ] } , "200": {}}'
    assert check(tricky) == (0, 2)
    assert check(tricky, 72) == (0, 1)
    assert check(tricky, 5) == (0, 0)
    assert check("") == (0, 0)
    for bad in ('{"148": {"h": ["k", 1]', '{"148": {"h": ["k"]}}', '{"148": {"h": "k"}}', '[1, 2]', '{"148": {"h": ["k", 1]}} x', '{"148": {h: ["k", 1]}}'):
        st, _ = check(bad)
        assert st == abi.INVALID_ARG, bad
