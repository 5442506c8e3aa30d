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
