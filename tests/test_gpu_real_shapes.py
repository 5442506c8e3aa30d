"""Layer-by-layer parity at the full size of the benchmark configurations, with the tile shapes the shipped tuning cache
holds for them.

Each network is built at its benchmark batch (ResNet-50 int8 at 256, MobileNet-v2 int8 at 128, AlexNet int8 / fp16 at 256,
VGG16 fp16 at 32) the way bench.py builds it -- optimising build, tile shapes from cldnn_b200/cache/tuning_cache.json -- with
every layer's result requested as an output.  Images are independent, so the CPU oracle runs the same topology on a few
images of the batch only (the first and the last: the last image ends in the tail tiles of every layer) and every layer's
rows for those images are compared: bit-exact for integer results (fused_conv_eltwise_gpu_ref.cl:65-234 and the tail
kernels), 1e-2 of the layer's scale for fp16.
"""
import os

import numpy as np
import pytest

import oracle_net
from cldnn_b200 import cldnn as cl
from cldnn_b200 import topologies

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIPPED_CACHE = os.path.join(ROOT, "cldnn_b200", "cache", "tuning_cache.json")

# name: (constructor, batch, images the oracle computes, integer network, the oracle folds ReLU6 like the optimising build)
NETWORKS = {
    "resnet50_int8": (topologies.resnet50_int8, 256, (0, 255), True, False),
    "mobilenet_v2_int8": (topologies.mobilenet_v2_int8, 128, (0, 127), True, True),
    "alexnet_int8": (topologies.alexnet_int8, 256, (0, 255), True, False),
    "alexnet_fp16": (topologies.alexnet_fp16, 256, (0, 255), False, False),
    "vgg16_fp16": (topologies.vgg16_fp16, 32, (31,), False, False),
}


def _visible_layers(spec):
    """Ids whose values the optimising build still produces: a convolution whose only reader is an activation or a sum is
    folded into that reader (prepare_primitive_fusing.cpp:396-433, :181-337), so the reader's id is taken instead."""
    users = {}
    for p in spec.prims:
        for k in ("input", "input2"):
            if p.args.get(k):
                users.setdefault(p.args[k], []).append(p)
    ids = []
    for p in spec.prims:
        if p.kind in ("data", "input_layout"):
            continue
        u = users.get(p.id, [])
        if p.kind == "convolution" and len(u) == 1 and u[0].kind in ("activation", "eltwise"):
            continue
        ids.append(p.id)
    return ids


def _images(spec, n, seed):
    lay = spec.input_layout
    shape = (n, lay.size.feature, lay.size.y, lay.size.x)
    rng = np.random.default_rng(seed)
    if lay.data_type == cl.data_types.u8:
        return rng.integers(0, 256, size=shape, dtype=np.int64).astype(np.uint8)
    return rng.standard_normal(shape).astype(np.float16)


@pytest.mark.parametrize("name", sorted(NETWORKS))
def test_every_layer_at_benchmark_size_with_shipped_tile_shapes(name):
    make, batch, picks, integer, fold = NETWORKS[name]
    spec = make(batch)
    layers = _visible_layers(spec)
    x = _images(spec, batch, seed=4242)
    eng = cl.engine(0)
    topo, keep = spec.realise(eng)
    net = cl.network(eng, topo, cl.build_options(optimize_data=True, outputs=layers, tuning=cl.tuning_mode.tuning_use_cache,
                                                 tuning_cache_path=SHIPPED_CACHE))
    net.set_input_data(spec.input_id, cl.memory.from_numpy(eng, x))
    net.execute()
    info = net.primitives_info()
    tc = [r for r in info if r["kernel"] in ("conv_i8_tc", "conv_f16_tc")]
    assert len(tc) >= 5
    # the shipped cache knows these shapes: every tensor-core launch runs a tuned tile shape (index 0 is the untuned default)
    missing = [r["id"] for r in tc if r["tune"] == 0]
    assert not missing, "no shipped tile shape for " + ", ".join(missing)

    small = make(len(picks))
    want = oracle_net.run(small, {small.input_id: x[list(picks)]}, keep=layers, fuse_activations=fold)
    bad = []
    for lid in layers:
        got = net.get_output(lid).to_numpy()[list(picks)]
        w = want[lid]
        assert got.shape == w.shape, lid
        if w.dtype.kind in "iu":
            n = int((w != got).sum())
            if n:
                bad.append("%s: %d of %d values differ" % (lid, n, w.size))
        else:
            w32, g32 = w.astype(np.float32), got.astype(np.float32)
            scale = float(np.abs(w32).max())
            err = float(np.abs(g32 - w32).max())
            # integer networks end in a float tail (softmax of exact logits): exp() rounding only
            tol = (1e-4 if integer else 1e-2) * scale
            if not err <= tol:
                bad.append("%s: max abs error %.4g on scale %.4g" % (lid, err, scale))
    assert not bad, "; ".join(bad[:8])
    logits = want[spec.outputs[1]]
    assert len(np.unique(logits)) > 8                      # the comparison is not on a constant
    del net
