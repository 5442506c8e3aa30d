"""Per-layer convolution sweeps of the benchmark configurations, through the C ABI.

    python -m cldnn_b200.sweep vgg16_fp16 [--batch 32]
    python -m cldnn_b200.sweep alexnet_fp16 | alexnet_int8 | vgg16_fp16_net | mobilenet_v2_int8 | resnet50_int8 [--batch N]

VGG16 fp16 (13 3x3 pad-1 layers, 64 -> 512 features, 224 -> 14 maps; weights N(0, sqrt(2 / fan_in)), inputs N(0, 1),
fp32 accumulation): every layer is timed on the direct tensor-core kernel (conv_f16_tc, best tile shape of its tuning
variants) and on the Winograd F(2x2, 3x3) path (conv_f16_winograd); TFLOP/s are quoted on the direct form's operation
count for both, so the two columns compare wall time.  One JSON line per layer, then a summary line.
"""
import argparse
import ctypes as C
import json
import sys

import numpy as np

from . import abi, engine as eng, topologies


def _conv_params(batch, cin, cout, size, f_align=16):
    p = abi.ConvParams()
    cs = -(-cin // f_align) * f_align
    p.in_, n_in = abi.tensor(abi.F16, batch, cin, size, size, "byxf", f_align)
    p.out, n_out = abi.tensor(abi.F16, batch, cout, size, size, "byxf", f_align)
    abi.set_weights(p, abi.F16, 1, cout, cin, 3, 3, "oyxi", f_align)
    p.stride_x = p.stride_y = p.dil_x = p.dil_y = 1
    p.pad_x = p.pad_y = 1
    p.bias_dtype = abi.F32
    p.act = abi.ACT_RELU
    p.eltw_stride_x = p.eltw_stride_y = 1
    p.i_qf = p.o_qf = 1.0
    return p, n_in, n_out, cs


def _time_best(E, kernel, p, args_for, runs):
    """Best tuning variant of `kernel` for the launch constants `p`: (ns, tune, scratch bytes) or None."""
    k = E.kernel(kernel)
    if not k.supports(p):
        return None
    sb = C.c_size_t()
    E.lib.cldnn_b200_kernel_scratch_bytes(k.handle, C.byref(p), C.sizeof(p), C.byref(sb))
    scratch = E.alloc(sb.value) if sb.value else None
    args = args_for(scratch)
    best = None
    for tune in range(1 if k.tune_count(p) > 1 else 0, k.tune_count(p)):
        q = abi.ConvParams.from_buffer_copy(bytes(p))
        q.tune = tune
        if not k.supports(q):
            continue
        pr = k.prepare(q, args)
        ns = pr.time_ns(3, runs)
        pr.destroy()
        if best is None or ns < best[0]:
            best = (ns, tune, sb.value)
    if scratch is not None:
        scratch.free()
    return best


def _first_layer(E, rng, batch, cin, cout, size, runs):
    """The image layer on conv_first_tc: planar (bfyx) input read in place, weights oiyx, dense K = C*9."""
    p = abi.ConvParams()
    p.in_, n_in = abi.tensor(abi.F16, batch, cin, size, size, "bfyx", 1)
    p.out, n_out = abi.tensor(abi.F16, batch, cout, size, size, "byxf", 16)
    abi.set_weights(p, abi.F16, 1, cout, cin, 3, 3, "oiyx")
    p.stride_x = p.stride_y = p.dil_x = p.dil_y = 1
    p.pad_x = p.pad_y = 1
    p.bias_dtype = abi.F32
    p.act = abi.ACT_RELU
    p.eltw_stride_x = p.eltw_stride_y = 1
    p.i_qf = p.o_qf = 1.0
    x = rng.standard_normal(n_in).astype(np.float16)
    w = (rng.standard_normal(cout * cin * 9) * np.sqrt(2.0 / (cin * 9))).astype(np.float16)
    bias = (rng.standard_normal(cout) * 0.05).astype(np.float32)
    mx, mw, mb, mo = E.upload(x), E.upload(w), E.upload(bias), E.alloc(n_out * 2)
    best = _time_best(E, "conv_first_tc", p, lambda scratch: eng.make_args(input0=mx, output=mo, weights=mw, bias=mb, scratch=scratch), runs)
    for m in (mx, mw, mb, mo):
        m.free()
    return best


def vgg16_fp16(batch=32, runs=20, out=sys.stdout):
    E = eng.Engine(0)
    rng = np.random.default_rng(16)
    rows = []
    for name, cin, cout, size in topologies.vgg16_conv_layers():
        p, n_in, n_out, cs = _conv_params(batch, cin, cout, size)
        x = np.zeros(n_in, dtype=np.float16)
        x.reshape(batch, size, size, cs)[..., :cin] = rng.standard_normal((batch, size, size, cin)).astype(np.float16)
        w = np.zeros((cout, 3, 3, cs), dtype=np.float16)
        w[..., :cin] = (rng.standard_normal((cout, 3, 3, cin)) * np.sqrt(2.0 / (cin * 9))).astype(np.float16)
        bias = (rng.standard_normal(cout) * 0.05).astype(np.float32)
        mx, mw, mb = E.upload(x), E.upload(w.reshape(-1)), E.upload(bias)
        mo = E.alloc(n_out * 2)
        flops = 2.0 * batch * size * size * cout * cin * 9
        res = {"layer": name, "features_in": cin, "features_out": cout, "map": size, "batch": batch, "gflop": flops / 1e9}
        for kernel in ("conv_f16_tc", "conv_f16_winograd"):
            k = E.kernel(kernel)
            sb = C.c_size_t()
            E.lib.cldnn_b200_kernel_scratch_bytes(k.handle, C.byref(p), C.sizeof(p), C.byref(sb))
            scratch = E.alloc(sb.value) if sb.value else None
            args = eng.make_args(input0=mx, output=mo, weights=mw, bias=mb, scratch=scratch)
            best = None
            for tune in range(1 if k.tune_count(p) > 1 else 0, k.tune_count(p)):
                q = abi.ConvParams.from_buffer_copy(bytes(p))
                q.tune = tune
                if not k.supports(q):
                    continue
                pr = k.prepare(q, args)
                ns = pr.time_ns(3, runs)
                pr.destroy()
                if best is None or ns < best[0]:
                    best = (ns, tune)
            if best:
                res[kernel] = {"us": best[0] / 1e3, "tune": best[1], "tflops": flops / best[0] / 1e3, "scratch_mb": sb.value / 1e6}
            if scratch is not None:
                scratch.free()
        if cin <= 4:
            b = _first_layer(E, rng, batch, cin, cout, size, runs)
            if b:
                res["conv_first_tc"] = {"us": b[0] / 1e3, "tune": b[1], "tflops": flops / b[0] / 1e3, "scratch_mb": b[2] / 1e6}
        res["device_status"] = E.device_status()
        rows.append(res)
        print(json.dumps(res), file=out, flush=True)
        for m in (mx, mw, mb, mo):
            m.free()
    # direct form: the image layer on its own kernel where that is faster, every other layer on conv_f16_tc
    direct = sum(min(r["conv_f16_tc"]["us"], r.get("conv_first_tc", r["conv_f16_tc"])["us"]) for r in rows)
    best = sum(min(r["conv_f16_tc"]["us"], r.get("conv_first_tc", r["conv_f16_tc"])["us"], r.get("conv_f16_winograd", r["conv_f16_tc"])["us"]) for r in rows)
    total = sum(r["gflop"] for r in rows)
    print(json.dumps({"summary": "vgg16_fp16", "batch": batch, "direct_us": direct, "direct_tflops": total / direct * 1e3,
                      "best_of_both_us": best, "winograd_wins": [r["layer"] for r in rows if "conv_f16_winograd" in r and r["conv_f16_winograd"]["us"] < r["conv_f16_tc"]["us"]]}),
          file=out, flush=True)
    E.close()
    return rows


NETWORKS = {
    "alexnet_fp16": (lambda b: topologies.alexnet_fp16(b), 256),
    "alexnet_int8": (lambda b: topologies.alexnet_int8(b), 256),
    "vgg16_fp16_net": (lambda b: topologies.vgg16_fp16(b), 32),
    "mobilenet_v2_int8": (lambda b: topologies.mobilenet_v2_int8(b), 128),
    "resnet50_int8": (lambda b: topologies.resnet50_int8(b), 256),
}


def network(name, batch=None, steps=10, cache="", out=sys.stdout):
    """A whole topology through the host API (optimising build, tile shapes tuned on the device): images/s over `steps`
    executions (wall clock around a synchronised loop of CUDA-graph launches, inputs resident on the device), then one
    JSON line per primitive with its kernel, device time (CUDA events on a profiling engine) and, for convolutions and
    inner products, the achieved TFLOP/s on the direct form's operation count."""
    import time
    from . import cldnn as cl
    make, default_batch = NETWORKS[name]
    batch = batch or default_batch
    spec = make(batch)
    total_ops, per_layer = topologies.conv_ops(spec)
    ops_by_id = {pid: ops for pid, kind, ops, shape in per_layer}
    lay = spec.input_layout
    rng = np.random.default_rng(1)
    shape = (lay.size.batch, lay.size.feature, lay.size.y, lay.size.x)
    x = rng.integers(0, 256, size=shape).astype(np.uint8) if lay.data_type == cl.data_types.u8 else rng.standard_normal(shape).astype(np.float16)

    def build(profiling):
        e = cl.engine(0, enable_profiling=profiling)
        topo, keep = spec.realise(e)
        opts = cl.build_options(optimize_data=True, outputs=[spec.outputs[0]], tuning=cl.tuning_mode.tuning_tune_and_cache, tuning_cache_path=cache)
        net = cl.network(e, topo, opts)
        xin = cl.memory.from_numpy(e, x)
        net.set_input_data(spec.input_id, xin)
        return e, net, (keep, xin)

    e, net, keep = build(False)
    for _ in range(3):
        net.execute()
    net.wait()
    t0 = time.perf_counter()
    for _ in range(steps):
        net.execute()
    net.wait()
    dt = (time.perf_counter() - t0) / steps
    first = net.get_output(spec.outputs[0]).to_numpy().reshape(-1)[:4].astype(float).tolist()
    print(json.dumps({"network": name, "batch": batch, "ms_per_step": dt * 1e3, "images_per_s": batch / dt, "gop_per_image": total_ops / 1e9,
                      "tflops": total_ops * batch / dt / 1e12, "launches_per_step": net.stats()["launches_per_execute"], "first_outputs": first}), file=out, flush=True)
    del net
    ep, netp, keepp = build(True)
    for _ in range(2):
        netp.execute()
    netp.wait()
    acc, reps = {}, 3
    for _ in range(reps):
        netp.execute()
        netp.wait()
        for k, v in netp.profiling_info().items():
            acc[k] = acc.get(k, 0) + v
    info = {r["id"]: r for r in netp.primitives_info()}
    for k, v in acc.items():
        ns = v / reps
        row = {"id": k, "type": info[k]["type"], "kernel": info[k]["kernel"], "us": ns / 1e3}
        if k in ops_by_id:
            row["tflops"] = ops_by_id[k] * batch / ns / 1e3
        print(json.dumps(row), file=out, flush=True)
    print(json.dumps({"summary": name, "profiled_us": sum(acc.values()) / reps / 1e3}), file=out, flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("config", choices=["vgg16_fp16"] + sorted(NETWORKS))
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--cache", default="", help="tuning cache file to read and extend (default: tune in memory)")
    a = ap.parse_args()
    if a.config == "vgg16_fp16":
        vgg16_fp16(a.batch or 32)
    else:
        network(a.config, a.batch, a.steps, a.cache)
