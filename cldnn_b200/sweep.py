"""Per-layer convolution sweeps of the benchmark configurations, through the C ABI.

    python -m cldnn_b200.sweep vgg16_fp16 [--batch 32]

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
        res["device_status"] = E.device_status()
        rows.append(res)
        print(json.dumps(res), file=out, flush=True)
        for m in (mx, mw, mb, mo):
            m.free()
    direct = sum(r["conv_f16_tc"]["us"] for r in rows)
    best = sum(min(r["conv_f16_tc"]["us"], r.get("conv_f16_winograd", r["conv_f16_tc"])["us"]) for r in rows)
    total = sum(r["gflop"] for r in rows)
    print(json.dumps({"summary": "vgg16_fp16", "batch": batch, "direct_us": direct, "direct_tflops": total / direct * 1e-3 * 1e3,
                      "best_of_both_us": best, "winograd_wins": [r["layer"] for r in rows if "conv_f16_winograd" in r and r["conv_f16_winograd"]["us"] < r["conv_f16_tc"]["us"]]}),
          file=out, flush=True)
    E.close()
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("config", choices=["vgg16_fp16"])
    ap.add_argument("--batch", type=int, default=32)
    a = ap.parse_args()
    vgg16_fp16(a.batch)
