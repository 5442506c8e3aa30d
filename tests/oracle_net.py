"""Runs a topology spec on the CPU oracle, primitive by primitive, in the
caller's bfyx layout -- the reference network with build_option::optimize_data
off, where every primitive runs its reference kernel.  Test infrastructure.
"""
import numpy as np

import oracle_lib
from cldnn_b200 import abi
from cldnn_b200 import cldnn as cl


def _act(with_activation, slope):
    if not with_activation:
        return abi.ACT_NONE, 0.0
    return (abi.ACT_RELU, 0.0) if slope == 0.0 else (abi.ACT_RELU_NEGATIVE_SLOPE, slope)


def _tensor(arr):
    b, f, y, x = arr.shape
    return abi.tensor(abi.dtype_of(arr.dtype), b, f, y, x, "bfyx")[0]


def _fusable_activations(spec):
    """The activation folding of the optimising build (prepare_primitive_fusing.cpp, fuse_activation): an `activation`
    whose only producer is a convolution without an activation of its own, consumed by nobody else and not an output,
    moves into the convolution, where it acts on the dequantised value before the requantisation.
    Returns {convolution id: (func, a, b)} and {activation id: convolution id}."""
    users = {}
    for p in spec.prims:
        for k in ("input", "input2"):
            if k in p.args:
                users.setdefault(p.args[k], []).append(p.id)
    by_id = {p.id: p for p in spec.prims}
    into, alias = {}, {}
    for p in spec.prims:
        if p.kind != "activation":
            continue
        prod = by_id.get(p.args["input"])
        if prod is None or prod.kind not in ("convolution",) or prod.args["with_activation"]:
            continue
        if users.get(prod.id, []) != [p.id] or prod.id in spec.outputs or prod.id in into:
            continue
        into[prod.id] = (p.args["func"], p.args["a"], p.args["b"])
        alias[p.id] = prod.id
    return into, alias


def run(spec, inputs, threads=0, stats=None, keep=None, conv_impl="oracle", fuse_activations=False):
    """inputs: {input id: logical [b,f,y,x] array}.  Returns {primitive id: logical array} for spec.outputs
    (or for the ids in `keep`; keep=True keeps everything).  `stats`, if a dict, receives per-primitive
    fractions of zero / saturated outputs for 8-bit results.  conv_impl="reference" runs the convolutions on the reference's
    own kernel source (oracle/_ref) where a variant exists, the C restatement elsewhere."""
    vals = dict(inputs)
    act_into, act_alias = _fusable_activations(spec) if fuse_activations else ({}, {})
    users = {}
    for p in spec.prims:
        for k in ("input", "input2"):
            if k in p.args:
                users[p.args[k]] = p.id
    wanted = set(spec.outputs) if keep is None else (None if keep is True else set(keep) | set(spec.outputs))
    for p in spec.prims:
        a, k = p.args, p.kind
        if k == "data":
            arr = a["array"]
            vals[p.id] = arr.reshape(1, 1, 1, -1) if arr.ndim == 1 else arr
            continue
        if k == "input_layout":
            assert p.id in vals, "missing input " + p.id
            continue
        if p.id in act_alias:                      # folded into its convolution
            vals[p.id] = vals[act_alias[p.id]]
            continue
        x = vals[a["input"]]
        if k in ("convolution", "fused_conv_eltwise"):
            w = vals[a["weights"]]
            cp = abi.ConvParams()
            cp.in_ = _tensor(x)
            groups = a.get("groups", 1)
            K, ifm, kh, kw = w.shape
            P = oracle_lib.conv_out_size(x.shape[2], kh, a["input_offset"][1], a["stride"][1], a["dilation"][1])
            Q = oracle_lib.conv_out_size(x.shape[3], kw, a["input_offset"][0], a["stride"][0], a["dilation"][0])
            odt = abi.np_dtype_of(a["output_data_type"]) if a["output_data_type"] != abi.NONE else x.dtype
            out = np.zeros((x.shape[0], K, P, Q), dtype=odt)
            cp.out = _tensor(out)
            abi.set_weights(cp, abi.dtype_of(w.dtype), groups, K // groups, ifm, kh, kw)
            cp.stride_x, cp.stride_y = a["stride"]
            cp.pad_x, cp.pad_y = max(-a["input_offset"][0], 0), max(-a["input_offset"][1], 0)
            cp.dil_x, cp.dil_y = a["dilation"]
            bias = vals[a["bias"]].reshape(-1) if a["bias"] else None
            cp.bias_dtype = abi.dtype_of(bias.dtype) if bias is not None else abi.NONE
            quant = vals[a["weights_quantization_factors"]].reshape(-1) if a["weights_quantization_factors"] else None
            calib = vals[a["output_calibration_factors"]].reshape(-1) if a["output_calibration_factors"] else None
            cp.quantization, cp.calibration = int(quant is not None), int(calib is not None)
            cp.i_qf = a["input_quantization_factor"]
            cp.o_qf = a.get("output_quantization_factor", 1.0)
            cp.act, cp.act_m = _act(a["with_activation"], a["activation_negative_slope"])
            if p.id in act_into:
                cp.act, cp.act_m, cp.act_n = act_into[p.id]
            cp.eltw_stride_x = cp.eltw_stride_y = 1
            eltw = ecal = None
            if k == "fused_conv_eltwise":
                eltw = vals[a["input2"]]
                cp.fused_eltw = 1
                cp.eltw = _tensor(eltw)
                cp.has_o_qf = cp.quantization
                cp.has_non_conv_scale = int(a["non_conv_scale"] != 1.0)
                cp.non_conv_scale = a["non_conv_scale"]
                cp.eltw_act, cp.eltw_m = _act(a["eltw_activation"], a["eltw_activation_negative_slope"])
                ecal = vals[a["eltw_output_calibration_factors"]].reshape(-1) if a["eltw_output_calibration_factors"] else None
                cp.eltw_calibration = int(ecal is not None)
                cp.eltw_stride_x, cp.eltw_stride_y = a["eltw_stride"]
            else:
                cp.has_o_qf = int(cp.o_qf != 1.0 and not cp.calibration)
            impl = oracle_lib
            if conv_impl == "reference":
                import ref_lib
                if ref_lib.available(cp):
                    impl = ref_lib
                    if stats is not None:
                        stats["reference_kernel_convs"] = stats.get("reference_kernel_convs", 0) + 1
            flat = impl.conv(cp, x.reshape(-1), w.reshape(-1), bias, quant, calib,
                             eltw.reshape(-1) if eltw is not None else None, ecal, threads=threads or oracle_lib.num_threads())
            res = flat.reshape(out.shape)
        elif k == "pooling":
            pp = abi.PoolParams()
            pp.in_ = _tensor(x)
            glob = a["global_pooling"]
            sx, sy = (x.shape[3], x.shape[2]) if glob else a["size"]
            stx, sty = (1, 1) if glob else a["stride"]
            ox, oy = a["input_offset"]
            P = 1 if glob else oracle_lib.pool_out_size(x.shape[2], sy, oy, sty)
            Q = 1 if glob else oracle_lib.pool_out_size(x.shape[3], sx, ox, stx)
            out = np.zeros((x.shape[0], x.shape[1], P, Q), dtype=x.dtype)
            pp.out = _tensor(out)
            pp.size_x, pp.size_y, pp.stride_x, pp.stride_y = sx, sy, stx, sty
            pp.pad_x, pp.pad_y = max(-ox, 0), max(-oy, 0)
            pp.mode = abi.POOL_MAX if a["mode"] == cl.pooling_mode.max else abi.POOL_AVG
            dyn = ((Q - 1) * stx + sx) > 2 * pp.pad_x + x.shape[3] or ((P - 1) * sty + sy) > 2 * pp.pad_y + x.shape[2]
            if a["mode"] == cl.pooling_mode.average and dyn:
                pp.div_mode = abi.DIV_DYNAMIC_WITH_PADDING
            else:
                pp.div_mode = abi.DIV_DYNAMIC if a["mode"] == cl.pooling_mode.average_no_padding else abi.DIV_FIXED
            res = oracle_lib.pooling(pp, x.reshape(-1), threads=threads).reshape(out.shape)
        elif k == "fully_connected":
            w = vals[a["weights"]]
            fp = abi.FcParams()
            fp.in_ = _tensor(x)
            out = np.zeros((x.shape[0], w.shape[0], 1, 1), dtype=x.dtype)
            fp.out = _tensor(out)
            fp.w_dtype = abi.dtype_of(w.dtype)
            fp.w_px, fp.w_py, fp.w_pi, fp.w_po = 1, w.shape[3], w.shape[3] * w.shape[2], w.shape[3] * w.shape[2] * w.shape[1]
            bias = vals[a["bias"]].reshape(-1) if a["bias"] else None
            fp.bias_dtype = abi.dtype_of(bias.dtype) if bias is not None else abi.NONE
            quant = vals[a["weights_quantization_factors"]].reshape(-1) if a["weights_quantization_factors"] else None
            calib = vals[a["output_calibration_factors"]].reshape(-1) if a["output_calibration_factors"] else None
            fp.quantization, fp.calibration = int(quant is not None), int(calib is not None)
            fp.i_qf, fp.o_qf = a["input_quantization_factor"], a["output_quantization_factor"]
            fp.act, fp.act_m = _act(a["with_activation"], a["activation_negative_slope"])
            flat, oor = oracle_lib.fc(fp, x.reshape(-1), w.reshape(-1), bias, quant, calib, threads=threads)
            if stats is not None:
                stats[p.id + ":out_of_range"] = oor
            res = flat.reshape(out.shape)
        elif k == "softmax":
            sp = abi.SoftmaxParams()
            sp.in_ = _tensor(x)
            sp.out = _tensor(x)
            sp.dimension = int(a.get("dimension", abi.SOFTMAX_FYX))
            res = oracle_lib.softmax(sp, x.reshape(-1)).reshape(x.shape)
        elif k == "reorder":
            odt = abi.np_dtype_of(a["out_data_type"]) if a["out_data_type"] != abi.NONE else x.dtype
            rp = abi.ReorderParams()
            rp.in_ = _tensor(x)
            out = np.zeros(x.shape, dtype=odt)
            rp.out = _tensor(out)
            sub = a["subtract_per_feature"]
            if sub:
                rp.has_mean = 1
                for i in range(4):
                    rp.mean[i] = sub[min(i, len(sub) - 1)]
            res = oracle_lib.reorder(rp, x.reshape(-1)).reshape(out.shape)     # logical values only: layout is a storage detail
        elif k == "eltwise":
            y2 = vals[a["input2"]]
            ep = abi.EltwiseParams()
            ep.in0, ep.in1 = _tensor(x), _tensor(y2)
            out = np.zeros(tuple(max(i, j) for i, j in zip(x.shape, y2.shape)), dtype=x.dtype)
            ep.out = _tensor(out)
            ep.mode = a["mode"]
            ep.stride_x0 = ep.stride_y0 = ep.stride_x1 = ep.stride_y1 = 1
            calib = vals[a["output_calibration_factors"]].reshape(-1) if a["output_calibration_factors"] else None
            ep.quantization, ep.calibration, ep.o_qf = int(a["quantized"]), int(calib is not None), a["output_quantization_factor"]
            ep.act, ep.act_m = _act(a["with_activation"], a["activation_negative_slope"])
            res = oracle_lib.eltwise(ep, x.reshape(-1), y2.reshape(-1), calib).reshape(out.shape)
        elif k == "activation":
            ap = abi.ActivationParams()
            ap.in_, ap.out = _tensor(x), _tensor(x)
            ap.act, ap.act_m, ap.act_n = a["func"], a["a"], a["b"]
            res = oracle_lib.activation(ap, x.reshape(-1)).reshape(x.shape)
        elif k == "lrn":
            lp = abi.LrnParams()
            lp.in_, lp.out = _tensor(x), _tensor(x)
            lp.size, lp.k, lp.alpha, lp.beta = a["size"], a["k"], a["alpha"], a["beta"]
            res = oracle_lib.lrn(lp, x.reshape(-1)).reshape(x.shape)
        elif k == "concatenation":
            # concatenation_gpu_ref.cl: every input copied to its offset along the axis (tensor sizes are b, f, x, y; arrays are [b, f, y, x])
            res = np.concatenate([vals[i] for i in a["inputs"]], axis={0: 0, 1: 1, 2: 3, 3: 2}[a["axis"]])
        else:
            raise ValueError("oracle_net: primitive kind " + k)
        vals[p.id] = res
        if stats is not None and res.dtype.kind in "iu" and res.dtype.itemsize == 1:
            hi = np.iinfo(res.dtype).max
            stats[p.id] = dict(zero=float((res == 0).mean()), saturated=float((res == hi).mean()))
    if wanted is None:
        return vals
    return {k: v for k, v in vals.items() if k in wanted}
