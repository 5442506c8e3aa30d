"""Python binding of the host layer (include/cldnn_host.h), shaped like clDNN's
C++ API (api/CPP/*.hpp): engine, memory, layout, tensor, topology, the
primitives of the convolution path, build options and network.

Only plumbing lives here.  Topologies are built and run by libcldnn_host.so,
every kernel by libcldnn_b200.so; a missing library or device raises.
"""
import ctypes as C
import os

import numpy as np

from . import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
HOST_LIB_PATH = os.path.join(_HERE, "libcldnn_host.so")


class data_types:
    i8, u8, i32, f16, f32, none = abi.I8, abi.U8, abi.I32, abi.F16, abi.F32, abi.NONE


class format:
    yxfb, byxf, bfyx, byxf_af32 = 0, 1, 2, 21
    names = {0: "yxfb", 1: "byxf", 2: "bfyx", 21: "byxf_af32"}


class eltwise_mode:
    sum, sub, max, prod, min = 0, 1, 2, 3, 4


class pooling_mode:
    max, average, average_no_padding = 0, 1, 2


class tuning_mode:
    tuning_disabled, tuning_use_cache, tuning_tune_and_cache = 0, 1, 2


class activation_func:
    none, relu, relu_negative_slope, clamp = abi.ACT_NONE, abi.ACT_RELU, abi.ACT_RELU_NEGATIVE_SLOPE, abi.ACT_CLAMP
    logistic, hyperbolic_tan, abs, linear, square, sqrt, elu = (abi.ACT_LOGISTIC, abi.ACT_TANH, abi.ACT_ABS, abi.ACT_LINEAR,
                                                                abi.ACT_SQUARE, abi.ACT_SQRT, abi.ACT_ELU)


class _BuildOptions(C.Structure):
    _fields_ = [("optimize_data", C.c_uint32), ("fuse_any_conv_eltwise", C.c_uint32), ("tuning_mode", C.c_uint32),
                ("tuning_cache_path", C.c_char_p), ("outputs", C.c_char_p), ("use_graph", C.c_uint32),
                ("force_kernel", C.c_char_p)]


_vp, _cp, _i, _u, _f = C.c_void_p, C.c_char_p, C.c_int32, C.c_uint32, C.c_float
_SIGNATURES = {
    "cldnn_host_last_error": (C.c_char_p, []),
    "cldnn_host_engine_create": (_i, [_i, _u, C.POINTER(_vp)]),
    "cldnn_host_engine_release": (_i, [_vp]),
    "cldnn_host_engine_info": (_i, [_vp, C.POINTER(abi.EngineInfo)]),
    "cldnn_host_engine_stream": (_i, [_vp, C.POINTER(_vp)]),
    "cldnn_host_memory_allocate": (_i, [_vp, _i, _i, _i, _i, _i, _i, C.POINTER(_vp)]),
    "cldnn_host_memory_attach": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, C.POINTER(_vp)]),
    "cldnn_host_memory_release": (_i, [_vp]),
    "cldnn_host_memory_write": (_i, [_vp, _vp, C.c_size_t]),
    "cldnn_host_memory_read": (_i, [_vp, _vp, C.c_size_t]),
    "cldnn_host_memory_layout": (_i, [_vp] + [C.POINTER(_i)] * 6 + [C.POINTER(C.c_size_t)]),
    "cldnn_host_memory_device_ptr": (_i, [_vp, C.POINTER(_vp)]),
    "cldnn_host_topology_create": (_i, [C.POINTER(_vp)]),
    "cldnn_host_topology_release": (_i, [_vp]),
    "cldnn_host_add_input_layout": (_i, [_vp, _cp, _i, _i, _i, _i, _i, _i]),
    "cldnn_host_add_data": (_i, [_vp, _cp, _vp]),
    "cldnn_host_add_reorder": (_i, [_vp, _cp, _cp, _i, _i, C.POINTER(_f), C.c_size_t]),
    "cldnn_host_add_convolution": (_i, [_vp, _cp, _cp, _cp, _cp, _cp, _cp, _f, _f, _i, _i, _i, _i, _i, _i, _i, _u, _f, _u]),
    "cldnn_host_add_fused_conv_eltwise": (_i, [_vp, _cp, _cp, _cp, _cp, _cp, _cp, _cp, _f, _f, _cp, _i, _i, _i, _i, _i, _i, _i, _i,
                                               _u, _f, _u, _f, _i]),
    "cldnn_host_add_eltwise": (_i, [_vp, _cp, _cp, _cp, _i, _u, _f, _cp, _f, _u]),
    "cldnn_host_add_activation": (_i, [_vp, _cp, _cp, _i, _f, _f]),
    "cldnn_host_add_pooling": (_i, [_vp, _cp, _cp, _i, _u, _i, _i, _i, _i, _i, _i]),
    "cldnn_host_add_fully_connected": (_i, [_vp, _cp, _cp, _cp, _cp, _cp, _cp, _f, _f, _u, _f]),
    "cldnn_host_add_softmax": (_i, [_vp, _cp, _cp]),
    "cldnn_host_add_softmax_dim": (_i, [_vp, _cp, _cp, C.c_int32]),
    "cldnn_host_add_lrn": (_i, [_vp, _cp, _cp, _u, _f, _f, _f]),
    "cldnn_host_add_concatenation": (_i, [_vp, _cp, _cp, _i]),
    "cldnn_host_tuning_cache_check": (_i, [_cp, _u, C.POINTER(C.c_size_t)]),
    "cldnn_host_network_build": (_i, [_vp, _vp, C.POINTER(_BuildOptions), C.POINTER(_vp)]),
    "cldnn_host_network_release": (_i, [_vp]),
    "cldnn_host_network_set_input": (_i, [_vp, _cp, _vp]),
    "cldnn_host_network_execute": (_i, [_vp]),
    "cldnn_host_network_wait": (_i, [_vp]),
    "cldnn_host_network_get_output": (_i, [_vp, _cp, C.POINTER(_vp)]),
    "cldnn_host_network_info": (_i, [_vp, _cp, C.c_size_t, C.POINTER(C.c_size_t)]),
    "cldnn_host_network_profiling": (_i, [_vp, _cp, C.c_size_t, C.POINTER(C.c_size_t)]),
    "cldnn_host_network_stats": (_i, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_size_t)]),
}

_lib = None


class error(RuntimeError):
    def __init__(self, status, message):
        super().__init__("cldnn status %d: %s" % (status, message))
        self.status = status


def load_library():
    global _lib
    if _lib is None:
        if not os.path.exists(HOST_LIB_PATH):
            raise error(abi.ERROR, "%s is missing: build it with `make -C cldnn_b200/host` (there is no CPU fallback)" % HOST_LIB_PATH)
        lib = C.CDLL(HOST_LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def declared_symbols():
    return sorted(_SIGNATURES)


def _check(status):
    if status != abi.SUCCESS:
        raise error(status, load_library().cldnn_host_last_error().decode("utf-8", "replace"))


def _b(s):
    return (s or "").encode()


class tensor:
    """cldnn::tensor(batch, feature, x, y)."""

    def __init__(self, batch=1, feature=1, x=1, y=1):
        self.batch, self.feature, self.x, self.y = batch, feature, x, y

    def __eq__(self, o):
        return (self.batch, self.feature, self.x, self.y) == (o.batch, o.feature, o.x, o.y)

    def __repr__(self):
        return "tensor(b=%d, f=%d, x=%d, y=%d)" % (self.batch, self.feature, self.x, self.y)


class layout:
    def __init__(self, data_type, fmt, size):
        self.data_type, self.format, self.size = data_type, fmt, size

    def np_dtype(self):
        return abi.np_dtype_of(self.data_type)

    def fmt_name(self):
        return "byxf" if self.format == format.byxf_af32 else format.names[self.format]

    def f_align(self):
        return 32 if self.format == format.byxf_af32 else 1


class engine:
    def __init__(self, device=0, enable_profiling=False):
        self.lib = load_library()
        self.handle = _vp()
        _check(self.lib.cldnn_host_engine_create(device, int(enable_profiling), C.byref(self.handle)))

    def get_info(self):
        info = abi.EngineInfo()
        _check(self.lib.cldnn_host_engine_info(self.handle, C.byref(info)))
        return info

    def stream(self):
        s = _vp()
        _check(self.lib.cldnn_host_engine_stream(self.handle, C.byref(s)))
        return s.value

    def release(self):
        if self.handle:
            self.lib.cldnn_host_engine_release(self.handle)
            self.handle = _vp()


class memory:
    def __init__(self, lib, handle):
        self.lib, self.handle = lib, handle
        dt, fmt, b, f, x, y, nbytes = _i(), _i(), _i(), _i(), _i(), _i(), C.c_size_t()
        _check(lib.cldnn_host_memory_layout(handle, C.byref(dt), C.byref(fmt), C.byref(b), C.byref(f), C.byref(x), C.byref(y), C.byref(nbytes)))
        self._layout = layout(dt.value, fmt.value, tensor(b.value, f.value, x.value, y.value))
        self.nbytes = nbytes.value

    @staticmethod
    def allocate(eng, lay):
        h = _vp()
        _check(eng.lib.cldnn_host_memory_allocate(eng.handle, lay.data_type, lay.format, lay.size.batch, lay.size.feature, lay.size.x, lay.size.y, C.byref(h)))
        return memory(eng.lib, h)

    @staticmethod
    def attach(eng, lay, device_ptr):
        """Wrap device memory owned by the caller (cldnn::memory::attach)."""
        h = _vp()
        _check(eng.lib.cldnn_host_memory_attach(eng.handle, lay.data_type, lay.format, lay.size.batch, lay.size.feature, lay.size.x, lay.size.y,
                                                device_ptr, C.byref(h)))
        return memory(eng.lib, h)

    @staticmethod
    def from_numpy(eng, arr_bfyx, fmt=format.bfyx):
        """Allocate a memory for a logical [b, f, y, x] array and fill it (set_values of the reference's tests)."""
        a = np.asarray(arr_bfyx)
        if a.ndim == 1:
            a = a.reshape(1, 1, 1, -1)              # per-feature constants: tensor(1, 1, n, 1) like the reference's tests
        b, f, y, x = a.shape
        m = memory.allocate(eng, layout(abi.dtype_of(a.dtype), fmt, tensor(b, f, x, y)))
        m.set_values(a)
        return m

    def get_layout(self):
        return self._layout

    def set_values(self, arr_bfyx):
        lay = self._layout
        flat = abi.to_layout(np.asarray(arr_bfyx, dtype=lay.np_dtype()).reshape(lay.size.batch, lay.size.feature, lay.size.y, lay.size.x),
                             lay.fmt_name(), lay.f_align())
        self.write_flat(flat)

    def write_flat(self, flat):
        flat = np.ascontiguousarray(flat)
        _check(self.lib.cldnn_host_memory_write(self.handle, flat.ctypes.data_as(_vp), flat.nbytes))

    def read_flat(self):
        out = np.empty(self.nbytes // self._layout.np_dtype().itemsize, dtype=self._layout.np_dtype())
        _check(self.lib.cldnn_host_memory_read(self.handle, out.ctypes.data_as(_vp), out.nbytes))
        return out

    def to_numpy(self):
        """Logical [b, f, y, x] view of the contents (memory::pointer<T> of the reference)."""
        lay = self._layout
        return abi.from_layout(self.read_flat(), (lay.size.batch, lay.size.feature, lay.size.y, lay.size.x), lay.fmt_name(), lay.f_align())

    def device_ptr(self):
        p = _vp()
        _check(self.lib.cldnn_host_memory_device_ptr(self.handle, C.byref(p)))
        return p.value

    def release(self):
        if self.handle:
            self.lib.cldnn_host_memory_release(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class primitive:
    """A topology entry; `kind` is the reference's primitive name, `args` its descriptor fields."""

    def __init__(self, kind, id, **args):
        self.kind, self.id, self.args = kind, id, args

    def __getattr__(self, name):
        try:
            return self.__dict__["args"][name]
        except KeyError:
            raise AttributeError(name)


def _xy(t, default=(1, 1)):
    if t is None:
        return default
    if isinstance(t, tensor):
        return (t.x, t.y)
    return tuple(t)


def input_layout(id, lay):
    return primitive("input_layout", id, layout=lay)


def data(id, mem):
    return primitive("data", id, mem=mem)


def reorder(id, input, out_format, out_data_type=data_types.none, subtract_per_feature=()):
    return primitive("reorder", id, input=input, out_format=out_format, out_data_type=out_data_type, subtract_per_feature=tuple(subtract_per_feature))


def convolution(id, input, weights, bias="", weights_quantization_factors="", output_calibration_factors="",
                input_quantization_factor=1.0, output_data_type=data_types.none, stride=(1, 1), input_offset=(0, 0),
                dilation=(1, 1), with_activation=False, activation_negative_slope=0.0, groups=1, output_quantization_factor=1.0):
    return primitive("convolution", id, input=input, weights=weights, bias=bias, weights_quantization_factors=weights_quantization_factors,
                     output_calibration_factors=output_calibration_factors, input_quantization_factor=input_quantization_factor,
                     output_quantization_factor=output_quantization_factor, output_data_type=output_data_type, stride=_xy(stride),
                     input_offset=_xy(input_offset, (0, 0)), dilation=_xy(dilation), with_activation=with_activation,
                     activation_negative_slope=activation_negative_slope, groups=groups)


def fused_conv_eltwise(id, input, input2, weights, bias="", conv_w_quantization_factor="", conv_output_calibration_factors="",
                       conv_i_quantization_factor=1.0, non_conv_scale=1.0, eltw_output_calibration_factors="", eltw_stride=(1, 1),
                       stride=(1, 1), input_offset=(0, 0), dilation=(1, 1), conv_with_activation=False, conv_activation_slp=0.0,
                       eltw_activation=False, eltw_activation_slp=0.0, output_data_type=data_types.none):
    return primitive("fused_conv_eltwise", id, input=input, input2=input2, weights=weights, bias=bias,
                     weights_quantization_factors=conv_w_quantization_factor, output_calibration_factors=conv_output_calibration_factors,
                     input_quantization_factor=conv_i_quantization_factor, non_conv_scale=non_conv_scale,
                     eltw_output_calibration_factors=eltw_output_calibration_factors, eltw_stride=_xy(eltw_stride), stride=_xy(stride),
                     input_offset=_xy(input_offset, (0, 0)), dilation=_xy(dilation), with_activation=conv_with_activation,
                     activation_negative_slope=conv_activation_slp, eltw_activation=eltw_activation,
                     eltw_activation_negative_slope=eltw_activation_slp, output_data_type=output_data_type)


def eltwise(id, input, input2, mode=eltwise_mode.sum, with_activation=False, activation_negative_slope=0.0,
            output_calibration_factors="", output_quantization_factor=1.0, quantized=False):
    return primitive("eltwise", id, input=input, input2=input2, mode=mode, with_activation=with_activation,
                     activation_negative_slope=activation_negative_slope, output_calibration_factors=output_calibration_factors,
                     output_quantization_factor=output_quantization_factor,
                     quantized=bool(quantized or output_calibration_factors or output_quantization_factor != 1.0))


def activation(id, input, func, a=0.0, b=0.0):
    return primitive("activation", id, input=input, func=func, a=a, b=b)


def pooling(id, input, mode, size=(1, 1), stride=(1, 1), input_offset=(0, 0), global_pooling=False):
    return primitive("pooling", id, input=input, mode=mode, size=_xy(size), stride=_xy(stride), input_offset=_xy(input_offset, (0, 0)),
                     global_pooling=global_pooling)


def fully_connected(id, input, weights, bias="", weights_quantization_factors="", output_calibration_factors="",
                    input_quantization_factor=1.0, output_quantization_factor=1.0, with_activation=False, activation_negative_slope=0.0):
    return primitive("fully_connected", id, input=input, weights=weights, bias=bias, weights_quantization_factors=weights_quantization_factors,
                     output_calibration_factors=output_calibration_factors, input_quantization_factor=input_quantization_factor,
                     output_quantization_factor=output_quantization_factor, with_activation=with_activation,
                     activation_negative_slope=activation_negative_slope)


class softmax_dimension:
    """softmax::dimension_t (api/CPP/softmax.hpp:44-50)."""
    normalize_f, normalize_x, normalize_y, normalize_fyx = 0, 1, 2, 3


def softmax(id, input, dimension=softmax_dimension.normalize_fyx):
    return primitive("softmax", id, input=input, dimension=dimension)


def lrn(id, input, size=5, k=1.0, alpha=1e-4, beta=0.75):
    return primitive("lrn", id, input=input, size=size, k=k, alpha=alpha, beta=beta)


class concatenation_axis:
    """concatenation::concatenation_axis (api/CPP/concatenation.hpp:44-52): the index into the tensor's sizes."""
    along_b, along_f, along_x, along_y = 0, 1, 2, 3


def concatenation(id, inputs, axis=concatenation_axis.along_f):
    inputs = list(inputs)
    return primitive("concatenation", id, input=inputs[0], inputs=inputs, axis=axis)


class topology:
    def __init__(self, *prims):
        self.prims = []
        for p in prims:
            self.add(p)

    def add(self, *prims):
        for p in prims:
            self.prims.append(p)
        return self

    def _realise(self, lib):
        h = _vp()
        _check(lib.cldnn_host_topology_create(C.byref(h)))
        try:
            for p in self.prims:
                a, k = p.args, p.kind
                if k == "input_layout":
                    lay = a["layout"]
                    st = lib.cldnn_host_add_input_layout(h, _b(p.id), lay.data_type, lay.format, lay.size.batch, lay.size.feature, lay.size.x, lay.size.y)
                elif k == "data":
                    st = lib.cldnn_host_add_data(h, _b(p.id), a["mem"].handle)
                elif k == "reorder":
                    sub = a["subtract_per_feature"]
                    arr = (_f * len(sub))(*sub) if sub else None
                    st = lib.cldnn_host_add_reorder(h, _b(p.id), _b(a["input"]), a["out_format"], a["out_data_type"], arr, len(sub))
                elif k == "convolution":
                    st = lib.cldnn_host_add_convolution(h, _b(p.id), _b(a["input"]), _b(a["weights"]), _b(a["bias"]), _b(a["weights_quantization_factors"]),
                                                        _b(a["output_calibration_factors"]), a["input_quantization_factor"], a["output_quantization_factor"],
                                                        a["output_data_type"], a["stride"][0], a["stride"][1], a["input_offset"][0], a["input_offset"][1],
                                                        a["dilation"][0], a["dilation"][1], int(a["with_activation"]), a["activation_negative_slope"], a["groups"])
                elif k == "fused_conv_eltwise":
                    st = lib.cldnn_host_add_fused_conv_eltwise(h, _b(p.id), _b(a["input"]), _b(a["input2"]), _b(a["weights"]), _b(a["bias"]),
                                                               _b(a["weights_quantization_factors"]), _b(a["output_calibration_factors"]),
                                                               a["input_quantization_factor"], a["non_conv_scale"], _b(a["eltw_output_calibration_factors"]),
                                                               a["eltw_stride"][0], a["eltw_stride"][1], a["stride"][0], a["stride"][1],
                                                               a["input_offset"][0], a["input_offset"][1], a["dilation"][0], a["dilation"][1],
                                                               int(a["with_activation"]), a["activation_negative_slope"], int(a["eltw_activation"]),
                                                               a["eltw_activation_negative_slope"], a["output_data_type"])
                elif k == "eltwise":
                    st = lib.cldnn_host_add_eltwise(h, _b(p.id), _b(a["input"]), _b(a["input2"]), a["mode"], int(a["with_activation"]),
                                                    a["activation_negative_slope"], _b(a["output_calibration_factors"]), a["output_quantization_factor"],
                                                    int(a["quantized"]))
                elif k == "activation":
                    st = lib.cldnn_host_add_activation(h, _b(p.id), _b(a["input"]), a["func"], a["a"], a["b"])
                elif k == "pooling":
                    st = lib.cldnn_host_add_pooling(h, _b(p.id), _b(a["input"]), a["mode"], int(a["global_pooling"]), a["size"][0], a["size"][1],
                                                    a["stride"][0], a["stride"][1], a["input_offset"][0], a["input_offset"][1])
                elif k == "fully_connected":
                    st = lib.cldnn_host_add_fully_connected(h, _b(p.id), _b(a["input"]), _b(a["weights"]), _b(a["bias"]), _b(a["weights_quantization_factors"]),
                                                            _b(a["output_calibration_factors"]), a["input_quantization_factor"], a["output_quantization_factor"],
                                                            int(a["with_activation"]), a["activation_negative_slope"])
                elif k == "softmax":
                    st = lib.cldnn_host_add_softmax_dim(h, _b(p.id), _b(a["input"]), int(a.get("dimension", 3)))
                elif k == "lrn":
                    st = lib.cldnn_host_add_lrn(h, _b(p.id), _b(a["input"]), a["size"], a["k"], a["alpha"], a["beta"])
                elif k == "concatenation":
                    st = lib.cldnn_host_add_concatenation(h, _b(p.id), _b(",".join(a["inputs"])), a["axis"])
                else:
                    raise error(abi.UNSUPPORTED_FORMAT, "primitive type '%s' is outside the supported path" % k)
                _check(st)
        except Exception:
            lib.cldnn_host_topology_release(h)
            raise
        return h


class build_options:
    """build_option::optimize_data / tuning_config / outputs (api/CPP/program.hpp:108-138)."""

    def __init__(self, optimize_data=False, fuse_any_conv_eltwise=True, tuning=tuning_mode.tuning_disabled, tuning_cache_path=None,
                 outputs=None, use_graph=True, force_kernel=None):
        self.optimize_data, self.fuse_any_conv_eltwise, self.tuning = optimize_data, fuse_any_conv_eltwise, tuning
        self.tuning_cache_path, self.outputs, self.use_graph, self.force_kernel = tuning_cache_path, outputs, use_graph, force_kernel


class network:
    def __init__(self, eng, topo, options=None):
        self.engine, self.lib = eng, eng.lib
        o = options or build_options()
        bo = _BuildOptions(int(o.optimize_data), int(o.fuse_any_conv_eltwise), int(o.tuning),
                           _b(o.tuning_cache_path) if o.tuning_cache_path else None,
                           _b(",".join(o.outputs)) if o.outputs else None, int(o.use_graph),
                           _b(o.force_kernel) if o.force_kernel else None)
        th = topo._realise(self.lib)
        self.handle = _vp()
        try:
            _check(self.lib.cldnn_host_network_build(eng.handle, th, C.byref(bo), C.byref(self.handle)))
        finally:
            self.lib.cldnn_host_topology_release(th)
        self._keep = [p.args["mem"] for p in topo.prims if p.kind == "data"]

    def set_input_data(self, id, mem):
        _check(self.lib.cldnn_host_network_set_input(self.handle, _b(id), mem.handle))
        self._keep.append(mem)

    def execute(self):
        _check(self.lib.cldnn_host_network_execute(self.handle))
        return self

    def wait(self):
        _check(self.lib.cldnn_host_network_wait(self.handle))

    def get_output(self, id):
        h = _vp()
        _check(self.lib.cldnn_host_network_get_output(self.handle, _b(id), C.byref(h)))
        return memory(self.lib, h)

    def primitives_info(self):
        need = C.c_size_t()
        _check(self.lib.cldnn_host_network_info(self.handle, None, 0, C.byref(need)))
        buf = C.create_string_buffer(need.value)
        _check(self.lib.cldnn_host_network_info(self.handle, buf, need.value, None))
        rows = []
        for line in buf.value.decode().splitlines():
            pid, kind, kernel, tune, fmt, dt, dims, fused, is_out, in_place = line.split("|")
            rows.append(dict(id=pid, type=kind, kernel=kernel, tune=int(tune), format=fmt, data_type=int(dt),
                             dims=tuple(int(v) for v in dims.split(",")), fused=[f for f in fused.split(",") if f], is_output=is_out == "1",
                             in_place=in_place == "1"))
        return rows

    def profiling_info(self):
        """{primitive id: device nanoseconds} of the last execute (engine created with enable_profiling)."""
        need = C.c_size_t()
        _check(self.lib.cldnn_host_network_profiling(self.handle, None, 0, C.byref(need)))
        buf = C.create_string_buffer(need.value)
        _check(self.lib.cldnn_host_network_profiling(self.handle, buf, need.value, None))
        return {l.split("|")[0]: int(l.split("|")[1]) for l in buf.value.decode().splitlines()}

    def stats(self):
        launches, pool = C.c_uint64(), C.c_size_t()
        _check(self.lib.cldnn_host_network_stats(self.handle, C.byref(launches), C.byref(pool)))
        return dict(launches_per_execute=launches.value, pool_bytes=pool.value)

    def release(self):
        if self.handle:
            self.lib.cldnn_host_network_release(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass
