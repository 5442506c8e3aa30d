"""ctypes binding of libcldnn_b200.so (include/cldnn_b200.h).

This is host plumbing only: it loads the CUDA library, owns handles and moves
bytes.  All compute happens in the library's sm_100a kernels; when the library
or a CUDA device is missing the calls raise, there is no fallback.
"""
import ctypes as C
import os

import numpy as np

from . import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcldnn_b200.so")

# every symbol include/cldnn_b200.h declares, with its argument types
_SIGNATURES = {
    "cldnn_b200_last_error": (C.c_char_p, []),
    "cldnn_b200_device_count": (C.c_int32, [C.POINTER(C.c_int32)]),
    "cldnn_b200_ctx_create": (C.c_int32, [C.c_int32, C.c_uint32, C.POINTER(C.c_void_p)]),
    "cldnn_b200_ctx_destroy": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_ctx_info": (C.c_int32, [C.c_void_p, C.POINTER(abi.EngineInfo)]),
    "cldnn_b200_ctx_flush": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_ctx_sync": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_ctx_stream": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "cldnn_b200_ctx_launch_count": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "cldnn_b200_ctx_device_status": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "cldnn_b200_mem_alloc": (C.c_int32, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "cldnn_b200_mem_attach": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "cldnn_b200_mem_free": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_mem_size": (C.c_int32, [C.c_void_p, C.POINTER(C.c_size_t)]),
    "cldnn_b200_mem_devptr": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "cldnn_b200_mem_map": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "cldnn_b200_mem_unmap": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_mem_fill": (C.c_int32, [C.c_void_p, C.c_uint8]),
    "cldnn_b200_mem_write": (C.c_int32, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "cldnn_b200_mem_read": (C.c_int32, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "cldnn_b200_mem_write_async": (C.c_int32, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "cldnn_b200_mem_read_async": (C.c_int32, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "cldnn_b200_host_alloc": (C.c_int32, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "cldnn_b200_host_free": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_event_create": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "cldnn_b200_event_record": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_event_wait": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_event_query": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32)]),
    "cldnn_b200_event_elapsed_ns": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint64)]),
    "cldnn_b200_event_destroy": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_kernel_count": (C.c_int32, []),
    "cldnn_b200_kernel_name": (C.c_char_p, [C.c_int32]),
    "cldnn_b200_kernel_lookup": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]),
    "cldnn_b200_kernel_supports": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_int32)]),
    "cldnn_b200_kernel_tune_count": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_int32)]),
    "cldnn_b200_kernel_scratch_bytes": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "cldnn_b200_launch": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(abi.Args)]),
    "cldnn_b200_prepare": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(abi.Args), C.POINTER(C.c_void_p)]),
    "cldnn_b200_run": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_prepared_destroy": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_time": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_uint64)]),
    "cldnn_b200_conv_first_noalloc": (C.c_int32, [C.c_void_p, C.POINTER(abi.ConvParams), C.POINTER(abi.Args)]),
    "cldnn_b200_tensor_peak": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_double)]),
    "cldnn_b200_graph_begin": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_graph_end": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "cldnn_b200_graph_launch": (C.c_int32, [C.c_void_p]),
    "cldnn_b200_graph_destroy": (C.c_int32, [C.c_void_p]),
}

_lib = None


class EngineError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("cldnn_b200 status %d: %s" % (status, message))
        self.status = status


def load_library():
    """Load libcldnn_b200.so and bind every declared entry point."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise EngineError(abi.ERROR, "%s is missing: build it with `make -C cldnn_b200/csrc` "
                                         "(there is no CPU fallback)" % LIB_PATH)
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def declared_symbols():
    return sorted(_SIGNATURES)


def _check(status):
    if status != abi.SUCCESS:
        raise EngineError(status, load_library().cldnn_b200_last_error().decode("utf-8", "replace"))


class Memory:
    """A device buffer (gpu_buffer of the reference, src/gpu/memory_gpu.h:62-83)."""

    def __init__(self, engine, nbytes):
        self.engine = engine
        self.nbytes = int(nbytes)
        self.handle = C.c_void_p()
        _check(engine.lib.cldnn_b200_mem_alloc(engine.handle, self.nbytes, C.byref(self.handle)))
        ptr = C.c_void_p()
        _check(engine.lib.cldnn_b200_mem_devptr(self.handle, C.byref(ptr)))
        self.ptr = ptr.value

    def write(self, array, offset=0):
        a = np.ascontiguousarray(array)
        _check(self.engine.lib.cldnn_b200_mem_write(self.handle, offset, a.ctypes.data_as(C.c_void_p), a.nbytes))

    def read(self, dtype, count=None, offset=0):
        dtype = np.dtype(dtype)
        if count is None:
            count = (self.nbytes - offset) // dtype.itemsize
        out = np.empty(count, dtype=dtype)
        _check(self.engine.lib.cldnn_b200_mem_read(self.handle, offset, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def fill(self, byte):
        _check(self.engine.lib.cldnn_b200_mem_fill(self.handle, byte))

    def free(self):
        # a buffer must not outlive its context: after Engine.close() only drop the handle
        if self.handle and self.engine.handle:
            self.engine.lib.cldnn_b200_mem_free(self.handle)
        self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Prepared:
    def __init__(self, engine, handle):
        self.engine, self.handle = engine, handle

    def run(self):
        _check(self.engine.lib.cldnn_b200_run(self.handle))

    def time_ns(self, warmup=3, runs=10):
        ns = C.c_uint64()
        _check(self.engine.lib.cldnn_b200_time(self.handle, warmup, runs, C.byref(ns)))
        return ns.value

    def destroy(self):
        if self.handle:
            self.engine.lib.cldnn_b200_prepared_destroy(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class Kernel:
    def __init__(self, engine, name):
        self.engine, self.name = engine, name
        self.handle = C.c_void_p()
        _check(engine.lib.cldnn_b200_kernel_lookup(engine.handle, name.encode(), C.byref(self.handle)))

    def supports(self, params):
        yes = C.c_int32()
        _check(self.engine.lib.cldnn_b200_kernel_supports(self.handle, C.byref(params), C.sizeof(params), C.byref(yes)))
        return bool(yes.value)

    def tune_count(self, params):
        n = C.c_int32()
        _check(self.engine.lib.cldnn_b200_kernel_tune_count(self.handle, C.byref(params), C.sizeof(params), C.byref(n)))
        return n.value

    def launch(self, params, args):
        _check(self.engine.lib.cldnn_b200_launch(self.handle, C.byref(params), C.sizeof(params), C.byref(args)))

    def prepare(self, params, args):
        h = C.c_void_p()
        _check(self.engine.lib.cldnn_b200_prepare(self.handle, C.byref(params), C.sizeof(params), C.byref(args), C.byref(h)))
        return Prepared(self.engine, h)


class Engine:
    """One CUDA context + stream on one B200 (gpu_toolkit of the reference,
    src/gpu/ocl_toolkit.h:59-137)."""

    def __init__(self, device=0, enable_profiling=False):
        self.lib = load_library()
        self.handle = C.c_void_p()
        _check(self.lib.cldnn_b200_ctx_create(device, int(enable_profiling), C.byref(self.handle)))
        self._kernels = {}

    def info(self):
        info = abi.EngineInfo()
        _check(self.lib.cldnn_b200_ctx_info(self.handle, C.byref(info)))
        return info

    def kernel(self, name):
        if name not in self._kernels:
            self._kernels[name] = Kernel(self, name)
        return self._kernels[name]

    def kernel_names(self):
        return [self.lib.cldnn_b200_kernel_name(i).decode() for i in range(self.lib.cldnn_b200_kernel_count())]

    def alloc(self, nbytes):
        return Memory(self, nbytes)

    def upload(self, array):
        a = np.ascontiguousarray(array)
        m = Memory(self, max(a.nbytes, 1))
        if a.nbytes:
            m.write(a)
        return m

    def sync(self):
        _check(self.lib.cldnn_b200_ctx_sync(self.handle))

    def stream(self):
        s = C.c_void_p()
        _check(self.lib.cldnn_b200_ctx_stream(self.handle, C.byref(s)))
        return s.value

    def launch_count(self):
        n = C.c_uint64()
        _check(self.lib.cldnn_b200_ctx_launch_count(self.handle, C.byref(n)))
        return n.value

    def tensor_peak(self, dtype=abi.I8, n=256):
        """Measured tensor-core peak of this device in tera-operations per second (cldnn_b200_tensor_peak)."""
        v = C.c_double()
        _check(self.lib.cldnn_b200_tensor_peak(self.handle, dtype, n, C.byref(v)))
        return v.value

    def device_status(self):
        s = C.c_uint32()
        _check(self.lib.cldnn_b200_ctx_device_status(self.handle, C.byref(s)))
        return s.value

    def close(self):
        if self.handle:
            self.lib.cldnn_b200_ctx_destroy(self.handle)
            self.handle = C.c_void_p()


def make_args(input0=None, input1=None, output=None, weights=None, bias=None, quant=None, calib=None, eltw_calib=None,
              scratch=None):
    """Argument block from Memory objects (or raw device addresses)."""
    def p(m):
        if m is None:
            return None
        return m.ptr if isinstance(m, Memory) else int(m)
    a = abi.Args()
    a.input0, a.input1, a.output, a.weights, a.bias = p(input0), p(input1), p(output), p(weights), p(bias)
    a.weights_quantization_factors, a.output_calibration_factors = p(quant), p(calib)
    a.eltw_output_calibration_factors = p(eltw_calib)
    a.scratch = p(scratch)
    a.scratch_bytes = scratch.nbytes if isinstance(scratch, Memory) else 0
    return a
