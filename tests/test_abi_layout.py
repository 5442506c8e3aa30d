"""Host-only checks of the C ABI: the ctypes mirror matches the header, the
library loads without a GPU, exports every declared symbol, and fails loudly
(no fallback) when asked for a device that is not there."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import pytest

from cldnn_b200 import abi, engine

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "cldnn_b200.h")

STRUCTS = {
    "cldnn_b200_tensor": abi.Tensor, "cldnn_b200_conv_params": abi.ConvParams, "cldnn_b200_args": abi.Args,
    "cldnn_b200_pool_params": abi.PoolParams, "cldnn_b200_fc_params": abi.FcParams,
    "cldnn_b200_softmax_params": abi.SoftmaxParams, "cldnn_b200_eltwise_params": abi.EltwiseParams,
    "cldnn_b200_reorder_params": abi.ReorderParams, "cldnn_b200_lrn_params": abi.LrnParams,
    "cldnn_b200_activation_params": abi.ActivationParams, "cldnn_b200_engine_info": abi.EngineInfo,
}


def test_ctypes_mirror_matches_header_sizes():
    src = '#include <stdio.h>\n#include "%s"\nint main(){\n' % HEADER
    for name in STRUCTS:
        src += 'printf("%s %%zu\\n", sizeof(%s));\n' % (name, name)
    src += 'printf("tune_off %zu\\n", offsetof(cldnn_b200_conv_params, tune));\n'
    src += 'printf("act_off %zu\\n", offsetof(cldnn_b200_conv_params, act));\nreturn 0;}\n'
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        subprocess.check_call(["/usr/bin/gcc", "-std=c99", c, "-o", os.path.join(d, "s")])
        out = subprocess.check_output([os.path.join(d, "s")]).decode().split()
    sizes = dict(zip(out[::2], map(int, out[1::2])))
    for name, cls in STRUCTS.items():
        assert sizes[name] == C.sizeof(cls), name
    assert sizes["tune_off"] == abi.ConvParams.tune.offset
    assert sizes["act_off"] == abi.ConvParams.act.offset


def test_library_exports_every_declared_symbol():
    declared = set(re.findall(r"CLDNN_B200_API\s+[\w\s\*]+?\b(cldnn_b200_\w+)\s*\(", open(HEADER).read()))
    assert declared == set(engine.declared_symbols())
    lib = engine.load_library()
    for name in declared:
        assert getattr(lib, name) is not None


def test_kernel_table_lists_the_hot_path():
    lib = engine.load_library()
    names = [lib.cldnn_b200_kernel_name(i).decode() for i in range(lib.cldnn_b200_kernel_count())]
    for k in ("conv_i8_tc", "conv_ref", "pooling_i8_byxf", "pooling_ref", "fc_ref", "softmax", "eltwise_ref", "reorder_ref"):
        assert k in names
    assert lib.cldnn_b200_kernel_name(len(names)) is None


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(engine.EngineError) as e:
        engine.Engine(0)
    assert e.value.status == abi.DEVICE_ERROR
    assert "no CPU fallback" in str(e.value)
