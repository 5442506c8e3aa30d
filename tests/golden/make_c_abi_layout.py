"""Regenerates tests/golden/cldnn_c_abi_layout.txt: the binary layout of clDNN's public C boundary as the reference's own
headers define it (api/C/cldnn.h and the api/C/<primitive>.h descriptors).  Needs the clDNN source tree:

    python tests/golden/make_c_abi_layout.py <path to the clDNN tree>

The probe (tests/api_cpp/abi_probe.cpp) is compiled against those headers and its output stored; tests/test_public_api_layout.py
compiles the same probe against include/cldnn_c_api.h and requires the same text."""
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
PROBE = os.path.join(HERE, "..", "api_cpp", "abi_probe.cpp")


def layout_from_reference(ref):
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "probe")
        subprocess.check_call(["g++", "-std=c++14", "-w", "-DUSE_REFERENCE_HEADERS", "-I" + ref, "-I" + os.path.join(ref, "api"), "-o", exe, PROBE])
        return subprocess.check_output([exe]).decode()


if __name__ == "__main__":
    text = layout_from_reference(sys.argv[1])
    with open(os.path.join(HERE, "cldnn_c_abi_layout.txt"), "w") as f:
        f.write(text)
    print("wrote %d lines" % len(text.splitlines()))
