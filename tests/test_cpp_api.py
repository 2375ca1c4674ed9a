"""The C++ host API (include/flexllm/*.hpp) compiles as plain C++17 and links against the library
(no GPU needed: nothing is launched; argument validation answers on the host)."""
import os
import subprocess
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SRC = r'''
#include <flexllm/flexllm.hpp>
#include <cstdio>
int main() {
    using namespace flexllm;
    // null pointers are rejected before any CUDA call
    if (pref_quant_layer_fp32_qint(nullptr, nullptr, nullptr, 8, 64) != FLEXLLM_EINVAL) return 1;
    if (pref_FHT(nullptr, nullptr, 1, 64, 8.0f) != FLEXLLM_EINVAL) return 2;
    if (pref_Linear_Layer_i8xi8(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 8, 64, 64) != FLEXLLM_EINVAL) return 3;
    if (dec_Layer_Norm(nullptr, nullptr, nullptr, nullptr, nullptr, 1, 2048) != FLEXLLM_EINVAL) return 4;
    if (MHA_i8xi8_Prefilling_workspace(4, 1024, 32, 8) == 0) return 5;
    if (pref_quant_layer_fp32_qint_asym(nullptr, nullptr, nullptr, nullptr, 8, 64) != FLEXLLM_EINVAL) return 6;
    if (pref_Linear_Layer_i4xi4(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 8, 64, 64) != FLEXLLM_EINVAL) return 7;
    HMT hmt; SpinQuantModel model;
    if (hmt.Prefilling(nullptr, 16) != FLEXLLM_EINVAL) return 8;
    std::printf("%s\n", status_string(FLEXLLM_EINVAL));
    return 0;
}
'''


def test_cpp_api_compiles_and_links():
    from flexllm_b200 import build
    lib = build.build()
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.cpp"); exe = os.path.join(d, "t")
        open(src, "w").write(SRC)
        r = subprocess.run(["/usr/bin/g++", "-std=c++17", "-Wall", "-I", os.path.join(ROOT, "include"), src, "-o", exe, lib,
                            "-Wl,-rpath," + os.path.dirname(lib)], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        r = subprocess.run([exe], capture_output=True, text=True)
        assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
        assert "invalid" in r.stdout
