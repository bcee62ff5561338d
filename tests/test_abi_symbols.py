"""The C-ABI library loads and exports every symbol include/ovk_cuda.h declares
(no compute calls: runs without a GPU)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ovk_cuda.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"OVK_API\s+[\w\s\*]+?\b(ovk_\w+)\s*\(", text)))


def test_header_declares_the_operator_entry_points():
    names = declared_symbols()
    for must in ("ovk_ctx_create", "ovk_flush", "ovk_nbits_prepack", "ovk_matmul_nbits",
                 "ovk_dynamic_quantize", "ovk_mmi_prepack", "ovk_matmul_integer",
                 "ovk_matmul_integer_scale_bias", "ovk_qlinear_matmul", "ovk_qconv_prepack",
                 "ovk_conv_integer", "ovk_qlinear_conv", "ovk_requantize"):
        assert must in names


def test_library_exports_every_declared_symbol():
    import ovk_b200
    if not os.path.exists(ovk_b200.LIB_PATH):
        import subprocess, sys
        subprocess.run([sys.executable, os.path.join(ROOT, "onnx-vulkan-rs_b200", "build.py")], check=True)
    lib = ctypes.CDLL(ovk_b200.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_covers_every_declared_symbol():
    import ovk_b200
    assert sorted(ovk_b200.SIGNATURES) == declared_symbols()


def test_no_gpu_means_a_loud_failure_not_a_fallback():
    import torch
    import ovk_b200
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(ovk_b200.OvkError):
        ovk_b200.Context(0)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "onnx-vulkan-rs_b200")
    for dirpath, _, files in os.walk(pkg):
        if "build" in dirpath.split(os.sep):
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f
