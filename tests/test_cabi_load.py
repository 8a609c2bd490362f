"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header
declares, and rejects bad arguments with status codes before touching a device."""
import ctypes
import os
import re

import pytest

from apnn_tc_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    text = open(os.path.join(ROOT, "include", "apnn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(apnn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = _cabi.lib()
    declared = _header_functions()
    assert set(declared) == set(_cabi.EXPORTS)
    for name in declared:
        assert hasattr(L, name), name


def test_status_strings_and_version():
    L = _cabi.lib()
    assert L.apnn_version() >= 100
    assert L.apnn_status_string(0) == b"ok"
    for s in range(1, 8):
        assert L.apnn_status_string(s) not in (b"ok", b"unknown status")


def test_argument_validation_returns_status_codes():
    L = _cabi.lib()
    buf = (ctypes.c_uint32 * 64)()
    base = ctypes.addressof(buf)
    p = base + (-base % 16)
    # null pointers / sizes
    assert L.apnn_gemm_ex(None, 0, 1, 2, None, p, p, 64, 64, 128, None, None, 0) == 1
    assert L.apnn_gemm_ex(None, 0, 1, 2, p, p, p, 0, 64, 128, None, None, 0) == 1
    # K not a multiple of 128, misaligned pointer
    assert L.apnn_gemm_ex(None, 0, 1, 2, p, p, p, 64, 64, 96, None, None, 0) == 3
    assert L.apnn_gemm_ex(None, 0, 1, 2, p + 4, p, p, 64, 64, 128, None, None, 0) == 3
    # unsupported widths, packed output with N % 32 != 0, signed operand wider than 1 bit
    assert L.apnn_gemm_ex(None, 0, 3, 3, p, p, p, 64, 64, 128, None, None, 0) == 4   # int8 path only: needs a workspace
    assert L.apnn_gemm_ex(None, 0, 5, 5, p, p, p, 64, 64, 128, None, None, 0) == 2
    e = _cabi.Epilogue(out_mode=1, out_bits=2)
    assert L.apnn_gemm_ex(None, 0, 1, 2, p, p, p, 64, 48, 128, ctypes.byref(e), None, 0) == 2
    e = _cabi.Epilogue(out_mode=0, signed_operand=2)
    assert L.apnn_gemm_ex(None, 0, 1, 2, p, p, p, 64, 64, 128, ctypes.byref(e), None, 0) == 2
    e = _cabi.Epilogue(out_mode=2, out_bits=2)  # thresholds missing
    assert L.apnn_gemm_ex(None, 0, 1, 2, p, p, p, 64, 64, 128, ctypes.byref(e), None, 0) == 1
    # a descriptor whose recorded size is not this library's structure (a caller built against another layout)
    e = _cabi.Epilogue(out_mode=1, out_bits=2)
    e.struct_size = 64
    assert L.apnn_gemm_ex(None, 0, 1, 2, p, p, p, 64, 64, 128, ctypes.byref(e), None, 0) == 1
    # the float affine output exists on the int8 entry points only; there it needs both vectors
    e = _cabi.Epilogue(out_mode=3)
    assert L.apnn_gemm_ex(None, 0, 1, 2, p, p, p, 64, 64, 128, ctypes.byref(e), None, 0) == 2
    flag = (ctypes.c_int * 1)()
    assert L.apnn_gemm_i8(None, p, p, p, 64, 64, 128, 0, 0, ctypes.byref(e), ctypes.addressof(flag)) == 1
    # activations from planes: 1..4 planes, a -1/+1 plane only alone, no int8-row / float outputs
    assert L.apnn_gemm_w8(None, p, 5, p, p, 64, 64, 128, 0, 0, None, ctypes.addressof(flag)) == 2
    assert L.apnn_gemm_w8(None, p, 2, p, p, 64, 64, 128, 0, 1, None, ctypes.addressof(flag)) == 2
    assert L.apnn_gemm_w8(None, p, 2, p, p, 64, 64, 100, 0, 0, None, ctypes.addressof(flag)) == 3
    assert L.apnn_gemm_w8(None, p, 2, p, p, 64, 64, 128, 0, 0, None, None) == 1
    # 4-bit floating-point path: one or two planes, K a multiple of 256 and small enough for exact fp32 sums
    assert L.apnn_expand_planes_fp4(None, p, p, 64, 256, 3, 0) == 2
    assert L.apnn_expand_planes_fp4(None, p, p, 64, 256, 2, 1) == 2
    assert L.apnn_expand_planes_fp4(None, p, p, 64, 128, 2, 0) == 3
    assert L.apnn_gemm_fp4(None, p, p, p, 64, 64, 128, None, ctypes.addressof(flag)) == 3
    assert L.apnn_gemm_fp4(None, p, p, p, 64, 64, 1 << 21, None, ctypes.addressof(flag)) == 2
    # tcgen05 path without a workspace
    assert L.apnn_gemm_ex(None, 3, 1, 2, p, p, p, 128, 256, 128, None, None, 0) == 4
    assert L.apnn_gemm_workspace_bytes(3, 1, 2, 128, 256, 128) >= (128 + 256) * 128
    assert L.apnn_gemm_workspace_bytes(2, 1, 2, 128, 256, 128) == 0
    # conv rules
    assert L.apnn_conv2d(None, 1, 2, p, p, p, 1, 8, 8, 96, 64, 3, 1, None) == 3
    assert L.apnn_conv2d(None, 1, 2, p, p, p, 1, 8, 8, 128, 64, 4, 1, None) == 2
    assert L.apnn_conv2d(None, 1, 2, p, p, p, 1, 8, 8, 128, 64, 13, 1, None) == 2
    assert L.apnn_conv2d(None, 1, 2, p, p, p, 1, 8, 8, 128, 64, 3, 5, None) == 2
    e = _cabi.Epilogue(out_mode=1, out_bits=2, pool=1)
    assert L.apnn_conv2d(None, 1, 2, p, p, p, 1, 7, 8, 128, 64, 3, 1, ctypes.byref(e)) == 2
    # packers
    assert L.apnn_bit_compress(None, p, p, 0, 3, 2) == 1
    assert L.apnn_quantize_pack(None, p, p, 4, 3, 9) == 1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _cabi.lib()


def test_reference_named_shims_compile(tmp_path):
    """include/apnn_b200_shims.h (the reference's kernel, packer and layer-launch names over the
    C ABI) compiles as C++/CUDA host code against structs with the reference's field names."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc")
    if nvcc is None:
        import pytest
        pytest.skip("nvcc not on PATH")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "shim_user.cu"
    src.write_text(r'''
#include "apnn_b200_shims.h"
struct ConvP { uin32 *filter_gpu, *input_gpu, *output_gpu; int batch, input_height, input_width, input_channels, output_channels; };
struct FcP { uin32 *input_gpu, *weight_gpu, *output_gpu; int input_height, input_width, weight_width; };
void use(ConvP* c, FcP* f, float* h, float* d, uin32* planes, int4* w, int4* x, int* out) {
  Conv_new_global(c); FC_new_global(f); Output_new_global(f);
  uin32* img = images_quantization(h, 8, 224, 224, 3, 2); uin32* flt = nullptr;
  filter_quantization(flt, d, 64, 3, 3, 128, 1); weight_quantization(planes, d, 512, 1000, 1);
  weight_quantization_fc_hidden(planes, d, 512, 512, 1);
  apmm_w1a2(w, x, out, 64, 1024, 1024); apmm_w1a3(w, x, out, 64, 1024, 1024); apmm_w1a4(w, x, out, 64, 1024, 1024);
  apmm_w2a2(w, x, out, 64, 1024, 1024); apmm_w1a2_decompose(w, x, out, 64, 1024, 1024);
  APConv_w1a2_pack(w, x, out, 16, 16, 128, 128); APConv_w1a2_pack_pool(w, x, out, 16, 16, 128, 128);
  APConv_w2a2_pack(w, x, out, 16, 16, 128, 128); compute_conv_imma(w, x, out, 16, 16, 128, 128, 1, 2);
  (void)img;
}
''')
    r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(root, "include"), "-c",
                        str(src), "-o", str(tmp_path / "shim_user.o")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
