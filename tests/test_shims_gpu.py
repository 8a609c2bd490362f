"""The reference-named C++ shims (include/apnn_b200_shims.h) RUN on a GPU: a C++ program, written the way the
reference's own main() programs and layer wrappers call their kernels, is compiled with nvcc, linked against
libapnn_b200.so and against the reference's unmodified host functions (oracle/_ref/libref_66.so), and checked
by the reference's own compute_ref / compute_ref_pack + validate_results[_pack]."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_style_program_passes_the_references_own_validation(cuda_device, tmp_path):
    nvcc = shutil.which("nvcc")
    ref_lib = os.path.join(ROOT, "oracle", "_ref", "libref_66.so")
    if nvcc is None or not os.path.exists(ref_lib):
        pytest.skip("needs nvcc and oracle/_ref/libref_66.so (make -C oracle ref)")
    exe = str(tmp_path / "shim_program")
    lib_dir, ref_dir = os.path.join(ROOT, "apnn_tc_b200"), os.path.join(ROOT, "oracle", "_ref")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "shim_program.cu"), "-o", exe, "-L", lib_dir, "-lapnn_b200", "-L", ref_dir,
           "-lref_66", "-Xlinker", "-rpath=" + lib_dir, "-Xlinker", "-rpath=" + ref_dir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("Result = PASS") == 3 and "Result = FAIL" not in r.stdout
    assert "apmm_w1a2 checksum 49072252" in r.stdout     # the reference's own operands: sum D of its first case
    assert "failures 0" in r.stdout
