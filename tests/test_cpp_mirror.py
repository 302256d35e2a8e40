"""The C++ host mirror (include/axc_runtime.hpp): compiled with g++ against libaxc_cuda.so and run.

Host-only part everywhere (typed bring-up failure without a device, plan shape and hashing);
the device part on a B200, with the expected value of the reference's LCG fixture (n = 128, seed
0xDEADBEEF, the AT-1324 case) computed here by the CPU oracle."""
import os
import shutil
import subprocess

import pytest

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "runtime_test")


def build_binary(axc):
    lib_dir = os.path.dirname(axc.library_path())
    if not os.path.exists(axc.library_path()):
        pytest.skip("library not built")
    cxx = shutil.which("g++")
    assert cxx, "g++ is needed for the C++ mirror test"
    cuda_inc = "/usr/local/cuda/include"
    cmd = [cxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", cuda_inc,
           os.path.join(ROOT, "tests", "cpp", "runtime_test.cpp"), "-o", BIN,
           "-L", lib_dir, "-laxc_cuda", f"-Wl,-rpath,{lib_dir}"]
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    res = subprocess.run(cmd, capture_output=True, text=True, env=env)
    assert res.returncode == 0, res.stderr[-3000:]
    return BIN


def test_cpp_mirror_host_part(axc):
    exe = build_binary(axc)
    res = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "host-only ok" in res.stdout


@pytest.mark.gpu
def test_cpp_mirror_device_part(axc, tmp_path):
    exe = build_binary(axc)
    q, x = oracle.generate_q4km_test_data(128, 0xDEADBEEF)
    expected = float(oracle.q4km_dequant_matvec_cpu(q, x, 128))
    fixture = tmp_path / "lcg_n128.bin"
    fixture.write_bytes(q.tobytes() + x.tobytes())
    res = subprocess.run([exe, "--gpu", repr(expected), str(fixture)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "gpu ok" in res.stdout
