"""The C-ABI library loads and exports every symbol include/axc_cuda.h declares; host-side
behaviour that needs no GPU (validation, error text, launch planning)."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT, load_pkg


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "axc_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(axc_cuda_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(ffi):
    names = declared_symbols()
    assert len(names) >= 25
    raw = C.CDLL(ffi.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"libaxc_cuda.so lacks {n}"
    assert set(names) == set(ffi.SYMBOLS), set(names) ^ set(ffi.SYMBOLS)


def test_version_and_strerror(ffi):
    L = ffi.lib()
    assert L.axc_cuda_version() >= 100
    assert L.axc_cuda_strerror(0) == b"ok"
    assert L.axc_cuda_strerror(ffi.AXC_ERR_FENCE_TIMEOUT) == b"FenceTimeout"
    assert L.axc_cuda_strerror(ffi.AXC_ERR_BINDING_COUNT_MISMATCH) == b"BindingCountMismatch"
    assert L.axc_cuda_strerror(12345) == b"Unknown"


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    ffi = load_pkg("_ffi")
    monkeypatch.setattr(ffi, "_lib", None)
    monkeypatch.setattr(ffi, "LIB_PATH", str(tmp_path / "libaxc_cuda.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ffi.lib()


def test_product_package_never_touches_the_oracle():
    pkg_dir = os.path.join(ROOT, "axiom-compute_b200")
    for dirpath, _dirs, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src, f
                assert "libaxc_oracle" not in src and "axc_oracle_" not in src, f


def test_no_gpu_here_means_typed_no_supported_device(axc, ffi):
    if ffi.lib().axc_cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    assert axc.probe_vulkan_available() is False
    with pytest.raises(axc.errors.NoSupportedDevice):
        axc.CudaContext.new()


def test_launch_plan_geometry(ops):
    p = ops.q4k_matvec_plan(14336, 16)
    assert p["grid"] == 296 and p["block"] == 256 and p["smem"] <= 114 * 1024   # 2 CTAs per SM
    assert p["tile_rows"] * p["stages"] >= 32           # most of a CTA's 48-49 rows in flight
    p = ops.q4k_matvec_plan(4096, 56)
    assert p["block"] % 224 == 0 and p["block"] <= 512   # groups of 7 warps cover the 56 superblocks
    p = ops.q4k_matvec_plan(8192, 112)
    assert p["grid"] == 148 and p["block"] == 448 and p["smem"] <= 227 * 1024
    p = ops.q4k_matvec_plan(1, 128)
    assert p["grid"] == 1 and p["block"] == 512
    p = ops.q4k_matvec_plan(8, 16)
    assert p["grid"] == 2
    p = ops.q4k_matvec_plan(3, 1000)                    # K segmented: 64 superblocks at a time
    assert p["grid"] == 3 and p["block"] == 256
    p = ops.q4k_matvec_plan(229376, 16)                 # tall: the ring is recycled
    assert p["grid"] == 296 and p["tile_rows"] * p["stages"] < 775
    p = ops.q4k_matvec_plan(14336, 16, ops.make_tuning(threads=512, ctas_per_sm=1))
    assert p["grid"] == 148 and p["block"] == 512


def test_device_layer_rejects_bad_pointers_without_a_gpu(ffi):
    L = ffi.lib()
    assert L.axc_cuda_q4k_matvec(None, None, None, 4, 1, None, None, None) == ffi.AXC_ERR_INVALID_ARGUMENT
    assert "null device pointer" in ffi.last_error_detail()
    assert L.axc_cuda_q4k_matvec(16, 32, 48 + 4, 4, 1, None, None, None) == ffi.AXC_ERR_INVALID_ARGUMENT
    assert "16-byte aligned" in ffi.last_error_detail()
    assert L.axc_cuda_q4k_matvec(None, None, None, 0, 1, None, None, None) == ffi.AXC_OK  # rows = 0
