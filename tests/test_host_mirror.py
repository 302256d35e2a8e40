"""Host-side mirror of axc-runtime's types: metadata sidecar, binding plan, error enum.  No GPU.
Mirrors crates/axc-runtime/tests/metadata_roundtrip.rs (AT-512/513) and error.rs at_801."""
import json

import pytest


def test_error_enum_has_the_reference_25_variants(axc):
    E = axc.errors
    assert len(E.ALL_VARIANTS) == 25
    assert len({v.variant for v in E.ALL_VARIANTS}) == 25
    for v in E.ALL_VARIANTS:
        assert issubclass(v, axc.DispatchError)
    e = E.BindingCountMismatch("binding count mismatch: expected 3, got 2", expected=3, provided=2)
    assert (e.expected, e.provided) == (3, 2) and "expected 3, got 2" in str(e)
    assert E.CopyDirection.HostToDevice.value == 0 and E.CopyDirection.DeviceToHost.value == 1


def test_q4_binding_plan_layout(axc):
    for kernel, scalar in (("q4km_dequant_matvec", "n_superblocks"), ("q4_0_dequant_matvec", "n_blocks")):
        plan = axc.q4_matvec_binding_plan(kernel)
        assert [b.name for b in plan.buffers] == ["q", "x", "y"]
        assert [b.buffer_position for b in plan.buffers] == [0, 1, 2]      # bindings {0,1,2}
        assert [(b.ty.elem, b.ty.access) for b in plan.buffers] == [
            ("U8", "ReadOnly"), ("F32", "ReadOnly"), ("F32", "ReadWrite")]
        assert len(plan.scalars) == 1 and plan.scalars[0].name == scalar
        assert plan.scalars[0].ty == "U32" and plan.scalars[0].offset == 0
        assert plan.scalars[0].position == 3 and plan.push_constant_total_bytes == 4


def test_metadata_round_trip_at_512(axc, tmp_path):
    plan = axc.q4_matvec_binding_plan()
    meta = axc.KernelMetadata.new("q4km_dequant_matvec", [64, 1, 1], plan, "q4km_dequant_matvec")
    assert meta.schema_version == 1 and meta.push_constant_total_bytes == 4
    p = tmp_path / "k.axc.meta.json"
    meta.save(p)
    raw = json.loads(p.read_text())
    assert raw["binding_plan"]["buffers"][0]["ty"] == {"elem": "U8", "access": "ReadOnly"}
    assert raw["binding_plan"]["scalars"][0]["ty"] == "U32"
    assert "span" not in raw["binding_plan"]["buffers"][0]
    back = axc.load_kernel_metadata(p)
    assert back == meta and back.binding_plan.hash64() == plan.hash64()


def test_metadata_schema_mismatch_at_513(axc, tmp_path):
    plan = axc.q4_matvec_binding_plan()
    meta = axc.KernelMetadata.new("k", [64, 1, 1], plan, "k")
    meta.schema_version = 2
    p = tmp_path / "k.json"
    meta.save(p)
    with pytest.raises(axc.errors.MetadataSchemaMismatch) as ei:
        axc.load_kernel_metadata(p)
    assert ei.value.got == 2 and ei.value.supported == 1
    p.write_text("{ not json")
    with pytest.raises(axc.errors.MetadataParseError):
        axc.load_kernel_metadata(p)
    with pytest.raises(axc.errors.MetadataIoError):
        axc.load_kernel_metadata(tmp_path / "absent.json")


def test_plan_hash_is_deterministic_and_sensitive(axc):
    a = axc.q4_matvec_binding_plan("q4km_dequant_matvec")
    b = axc.q4_matvec_binding_plan("q4km_dequant_matvec")
    c = axc.q4_matvec_binding_plan("q4_0_dequant_matvec")
    assert a.hash64() == b.hash64() != c.hash64()


def test_context_options_from_env(axc, monkeypatch):
    monkeypatch.setenv("AXC_PHYSICAL_DEVICE_INDEX", "3")
    monkeypatch.setenv("AXC_FENCE_TIMEOUT_MS", "250")
    o = axc.CudaContextOptions.from_env()
    assert o.physical_device_index == 3 and o.fence_timeout_ms == 250 and o.pipeline_cache_path is None
    monkeypatch.setenv("AXC_FENCE_TIMEOUT_MS", "soon")
    assert axc.CudaContextOptions.from_env().fence_timeout_ms is None
    monkeypatch.setenv("AXC_ENABLE_GPU_TESTS", "1")
    assert axc.gpu_tests_enabled() is True
    monkeypatch.setenv("AXC_ENABLE_GPU_TESTS", "true")
    assert axc.gpu_tests_enabled() is False
    assert axc.captured_icd_path() == ""
