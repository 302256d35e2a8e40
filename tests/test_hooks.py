"""Host logic of the bench_variant / grid_search hooks (no GPU): the reference's own unit tests
for these tools, restated (crates/axc-driver/src/mcp/tools/bench_variant.rs:513-631,
crates/axc-optimize/src/grid_search.rs:323-526)."""
import base64
import json
import struct

import pytest

from conftest import load_pkg

hooks = load_pkg("hooks")
runtime = load_pkg("runtime")


def test_at_1121_derive_workgroups_ceiling_divide():
    assert hooks.derive_workgroups([4096, 4096], [64, 1, 1], None) == [16, 1, 1]
    assert hooks.derive_workgroups([4096, 4096], [64, 1, 1], [8, 8, 1]) == [8, 8, 1]
    assert hooks.derive_workgroups([], [64, 1, 1], None) == [1, 1, 1]


def test_derive_workgroups_for_q4_kernels_counts_rows():
    pc = struct.pack("<I", 16)
    sizes = [100 * 16 * 144, 4096 * 4, 100 * 4]
    assert hooks.derive_workgroups(sizes, [64, 1, 1], None, kernel_name="q4km_dequant_matvec",
                                   push_constants=pc) == [100, 1, 1]
    # y shorter than the rows q holds: the output size wins
    assert hooks.derive_workgroups(sizes, [64, 1, 1], None, kernel_name="q4km_dequant_matvec",
                                   push_constants=pc, output_sizes=[0, 0, 28]) == [7, 1, 1]
    # n = 0 keeps the reference's single invocation (y[0] = 0)
    assert hooks.derive_workgroups(sizes, [64, 1, 1], None, kernel_name="q4_0_dequant_matvec",
                                   push_constants=struct.pack("<I", 0)) == [1, 1, 1]
    assert hooks.derive_workgroups([128 * 18 * 5, 16384, 20], [64, 1, 1], None,
                                   kernel_name="q4_0_dequant_matvec",
                                   push_constants=struct.pack("<I", 128)) == [5, 1, 1]
    # an override always wins
    assert hooks.derive_workgroups(sizes, [64, 1, 1], [3, 1, 1], kernel_name="q4km_dequant_matvec",
                                   push_constants=pc) == [3, 1, 1]


def test_at_1122_seeded_inputs_deterministic():
    v1, v2, v3 = hooks.seeded_inputs([16, 32], 42), hooks.seeded_inputs([16, 32], 42), hooks.seeded_inputs([16, 32], 43)
    assert v1 == v2 and v1 != v3
    assert [len(b) for b in hooks.seeded_inputs([100, 200, 50], 0)] == [100, 200, 50]


def test_seeded_q4_inputs_are_well_formed_and_sized():
    import numpy as np
    sizes = [5 * 4 * 144 + 7, 4 * 256 * 4, 5 * 4]
    q, x, y = hooks.seeded_q4_inputs("q4km_dequant_matvec", sizes, 4, 9)
    assert [len(q), len(x), len(y)] == sizes and y == bytes(20)
    d = np.frombuffer(q[:5 * 4 * 144], np.uint8).reshape(-1, 144)[:, :4].copy().view(np.float16)
    assert np.isfinite(d.astype(np.float32)).all()
    assert hooks.seeded_q4_inputs("q4km_dequant_matvec", sizes, 4, 9)[0] == q
    q0, _, _ = hooks.seeded_q4_inputs("q4_0_dequant_matvec", [3 * 8 * 18, 8 * 32 * 4, 12], 8, 1)
    assert len(q0) == 3 * 8 * 18


def test_pick_reference():
    plan = runtime.q4_matvec_binding_plan("q4km_dequant_matvec")
    assert hooks.pick_reference("q4km_dequant_matvec", plan) == "strict_order_kernel"
    assert hooks.pick_reference("q4_0_dequant_matvec", plan) == "strict_order_kernel"
    assert hooks.pick_reference("unknown_kernel", runtime.ParamBindingPlan([], [], 0)) is None


def test_correctness_status_serde():
    assert json.dumps(hooks.CorrectnessStatus.ok().to_json_obj()) == '{"status": "ok"}'
    s = json.dumps(hooks.CorrectnessStatus.failed("3/10 exceeded ULP").to_json_obj())
    assert "failed" in s and "3/10 exceeded ULP" in s
    assert "not_checked" in json.dumps(hooks.CorrectnessStatus.not_checked("no oracle").to_json_obj())


def test_push_constants_decode_and_length_check():
    assert hooks.build_push_constants(None, 4) == bytes(4)
    assert hooks.build_push_constants(base64.b64encode(struct.pack("<I", 16)).decode(), 4) == struct.pack("<I", 16)
    with pytest.raises(hooks.InvalidParams, match="decoded to 8 bytes, but kernel expects 4"):
        hooks.build_push_constants(base64.b64encode(bytes(8)).decode(), 4)
    with pytest.raises(hooks.InvalidParams):
        hooks.build_push_constants("!!!not base64", 4)


def test_variant_id_is_canonical_and_zero_without_assignments():
    assert hooks.compute_variant_id({}) == 0
    a = hooks.compute_variant_id({"stages": 2, "tile_rows": 16})
    assert a == hooks.compute_variant_id({"tile_rows": 16, "stages": 2}) != hooks.compute_variant_id({"stages": 3, "tile_rows": 16})


def test_enumerate_strategy_mixed_radix_order():
    v = hooks.enumerate_strategy({"b": [10, 20], "a": [1, 2, 3]})
    assert [x.ordinal for x in v] == list(range(6))
    assert [(x.assignments["a"], x.assignments["b"]) for x in v] == [(1, 10), (1, 20), (2, 10), (2, 20), (3, 10), (3, 20)]
    assert len({x.variant_id for x in v}) == 6
    with pytest.raises(hooks.GridSearchError, match="EmptyStrategy"):
        hooks.enumerate_strategy({})


def _stats(ns):
    return hooks.SampleStats(ns, ns - 10, ns + 10, 3)


def test_at_1022_no_strategy_is_an_error():
    with pytest.raises(hooks.GridSearchError, match="NoStrategy"):
        hooks.grid_search(None, hooks.CorrectnessPolicy(), None, lambda a: _stats(1000))


def test_at_1023_picks_fastest_variant_and_at_1040_1041_1042():
    times = {32: 3000, 64: 1000, 128: 2000}
    r = hooks.grid_search({"workgroup_x": [32, 64, 128]}, hooks.CorrectnessPolicy(), None,
                          lambda a: _stats(times[a["workgroup_x"]]))
    assert r.winner_assignments == {"workgroup_x": 64} and r.winner_ordinal == 1
    assert r.winner_variant_id == hooks.enumerate_strategy({"workgroup_x": [32, 64, 128]})[1].variant_id
    assert r.fallback_used is False
    assert [x.ordinal for x in r.results] == [0, 1, 2]


def test_at_1024_fallback_to_ordinal_zero_when_all_benchmarks_fail():
    def bench(a):
        raise RuntimeError("device lost")
    r = hooks.grid_search({"workgroup_x": [32, 64]}, hooks.CorrectnessPolicy(), None, bench)
    assert r.fallback_used and r.winner_ordinal == 0
    assert all(x.outcome == ("Failed", "device lost") for x in r.results)


def test_at_1025_correctness_failure_excludes_variant():
    r = hooks.grid_search({"workgroup_x": [32, 64]}, hooks.CorrectnessPolicy("BitExact"),
                          lambda a: ("BitMismatch", 3) if a["workgroup_x"] == 32 else None,
                          lambda a: _stats(500 if a["workgroup_x"] == 32 else 900))
    assert r.winner_assignments == {"workgroup_x": 64}
    assert r.results[0].outcome == ("CorrectnessRejected", ("BitMismatch", 3))
    # with policy None the correctness closure is not consulted
    r2 = hooks.grid_search({"workgroup_x": [32, 64]}, hooks.CorrectnessPolicy(), lambda a: ("BitMismatch", 1),
                           lambda a: _stats(500 if a["workgroup_x"] == 32 else 900))
    assert r2.winner_assignments == {"workgroup_x": 32}


def test_at_1026_cartesian_warning_threshold():
    assert hooks.CARTESIAN_WARN_THRESHOLD == 100
    r = hooks.grid_search({"a": list(range(11)), "b": list(range(10))}, hooks.CorrectnessPolicy(), None,
                          lambda a: _stats(1000 + a["a"]))
    assert any("exceeds CARTESIAN_WARN_THRESHOLD" in w for w in r.warnings)
    assert len(r.results) == 110


def test_correctness_policy_parse():
    P = hooks.CorrectnessPolicy
    assert P.parse("none") == P("None") and P.parse("bit-exact") == P("BitExact")
    assert P.parse("fp-tol:4") == P("EquivFpTol", 4)
    assert P.parse("fp-tol:x") == P("EquivFpTol", 4) and P.parse("whatever") == P("None")   # optimize.rs:121-135


def test_policy_is_applied_to_the_output_bytes():
    """A variant one unit in the last place away from the ordinal-0 variant: rejected under
    bit-exact, accepted under fp-tol:1, rejected again under fp-tol:0 (grid_search.rs:54-75)."""
    import numpy as np
    ref = np.array([1.0, -2.5, 0.0, 1e-3], np.float32)
    got = ref.copy()
    got.view(np.uint32)[1] += 1
    P = hooks.CorrectnessPolicy
    assert hooks.policy_failure(P.parse("none"), got.tobytes(), ref.tobytes()) is None
    assert hooks.policy_failure(P.parse("bit-exact"), ref.tobytes(), ref.tobytes()) is None
    assert hooks.policy_failure(P.parse("bit-exact"), got.tobytes(), ref.tobytes()) == ("BitMismatch", 1)
    assert hooks.policy_failure(P.parse("fp-tol:1"), got.tobytes(), ref.tobytes()) is None
    assert hooks.policy_failure(P.parse("fp-tol:0"), got.tobytes(), ref.tobytes()) == ("UlpExceeded", 1, 1)
    assert hooks.policy_failure(P.parse("bit-exact"), got.tobytes(), ref.tobytes()[:8])[0] == "OracleError"
    # and through grid_search: the rejected variant cannot win however fast it is
    outs = {32: got.tobytes(), 64: ref.tobytes()}
    fail = lambda a: hooks.policy_failure(P.parse("bit-exact"), outs[a["workgroup_x"]], outs[64])
    r = hooks.grid_search({"workgroup_x": [64, 32]}, P.parse("bit-exact"), fail,
                          lambda a: _stats(100 if a["workgroup_x"] == 32 else 900))
    assert r.winner_assignments == {"workgroup_x": 64}
    assert r.results[1].outcome == ("CorrectnessRejected", ("BitMismatch", 1))


def test_tuning_from_assignments_rejects_unknown_holes():
    t = hooks.tuning_from_assignments({"stages": 3, "tile_rows": 8})
    assert (t.stages, t.tile_rows, t.ctas_per_sm, t.pdl, t.evict_first) == (3, 8, 0, -1, -1)
    with pytest.raises(hooks.InvalidParams, match="unknown tunable"):
        hooks.tuning_from_assignments({"workgroup_x": 64})


def test_ulp_distance():
    import numpy as np
    a = np.array([1.0, -1.0, 0.0, 1.0], np.float32)
    b = np.array([np.nextafter(np.float32(1), np.float32(2)), -1.0, -0.0, 1.0], np.float32)
    assert hooks.ulp_distance(a, b).tolist() == [1, 0, 0, 0]


def test_history_append_is_one_json_line_per_entry(tmp_path):
    p = tmp_path / "h.jsonl"
    hooks.append_history_entry(str(p), {"a": 1})
    hooks.append_history_entry(str(p), {"b": [1, 2]})
    assert [json.loads(l) for l in p.read_text().splitlines()] == [{"a": 1}, {"b": [1, 2]}]


def test_request_validation_happens_before_any_gpu_use():
    ctx = hooks.McpContext()
    meta = hooks.q4_metadata("q4km_dequant_matvec")
    with pytest.raises(hooks.InvalidParams, match="sample_count must be >= 1"):
        hooks.bench_variant(hooks.BenchVariantRequest([1, 2, 3], 0, metadata=meta), ctx)
    with pytest.raises(hooks.InvalidParams, match="input_sizes.len\\(\\) == 2 but kernel has 3 buffer bindings"):
        hooks.bench_variant(hooks.BenchVariantRequest([1, 2], 1, metadata=meta), ctx)
    with pytest.raises(hooks.InvalidParams, match="exactly one of"):
        hooks.bench_variant(hooks.BenchVariantRequest([1, 2, 3], 1), ctx)
    assert ctx.cuda._ctx is None and ctx.cuda._err is None


def test_once_cuda_caches_the_failure(axc):
    """mcp/dispatch.rs:78-129: a failed bring-up is remembered, not retried."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: bring-up succeeds")
    once = hooks.OnceCuda()
    with pytest.raises(axc.DispatchError) as e1:
        once.get_or_init()
    with pytest.raises(axc.DispatchError) as e2:
        once.get_or_init()
    assert e1.value is e2.value
