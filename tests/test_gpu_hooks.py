"""bench_variant / grid_search against a real device, through the C ABI
(crates/axc-driver/src/mcp/tools/bench_variant.rs:214-320, mcp/tools/grid_search.rs)."""
import base64
import json
import struct

import numpy as np
import pytest

import oracle
from conftest import load_pkg

pytestmark = pytest.mark.gpu

hooks = load_pkg("hooks")


def b64(n):
    return base64.b64encode(struct.pack("<I", n)).decode()


@pytest.fixture(scope="module")
def mcp():
    return hooks.McpContext(git_sha="abc1234")


@pytest.mark.parametrize("kernel,blk,elems,rows,n", [("q4km_dequant_matvec", 144, 256, 300, 16),
                                                     ("q4_0_dequant_matvec", 18, 32, 257, 128)])
def test_bench_variant_times_and_checks_both_q4_kernels(mcp, kernel, blk, elems, rows, n):
    sizes = [rows * n * blk, n * elems * 4, rows * 4]
    resp = hooks.bench_variant(hooks.BenchVariantRequest(
        sizes, 5, metadata=hooks.q4_metadata(kernel), push_constants_base64=b64(n)), mcp)
    assert resp.workgroups == [rows, 1, 1]                 # derived from the buffers, not from q's bytes / 256
    assert len(resp.samples) == 5 and resp.median_ns == sorted(resp.samples)[2]
    assert len(resp.device_samples) == 5 and 0 < resp.device_median_ns <= resp.median_ns
    assert resp.correctness.kind == "Ok", resp.correctness.reason
    assert "B200" in resp.machine.device_name and resp.machine.git_sha == "abc1234"
    json.dumps(resp.to_json_obj())


def test_bench_variant_output_matches_the_oracle(mcp):
    """The inputs the tool generates, pushed through the same dispatch, give the oracle's y."""
    rows, n = 64, 8
    sizes = [rows * n * 144, n * 256 * 4, rows * 4]
    q, x, y = hooks.seeded_q4_inputs("q4km_dequant_matvec", sizes, n, 0)
    meta = hooks.q4_metadata("q4km_dequant_matvec")
    cuda = mcp.cuda.get_or_init()
    h = cuda.prepare_kernel([1, 2, 3], meta.binding_plan, 4, meta.entry_point)
    out = cuda.dispatch_handle(h, [rows, 1, 1], [q, x, y], sizes, struct.pack("<I", n))
    h.drop()
    qa, xa = np.frombuffer(q, np.uint8), np.frombuffer(x, np.float32)
    y_ref = oracle.matvec_rows("q4k", qa, xa, rows, n)
    _y64, mag = oracle.matvec_rows_f64("q4k", qa, xa, rows, n)
    assert (np.abs(np.frombuffer(bytes(out[2]), np.float32) - y_ref) / mag).max() <= 1e-5


def test_bench_variant_detects_a_wrong_result(mcp):
    """The verdict is a real comparison: a corrupted y is reported as Failed."""
    rows, n = 32, 4
    sizes = [rows * n * 144, n * 256 * 4, rows * 4]
    meta = hooks.q4_metadata("q4km_dequant_matvec")
    cuda = mcp.cuda.get_or_init()
    inputs = hooks.seeded_q4_inputs("q4km_dequant_matvec", sizes, n, 0)
    pc = struct.pack("<I", n)
    h = cuda.prepare_kernel([4, 5, 6], meta.binding_plan, 4, meta.entry_point)
    out = cuda.dispatch_handle(h, [rows, 1, 1], inputs, sizes, pc)
    h.drop()
    assert hooks.check_against_strict(cuda, meta, [rows, 1, 1], inputs, sizes, pc, out).kind == "Ok"
    bad = np.frombuffer(bytes(out[2]), np.float32).copy()
    bad[5] += 0.5 * np.abs(bad).max() + 1.0
    verdict = hooks.check_against_strict(cuda, meta, [rows, 1, 1], inputs, sizes, pc,
                                         [out[0], out[1], bad.tobytes()])
    assert verdict.kind == "Failed" and "1/32 rows" in verdict.reason


def test_bench_variant_with_tunables_and_unknown_kernel(mcp):
    rows, n = 512, 16
    sizes = [rows * n * 144, n * 256 * 4, rows * 4]
    meta = hooks.q4_metadata("q4km_dequant_matvec")
    r = hooks.bench_variant(hooks.BenchVariantRequest(sizes, 3, metadata=meta, push_constants_base64=b64(n),
                                                      assignments={"stages": 3, "tile_rows": 8}), mcp)
    assert r.correctness.kind == "Ok"
    with pytest.raises(hooks.InvalidParams, match="unknown tunable"):
        hooks.bench_variant(hooks.BenchVariantRequest(sizes, 3, metadata=meta, push_constants_base64=b64(n),
                                                      assignments={"workgroup_x": 64}), mcp)
    other = hooks.q4_metadata("q4km_dequant_matvec")
    other.kernel_name = other.entry_point = "saxpy"
    axc = load_pkg("errors")
    with pytest.raises(axc.DispatchError, match="unsupported kernel"):   # no CPU fallback, no other kernels
        hooks.bench_variant(hooks.BenchVariantRequest(sizes, 1, metadata=other, push_constants_base64=b64(n)), mcp)


def test_grid_search_tool_ranks_tunable_variants(mcp, tmp_path):
    rows, n = 2048, 16
    sizes = [rows * n * 144, n * 256 * 4, rows * 4]
    mcp2 = hooks.McpContext(cuda=mcp.cuda, git_sha="abc1234", history_dir=str(tmp_path))
    # policy "none": every variant is still checked against the reference-order kernel by bench_variant
    # (correctness.kind below); the policies that compare variants with the ordinal-0 variant are
    # exercised further down (tile heights change the order of the row sum, so they are not bit-equal)
    req = hooks.GridSearchRequest(sizes, 5, {"tile_rows": [8, 16], "stages": [2, 3]},
                                  metadata=hooks.q4_metadata("q4km_dequant_matvec"),
                                  correctness="none", push_constants_base64=b64(n))
    resp = hooks.grid_search_tool(req, mcp2)
    assert len(resp.ranked) == 4 and all(v.outcome == "ok" and v.correctness.kind == "Ok" for v in resp.ranked)
    meds = [v.median_ns for v in resp.ranked]
    assert meds == sorted(meds) and resp.winner_median_ns == meds[0]
    assert resp.winner_assignments == resp.ranked[0].assignments and not resp.fallback_used
    assert {tuple(sorted(v.assignments.items())) for v in resp.ranked} == {
        (("stages", s), ("tile_rows", t)) for s in (2, 3) for t in (8, 16)}
    rec = [json.loads(l) for l in open(resp.history_path)]
    assert len(rec) == 1 and rec[0]["grid_search"]["winner_variant_id"] == resp.winner_variant_id
    assert rec[0]["grid_search"]["ranked"][0]["correctness"] == {"status": "ok"}


def test_grid_search_tool_applies_the_stated_policy(mcp):
    """bit-exact / fp-tol compare each variant's output bytes with the ordinal-0 variant's
    (grid_search.rs:54-75).  The ring depth does not touch the arithmetic, so those variants pass
    bit-exact; a variant may only be rejected with the failure its policy defines, and a rejected
    variant never wins."""
    rows, n = 2048, 16
    sizes = [rows * n * 144, n * 256 * 4, rows * 4]
    meta = hooks.q4_metadata("q4km_dequant_matvec")
    same = hooks.grid_search_tool(hooks.GridSearchRequest(sizes, 3, {"stages": [2, 3, 4]}, metadata=meta,
                                                          correctness="bit-exact", push_constants_base64=b64(n)), mcp)
    assert all(v.outcome == "ok" for v in same.ranked)
    mixed = hooks.grid_search_tool(hooks.GridSearchRequest(sizes, 3, {"tile_rows": [8, 16], "stages": [2, 3]},
                                                           metadata=meta, correctness="bit-exact",
                                                           push_constants_base64=b64(n)), mcp)
    by_assign = {tuple(sorted(v.assignments.items())): v for v in mixed.ranked}
    assert by_assign[(("stages", 2), ("tile_rows", 8))].outcome == "ok"       # ordinal 0 against itself
    assert by_assign[(("stages", 3), ("tile_rows", 8))].outcome == "ok"       # same arithmetic
    for v in mixed.ranked:
        assert v.outcome == "ok" or v.outcome.startswith("correctness_rejected: ('BitMismatch'"), v.outcome
    assert by_assign[tuple(sorted(mixed.winner_assignments.items()))].outcome == "ok"
    loose = hooks.grid_search_tool(hooks.GridSearchRequest(sizes, 3, {"tile_rows": [8, 16]}, metadata=meta,
                                                           correctness="fp-tol:4294967295",
                                                           push_constants_base64=b64(n)), mcp)
    assert all(v.outcome == "ok" for v in loose.ranked)


def test_run_optimize_writes_winner_metadata_and_strategy_sidecar(mcp, tmp_path):
    rows, n = 1024, 16
    sizes = [rows * n * 144, n * 256 * 4, rows * 4]
    out = tmp_path / "q4km.tuned.json"
    req = hooks.GridSearchRequest(sizes, 3, {"stages": [2, 3]}, metadata=hooks.q4_metadata("q4km_dequant_matvec"),
                                  correctness="fp-tol:4", push_constants_base64=b64(n))
    resp = hooks.run_optimize(req, str(out), mcp)
    runtime = load_pkg("runtime")
    assert runtime.load_kernel_metadata(out).kernel_name == "q4km_dequant_matvec"
    side = json.loads(open(hooks.strategy_sidecar_path(str(out))).read())
    assert hooks.strategy_sidecar_path("out.spv") == "out.spv.axc.strategy.json"
    assert side["winner_assignments"]["values"] == resp.winner_assignments and len(side["results"]) == 2
    assert [r["ordinal"] for r in side["results"]] == [0, 1] and side["fallback_used"] is False
