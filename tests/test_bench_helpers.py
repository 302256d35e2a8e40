"""Host-side helpers of bench.py that the multi-GPU parity check relies on: any row of any rank's
matrix can be rebuilt from the one seeded base matrix, and both arms describe the workload alike."""
import importlib.util
import os

import numpy as np

from conftest import ROOT


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_matrix_rows_agree_with_the_whole_matrix():
    b = _bench()
    rng = np.random.default_rng(3)
    base = rng.integers(0, 256, size=(b.ROWS, b.ROW_BYTES), dtype=np.uint8)
    for m, shard in ((0, 0), (7, 0), (3, 5), (15, 7)):
        full = b.build_matrix(base, m, shard)
        assert full.shape == base.shape
        for begin, count in ((0, 64), (b.ROWS - 64, 64), (1792 * 3, 128)):
            assert np.array_equal(b.matrix_rows(base, m, shard, begin, count), full[begin:begin + count])
    # distinct matrices: different rotation and one flipped byte lane
    assert not np.array_equal(b.build_matrix(base, 1, 0), b.build_matrix(base, 2, 0))
    assert not np.array_equal(b.build_matrix(base, 1, 0), b.build_matrix(base, 1, 1))
    assert np.array_equal(b.build_matrix(base, 0, 0), base)


def test_both_arms_print_the_same_config():
    b = _bench()
    for world in (1, 2, 8):
        ours = b.bench_config(world, True)
        assert ours == b.bench_config(world, True)
        assert ours["rows"] == b.ROWS and ours["cols"] == b.K_COLS and "larger than L2" in ours["l2"]
    assert b.bench_config(4, False)["rows"] == 4 * b.ROWS          # the weak-scaling variant says so
    assert b.ALGO_BYTES_PER_CALL == 33_103_872


def test_error_figures_shape():
    b = _bench()
    y_ref = np.array([1.0, -2.0, 0.0, 4.0], np.float32)
    y_gpu = y_ref + np.array([1e-7, 0.0, 1e-9, -4e-6], np.float32)
    mag = np.array([10.0, 20.0, 1.0, 40.0])
    f = b.error_figures(y_gpu, y_ref, y_ref.astype(np.float64), mag)
    assert f["rows"] == 4 and f["normwise_vs_cpu_f32"]["gate"] == 1e-5
    assert f["normwise_vs_cpu_f32"]["max"] <= 1.1e-7
    assert 0.0 <= f["strict_rel_vs_cpu_f32"]["frac_within_1e-5"] <= 1.0
    assert f["strict_rel_vs_cpu_f32"]["max"] >= 9e-10            # the zero row is measured absolutely
