"""Parity of the CUDA kernels with the CPU oracle, through the C ABI (device layer).

Bars: dequantised weights bit-exact; reference-order kernels bit-exact in y; the fast kernels
within 1e-5 of the oracle per row, measured norm-wise (|dy| / sum_i |w_i x_i|), because the
reference's own sequential fp32 sum misses the exact dot product by more than 1e-5 of |y| on a
few percent of rows (cancellation), so no reordered sum can meet a strict |dy|/|y| bound on
every row.  The strict figure is still computed and bounded in distribution.
"""
import hashlib

import numpy as np
import pytest

import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

NORMWISE_TOL = 1e-5     # the stated output tolerance
REFERENCE_TOL = 1e-3    # the reference's own GPU-vs-CPU tolerance (compile_q4km_dequant_matvec.rs:946-956)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_err_reference_rule(gpu, cpu):
    """|gpu - cpu| / |cpu| when |cpu| > 1e-10, else absolute (the reference's rule)."""
    gpu, cpu = np.asarray(gpu, np.float64), np.asarray(cpu, np.float64)
    d = np.abs(gpu - cpu)
    return np.where(np.abs(cpu) > 1e-10, d / np.maximum(np.abs(cpu), 1e-300), d)


def check_fast(fmt, y_gpu, q, x, rows, n):
    y_ref = oracle.matvec_rows(fmt, q, x, rows, n)
    y64, mag = oracle.matvec_rows_f64(fmt, q, x, rows, n)
    y_gpu = np.asarray(y_gpu, np.float64)
    mag = np.maximum(mag, 1e-300)
    normwise = np.abs(y_gpu - y_ref) / mag
    assert normwise.max() <= NORMWISE_TOL, f"norm-wise error {normwise.max():.3e}"
    # against exact arithmetic the GPU must be at least as good as the fp32-sequential reference
    e_gpu = np.abs(y_gpu - y64) / mag
    e_ref = np.abs(y_ref - y64) / mag
    assert e_gpu.max() <= max(2.0 * e_ref.max(), 5e-7), (e_gpu.max(), e_ref.max())
    return rel_err_reference_rule(y_gpu, y_ref)   # strict figure, for callers that bound it


# ---------------------------------------------------------------------------------- Q4_K_M

@pytest.mark.parametrize("rows,n_sb", [(1, 1), (3, 2), (8, 16), (9, 3), (7, 56), (2, 128), (5, 200)])
def test_q4k_dequant_is_bit_exact(ops, synth, rows, n_sb):
    q = synth.q4k_weights(rows, n_sb, 100 + rows * 7 + n_sb)
    w = ops.q4k_dequant(dev(q), rows, n_sb).cpu().numpy()
    w_ref = oracle.dequant_rows("q4k", q, rows, n_sb)
    assert (w.view(np.uint32) == w_ref.view(np.uint32)).all()


def test_q4k_dequant_lcg_fixture_matches_golden_hash(ops, golden):
    for fx in golden["lcg"]["fixtures"]:
        q, _x = oracle.generate_q4km_test_data(fx["n_superblocks"], fx["seed"])
        w = ops.q4k_dequant(dev(q), 1, fx["n_superblocks"]).cpu().numpy()
        assert hashlib.sha256(w.tobytes()).hexdigest() == fx["w_sha256"]


def test_q4k_dequant_special_scales_bit_exact(ops, synth):
    """fp16 subnormals, zeros, Inf and NaN in d / dmin are widened exactly and propagate."""
    rows, n_sb = 4, 8
    q = synth.q4k_weights(rows, n_sb, 9).reshape(-1, 144)
    specials = [0x0001, 0x03FF, 0x0000, 0x8000, 0x7C00, 0xFC00, 0x7E00, 0x0400, 0x7BFF]
    for i in range(q.shape[0]):
        q[i, 0:2] = np.frombuffer(np.uint16(specials[i % len(specials)]).tobytes(), np.uint8)
        q[i, 2:4] = np.frombuffer(np.uint16(specials[(i * 5 + 3) % len(specials)]).tobytes(), np.uint8)
    q = q.reshape(-1)
    w = ops.q4k_dequant(dev(q), rows, n_sb).cpu().numpy().view(np.uint32)
    w_ref = oracle.dequant_rows("q4k", q, rows, n_sb).view(np.uint32)
    nan = (w_ref & 0x7FFFFFFF) > 0x7F800000
    assert ((w == w_ref) | nan).all()
    assert (((w & 0x7FFFFFFF) > 0x7F800000) == nan).all()


def test_q4k_seq_kernel_is_bit_identical_on_the_reference_fixture(ops, golden):
    """The reference's own parity case (AT-1324 / AT-1331: n = 128, seed 0xDEADBEEF, one output)
    and its bench pre-flight seed, in reference operation order: same bits as the CPU function."""
    for fx in golden["lcg"]["fixtures"]:
        n = fx["n_superblocks"]
        q, x = oracle.generate_q4km_test_data(n, fx["seed"])
        y = ops.q4k_matvec_seq(dev(q), dev(x), 1, n).cpu().numpy()
        assert int(y.view(np.uint32)[0]) == fx["y_bits"]


@pytest.mark.parametrize("rows,n_sb", [(8, 16), (33, 5), (4, 56)])
def test_q4k_seq_kernel_bit_identical_rows(ops, synth, rows, n_sb):
    q = synth.q4k_weights(rows, n_sb, 31 + rows)
    x = synth.activations(n_sb * 256, 32 + rows)
    y = ops.q4k_matvec_seq(dev(q), dev(x), rows, n_sb).cpu().numpy()
    y_ref = oracle.matvec_rows("q4k", q, x, rows, n_sb)
    assert (y.view(np.uint32) == y_ref.view(np.uint32)).all()


def test_q4k_fast_kernel_on_the_reference_fixture(ops, golden):
    for fx in golden["lcg"]["fixtures"]:
        n = fx["n_superblocks"]
        q, x = oracle.generate_q4km_test_data(n, fx["seed"])
        st = ops.new_status()
        y = ops.q4k_matvec(dev(q), dev(x), 1, n, status=st).cpu().numpy()
        assert int(st.item()) == 0
        cpu = np.array([fx["y_bits"]], np.uint32).view(np.float32)
        assert rel_err_reference_rule(y, cpu)[0] < 1e-5
        check_fast("q4k", y, q, x, 1, n)


@pytest.mark.parametrize("rows,n_sb", [
    (8, 16),        # config 0: 8 rows x 4096
    (1, 1), (1, 2), (2, 3), (7, 16), (9, 16), (1, 16), (300, 16), (1000, 16),
    (5, 56), (64, 56),          # down-projection row length (K = 14336)
    (6, 32), (3, 112),          # 70B-shaped rows (K = 8192, 28672)
    (2, 128), (3, 129), (2, 200), (1, 512),   # K segmented beyond 128 superblocks
])
def test_q4k_fast_kernel_matches_oracle(ops, synth, rows, n_sb):
    q = synth.q4k_weights(rows, n_sb, 1000 + rows * 13 + n_sb)
    x = synth.activations(n_sb * 256, 2000 + rows + n_sb)
    st = ops.new_status()
    y = ops.q4k_matvec(dev(q), dev(x), rows, n_sb, status=st).cpu().numpy()
    assert int(st.item()) == 0
    check_fast("q4k", y, q, x, rows, n_sb)


@pytest.mark.parametrize("scale_exp", [-100, -60, -20, 20, 60, 100])
def test_q4k_fast_kernel_is_scale_invariant(ops, synth, scale_exp):
    """Activations of any magnitude: the power-of-two pre-scaling must not lose them."""
    rows, n_sb = 16, 16
    q = synth.q4k_weights(rows, n_sb, 77)
    x = (synth.activations(n_sb * 256, 78).astype(np.float64) * 2.0 ** scale_exp).astype(np.float32)
    y = ops.q4k_matvec(dev(q), dev(x), rows, n_sb).cpu().numpy()
    check_fast("q4k", y, q, x, rows, n_sb)


def test_q4k_fast_kernel_mixed_magnitudes_and_zeros(ops, synth):
    rows, n_sb = 12, 16
    q = synth.q4k_weights(rows, n_sb, 79)
    x = synth.activations(n_sb * 256, 80)
    x[:64] = 0.0                      # a whole chunk of zeros
    x[64:128] *= 1e-30                # a tiny chunk
    x[128:192] *= 1e20                # a huge chunk
    x[300] = 0.0
    y = ops.q4k_matvec(dev(q), dev(x), rows, n_sb).cpu().numpy()
    check_fast("q4k", y, q, x, rows, n_sb)


def test_q4k_nonfinite_inputs_propagate_without_trapping(ops, synth):
    """bench_variant feeds uniform random bytes: fp16 scales and fp32 activations may be Inf/NaN.
    Rows the oracle makes non-finite must come out non-finite; finite rows must still match."""
    rows, n_sb = 32, 4
    rng = np.random.default_rng(5)
    q = rng.integers(0, 256, rows * n_sb * 144, dtype=np.uint8)
    x = synth.activations(n_sb * 256, 6)
    st = ops.new_status()
    y = ops.q4k_matvec(dev(q), dev(x), rows, n_sb, status=st).cpu().numpy()
    assert int(st.item()) == 0
    with np.errstate(all="ignore"):
        y_ref = oracle.matvec_rows("q4k", q, x, rows, n_sb)
    finite = np.isfinite(y_ref)
    assert (np.isfinite(y) == finite).all()
    x2 = x.copy()
    x2[5] = np.inf
    x2[700] = np.nan
    y2 = ops.q4k_matvec(dev(synth.q4k_weights(rows, n_sb, 8)), dev(x2), rows, n_sb).cpu().numpy()
    assert not np.isfinite(y2).any()


def test_q4k_zero_superblocks_writes_positive_zero(ops):
    q = torch.zeros(16, dtype=torch.uint8, device="cuda")
    x = torch.zeros(4, dtype=torch.float32, device="cuda")
    y = torch.full((5,), 7.0, dtype=torch.float32, device="cuda")
    ops.q4k_matvec(q, x, 5, 0, y=y)
    assert (y.cpu().numpy().view(np.uint32) == 0).all()


def test_q4k_tuning_variants_agree(ops, synth):
    rows, n_sb = 513, 16
    q = synth.q4k_weights(rows, n_sb, 91)
    x = synth.activations(n_sb * 256, 92)
    y_ref = oracle.matvec_rows("q4k", q, x, rows, n_sb)
    _y64, mag = oracle.matvec_rows_f64("q4k", q, x, rows, n_sb)
    for kw in (dict(ctas_per_sm=1), dict(ctas_per_sm=2, tile_rows=4, stages=2), dict(tile_rows=16),
               dict(stages=1), dict(evict_first=1), dict(ctas_per_sm=1, tile_rows=32, stages=3), dict(pdl=3),
               dict(pdl=0), dict(threads=512, ctas_per_sm=1), dict(threads=128, ctas_per_sm=4)):
        for _ in range(2):   # back to back: exercises the programmatic-dependent-launch modes
            y_d = ops.q4k_matvec(dev(q), dev(x), rows, n_sb, tuning=ops.make_tuning(**kw))
        y = y_d.cpu().numpy()
        assert (np.abs(y - y_ref) / mag).max() <= NORMWISE_TOL, kw


def test_q4k_ring_refill_path(ops, synth):
    """More rows per CTA than the shared-memory ring holds: stages are recycled through the
    empty-barrier / claim protocol (also forced with one- and two-stage rings)."""
    rows, n_sb = 20000, 16
    q = synth.q4k_weights(rows, n_sb, 93)
    x = synth.activations(n_sb * 256, 94)
    y_ref = oracle.matvec_rows("q4k", q, x, rows, n_sb)
    _y64, mag = oracle.matvec_rows_f64("q4k", q, x, rows, n_sb)
    qd, xd = dev(q), dev(x)
    for kw in (dict(), dict(stages=1), dict(stages=2, tile_rows=4), dict(ctas_per_sm=1, stages=3),
               dict(stages=2, tile_rows=16, pdl=0)):
        st = ops.new_status()
        for _ in range(3):   # back-to-back launches also exercise programmatic dependent launch
            y = ops.q4k_matvec(qd, xd, rows, n_sb, status=st, tuning=ops.make_tuning(**kw))
        assert int(st.item()) == 0, kw
        assert (np.abs(y.cpu().numpy() - y_ref) / mag).max() <= NORMWISE_TOL, kw


def test_q4k_fused_allgather_epilogue_single_rank(synth):
    """The all-gather epilogue with world = 1 (peer table = own buffer): every slice lands at the
    row offset of its slot as (value, epoch) words in the copy of the step's parity, finish()
    unpacks exactly the plain matvec's values and ends the step (epoch advanced, done word set)."""
    from conftest import load_pkg
    coll = load_pkg("collective")
    ops_ = load_pkg("ops")
    rows, n_sb, slots = 777, 16, 3
    pg = coll.PeerGather(rows, slots, "cuda")
    assert (pg.world, pg.rank, pg.row_offset, pg.rows_local) == (1, 0, 0, rows)
    st = ops_.new_status()
    n = rows * slots
    for it in range(3):
        epoch = it + 1
        assert int(pg.epoch.item()) == epoch
        cases = []
        for slot in range(slots):
            q = synth.q4k_weights(rows, n_sb, 4000 + 10 * it + slot)
            x = synth.activations(n_sb * 256, 4100 + 10 * it + slot)
            pg.matvec(dev(q), dev(x), n_sb, slot, status=st,
                      tuning=ops_.make_tuning(pdl=3 if slot else 2))
            cases.append((q, x))
        # on odd iterations the finish launch lets the launches behind it start while it waits
        pg.finish(st, let_next_start=bool(it % 2))
        for slot, (q, x) in enumerate(cases):
            y = pg.vector(slot)
            y_plain = ops_.q4k_matvec(dev(q), dev(x), rows, n_sb)
            assert torch.equal(y, y_plain)
            y_ref = oracle.matvec_rows("q4k", q, x, rows, n_sb)
            _y64, mag = oracle.matvec_rows_f64("q4k", q, x, rows, n_sb)
            assert (np.abs(y.cpu().numpy() - y_ref) / mag).max() <= NORMWISE_TOL
        assert int(pg.epoch.item()) == epoch + 1                   # finish ended the step
        words = pg.pairs.cpu().numpy()
        copy = words[(epoch & 1) * n:(epoch & 1) * n + n]
        assert ((copy >> 32) == epoch).all()                       # every word carries the step's epoch
        other = words[(1 - (epoch & 1)) * n:(1 - (epoch & 1)) * n + n]
        assert ((other >> 32) == max(epoch - 1, 0)).all()          # the other copy still holds the step before
        assert int(words[2 * n:].view(np.int32)[0]) == epoch       # this rank's done word
    assert int(st.item()) == 0


def test_gather_finish_times_out_without_faulting():
    """A word whose epoch never arrives: finish() gives up after its bounded wait, sets the
    peer-wait bit in the status word and leaves the context usable."""
    from conftest import load_pkg
    coll = load_pkg("collective")
    ops_ = load_pkg("ops")
    pg = coll.PeerGather(8, 1, "cuda")      # epoch 1, nothing stores
    st = ops_.new_status()
    pg.finish(st)
    torch.cuda.synchronize()
    assert int(st.item()) & 4
    assert torch.zeros(4, device="cuda").sum().item() == 0.0


def test_gather_finish_reports_a_word_from_a_later_epoch():
    """A producer that ran ahead of the reader (storage reused too early) is reported, not
    accepted: a word of epoch 3 in the copy that epoch 1 reads sets bit 8."""
    from conftest import load_pkg
    coll = load_pkg("collective")
    ops_ = load_pkg("ops")
    pg = coll.PeerGather(8, 1, "cuda")
    words = torch.full((8,), (1 << 32) | 0x3F800000, dtype=torch.int64, device="cuda")
    words[5] = (3 << 32) | 0x40000000
    pg.pairs[8:16] = words                  # epoch 1 is odd: second copy
    st = ops_.new_status()
    pg.finish(st)
    torch.cuda.synchronize()
    assert int(st.item()) == 8
    assert pg.vector(0)[0].item() == 1.0


# ---------------------------------------------------------------------------------- Q4_0

@pytest.mark.parametrize("rows,n", [(1, 1), (3, 2), (5, 7), (8, 128), (2, 1024), (2, 1030)])
def test_q4_0_dequant_is_bit_exact(ops, synth, rows, n):
    q = synth.q4_0_weights(rows, n, 300 + rows + n)
    w = ops.q4_0_dequant(dev(q), rows, n).cpu().numpy()
    w_ref = oracle.dequant_rows("q4_0", q, rows, n)
    assert (w.view(np.uint32) == w_ref.view(np.uint32)).all()


def test_q4_0_reference_layout_fixtures_on_gpu(ops, golden):
    for case in golden["known"]["q4_0_layout"]:
        q = np.zeros(32, np.uint8)
        q[:18] = case["q"]
        x = np.array(case["x"], np.float32)
        for fn in (ops.q4_0_matvec, ops.q4_0_matvec_seq):
            y = fn(dev(q), dev(x), 1, 1).cpu().numpy()
            assert abs(float(y[0]) - case["expected"]) < case["abs_tol"]


@pytest.mark.parametrize("rows,n", [(1, 128), (1, 1024), (17, 5), (40, 128)])
def test_q4_0_seq_kernel_is_bit_identical(ops, synth, rows, n):
    q = synth.q4_0_weights(rows, n, 400 + rows + n)
    x = np.random.default_rng(n).uniform(-1, 1, n * 32).astype(np.float32)
    y = ops.q4_0_matvec_seq(dev(q), dev(x), rows, n).cpu().numpy()
    y_ref = oracle.matvec_rows("q4_0", q, x, rows, n)
    assert (y.view(np.uint32) == y_ref.view(np.uint32)).all()


@pytest.mark.parametrize("rows,n", [
    (1, 128), (1, 1024),            # the reference's bench sizes (one output)
    (1, 1), (1, 2), (3, 3), (5, 7), (9, 2), (7, 10), (33, 64), (100, 128), (513, 128),
    (3, 66), (2, 448), (4, 1024), (2, 1026), (3, 2049),
])
def test_q4_0_fast_kernel_matches_oracle(ops, synth, rows, n):
    q = synth.q4_0_weights(rows, n, 500 + rows * 3 + n)
    x = synth.activations(n * 32, 600 + rows + n)
    pad = np.zeros(((q.size + 31) // 16) * 16, np.uint8)   # spare tail, as any allocator gives
    pad[:q.size] = q
    st = ops.new_status()
    y = ops.q4_0_matvec(dev(pad), dev(x), rows, n, status=st).cpu().numpy()
    assert int(st.item()) == 0
    check_fast("q4_0", y, q, x, rows, n)


def test_q4_0_zero_blocks_writes_positive_zero(ops):
    q = torch.zeros(32, dtype=torch.uint8, device="cuda")
    x = torch.zeros(4, dtype=torch.float32, device="cuda")
    y = torch.full((3,), -1.0, dtype=torch.float32, device="cuda")
    ops.q4_0_matvec(q, x, 3, 0, y=y)
    assert (y.cpu().numpy().view(np.uint32) == 0).all()


# ------------------------------------------------------------------- full benchmark sizes

def _full_size_check(ops, fmt, q_np, x_np, rows, n, sample_rows, tuning=None, calls=1):
    """Full-size run: every row against an fp64 product of the GPU's own bit-exact dequantised
    weights (themselves checked against the oracle on a row sample), the oracle on the sample.
    `calls` back-to-back launches with `tuning` (each into its own y; all must agree bit for bit)."""
    q, x = dev(q_np), dev(x_np)
    blk_b, blk_e = (144, 256) if fmt == "q4k" else (18, 32)
    matvec_ = ops.q4k_matvec if fmt == "q4k" else ops.q4_0_matvec
    matvec = lambda *a, **kw: matvec_(*a, tuning=tuning, **kw)
    dequant = ops.q4k_dequant if fmt == "q4k" else ops.q4_0_dequant
    st = ops.new_status()
    ys = [torch.full((rows,), float("nan"), dtype=torch.float32, device="cuda") for _ in range(calls)]
    for yy in ys:
        matvec(q, x, rows, n, y=yy, status=st)
    y = ys[0]
    assert int(st.item()) == 0
    for yy in ys[1:]:
        assert torch.equal(yy, y)
    w = dequant(q, rows, n)
    for r in sample_rows:
        w_ref = oracle.dequant_rows(fmt, q_np[r * n * blk_b:(r + 1) * n * blk_b], 1, n)[0]
        assert (w[r].cpu().numpy().view(np.uint32) == w_ref.view(np.uint32)).all()
    xd = x.double()
    y64 = w.double() @ xd
    mag = w.double().abs() @ xd.abs()
    normwise = ((y.double() - y64).abs() / mag).max().item()
    assert normwise <= NORMWISE_TOL, normwise
    idx = np.array(sample_rows)
    y_ref = np.array([oracle.matvec_rows(fmt, q_np[r * n * blk_b:(r + 1) * n * blk_b], x_np, 1, n)[0]
                      for r in sample_rows])
    got = y.cpu().numpy()[idx]
    assert (np.abs(got - y_ref) / mag.cpu().numpy()[idx]).max() <= NORMWISE_TOL
    # linearity: y(a*x) == a*y(x) exactly for a power of two
    y2 = matvec(q, x * 4.0, rows, n)
    assert torch.equal(y2, y * 4.0)
    return y


def test_q4k_full_size_up_gate_14336x4096(ops, synth):
    rows, n = 14336, 16
    q = synth.q4k_weights(rows, n, synth.config_seed(2, 0))
    x = synth.activations(n * 256, synth.config_seed(2, 1))
    y = _full_size_check(ops, "q4k", q, x, rows, n, [0, 1, 48, 49, 7167, 14335])
    # strict relative figure against the oracle on a 2048-row sample, in distribution
    rs = 2048
    y_ref = oracle.matvec_rows("q4k", q[:rs * n * 144], x, rs, n)
    strict = rel_err_reference_rule(y.cpu().numpy()[:rs], y_ref)
    assert np.median(strict) < 5e-6 and (strict <= 1e-5).mean() > 0.90 and strict.max() < 1e-1


def test_q4k_full_size_down_4096x14336(ops, synth):
    rows, n = 4096, 56
    q = synth.q4k_weights(rows, n, synth.config_seed(2, 2))
    x = synth.activations(n * 256, synth.config_seed(2, 3))
    _full_size_check(ops, "q4k", q, x, rows, n, [0, 27, 28, 2047, 4095])


def test_q4_0_full_size_4096x4096(ops, synth):
    rows, n = 4096, 128
    q = synth.q4_0_weights(rows, n, synth.config_seed(1, 0))
    x = synth.activations(n * 32, synth.config_seed(1, 1))
    _full_size_check(ops, "q4_0", q, x, rows, n, [0, 13, 14, 2048, 4095])


@pytest.mark.parametrize("shape", ["up_gate_14336x4096", "down_4096x14336", "q4_0_4096x4096"])
def test_full_size_under_the_benchmark_launch_geometry(ops, synth, shape):
    """The geometry the benchmark times: calls declared independent (pdl = 3: one small CTA per SM,
    several launches resident), three launches back to back, every row checked."""
    tn = ops.make_tuning(pdl=3)
    if shape == "up_gate_14336x4096":
        rows, n, fmt = 14336, 16, "q4k"
        q, x = synth.q4k_weights(rows, n, synth.config_seed(2, 0)), synth.activations(n * 256, synth.config_seed(2, 1))
    elif shape == "down_4096x14336":
        rows, n, fmt = 4096, 56, "q4k"
        q, x = synth.q4k_weights(rows, n, synth.config_seed(2, 2)), synth.activations(n * 256, synth.config_seed(2, 3))
    else:
        rows, n, fmt = 4096, 128, "q4_0"
        q, x = synth.q4_0_weights(rows, n, synth.config_seed(1, 0)), synth.activations(n * 32, synth.config_seed(1, 1))
    y3 = _full_size_check(ops, fmt, q, x, rows, n, [0, 1, rows // 2, rows - 1], tuning=tn, calls=3)
    # and the same values as the ordered geometry delivers
    y2 = (ops.q4k_matvec if fmt == "q4k" else ops.q4_0_matvec)(dev(q), dev(x), rows, n, tuning=ops.make_tuning(pdl=2))
    assert torch.equal(y3, y2)


def test_independent_launch_behind_an_ordered_one_sees_the_producer(ops, synth):
    """producer matvec -> ordered matvec (pdl 2) -> independent matvec (pdl 3), both consumers
    reading the producer's y as their x.  The independent launch reads x without waiting; the
    ordered launch in between lets it be scheduled only after its own wait, i.e. when the producer
    is complete, so both consumers must match the oracle on the oracle's own intermediate."""
    k0, mid, rows = 4096, 4096, 3000
    wp = synth.q4k_weights(mid, k0 // 256, 9101)
    wg = synth.q4k_weights(rows, mid // 256, 9102)
    wu = synth.q4k_weights(rows, mid // 256, 9103)
    x0 = synth.activations(k0, 9104)
    wpd, wgd, wud, x0d = dev(wp), dev(wg), dev(wu), dev(x0)
    v = torch.zeros(mid, device="cuda")
    yg, yu = torch.zeros(rows, device="cuda"), torch.zeros(rows, device="cuda")
    st = ops.new_status()
    for it in range(5):
        v.zero_()     # a consumer that ran ahead of the producer would read zeros
        ops.q4k_matvec(wpd, x0d, mid, k0 // 256, y=v, status=st, tuning=ops.make_tuning(pdl=2))
        ops.q4k_matvec(wgd, v, rows, mid // 256, y=yg, status=st, tuning=ops.make_tuning(pdl=2))
        ops.q4k_matvec(wud, v, rows, mid // 256, y=yu, status=st, tuning=ops.make_tuning(pdl=3))
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        v_np = v.cpu().numpy()
        check_fast("q4k", v_np, wp, x0, mid, k0 // 256)
        check_fast("q4k", yg.cpu().numpy(), wg, v_np, rows, mid // 256)
        check_fast("q4k", yu.cpu().numpy(), wu, v_np, rows, mid // 256)


def _log_uniform_x(k, spread_bits, seed):
    """|x| log-uniform over 2^0 .. 2^-spread_bits with random signs, independently per element, so
    every 64-column chunk holds the whole range (the fixed-point scale is per chunk)."""
    rng = np.random.default_rng(seed)
    return (np.exp2(-rng.uniform(0.0, spread_bits, k)) * rng.choice([-1.0, 1.0], k)).astype(np.float32)


@pytest.mark.parametrize("fmt,rows,n", [("q4k", 512, 16), ("q4k", 64, 112), ("q4_0", 512, 128)])
@pytest.mark.parametrize("spread_bits", [10, 30])
def test_magnitudes_spread_inside_every_chunk(ops, synth, fmt, rows, n, spread_bits):
    """Activations whose magnitudes span up to 2^30 INSIDE each 64-column chunk: elements below
    2^-24 of their chunk's maximum are flushed by the fixed point.  Observed norm-wise maximum
    against the oracle: below 1e-6 (a numpy model of the fixed point alone gives 6e-8; the rest is
    the summation-order difference to the fp32-sequential reference, about 3e-7)."""
    blk_e = 256 if fmt == "q4k" else 32
    q = (synth.q4k_weights if fmt == "q4k" else synth.q4_0_weights)(rows, n, 9200 + n)
    x = _log_uniform_x(n * blk_e, spread_bits, 9300 + spread_bits)
    y = (ops.q4k_matvec if fmt == "q4k" else ops.q4_0_matvec)(dev(q), dev(x), rows, n).cpu().numpy()
    y_ref = oracle.matvec_rows(fmt, q, x, rows, n)
    y64, mag = oracle.matvec_rows_f64(fmt, q, x, rows, n)
    assert (np.abs(y - y_ref) / mag).max() <= 1e-6
    assert (np.abs(y - y64) / mag).max() <= 1e-6       # and as close to exact arithmetic


def test_fixed_point_worst_case_stays_inside_its_derived_bound(ops, synth):
    """The adversarial input for a per-chunk fixed point: in every chunk one element at 1.0 placed
    where that row's |w| is smallest, the other 63 at 1.4 * 2^-24 (just above half a unit of the
    fixed point: they round to one unit, an error of 0.3 units each).  Relative to sum |w_i x_i| the
    error is then no longer small, which the derivation beside X_FRAC_BITS says; what must hold is
    the derived absolute bound  |dy| <= 2^-23 * sum_chunks M_c * sum_{i in c} |w_i|  (plus the fp32
    rounding of the row sum)."""
    rows, n = 8, 16
    q = synth.q4k_weights(rows, n, 9400)
    w = oracle.dequant_rows("q4k", q, rows, n).astype(np.float64)
    qd = dev(q)
    for r in range(rows):
        x = np.full(n * 256, 1.4 * 2.0 ** -24, np.float32)
        for c in range(0, n * 256, 64):
            x[c + int(np.argmin(np.abs(w[r, c:c + 64])))] = 1.0
        y = ops.q4k_matvec(qd, dev(x), rows, n).cpu().numpy()[r]
        exact = float(w[r] @ x.astype(np.float64))
        bound = 2.0 ** -23 * np.abs(w[r]).sum() + 1e-6 * float(np.abs(w[r]) @ np.abs(x.astype(np.float64)))
        assert abs(float(y) - exact) <= bound, (r, y, exact, bound)


def test_rows_whose_dequantised_weights_are_all_zero(ops, synth):
    """Rows the reference computes as exactly 0.0 (every dequantised weight is 0), measured by its
    own rule: |cpu| <= 1e-10, so the ABSOLUTE difference counts
    (crates/axc-driver/tests/compile_q4km_dequant_matvec.rs:946-950).
    Q4_0: all nibbles 8 -> (8 - 8) * d = 0; the kernel sums (q - 8) X in integers, so it returns
    exactly 0 too.  Q4_K_M: d = dmin, every nibble q0 and sc * q0 = m, so d*sc*q0 - dmin*m = 0; the
    kernel factors the sum as d*sc*sum(q X) - dmin*m*sum(X) over the same fixed-point X, which
    cancels to rounding: a residual of a few 1e-7 of the cancelled magnitude, held to 1e-5 of it."""
    # Q4_0
    rows, n = 6, 128
    q = synth.q4_0_weights(rows, n, 9500).reshape(rows, n, 18).copy()
    q[2, :, 2:] = 0x88
    q[5, :, 2:] = 0x88
    x = synth.activations(n * 32, 9501) * np.float32(1000.0)
    y = ops.q4_0_matvec(dev(q.reshape(-1)), dev(x), rows, n).cpu().numpy()
    y_cpu = oracle.matvec_rows("q4_0", q.reshape(-1), x, rows, n)
    assert y_cpu[2] == 0.0 and y_cpu[5] == 0.0
    assert y[2] == 0.0 and y[5] == 0.0
    keep = [0, 1, 3, 4]                # (a row of zero weights has no norm-wise figure)
    _y64, mag = oracle.matvec_rows_f64("q4_0", q.reshape(-1), x, rows, n)
    assert (np.abs(y[keep] - y_cpu[keep]) / mag[keep]).max() <= NORMWISE_TOL
    # Q4_K_M
    rows, n = 4, 16
    qk = synth.q4k_weights(rows, n, 9502).reshape(rows, n, 144).copy()
    sc, q0 = 5, 7                     # sc * q0 = 35 = m, both below 64
    one = np.array([0.01], np.float16).view(np.uint8)
    for sb in range(n):
        qk[1, sb, 0:2] = one
        qk[1, sb, 2:4] = one
        qk[1, sb, 4:16] = synth.pack_q4k_scales(np.full(8, sc), np.full(8, sc * q0))
        qk[1, sb, 16:] = q0 | (q0 << 4)
    xk = synth.activations(n * 256, 9503)
    yk = ops.q4k_matvec(dev(qk.reshape(-1)), dev(xk), rows, n).cpu().numpy()
    yk_cpu = oracle.matvec_rows("q4k", qk.reshape(-1), xk, rows, n)
    assert yk_cpu[1] == 0.0
    cancelled = float(np.float32(one.view(np.float16)[0]) * sc * q0 * np.abs(xk).sum())
    assert abs(float(yk[1])) <= 1e-5 * cancelled       # the reference's rule: absolute difference
    assert abs(float(yk[1])) <= 1e-3                   # and inside the reference's own 1e-3 bar
