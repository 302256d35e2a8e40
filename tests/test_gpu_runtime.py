"""Runtime layer through the C ABI with host buffers: the reference's dispatch semantics.

Mirrors crates/axc-driver/tests/compile_q4km_dequant_matvec.rs (AT-1324/1331 parity protocol),
crates/axc-driver/tests/compile_q4_0_dequant_matvec.rs (AT-918) and the runtime behaviour tests
under crates/axc-runtime/tests/ (AT-805 handle reuse + pow2 growth, AT-816 amortisation, AT-827
handle outlives context, AT-516 context lifecycle, AT-517/518/506a typed errors).
"""
import struct
import time

import numpy as np
import pytest

torch = pytest.importorskip("torch")

import oracle

pytestmark = pytest.mark.gpu

SPIRV_STANDIN = [0x07230203, 0x00010300, 0, 1, 0]   # only hashed for the cache key


def pc(n):
    return struct.pack("<I", n)


def f32(buf):
    return np.frombuffer(bytes(buf), np.float32)


@pytest.fixture(scope="module")
def ctx(axc):
    c = axc.CudaContext.new_with_options(axc.CudaContextOptions(None, None, None))
    yield c
    c.drop()


def rel_err(gpu, cpu):
    return abs(gpu - cpu) / abs(cpu) if abs(cpu) > 1e-10 else abs(gpu - cpu)


def test_context_reports_device_and_limits(axc, ctx):
    assert axc.probe_vulkan_available() is True
    assert "B200" in ctx.physical_device_name() or "NVIDIA" in ctx.physical_device_name()
    assert ctx.max_compute_work_group_count() == [2147483647, 65535, 65535]
    assert ctx.sm_count() >= 100


def test_at_1324_q4km_dispatch_matches_cpu_reference(axc, ctx):
    """The reference's parity test verbatim: n = 128, seed 0xDEADBEEF, workgroups [1,1,1], all
    three buffers uploaded and read back, y[0] within 1e-3 relative (here also within 1e-5)."""
    n = 128
    q, x = oracle.generate_q4km_test_data(n, 0xDEADBEEF)
    cpu = float(oracle.q4km_dequant_matvec_cpu(q, x, n))
    plan = axc.q4_matvec_binding_plan("q4km_dequant_matvec")
    req = axc.DispatchRequest(
        spirv=SPIRV_STANDIN, binding_plan=plan, workgroups=[1, 1, 1],
        inputs=[q.tobytes(), x.tobytes(), bytes(4)], output_sizes=[q.size, x.size * 4, 4],
        push_constants=pc(n), entry_point="q4km_dequant_matvec")
    out = ctx.dispatch(req)
    assert [len(o) for o in out] == [q.size, x.size * 4, 4]
    assert bytes(out[0]) == q.tobytes() and bytes(out[1]) == x.tobytes()   # inputs read back intact
    gpu = float(f32(out[2])[0])
    assert rel_err(gpu, cpu) < 1e-3
    assert rel_err(gpu, cpu) < 1e-5


def test_at_918_q4_0_dispatch_matches_cpu_reference(axc, ctx, synth):
    for n in (128, 1024):
        rng = np.random.default_rng(42)
        q = synth.q4_0_weights(1, n, 42)
        scale = rng.uniform(0.1, 1.0, n).astype(np.float32).astype(np.float16)
        q.reshape(n, 18)[:, 0:2] = scale.view(np.uint8).reshape(n, 2)
        x = rng.uniform(-1, 1, n * 32).astype(np.float32)
        cpu = float(oracle.q4_0_dequant_matvec_cpu(q, x, n))
        plan = axc.q4_matvec_binding_plan("q4_0_dequant_matvec")
        out = ctx.dispatch(axc.DispatchRequest(
            SPIRV_STANDIN, plan, [1, 1, 1], [q.tobytes(), x.tobytes(), bytes(4)],
            [q.size, x.size * 4, 4], pc(n), "q4_0_dequant_matvec"))
        gpu = float(f32(out[2])[0])
        assert rel_err(gpu, cpu) < 1e-3 and abs(gpu - cpu) < 1e-3   # test + bench pre-flight bars


def test_strict_order_handle_is_bit_identical(axc, ctx, golden):
    fx = [f for f in golden["lcg"]["fixtures"] if f["n_superblocks"] == 128 and f["seed"] == 0xCAFEBABE][0]
    q, x = oracle.generate_q4km_test_data(128, 0xCAFEBABE)
    plan = axc.q4_matvec_binding_plan()
    h = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x51)
    h.set_strict_order(True)
    out = ctx.dispatch_handle(h, (1, 1, 1), [q.tobytes(), x.tobytes(), b""], [0, 0, 4], pc(128))
    assert int(np.frombuffer(bytes(out[2]), np.uint32)[0]) == fx["y_bits"]
    h.set_strict_order(False)
    out2 = ctx.dispatch_handle(h, (1, 1, 1), [b"", b"", b""], [0, 0, 4], pc(128))
    assert rel_err(float(f32(out2[2])[0]), float(f32(out[2])[0])) < 1e-5


def test_rows_from_grid_and_resident_weights(axc, ctx, synth):
    """rows = workgroups.x; the push constant stays 'blocks per ROW'; an empty input keeps the
    device contents (upload q once, then dispatch with inputs [empty, x, empty])."""
    rows, n = 64, 16
    q = synth.q4k_weights(rows, n, 3)
    plan = axc.q4_matvec_binding_plan()
    h = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x52)
    x0 = synth.activations(n * 256, 4)
    out, st = ctx.dispatch_handle(h, (rows, 1, 1), [q, x0, b""], [0, 0, rows * 4], pc(n), stats=True)
    assert st.rows_effective == rows and st.blocks_per_row == n and st.kernel_ns > 0
    y_ref = oracle.matvec_rows("q4k", q, x0, rows, n)
    _y64, mag = oracle.matvec_rows_f64("q4k", q, x0, rows, n)
    assert (np.abs(f32(out[2]) - y_ref) / mag).max() < 1e-5
    assert len(out[0]) == 0 and len(out[1]) == 0
    for seed in (5, 6):
        x1 = synth.activations(n * 256, seed)
        out = ctx.dispatch_handle(h, (rows, 1, 1), [b"", x1, b""], [0, 0, rows * 4], pc(n))
        y_ref = oracle.matvec_rows("q4k", q, x1, rows, n)
        _y64, mag = oracle.matvec_rows_f64("q4k", q, x1, rows, n)
        assert (np.abs(f32(out[2]) - y_ref) / mag).max() < 1e-5


def test_rows_are_clamped_to_what_the_buffers_hold(axc, ctx, synth):
    """bench_variant derives workgroups.x from the byte length of q, which over-counts rows;
    the backend clamps to floor(q_len / row_bytes) and to y_len / 4 instead of overrunning."""
    rows, n = 8, 16
    q = synth.q4k_weights(rows, n, 13)
    x = synth.activations(n * 256, 14)
    plan = axc.q4_matvec_binding_plan()
    h = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x53)
    out, st = ctx.dispatch_handle(h, (72, 1, 1), [q, x, bytes(rows * 4)], [0, 0, rows * 4], pc(n), stats=True)
    assert st.rows_effective == rows
    out, st = ctx.dispatch_handle(h, (72, 1, 1), [q, x, bytes(12)], [0, 0, 12], pc(n), stats=True)
    assert st.rows_effective == 3
    y_ref = oracle.matvec_rows("q4k", q, x, 3, n)
    assert np.allclose(f32(out[2]), y_ref, rtol=1e-4)


def test_zero_push_constant_gives_positive_zero(axc, ctx):
    """grid_search dispatches with zeroed push constants: n = 0 must yield y[0] = +0.0."""
    plan = axc.q4_matvec_binding_plan()
    for entry in ("q4km_dequant_matvec", "q4_0_dequant_matvec"):
        h = ctx.prepare_kernel(SPIRV_STANDIN, axc.q4_matvec_binding_plan(entry), 4, entry, spirv_hash=0x54)
        out = ctx.dispatch_handle(h, (1, 1, 1), [bytes(4096), bytes(4096), b"\xff" * 4096],
                                  [4096, 4096, 4096], pc(0))
        assert bytes(out[2][:4]) == bytes(4)
    del plan


def test_at_805_handle_reuse_and_pow2_growth(axc, ctx, synth):
    plan = axc.q4_matvec_binding_plan()
    h1 = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x55)
    h2 = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x55)
    assert h1.inner_id() == h2.inner_id()                     # same key -> same inner object
    assert h1.cache_key() == h2.cache_key() and h1.cache_key().push_constant_bytes == 4
    h3 = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x56)
    assert h3.inner_id() != h1.inner_id()
    assert h1.buffer_sizes() == []
    q, x = oracle.generate_q4km_test_data(1, 1)
    ctx.dispatch_handle(h1, (1, 1, 1), [q, x, bytes(4)], [0, 0, 4], pc(1))
    assert h1.buffer_sizes() == [256, 1024, 4]                # round_up_pow2(144), 1024, min 4
    q, x = oracle.generate_q4km_test_data(3, 1)
    ctx.dispatch_handle(h1, (1, 1, 1), [q, x, bytes(4)], [0, 0, 4], pc(3))
    assert h1.buffer_sizes() == [512, 4096, 4]                # grew
    q, x = oracle.generate_q4km_test_data(1, 1)
    ctx.dispatch_handle(h2, (1, 1, 1), [q, x, bytes(4)], [0, 0, 4], pc(1))
    assert h2.buffer_sizes() == [512, 4096, 4]                # never shrinks
    clone = h1.clone()
    assert clone.inner_id() == h1.inner_id()
    h1.drop(); h2.drop()
    assert clone.buffer_sizes() == [512, 4096, 4]             # clone keeps it alive
    clone.drop(); h3.drop()
    h4 = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x55)
    assert h4.buffer_sizes() == []                            # all refs dropped -> rebuilt fresh


def test_at_816_amortised_dispatch(axc, ctx):
    """100 dispatches on a prepared handle cost less than 50 one-shot-style first calls."""
    n = 16
    q, x = oracle.generate_q4km_test_data(n, 7)
    plan = axc.q4_matvec_binding_plan()
    h = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x57)
    t0 = time.perf_counter()
    ctx.dispatch_handle(h, (1, 1, 1), [q, x, bytes(4)], [0, 0, 4], pc(n))
    first = time.perf_counter() - t0
    t0 = time.perf_counter()
    for _ in range(100):
        ctx.dispatch_handle(h, (1, 1, 1), [q, x, bytes(4)], [0, 0, 4], pc(n))
    hundred = time.perf_counter() - t0
    assert hundred < 50 * max(first, 2e-4)


def test_at_827_handle_outlives_context(axc):
    c = axc.CudaContext.new()
    plan = axc.q4_matvec_binding_plan()
    h = c.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec")
    q, x = oracle.generate_q4km_test_data(2, 9)
    c.dispatch_handle(h, (1, 1, 1), [q, x, bytes(4)], [0, 0, 4], pc(2))
    c.drop()
    assert h.buffer_sizes() == [512, 2048, 4]
    assert h.spirv_word_count() == len(SPIRV_STANDIN)
    h.drop()


def test_at_516_context_lifecycle_12x(axc):
    for _ in range(12):
        c = axc.CudaContext.new()
        assert c.physical_device_name()
        c.drop()


def test_typed_errors_before_any_allocation(axc, ctx):
    E = axc.errors
    plan = axc.q4_matvec_binding_plan()
    h = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x58)
    with pytest.raises(E.BindingCountMismatch) as ei:          # AT-517
        ctx.dispatch_handle(h, (1, 1, 1), [b"", b""], [0, 0, 4], pc(1))
    assert (ei.value.expected, ei.value.provided) == (3, 2)
    with pytest.raises(E.BindingCountMismatch) as ei:
        ctx.dispatch_handle(h, (1, 1, 1), [b"", b"", b""], [0, 4], pc(1))
    assert (ei.value.expected, ei.value.provided) == (3, 2)
    with pytest.raises(E.PushConstantSizeMismatch) as ei:      # AT-518
        ctx.dispatch_handle(h, (1, 1, 1), [b"", b"", b""], [0, 0, 4], b"\0" * 8)
    assert (ei.value.expected, ei.value.provided) == (4, 8)
    with pytest.raises(E.WorkgroupCountExceedsDeviceLimit) as ei:   # AT-506a
        ctx.dispatch_handle(h, (1, 70000, 1), [b"", b"", b""], [0, 0, 4], pc(1))
    assert ei.value.requested == [1, 70000, 1] and ei.value.max == [2147483647, 65535, 65535]
    assert h.buffer_sizes() == []                              # nothing was allocated
    # order: input count is reported before the push-constant size
    with pytest.raises(E.BindingCountMismatch):
        ctx.dispatch_handle(h, (1, 1, 1), [b""], [0, 0, 4], b"")
    with pytest.raises(E.PipelineCreationFailed, match="unsupported kernel for CUDA backend"):
        ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "saxpy")
    bad = axc.ParamBindingPlan(plan.buffers[:2], plan.scalars, 4)
    with pytest.raises(E.PipelineCreationFailed):
        ctx.prepare_kernel(SPIRV_STANDIN, bad, 4, "q4km_dequant_matvec")
    # x shorter than the push constant demands: a host-side error, never a device fault
    q, x = oracle.generate_q4km_test_data(4, 3)
    with pytest.raises(E.BufferAllocationFailed) as ei:
        ctx.dispatch_handle(h, (1, 1, 1), [q, x[:256], bytes(4)], [0, 0, 4], pc(4))
    assert ei.value.binding == 1
    with pytest.raises(E.BufferAllocationFailed) as ei:
        ctx.dispatch_handle(h, (1, 1, 1), [q[:144], x, bytes(4)], [0, 0, 4], pc(4))
    assert ei.value.binding == 0


def test_bench_dispatch_median_rule(axc, ctx):
    """bench_variant's loop: sample_count timed dispatch_handle calls, median = sorted[len/2]."""
    n = 128
    q, x = oracle.generate_q4km_test_data(n, 0xCAFEBABE)
    plan = axc.q4_matvec_binding_plan()
    h = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x59)
    median, samples, dev_ns, out = ctx.bench_dispatch(
        h, (1, 1, 1), [q, x, bytes(4)], [q.size, x.size * 4, 4], pc(n), 6)
    assert len(samples) == 6 and median == sorted(samples)[3]
    assert all(s > 0 for s in samples) and all(d > 0 for d in dev_ns)
    cpu = float(oracle.q4km_dequant_matvec_cpu(q, x, n))
    assert rel_err(float(f32(out[2])[0]), cpu) < 1e-5


def test_bound_dispatch_repeats_and_rereads_host_input(axc, ctx, synth):
    """``bind`` marshals once; every ``run`` re-reads the caller's host buffer and reuses the
    output buffers."""
    rows, n = 40, 4
    q = synth.q4k_weights(rows, n, 8801)
    x = synth.activations(n * 256, 8802)
    plan = axc.q4_matvec_binding_plan("q4km_dequant_matvec")
    h = ctx.prepare_kernel(SPIRV_STANDIN + [88], plan, 4, "q4km_dequant_matvec")
    xbuf = bytearray(x.tobytes())
    b = ctx.bind(h, (rows, 1, 1), [q, xbuf, b""], [0, 0, rows * 4], pc(n))
    out1 = f32(b.run()[2]).copy()
    y_ref = oracle.matvec_rows("q4k", q, x, rows, n)
    _y64, mag = oracle.matvec_rows_f64("q4k", q, x, rows, n)
    assert (np.abs(out1 - y_ref) / mag).max() <= 1e-5
    x2 = (2.0 * x).astype(np.float32)
    xbuf[:] = x2.tobytes()                      # same buffer object, new contents
    out2 = f32(b.run()[2])
    assert np.array_equal(out2, 2.0 * out1)     # scaling x by two is exact in every step of the kernel
    assert b.run() is b.outputs
    h.drop()


@pytest.mark.parametrize("entry,rows,n", [
    ("q4km_dequant_matvec", 14336, 16),    # one producer CTA for x
    ("q4km_dequant_matvec", 4096, 56),     # K = 14336: four producer CTAs
    ("q4km_dequant_matvec", 300, 128),     # K = 32768: eight
    ("q4km_dequant_matvec", 64, 1),
    ("q4_0_dequant_matvec", 4096, 128),
    ("q4km_dequant_matvec", 63, 16),       # below the row limit of the single-launch path: copy path
])
def test_single_launch_dispatch_matches_the_resident_path(axc, ctx, ops, synth, entry, rows, n):
    """dispatch_handle with resident weights and a fresh host x per call takes the single-launch
    path (x read from mapped host memory by the kernel's first CTAs, y copied to the host by its
    last CTA, completion polled): bit-identical to the device-resident call on the same inputs,
    call after call (a stale x image or an early completion flag would show), and to the timed
    (copy-and-event) path."""
    q4k = entry == "q4km_dequant_matvec"
    q = (synth.q4k_weights if q4k else synth.q4_0_weights)(rows, n, 8800 + rows + n)
    k = n * (256 if q4k else 32)
    plan = axc.q4_matvec_binding_plan(entry)
    h = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, entry, spirv_hash=0x5F00 + rows + n)
    x0 = synth.activations(k, 1)
    ctx.dispatch_handle(h, (rows, 1, 1), [q, x0, b""], [0, 0, rows * 4], pc(n))      # weights uploaded once
    qd = torch.from_numpy(q).cuda()
    fn = ops.q4k_matvec if q4k else ops.q4_0_matvec
    for it in range(12):
        x = synth.activations(k, 8900 + it) * np.float32(1.5 ** it)
        out = ctx.dispatch_handle(h, (rows, 1, 1), [b"", x, b""], [0, 0, rows * 4], pc(n))
        want = fn(qd, torch.from_numpy(x).cuda(), rows, n).cpu().numpy()
        assert np.array_equal(f32(out[2]), want), it
    out_t, st = ctx.dispatch_handle(h, (rows, 1, 1), [b"", b"", b""], [0, 0, rows * 4], pc(n), stats=True)
    assert np.array_equal(f32(out_t[2]), want) and st.rows_effective == rows      # resident x, copy path
    h.drop()


def test_dispatches_on_different_handles_run_concurrently(axc, ctx, ops, synth):
    """Same-handle dispatches serialise on the handle's mutex, different handles may run concurrently
    (crates/axc-runtime/src/context.rs:494-497): four threads, one handle each, many dispatches with
    per-thread x; every result bit-identical to the device-resident call."""
    from concurrent.futures import ThreadPoolExecutor
    rows, n = 2048, 16
    plan = axc.q4_matvec_binding_plan("q4km_dequant_matvec")
    qs = [synth.q4k_weights(rows, n, 9700 + t) for t in range(4)]
    xs = [synth.activations(n * 256, 9710 + t) for t in range(4)]
    hs = []
    for t in range(4):
        h = ctx.prepare_kernel(SPIRV_STANDIN, plan, 4, "q4km_dequant_matvec", spirv_hash=0x7700 + t)
        ctx.dispatch_handle(h, (rows, 1, 1), [qs[t], xs[t], b""], [0, 0, rows * 4], pc(n))
        hs.append(h)
    want = [ops.q4k_matvec(torch.from_numpy(qs[t]).cuda(), torch.from_numpy(xs[t]).cuda(), rows, n).cpu().numpy()
            for t in range(4)]

    def worker(t):
        bad = 0
        for _ in range(200):
            out = ctx.dispatch_handle(hs[t], (rows, 1, 1), [b"", xs[t], b""], [0, 0, rows * 4], pc(n))
            bad += not np.array_equal(f32(out[2]), want[t])
        return bad

    with ThreadPoolExecutor(4) as pool:
        assert list(pool.map(worker, range(4))) == [0, 0, 0, 0]
    for h in hs:
        h.drop()
