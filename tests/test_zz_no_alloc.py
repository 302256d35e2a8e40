"""The allocation-free entry point against the ordinary one (collected last on purpose: if it
fails under ``-x`` every other test has already run).

``axc_cuda_q4k_matvec_static`` serves callers that are not allowed to create device memory when
they need a matvec -- a plug-in inside a host program that owns the GPU's memory pool and bans
driver allocations after start-up, or a decode thread that must stay clear of cudaMalloc /
cudaFree because they synchronise the whole device.  It keeps its only scratch (x quantised into
digit words) in a fixed array inside the library, shared by all calls, so the test makes two
calls in a row with different activations and different shapes and checks each against
``axc_cuda_q4k_matvec`` on the same inputs: same arithmetic, so the results must agree far
inside the 1e-5 norm-wise tolerance of the parity tests (they are in fact bit-identical).
"""
import ctypes as C

import numpy as np
import pytest

import oracle

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

NORMWISE_TOL = 1e-5


def _call_static(ffi, q, x, y, rows, n_sb):
    rc = ffi.lib().axc_cuda_q4k_matvec_static(q.data_ptr(), x.data_ptr(), y.data_ptr(), rows, n_sb,
                                              int(torch.cuda.current_stream().cuda_stream))
    return rc


def test_static_entry_point_matches_allocating_entry_point_twice_in_a_row(ffi, ops, synth):
    cases = [(300, 16, 11), (37, 56, 12)]   # second call: other shape, other x, same scratch
    for rows, n_sb, seed in cases:
        q_np = synth.q4k_weights(rows, n_sb, 7000 + seed)
        x_np = synth.activations(n_sb * 256, 7100 + seed) * np.float32(3.0 ** seed)
        q = torch.from_numpy(q_np).cuda()
        x = torch.from_numpy(x_np).cuda()
        y_ref = ops.q4k_matvec(q, x, rows, n_sb)                      # existing entry point
        y = torch.full((rows,), float("nan"), dtype=torch.float32, device="cuda")
        assert _call_static(ffi, q, x, y, rows, n_sb) == ffi.AXC_OK
        torch.cuda.synchronize()
        _y64, mag = oracle.matvec_rows_f64("q4k", q_np, x_np, rows, n_sb)
        err = np.abs(y.cpu().numpy().astype(np.float64) - y_ref.cpu().numpy()) / mag
        assert err.max() <= NORMWISE_TOL
        assert torch.equal(y, y_ref)
        # and both agree with the CPU oracle
        y_cpu = oracle.matvec_rows("q4k", q_np, x_np, rows, n_sb)
        assert (np.abs(y.cpu().numpy() - y_cpu) / mag).max() <= NORMWISE_TOL


def test_static_entry_point_rejects_rows_longer_than_its_scratch(ffi):
    q = torch.zeros(144 * 129, dtype=torch.uint8, device="cuda")
    x = torch.zeros(256 * 129, dtype=torch.float32, device="cuda")
    y = torch.zeros(1, dtype=torch.float32, device="cuda")
    assert _call_static(ffi, q, x, y, 1, 129) == ffi.AXC_ERR_BUFFER_ALLOCATION_FAILED
    assert _call_static(ffi, q, x, y, 1, 0) == ffi.AXC_ERR_BUFFER_ALLOCATION_FAILED
    assert ffi.lib().axc_cuda_q4k_matvec_static(None, None, None, 1, 1, None) == ffi.AXC_ERR_INVALID_ARGUMENT
    assert _call_static(ffi, q, x, y, 0, 129) == ffi.AXC_OK      # nothing to do
    assert _call_static(ffi, q, x, y, 1, 128) == ffi.AXC_OK      # the stated maximum works
    torch.cuda.synchronize()
    assert float(y.item()) == 0.0


def test_static_entry_point_leaves_free_memory_unchanged_after_warmup(ffi, synth):
    """After the start-up warm-up (array looked up, every kernel of the path loaded) calls of
    different shapes, which take different tile heights of the matvec kernel, change nothing in
    the device's free memory: neither the entry point nor the runtime allocates on its behalf."""
    assert ffi.lib().axc_cuda_q4k_matvec_static_warmup() == ffi.AXC_OK
    shapes = [(4096, 16), (16, 128), (3, 1), (1000, 56)]
    bufs = []
    for rows, n_sb in shapes:       # the caller's own buffers exist before the measurement
        q = torch.from_numpy(synth.q4k_weights(rows, n_sb, 7300 + rows)).cuda()
        x = torch.from_numpy(synth.activations(n_sb * 256, 7400 + rows)).cuda()
        y = torch.zeros(rows, dtype=torch.float32, device="cuda")
        bufs.append((q, x, y, rows, n_sb))
    torch.cuda.synchronize()
    free_before, _total = torch.cuda.mem_get_info()
    for q, x, y, rows, n_sb in bufs:
        assert _call_static(ffi, q, x, y, rows, n_sb) == ffi.AXC_OK
    torch.cuda.synchronize()
    free_after, _total = torch.cuda.mem_get_info()
    assert free_after == free_before
