"""The fused-source matvec (x = a + b, unit RMS, (value, epoch) sources) and the decode sweep
built from it, against the CPU oracle's sweep on small shapes."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from conftest import load_pkg

pytestmark = pytest.mark.gpu
NORMWISE_TOL = 1e-5


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def fused(ffi, q, rows, n_sb, x=None, x2=None, xp=None, x2p=None, epoch=None, rms=False, gather=None, y=None, st=None,
          parity_stride=0):
    xs = ffi.AxcXSrc(x.data_ptr() if x is not None else None, x2.data_ptr() if x2 is not None else None,
                     xp.data_ptr() if xp is not None else None, x2p.data_ptr() if x2p is not None else None,
                     epoch.data_ptr() if epoch is not None else None, 1 if rms else 0, parity_stride)
    rc = ffi.lib().axc_cuda_q4k_matvec_fused(q.data_ptr(), C.byref(xs), y.data_ptr() if y is not None else None,
                                             rows, n_sb, C.byref(gather) if gather is not None else None,
                                             int(torch.cuda.current_stream().cuda_stream),
                                             st.data_ptr() if st is not None else None, None)
    return rc


@pytest.mark.parametrize("rows,n_sb", [(33, 1), (257, 16), (64, 112), (1000, 32)])
@pytest.mark.parametrize("second,rms", [(False, False), (True, False), (False, True), (True, True)])
def test_fused_source_matches_oracle(ffi, ops, synth, rows, n_sb, second, rms):
    q = synth.q4k_weights(rows, n_sb, 7000 + rows + n_sb)
    a = synth.activations(n_sb * 256, 7100 + rows)
    b = synth.activations(n_sb * 256, 7200 + rows)
    x = (a + b).astype(np.float32) if second else a
    x_eff = oracle.unit_rms(x) if rms else x
    y_ref = oracle.matvec_rows("q4k", q, x_eff, rows, n_sb)
    _y64, mag = oracle.matvec_rows_f64("q4k", q, x_eff, rows, n_sb)
    y = torch.empty(rows, device="cuda")
    st = ops.new_status()
    assert fused(ffi, dev(q), rows, n_sb, x=dev(a), x2=dev(b) if second else None, rms=rms, y=y, st=st) == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert (np.abs(y.cpu().numpy() - y_ref) / mag).max() <= NORMWISE_TOL


def test_fused_source_reads_epoch_words_and_chains(ffi, ops, synth):
    """Producer with the all-gather epilogue (world 1), consumer polling its words: g + u with
    unit RMS straight from the (value, epoch) vector, no finish launch in between."""
    coll = load_pkg("collective")
    ffn, hid = 512, 256
    gu_w = synth.q4k_weights(2 * ffn, hid // 256, 7301)
    dn_w = synth.q4k_weights(hid, ffn // 256, 7302)
    x = synth.activations(hid, 7303)
    pg = coll.PeerGather(2 * ffn, 1, "cuda")
    st = ops.new_status()
    y = torch.empty(hid, device="cuda")
    for it in range(3):
        pg.matvec(dev(gu_w), dev(x), hid // 256, 0, status=st)
        pairs = pg.pairs
        second = pairs[ffn:]
        assert fused(ffi, dev(dn_w), hid, ffn // 256, xp=pairs, x2p=second, epoch=pg.epoch, rms=True, y=y, st=st,
                     parity_stride=pg.parity_stride) == 0
        pg.finish(st)     # ends the step: the next one writes the other copy
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        gu = oracle.matvec_rows("q4k", gu_w, x, 2 * ffn, hid // 256)
        xin = oracle.unit_rms(gu[:ffn] + gu[ffn:])
        y_ref = oracle.matvec_rows("q4k", dn_w, xin, hid, ffn // 256)
        _y64, mag = oracle.matvec_rows_f64("q4k", dn_w, xin, hid, ffn // 256)
        assert (np.abs(y.cpu().numpy() - y_ref) / mag).max() <= 2e-5   # two chained fast kernels


def test_fused_source_times_out_on_missing_epoch(ffi, ops, synth):
    """Words that never arrive: bounded wait, status bit 4, context stays usable."""
    q = dev(synth.q4k_weights(8, 1, 7401))
    pairs = torch.zeros(256, dtype=torch.int64, device="cuda")
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")
    st = ops.new_status()
    y = torch.empty(8, device="cuda")
    assert fused(ffi, q, 8, 1, xp=pairs, epoch=epoch, y=y, st=st) == 0
    torch.cuda.synchronize()
    assert int(st.item()) & 4
    assert torch.ones(3, device="cuda").sum().item() == 3.0


def test_fused_source_argument_checks(ffi, ops, synth):
    q = dev(synth.q4k_weights(8, 1, 7501))
    x = dev(synth.activations(256, 7502))
    y = torch.empty(8, device="cuda")
    pairs = torch.zeros(256, dtype=torch.int64, device="cuda")
    assert fused(ffi, q, 8, 1, y=y) == 100                         # no source
    assert fused(ffi, q, 8, 1, x=x, xp=pairs, y=y) == 100          # two first sources
    assert fused(ffi, q, 8, 1, xp=pairs, y=y) == 100               # epoch words without the counter
    assert fused(ffi, q, 8, 1, x=x) == 100                         # nowhere to put y
    assert fused(ffi, q, 8, 129, x=x, y=y) == 100                  # row too long for this kernel


def test_gather_finish_overlapping_its_producer(ffi, ops, synth):
    """finish launched with the overlap flag right behind its producer: it starts early, polls
    for the producer's words and delivers exactly the plain kernel's values."""
    coll = load_pkg("collective")
    rows, n_sb = 3000, 16
    q, x = dev(synth.q4k_weights(rows, n_sb, 7601)), dev(synth.activations(n_sb * 256, 7602))
    pg = coll.PeerGather(rows, 1, "cuda")
    st = ops.new_status()
    out = torch.zeros(rows, device="cuda")
    s = int(torch.cuda.current_stream().cuda_stream)
    for it in range(3):
        pg.matvec(q, x, n_sb, 0, status=st)
        rc = ffi.lib().axc_cuda_gather_finish(pg.pairs.data_ptr(), pg.epoch.data_ptr(), out.data_ptr(), rows,
                                              s, st.data_ptr(), ffi.AXC_FINISH_OVERLAP_PREVIOUS, pg.parity_stride, None)
        assert rc == 0
        y = ops.q4k_matvec(q, x, rows, n_sb)
        assert torch.equal(out, y)
        out.zero_()
        assert ffi.lib().axc_cuda_gather_next_epoch(pg.epoch.data_ptr(), s) == 0
    # the end-of-step handshake advances the epoch, so it may not run ahead of the launch before it
    assert ffi.lib().axc_cuda_gather_finish(pg.pairs.data_ptr(), pg.epoch.data_ptr(), out.data_ptr(), rows, s,
                                            st.data_ptr(), ffi.AXC_FINISH_OVERLAP_PREVIOUS, pg.parity_stride,
                                            C.byref(pg._sync)) == 100
    assert int(st.item()) == 0


@pytest.mark.parametrize("rows,n_sb", [(33, 1), (257, 16), (64, 112), (300, 128)])
@pytest.mark.parametrize("second,rms", [(False, False), (True, True)])
def test_prepared_x_matches_oracle(ffi, ops, synth, rows, n_sb, second, rms):
    """prepare_x + matvec_prepared: same results as the oracle on x = a [+ b] (unit RMS optional);
    the plain copy of x that prepare_x can emit is exact."""
    q = synth.q4k_weights(rows, n_sb, 7700 + rows + n_sb)
    a = synth.activations(n_sb * 256, 7710 + rows)
    b = synth.activations(n_sb * 256, 7720 + rows)
    x = (a + b).astype(np.float32) if second else a
    x_eff = oracle.unit_rms(x) if rms else x
    y_ref = oracle.matvec_rows("q4k", q, x_eff, rows, n_sb)
    _y64, mag = oracle.matvec_rows_f64("q4k", q, x_eff, rows, n_sb)
    L = ffi.lib()
    img = torch.zeros(int(L.axc_cuda_q4k_prepared_x_bytes(n_sb)), dtype=torch.uint8, device="cuda")
    plain = torch.zeros(n_sb * 256, device="cuda")
    y = torch.empty(rows, device="cuda")
    st = ops.new_status()
    ad, bd, qd = dev(a), dev(b), dev(q)
    xs = ffi.AxcXSrc(ad.data_ptr(), bd.data_ptr() if second else None, None, None, None, 0, 0)
    s = int(torch.cuda.current_stream().cuda_stream)
    for _ in range(2):
        assert L.axc_cuda_q4k_prepare_x(C.byref(xs), img.data_ptr(), plain.data_ptr(), n_sb, s, st.data_ptr(), 0) == 0
        assert L.axc_cuda_q4k_matvec_prepared(qd.data_ptr(), img.data_ptr(), 1 if rms else 0, y.data_ptr(), rows, n_sb,
                                              None, s, st.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert np.array_equal(plain.cpu().numpy(), x)
    assert (np.abs(y.cpu().numpy() - y_ref) / mag).max() <= NORMWISE_TOL


def test_prepare_x_argument_checks(ffi, synth):
    L = ffi.lib()
    x = dev(synth.activations(256, 7801))
    pairs = torch.zeros(256, dtype=torch.int64, device="cuda")
    img = torch.zeros(int(L.axc_cuda_q4k_prepared_x_bytes(1)), dtype=torch.uint8, device="cuda")
    s = int(torch.cuda.current_stream().cuda_stream)
    plain_src = ffi.AxcXSrc(x.data_ptr(), None, None, None, None, 0, 0)
    assert L.axc_cuda_q4k_prepare_x(C.byref(plain_src), None, None, 1, s, None, 0) == 100
    assert L.axc_cuda_q4k_prepare_x(C.byref(plain_src), img.data_ptr(), None, 129, s, None, 0) == 100
    assert L.axc_cuda_q4k_prepare_x(C.byref(plain_src), img.data_ptr(), None, 1, s, None, 1) == 100   # plain source may not overlap
    no_epoch = ffi.AxcXSrc(None, None, pairs.data_ptr(), None, None, 0, 0)
    assert L.axc_cuda_q4k_prepare_x(C.byref(no_epoch), img.data_ptr(), None, 1, s, None, 0) == 100
    assert L.axc_cuda_q4k_prepared_x_bytes(16) == 17 * 64 * 16 + 128


@pytest.mark.parametrize("mode", ["prepared", "fused", "mixed"])
def test_decode_sweep_matches_oracle_on_a_small_stack(mode):
    decode = load_pkg("decode")
    shape = decode.SweepShape(hidden=512, kv=128, ffn=1024, layers=3)
    assert decode.DecodeSweep(decode.SweepShape(256, 64, 256, 1), "cuda").mode == "mixed"   # auto, one GPU
    sweep = decode.DecodeSweep(shape, "cuda", seed=4242, mode=mode)
    assert sweep.world == 1 and sweep.launches_per_token == {"prepared": 25, "fused": 13, "mixed": 13}[mode]
    rng = np.random.default_rng(5)
    h0 = rng.standard_normal(shape.hidden).astype(np.float32)
    weights = [tuple(w.cpu().numpy() for w in layer) for layer in sweep.weights]
    sweep.h.copy_(dev(h0))
    sweep.token(normalise_input=False)
    torch.cuda.synchronize()
    assert int(sweep.status.item()) == 0
    outs, d, h1, ksum = oracle.decode_token(weights, shape.hidden, shape.kv, shape.ffn, h0, normalise_input=False)
    # first layer's first linear sees identical inputs: the per-kernel bar applies
    _y64, mag = oracle.matvec_rows_f64("q4k", weights[0][0], h0, shape.hidden + 2 * shape.kv, shape.hidden // 256)
    assert (np.abs(sweep.output(0, 0).cpu().numpy() - outs[0][0]) / mag).max() <= NORMWISE_TOL
    # deeper vectors carry the rounding differences of every kernel before them
    for layer in range(shape.layers):
        for j in range(4):
            got, ref = sweep.output(layer, j).cpu().numpy(), outs[layer][j]
            assert np.abs(got - ref).max() <= 1e-3 * np.sqrt(np.mean(ref.astype(np.float64) ** 2)), (layer, j)
    assert np.abs(sweep.hidden_out().cpu().numpy() - h1).max() <= 1e-3
    assert abs(float(sweep.kv_checksum().item()) - ksum) <= 1e-3 * max(1.0, abs(ksum))
    # second token: h = unitRMS(d) through the first launch's normalisation
    sweep.advance()
    sweep.token()
    torch.cuda.synchronize()
    outs2, d2, h2, _ = oracle.decode_token(weights, shape.hidden, shape.kv, shape.ffn, d, normalise_input=True)
    assert np.abs(sweep.hidden_out().cpu().numpy() - h2).max() <= 2e-3
    assert int(sweep.status.item()) == 0
