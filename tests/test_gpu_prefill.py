"""Batched prefill on the tensor cores (tcgen05) against the CPU oracle's dequant-then-GEMM.

The reference has no M > 1 kernel; the bar is the one its north star states for this case:
1e-2 relative against the CPU dequantisation followed by a GEMM with bf16 operands and fp32
accumulation.  Both sides use the same bf16 operands, so the observed error is far smaller and
a norm-wise bound is asserted as well."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def bf16_operands(m, k, seed):
    rng = np.random.default_rng(seed)
    a32 = rng.standard_normal((m, k)).astype(np.float32)
    a_bf = torch.from_numpy(a32).to(torch.bfloat16)
    return a_bf, a_bf.to(torch.float32).numpy()


def check(ops, synth, m, n, n_sb, seed, form=0):
    q = synth.q4k_weights(n, n_sb, seed)
    a_bf, a32 = bf16_operands(m, n_sb * 256, seed + 1)
    st = ops.new_status()
    c = ops.q4k_prefill(torch.from_numpy(q).cuda(), a_bf.cuda(), m, n, n_sb, status=st, form=form)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ref = oracle.q4km_prefill(q, a32, m, n, n_sb)
    got = c.cpu().numpy()
    w = np.abs(oracle.dequant_rows("q4k", q, n, n_sb)).astype(np.float64)
    mag = np.abs(a32).astype(np.float64) @ w.T                      # sum_k |a w| per output
    assert (np.abs(got - ref) / np.maximum(mag, 1e-30)).max() <= 1e-5
    rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    assert (np.abs(got - ref) <= 1e-2 * np.maximum(np.abs(ref), rms)).all()
    return got


@pytest.mark.parametrize("m,n,n_sb", [(64, 128, 1), (256, 128, 2), (512, 256, 4), (300, 200, 2),
                                      (1, 128, 1), (17, 130, 3), (600, 384, 2), (1030, 128, 1), (130, 384, 1)])
@pytest.mark.parametrize("form", [1, 2])
def test_prefill_matches_oracle(ops, synth, m, n, n_sb, form):
    """form 1: one CTA per tile; form 2: CTA pairs (a 128-row matrix has one tile and runs as form 1)."""
    check(ops, synth, m, n, n_sb, 9000 + m + n + n_sb, form)


def test_prefill_forms_agree_bit_for_bit(ops, synth):
    """Both forms accumulate the same products in the same k order."""
    m, n, n_sb = 300, 640, 3
    q = torch.from_numpy(synth.q4k_weights(n, n_sb, 9050)).cuda()
    a_bf, _ = bf16_operands(m, n_sb * 256, 9051)
    a = a_bf.cuda()
    assert torch.equal(ops.q4k_prefill(q, a, m, n, n_sb, form=1), ops.q4k_prefill(q, a, m, n, n_sb, form=2))


def test_prefill_weights_are_the_bit_exact_bf16_dequant(ops, synth):
    """A = identity columns picks out bf16(W): every weight must be the reference's fp32 value
    rounded to nearest even, bit for bit."""
    n, n_sb = 128, 1
    q = synth.q4k_weights(n, n_sb, 9100)
    eye = torch.eye(256, dtype=torch.bfloat16)
    c = ops.q4k_prefill(torch.from_numpy(q).cuda(), eye.cuda(), 256, n, n_sb)
    w_ref = torch.from_numpy(oracle.dequant_rows("q4k", q, n, n_sb)).to(torch.bfloat16).to(torch.float32).numpy()
    got = c.cpu().numpy().T                                           # [n][k]
    assert (got.view(np.uint32) == w_ref.view(np.uint32)).all()


def test_prefill_rejects_bad_arguments(ffi, ops, synth):
    q = torch.from_numpy(synth.q4k_weights(128, 1, 9200)).cuda()
    a = torch.zeros((4, 256), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((4, 128), device="cuda")
    s = int(torch.cuda.current_stream().cuda_stream)
    L = ffi.lib()
    assert L.axc_cuda_q4k_prefill(q.data_ptr(), a.data_ptr(), c.data_ptr(), 4, 128, 0, s, None) == 100
    assert L.axc_cuda_q4k_prefill(None, a.data_ptr(), c.data_ptr(), 4, 128, 1, s, None) == 100
    assert L.axc_cuda_q4k_prefill(q.data_ptr(), a.data_ptr() + 2, c.data_ptr(), 4, 128, 1, s, None) == 100
    assert L.axc_cuda_q4k_prefill(q.data_ptr(), a.data_ptr(), c.data_ptr(), 0, 128, 1, s, None) == 0


def test_prefill_full_shape_linearity(ops, synth):
    """512 x 4096 x 14336: rows of C against oracle samples plus linearity in A (C(a1 + a2) rows
    equal C(a1) + C(a2) up to rounding) at the full size."""
    m, n, n_sb = 512, 14336, 16
    q = synth.q4k_weights(n, n_sb, 9300)
    a_bf, a32 = bf16_operands(m, n_sb * 256, 9301)
    qd = torch.from_numpy(q).cuda()
    c = ops.q4k_prefill(qd, a_bf.cuda(), m, n, n_sb)
    rows = np.array([0, 1, 127, 128, 5000, 14335])
    ref = oracle.q4km_prefill(np.ascontiguousarray(q.reshape(n, -1)[rows]).reshape(-1), a32, m, len(rows), n_sb)
    got = c[:, torch.from_numpy(rows).cuda()].cpu().numpy()
    rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    assert (np.abs(got - ref) <= 1e-2 * np.maximum(np.abs(ref), rms)).all()
    assert np.abs(got - ref).max() <= 1e-4 * rms


def test_prefill_independent_calls_back_to_back(ops, synth):
    """Calls declared independent of the launch before them may overlap it on idle SMs; every C
    is still exactly what the strictly ordered call produces."""
    m, n, n_sb = 200, 384, 2
    a_bf, _ = bf16_operands(m, n_sb * 256, 9400)
    a = a_bf.cuda()
    qs = [torch.from_numpy(synth.q4k_weights(n, n_sb, 9401 + j)).cuda() for j in range(4)]
    ref = [ops.q4k_prefill(q, a, m, n, n_sb) for q in qs]
    torch.cuda.synchronize()
    st = ops.new_status()
    outs = [torch.zeros((m, n), device="cuda") for _ in qs]
    for _ in range(3):
        for q, c in zip(qs, outs):
            ops.q4k_prefill(q, a, m, n, n_sb, c=c, status=st, independent=True)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    for r, c in zip(ref, outs):
        assert torch.equal(r, c)
