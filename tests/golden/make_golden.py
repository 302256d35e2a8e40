"""Regenerates the golden fixtures in this directory.

Two kinds of vectors:

* ``reference_known_answers.json`` -- the hand-verified known-answer cases of the reference's own
  tests, typed in from their source text (the reference is Rust and cannot be run here):
  AT-1312 (crates/axc-driver/tests/compile_q4km_dequant_matvec.rs:484-584), the two Q4_0 layout
  fixtures (crates/axc-driver/tests/common_helpers.rs:272-333) and n = 0 -> +0.0
  (compile_q4km_dequant_matvec.rs:850-856).  Expected values are the reference's, not ours.
* ``lcg_fixture_outputs.json`` -- outputs of the CPU oracle on the reference's reproducible LCG
  fixture (common_helpers.rs:476-519) for the seeds its tests and benches use.  The reference
  stores no numbers for these, so they are produced here and only committed after the C
  restatement, the .axc-body restatement and the numpy twin agree bit for bit (asserted below).
  They pin the oracle against drift and give the GPU tests fixed targets.

Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from oracle import oracle_np  # noqa: E402


def z12(**kv):
    s = [0] * 12
    for k, v in kv.items():
        s[int(k[1:])] = v
    return s


def known_answers():
    at_1312 = [{"scales": [0] * 12, "j": j, "sc": 0, "m": 0, "note": "all-zero scales"} for j in range(8)]
    at_1312 += [
        {"scales": z12(s0=0xFF, s4=0xC0), "j": 0, "sc": 63, "m": 0, "note": "j=0 high bits discarded"},
        {"scales": z12(s3=0x3F, s7=0x3F), "j": 3, "sc": 63, "m": 63, "note": "j=3"},
        {"scales": z12(s8=0xAB, s0=0xC0, s4=0xD0), "j": 4, "sc": 59, "m": 58, "note": "j=4 high branch"},
        {"scales": z12(s9=0xCD, s1=0x80, s5=0x40), "j": 5, "sc": 0x0D | (2 << 4), "m": 0x0C | (1 << 4), "note": "j=5"},
        {"scales": z12(s10=0x12, s2=0x55, s6=0xAA), "j": 6, "sc": 0x02 | (1 << 4), "m": 0x01 | (2 << 4), "note": "j=6"},
        {"scales": z12(s11=0xFF, s3=0xFF, s7=0xFF), "j": 7, "sc": 63, "m": 63, "note": "j=7"},
        {"scales": z12(s8=0x10, s4=0x80, s0=0x40), "j": 4, "sc": None, "m": 33,
         "note": "m-high uses scales[j] (33), not scales[j-4] (17)"},
    ]
    q4_0 = [
        {"name": "gguf_layout_index_k_and_k_plus_16", "q": [0x00, 0x3C] + [0x80] * 16,
         "x": [1.0] * 32, "n_blocks": 1, "expected": -128.0, "abs_tol": 1e-6},
        {"name": "layout_discriminating_fixture", "q": [0x00, 0x3C] + [0x12] * 16,
         "x": [1.0] * 16 + [0.0] * 16, "n_blocks": 1, "expected": -96.0, "abs_tol": 1e-6,
         "wrong_layout_would_give": -104.0},
    ]
    return {"source": "reference test text (see make_golden.py docstring)",
            "at_1312_unpack_scale_min_k4": at_1312, "q4_0_layout": q4_0,
            "q4km_n0": {"n_superblocks": 0, "expected_bits": 0}}


def lcg_outputs():
    out = []
    for seed, n in ((0xDEADBEEF, 16), (0xDEADBEEF, 128), (0xCAFEBABE, 128), (0xCAFEBABE, 512)):
        q, x = oracle.generate_q4km_test_data(n, seed)
        if n <= 128:
            qn, xn = oracle_np.generate_q4km_test_data(n, seed)
            assert (q == qn).all() and (x.view(np.uint32) == xn.view(np.uint32)).all()
        y = oracle.q4km_dequant_matvec_cpu(q, x, n)
        y2 = oracle.q4km_axc_body(q, x, n)
        y3 = oracle_np.q4km_dequant_matvec(q, x, n)
        assert y.view(np.uint32) == y2.view(np.uint32) == y3.view(np.uint32), (seed, n)
        w = oracle.dequant_rows("q4k", q, 1, n)
        out.append({"seed": seed, "n_superblocks": n,
                    "q_sha256": hashlib.sha256(q.tobytes()).hexdigest(),
                    "x_sha256": hashlib.sha256(x.tobytes()).hexdigest(),
                    "w_sha256": hashlib.sha256(w.tobytes()).hexdigest(),
                    "q_first16": [int(v) for v in q[:16]],
                    "x_first4_bits": [int(v) for v in x[:4].view(np.uint32)],
                    "y_bits": int(y.view(np.uint32)), "y": float(y)})
    return {"source": "CPU oracle on the reference's LCG fixture; C == .axc body == numpy",
            "fixtures": out}


if __name__ == "__main__":
    with open(os.path.join(HERE, "reference_known_answers.json"), "w") as f:
        json.dump(known_answers(), f, indent=1)
    with open(os.path.join(HERE, "lcg_fixture_outputs.json"), "w") as f:
        json.dump(lcg_outputs(), f, indent=1)
    print("wrote golden fixtures")
