"""numpy twin of the C oracle -- TEST INFRASTRUCTURE ONLY (cross-check, small sizes).

Written independently of ``axc_oracle.c`` from the same reference sources
(crates/axc-driver/tests/common_helpers.rs:365-381,411-461,476-519;
crates/axc-driver/benches/common.rs:212-259).  Binary16 widening uses numpy's float16
(exact); sequential fp32 sums use ``np.add.accumulate`` on float32, which adds left to right
with one rounding per add, like the reference's ``sum += ...``.
"""
from __future__ import annotations

import numpy as np

MASK64 = (1 << 64) - 1


def f16_le_to_f32(two_bytes: np.ndarray) -> np.ndarray:
    """Little-endian binary16 byte pairs (..., 2) -> float32, exactly."""
    b = np.ascontiguousarray(two_bytes, dtype=np.uint8)
    return b.view("<f2").astype(np.float32)[..., 0]


def unpack_scale_min_k4(scales, j: int) -> tuple[int, int]:
    s = [int(v) for v in scales]
    if j < 4:
        return s[j] & 63, s[j + 4] & 63
    sc = (s[j + 4] & 0x0F) | (((s[j - 4] >> 6) & 3) << 4)
    m = ((s[j + 4] >> 4) & 0x0F) | (((s[j] >> 6) & 3) << 4)
    return sc, m


def q4km_dequant_row(q: np.ndarray, n_sb: int) -> np.ndarray:
    """Bit-exact fp32 weights of one row, x-index order (d*sc and dmin*m rounded first)."""
    q = np.ascontiguousarray(q, dtype=np.uint8)[: n_sb * 144].reshape(n_sb, 144)
    d = f16_le_to_f32(q[:, 0:2].reshape(n_sb, 1, 2))[:, 0]
    dmin = f16_le_to_f32(q[:, 2:4].reshape(n_sb, 1, 2))[:, 0]
    w = np.zeros((n_sb, 256), np.float32)
    for sb in range(n_sb):
        scales = q[sb, 4:16]
        for chunk in range(4):
            sc0, m0 = unpack_scale_min_k4(scales, 2 * chunk)
            sc1, m1 = unpack_scale_min_k4(scales, 2 * chunk + 1)
            d1 = np.float32(d[sb]) * np.float32(sc0)
            m1f = np.float32(dmin[sb]) * np.float32(m0)
            d2 = np.float32(d[sb]) * np.float32(sc1)
            m2f = np.float32(dmin[sb]) * np.float32(m1)
            qs = q[sb, 16 + chunk * 32: 16 + chunk * 32 + 32]
            lo = (qs & 0x0F).astype(np.float32)
            hi = (qs >> 4).astype(np.float32)
            with np.errstate(all="ignore"):
                w[sb, chunk * 64: chunk * 64 + 32] = d1 * lo - m1f
                w[sb, chunk * 64 + 32: chunk * 64 + 64] = d2 * hi - m2f
    return w.reshape(-1)


def q4km_dequant_matvec(q: np.ndarray, x: np.ndarray, n_sb: int) -> np.float32:
    """Reference order: within a chunk, lo_l then hi_l for l = 0..31."""
    if n_sb == 0:
        return np.float32(0.0)
    w = q4km_dequant_row(q, n_sb).reshape(n_sb, 4, 2, 32)
    xs = np.ascontiguousarray(x, dtype=np.float32)[: n_sb * 256].reshape(n_sb, 4, 2, 32)
    with np.errstate(all="ignore"):
        terms = (w * xs).transpose(0, 1, 3, 2).reshape(-1)  # (sb, chunk, l, {lo, hi})
        seq = np.concatenate([np.zeros(1, np.float32), terms])
        return np.float32(np.add.accumulate(seq, dtype=np.float32)[-1])


def q4_0_dequant_row(q: np.ndarray, n_blocks: int) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)[: n_blocks * 18].reshape(n_blocks, 18)
    scale = f16_le_to_f32(q[:, 0:2].reshape(n_blocks, 1, 2))  # (n_blocks, 1)
    lo = (q[:, 2:] & 0x0F).astype(np.float32)
    hi = (q[:, 2:] >> 4).astype(np.float32)
    w = np.zeros((n_blocks, 32), np.float32)
    with np.errstate(all="ignore"):
        w[:, :16] = (lo - np.float32(8.0)) * scale
        w[:, 16:] = (hi - np.float32(8.0)) * scale
    return w.reshape(-1)


def q4_0_dequant_matvec(q: np.ndarray, x: np.ndarray, n_blocks: int) -> np.float32:
    if n_blocks == 0:
        return np.float32(0.0)
    w = q4_0_dequant_row(q, n_blocks).reshape(n_blocks, 2, 16)
    xs = np.ascontiguousarray(x, dtype=np.float32)[: n_blocks * 32].reshape(n_blocks, 2, 16)
    with np.errstate(all="ignore"):
        terms = (w * xs).transpose(0, 2, 1).reshape(-1)  # (block, k, {lo, hi})
        seq = np.concatenate([np.zeros(1, np.float32), terms])
        return np.float32(np.add.accumulate(seq, dtype=np.float32)[-1])


def generate_q4km_test_data(n_sb: int, seed: int):
    """The reference's LCG fixture (common_helpers.rs:476-519) in Python integers."""
    state = (seed ^ 0x9E3779B97F4A7C15) & MASK64
    two64 = np.float32(np.uint64(MASK64))  # u64::MAX as f32 == 2^64

    def nxt() -> int:
        nonlocal state
        state = (state * 6364136223846793005 + 1442695040888963407) & MASK64
        return state

    def unit() -> np.float32:
        return np.float32(np.uint64(nxt())) / two64

    q = np.zeros(n_sb * 144, np.uint8)
    p = 0
    for _ in range(n_sb):
        d_raw = np.float32(0.1) + unit() * np.float32(1.9)
        q[p:p + 2] = np.frombuffer(np.float16(d_raw).tobytes(), np.uint8)
        dmin_raw = unit() * np.float32(0.5)
        q[p + 2:p + 4] = np.frombuffer(np.float16(dmin_raw).tobytes(), np.uint8)
        p += 4
        for _k in range(140):
            q[p] = nxt() & 0xFF
            p += 1
    x = np.zeros(n_sb * 256, np.float32)
    for i in range(n_sb * 256):
        x[i] = unit() * np.float32(2.0) - np.float32(1.0)
    return q, x
