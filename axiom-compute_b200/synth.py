"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

These stand in for model weights (none are available): Q4_K_M superblocks with fp16
d, dmin = |N(0,1)| * 0.01, eight 6-bit scales and mins uniform in 0..63 packed in the ggml
Q4_K layout, nibbles uniform in 0..15; Q4_0 blocks with fp16 d = |N(0,1)| * 0.02.  Because the
12-byte scales field uses each of its 96 bits for exactly one of the sixteen 6-bit values,
uniform random bytes there ARE uniform independent 6-bit values, so the bulk generators draw
bytes directly; ``pack_q4k_scales`` spells the packing out for small cases and tests.
"""
from __future__ import annotations

import numpy as np

Q4K_SB_BYTES, Q4K_SB_ELEMS = 144, 256
Q4_0_BLK_BYTES, Q4_0_BLK_ELEMS = 18, 32


def pack_q4k_scales(sc: np.ndarray, m: np.ndarray) -> np.ndarray:
    """(…, 8) scales and mins in 0..63 -> (…, 12) packed bytes; inverse of get_scale_min_k4
    (crates/axc-driver/tests/common_helpers.rs:365-381)."""
    sc = np.asarray(sc, dtype=np.uint8)
    m = np.asarray(m, dtype=np.uint8)
    out = np.zeros(sc.shape[:-1] + (12,), np.uint8)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (m[..., 0:4] & 63) | ((m[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((m[..., 4:8] & 0x0F) << 4)
    return out


def q4k_weights(rows: int, n_sb: int, seed: int, explicit_pack: bool = False) -> np.ndarray:
    """rows * n_sb superblocks as a flat uint8 array (row-major, 144 B each)."""
    rng = np.random.default_rng(seed)
    total = rows * n_sb
    q = rng.integers(0, 256, size=(total, Q4K_SB_BYTES), dtype=np.uint8)
    dd = (np.abs(rng.standard_normal((total, 2), dtype=np.float32)) * np.float32(0.01))
    q[:, 0:4] = dd.astype(np.float16).view(np.uint8).reshape(total, 4)
    if explicit_pack:
        sc = rng.integers(0, 64, size=(total, 8), dtype=np.uint8)
        m = rng.integers(0, 64, size=(total, 8), dtype=np.uint8)
        q[:, 4:16] = pack_q4k_scales(sc, m)
    return q.reshape(-1)


def q4_0_weights(rows: int, n_blocks: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    total = rows * n_blocks
    q = rng.integers(0, 256, size=(total, Q4_0_BLK_BYTES), dtype=np.uint8)
    d = (np.abs(rng.standard_normal((total, 1), dtype=np.float32)) * np.float32(0.02))
    q[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(total, 2)
    return q.reshape(-1)


def activations(k: int, seed: int) -> np.ndarray:
    """fp32 ~ N(0, 1)."""
    return np.random.default_rng(seed).standard_normal(k, dtype=np.float32)


def config_seed(config: int, tensor_id: int) -> int:
    """One stream per tensor: 0xA0C0 + 16 * config + tensor id."""
    return 0xA0C0 + 16 * config + tensor_id
