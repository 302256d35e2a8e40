"""CPU oracle for the Q4_K_M / Q4_0 dequant-matvec path -- TEST INFRASTRUCTURE ONLY.

ctypes front end of ``libaxc_oracle.so`` (built from ``axc_oracle.c`` by ``make -C oracle``),
the C restatement of the reference's CPU functions
(crates/axc-driver/tests/common_helpers.rs:365-381,411-461,476-519 and
crates/axc-driver/benches/common.rs:212-259).  Only tests, the smoke check and the benchmark's
CPU-baseline / reference legs may import this package; the product package never does.

Parity pinning: checked against the reference's known-answer tests (AT-1312 scale/min pairs,
Q4_0 layout fixtures, n = 0) in ``tests/golden/reference_known_answers.json``; the reference
holds no stored outputs for its random fixtures, so beyond those cases the C restatement, the
``.axc``-body restatement and the numpy twin (``oracle_np.py``) pin each other bit for bit.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import threading

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libaxc_oracle.so")
_lock = threading.Lock()
_lib = None

Q4KM_SB_BYTES = 144
Q4KM_SB_ELEMS = 256
Q4_0_BLK_BYTES = 18
Q4_0_BLK_ELEMS = 32


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (no-op when the .so is newer than its source)."""
    src = os.path.join(_HERE, "axc_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libaxc_oracle.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    with _lock:
        if _lib is None:
            build()
            L = C.CDLL(_LIB_PATH)
            u8p, f32p, f64p = C.c_void_p, C.c_void_p, C.c_void_p
            sz = C.c_size_t
            L.axc_oracle_f16_bits_to_f32.restype = C.c_float
            L.axc_oracle_f16_bits_to_f32.argtypes = [C.c_uint16]
            L.axc_oracle_f32_to_f16_bits.restype = C.c_uint16
            L.axc_oracle_f32_to_f16_bits.argtypes = [C.c_float]
            L.axc_oracle_bf16_round.restype = C.c_float
            L.axc_oracle_bf16_round.argtypes = [C.c_float]
            L.axc_oracle_unpack_scale_min_k4.restype = None
            L.axc_oracle_unpack_scale_min_k4.argtypes = [u8p, C.c_int, u8p, u8p]
            L.axc_oracle_pack_scale_min_k4.restype = None
            L.axc_oracle_pack_scale_min_k4.argtypes = [u8p, u8p, u8p]
            for name in ("axc_oracle_q4km_dequant_matvec", "axc_oracle_q4_0_dequant_matvec"):
                f = getattr(L, name)
                f.restype = C.c_float
                f.argtypes = [u8p, f32p, sz]
            for name in ("axc_oracle_q4km_axc_body", "axc_oracle_q4_0_axc_body"):
                f = getattr(L, name)
                f.restype = C.c_float
                f.argtypes = [u8p, f32p, C.c_uint32]
            for name in ("axc_oracle_q4km_matvec_rows", "axc_oracle_q4_0_matvec_rows"):
                f = getattr(L, name)
                f.restype = None
                f.argtypes = [u8p, f32p, f32p, sz, sz, C.c_int]
            for name in ("axc_oracle_q4km_matvec_rows_f64", "axc_oracle_q4_0_matvec_rows_f64"):
                f = getattr(L, name)
                f.restype = None
                f.argtypes = [u8p, f32p, f64p, f64p, sz, sz, C.c_int]
            for name in ("axc_oracle_q4km_dequant_rows", "axc_oracle_q4_0_dequant_rows"):
                f = getattr(L, name)
                f.restype = None
                f.argtypes = [u8p, f32p, sz, sz, C.c_int]
            L.axc_oracle_q4km_prefill.restype = None
            L.axc_oracle_q4km_prefill.argtypes = [u8p, f32p, f32p, sz, sz, sz, C.c_int]
            L.axc_oracle_generate_q4km_test_data.restype = None
            L.axc_oracle_generate_q4km_test_data.argtypes = [C.c_uint32, C.c_uint64, u8p, f32p]
            L.axc_oracle_max_threads.restype = C.c_int
            L.axc_oracle_max_threads.argtypes = []
            _lib = L
    return _lib


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint8)
    return a


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def max_threads() -> int:
    return int(lib().axc_oracle_max_threads())


def f16_bits_to_f32(bits: int) -> np.float32:
    return np.float32(lib().axc_oracle_f16_bits_to_f32(int(bits) & 0xFFFF))


def f32_to_f16_bits(v: float) -> int:
    return int(lib().axc_oracle_f32_to_f16_bits(float(np.float32(v))))


def unpack_scale_min_k4(scales, j: int) -> tuple[int, int]:
    """(sc, m) of sub-block ``j`` from the 12-byte scales field (common_helpers.rs:365-381)."""
    s = _u8(scales)
    assert s.size == 12 and 0 <= j < 8
    sc = np.zeros(1, np.uint8)
    m = np.zeros(1, np.uint8)
    lib().axc_oracle_unpack_scale_min_k4(_p(s), j, _p(sc), _p(m))
    return int(sc[0]), int(m[0])


def pack_scale_min_k4(sc, m) -> np.ndarray:
    sc, m = _u8(sc), _u8(m)
    assert sc.size == 8 and m.size == 8
    out = np.zeros(12, np.uint8)
    lib().axc_oracle_pack_scale_min_k4(_p(sc), _p(m), _p(out))
    return out


def q4km_dequant_matvec_cpu(q, x, n_superblocks: int) -> np.float32:
    """One reference call (common_helpers.rs:411-461), including its size assertions."""
    q, x = _u8(q), _f32(x)
    if q.size != n_superblocks * Q4KM_SB_BYTES:
        raise AssertionError(f"q4km_dequant_matvec_cpu: q length mismatch: expected "
                             f"{n_superblocks * Q4KM_SB_BYTES}, got {q.size}")
    if x.size < n_superblocks * Q4KM_SB_ELEMS:
        raise AssertionError(f"q4km_dequant_matvec_cpu: x length too short: expected >= "
                             f"{n_superblocks * Q4KM_SB_ELEMS}, got {x.size}")
    return np.float32(lib().axc_oracle_q4km_dequant_matvec(_p(q), _p(x), n_superblocks))


def q4_0_dequant_matvec_cpu(q, x, n_blocks: int) -> np.float32:
    """One reference call (benches/common.rs:212-259), including its size assertions."""
    q, x = _u8(q), _f32(x)
    if q.size != n_blocks * Q4_0_BLK_BYTES:
        raise AssertionError(f"q4_0_dequant_matvec_cpu: q length mismatch: expected "
                             f"{n_blocks * Q4_0_BLK_BYTES}, got {q.size}")
    if x.size != n_blocks * Q4_0_BLK_ELEMS:
        raise AssertionError(f"q4_0_dequant_matvec_cpu: x length mismatch: expected "
                             f"{n_blocks * Q4_0_BLK_ELEMS}, got {x.size}")
    return np.float32(lib().axc_oracle_q4_0_dequant_matvec(_p(q), _p(x), n_blocks))


def q4km_axc_body(q, x, n_superblocks: int) -> np.float32:
    q, x = _u8(q), _f32(x)
    assert q.size >= n_superblocks * Q4KM_SB_BYTES and x.size >= n_superblocks * Q4KM_SB_ELEMS
    return np.float32(lib().axc_oracle_q4km_axc_body(_p(q), _p(x), n_superblocks))


def q4_0_axc_body(q, x, n_blocks: int) -> np.float32:
    q, x = _u8(q), _f32(x)
    assert q.size >= n_blocks * Q4_0_BLK_BYTES and x.size >= n_blocks * Q4_0_BLK_ELEMS
    return np.float32(lib().axc_oracle_q4_0_axc_body(_p(q), _p(x), n_blocks))


def _fmt(fmt: str) -> tuple[int, int, str]:
    if fmt == "q4k":
        return Q4KM_SB_BYTES, Q4KM_SB_ELEMS, "q4km"
    if fmt == "q4_0":
        return Q4_0_BLK_BYTES, Q4_0_BLK_ELEMS, "q4_0"
    raise ValueError(fmt)


def matvec_rows(fmt: str, q, x, rows: int, n: int, threads: int = 0) -> np.ndarray:
    """y[r] = reference call on row r (``n`` blocks per row) with the shared x, fp32 sequential."""
    bb, be, nm = _fmt(fmt)
    q, x = _u8(q), _f32(x)
    assert q.size >= rows * n * bb and x.size >= n * be
    y = np.zeros(max(rows, 0), np.float32)
    getattr(lib(), f"axc_oracle_{nm}_matvec_rows")(_p(q), _p(x), _p(y), rows, n, threads)
    return y


def matvec_rows_f64(fmt: str, q, x, rows: int, n: int, threads: int = 0):
    """(fp64 dot products of the bit-exact weights, per-row sum |w_i x_i|)."""
    bb, be, nm = _fmt(fmt)
    q, x = _u8(q), _f32(x)
    assert q.size >= rows * n * bb and x.size >= n * be
    y = np.zeros(rows, np.float64)
    a = np.zeros(rows, np.float64)
    getattr(lib(), f"axc_oracle_{nm}_matvec_rows_f64")(_p(q), _p(x), _p(y), _p(a), rows, n, threads)
    return y, a


def dequant_rows(fmt: str, q, rows: int, n: int, threads: int = 0) -> np.ndarray:
    """Bit-exact dequantised weights, shape (rows, n * elems_per_block), x-index order."""
    bb, be, nm = _fmt(fmt)
    q = _u8(q)
    assert q.size >= rows * n * bb
    w = np.zeros((rows, n * be), np.float32)
    getattr(lib(), f"axc_oracle_{nm}_dequant_rows")(_p(q), _p(w), rows, n, threads)
    return w


def q4km_prefill(q, a, m_rows: int, n_rows: int, n_sb: int, threads: int = 0) -> np.ndarray:
    """C[m, n] = sum_k bf16(A[m, k]) * bf16(W[n, k]) with fp32 accumulation in k order."""
    q, a = _u8(q), _f32(a)
    assert q.size >= n_rows * n_sb * Q4KM_SB_BYTES and a.size >= m_rows * n_sb * Q4KM_SB_ELEMS
    c = np.zeros((m_rows, n_rows), np.float32)
    lib().axc_oracle_q4km_prefill(_p(q), _p(a), _p(c), m_rows, n_rows, n_sb, threads)
    return c


def unit_rms(v) -> np.ndarray:
    """v / sqrt(mean(v^2)) in fp32 (the sweep's normalisation; no counterpart in the reference)."""
    v = _f32(v)
    ms = np.float32(np.sum(v * v, dtype=np.float32) / np.float32(v.size))
    return (v / np.float32(np.sqrt(ms))).astype(np.float32)


def decode_token(weights, hidden: int, kv: int, ffn: int, h, normalise_input: bool = True, threads: int = 0):
    """One token of the decode sweep on the CPU, every linear through the reference-order matvec.

    weights[layer] = (qkv, o, gate_up, down) Q4_K_M byte arrays of shapes (hidden + 2 kv, hidden),
    (hidden, hidden), (2 ffn, hidden), (hidden, ffn).  Dataflow: q,k,v = W h; o = Wo unitRMS(q);
    g,u = W unitRMS(o); d = Wdown unitRMS(g + u); h <- unitRMS(d).  Returns (outputs, d of the last
    layer, h after the token, sum of all k and v entries in fp64); outputs[layer] = the four vectors.
    """
    h = _f32(h)
    x = unit_rms(h) if normalise_input else h
    outs, ksum, d = [], 0.0, None
    for qkv_w, o_w, gu_w, down_w in weights:
        qkv = matvec_rows("q4k", qkv_w, x, hidden + 2 * kv, hidden // 256, threads)
        o = matvec_rows("q4k", o_w, unit_rms(qkv[:hidden]), hidden, hidden // 256, threads)
        gu = matvec_rows("q4k", gu_w, unit_rms(o), 2 * ffn, hidden // 256, threads)
        d = matvec_rows("q4k", down_w, unit_rms(gu[:ffn] + gu[ffn:]), hidden, ffn // 256, threads)
        ksum += float(np.sum(qkv[hidden:].astype(np.float64)))
        outs.append((qkv, o, gu, d))
        x = unit_rms(d)
    return outs, d, x, ksum


def generate_q4km_test_data(n_superblocks: int, seed: int):
    """The reference's LCG fixture (common_helpers.rs:476-519): (q bytes, x f32)."""
    q = np.zeros(n_superblocks * Q4KM_SB_BYTES, np.uint8)
    x = np.zeros(n_superblocks * Q4KM_SB_ELEMS, np.float32)
    lib().axc_oracle_generate_q4km_test_data(n_superblocks, seed & 0xFFFFFFFFFFFFFFFF, _p(q), _p(x))
    return q, x
