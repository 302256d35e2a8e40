"""GGUF ingestion: the reader against files written by the module's own writer and against a
file assembled field by field from the published layout (no file from another tool is available:
container parity stays unpinned), and the Q4 tensors it hands out against the oracle / the GPU
kernels."""
import struct

import numpy as np
import pytest

import oracle
from conftest import load_pkg

gguf = load_pkg("gguf")


@pytest.fixture()
def sample(tmp_path, synth):
    qk = synth.q4k_weights(24, 4, 6001)          # 24 rows x 1024 columns
    q0 = synth.q4_0_weights(10, 8, 6002)         # 10 rows x 256 columns
    f32 = np.arange(7, dtype=np.float32)
    path = tmp_path / "tiny.gguf"
    gguf.write_gguf(path, [("blk.0.ffn_up.weight", (1024, 24), gguf.GGML_TYPE_Q4_K, qk),
                           ("blk.0.attn_q.weight", (256, 10), gguf.GGML_TYPE_Q4_0, q0),
                           ("norm.weight", (7,), 0, f32.tobytes())],
                    {"general.architecture": "llama", "llama.block_count": 1, "general.file_type": 15,
                     "tokenizer.ggml.tokens": ["a", "bc"], "x.scale": 0.5, "x.flag": True, "x.big": 2 ** 40,
                     "x.neg": -3})
    return path, qk, q0, f32


def test_round_trip_of_header_metadata_and_directory(sample):
    path, qk, q0, f32 = sample
    with gguf.GgufFile(path) as g:
        assert g.version == 3 and g.alignment == 32 and g.data_start % 32 == 0
        assert g.metadata["general.architecture"] == "llama" and g.metadata["llama.block_count"] == 1
        assert g.metadata["tokenizer.ggml.tokens"] == ["a", "bc"] and g.metadata["x.flag"] is True
        assert g.metadata["x.big"] == 2 ** 40 and g.metadata["x.neg"] == -3 and g.metadata["x.scale"] == 0.5
        assert list(g.tensors) == ["blk.0.ffn_up.weight", "blk.0.attn_q.weight", "norm.weight"]
        t = g.tensors["blk.0.ffn_up.weight"]
        assert (t.shape, t.type_name, t.nbytes, t.offset % 32) == ((1024, 24), "Q4_K", 24 * 4 * 144, 0)
        assert g.q4_matrices() == ["blk.0.ffn_up.weight", "blk.0.attn_q.weight"]
        fmt, rows, n, data = g.q4_matrix("blk.0.ffn_up.weight")
        assert (fmt, rows, n) == ("q4k", 24, 4) and np.array_equal(data, qk) and not data.flags.writeable
        fmt, rows, n, data = g.q4_matrix("blk.0.attn_q.weight")
        assert (fmt, rows, n) == ("q4_0", 10, 8) and np.array_equal(data, q0)
        assert np.array_equal(g.tensor_bytes("norm.weight").view(np.float32), f32)
        with pytest.raises(gguf.GgufError, match="only Q4_K and Q4_0"):
            g.q4_matrix("norm.weight")


def test_tensors_from_the_file_feed_the_reference_arithmetic(sample, synth):
    """What the reader hands out is exactly what the oracle (and so the kernels) consume."""
    path, qk, q0, _ = sample
    with gguf.GgufFile(path) as g:
        fmt, rows, n, data = g.q4_matrix("blk.0.ffn_up.weight")
        x = synth.activations(n * 256, 6003)
        assert np.array_equal(oracle.matvec_rows(fmt, data, x, rows, n), oracle.matvec_rows("q4k", qk, x, rows, n))
        fmt, rows, n, data = g.q4_matrix("blk.0.attn_q.weight")
        x0 = synth.activations(n * 32, 6004)
        assert np.array_equal(oracle.matvec_rows(fmt, data, x0, rows, n), oracle.matvec_rows("q4_0", q0, x0, rows, n))


def test_custom_alignment_and_malformed_files(tmp_path, synth):
    q = synth.q4k_weights(2, 1, 6005)
    p = tmp_path / "a64.gguf"
    gguf.write_gguf(p, [("w", (256, 2), gguf.GGML_TYPE_Q4_K, q)], alignment=64)
    with gguf.GgufFile(p) as g:
        assert g.alignment == 64 and g.data_start % 64 == 0 and np.array_equal(g.q4_matrix("w")[3], q)
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + bytes(40))
    with pytest.raises(gguf.GgufError, match="bad magic"):
        gguf.GgufFile(bad)
    v9 = tmp_path / "v9.gguf"
    v9.write_bytes(struct.pack("<IIQQ", gguf.GGUF_MAGIC, 9, 0, 0))
    with pytest.raises(gguf.GgufError, match="version 9"):
        gguf.GgufFile(v9)
    raw = bytearray(p.read_bytes())
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(bytes(raw[:-100]))
    with pytest.raises(gguf.GgufError, match="past the end"):
        gguf.GgufFile(cut)
    with pytest.raises(gguf.GgufError, match="do not match"):
        gguf.write_gguf(tmp_path / "x.gguf", [("w", (256, 3), gguf.GGML_TYPE_Q4_K, q)])
    # a directory entry whose row length is not a whole number of blocks (hand-made header)
    name = b"w"
    hdr = struct.pack("<IIQQ", gguf.GGUF_MAGIC, 3, 1, 0) + struct.pack("<Q", len(name)) + name
    hdr += struct.pack("<IQQIQ", 2, 100, 2, gguf.GGML_TYPE_Q4_K, 0)
    odd = tmp_path / "odd.gguf"
    odd.write_bytes(hdr + bytes(256))
    with pytest.raises(gguf.GgufError, match="not a multiple of the block size"):
        gguf.GgufFile(odd)


@pytest.mark.gpu
def test_matvec_on_a_tensor_read_from_gguf(sample, ops, synth):
    import torch
    path, qk, _q0, _ = sample
    with gguf.GgufFile(path) as g:
        fmt, rows, n, data = g.q4_matrix("blk.0.ffn_up.weight")
        x = synth.activations(n * 256, 6006)
        y = ops.q4k_matvec(torch.from_numpy(np.array(data)).cuda(), torch.from_numpy(x).cuda(), rows, n).cpu().numpy()
    y_ref = oracle.matvec_rows("q4k", qk, x, rows, n)
    _y, mag = oracle.matvec_rows_f64("q4k", qk, x, rows, n)
    assert (np.abs(y - y_ref) / mag).max() <= 1e-5


def test_reader_on_bytes_assembled_by_hand_from_the_specification(tmp_path, synth):
    """A file laid out field by field here, independently of the module's writer, following the
    published GGUF v3 layout: magic "GGUF", u32 version, u64 tensor count, u64 key-value count;
    key-values as (string key, u32 value type, value) with strings as u64 length + bytes; tensor
    infos as (string name, u32 n_dims, u64 dims..., u32 ggml type, u64 offset into the data
    section); the data section starts at the next multiple of general.alignment (default 32)."""
    def gstr(t):
        b = t.encode()
        return struct.pack("<Q", len(b)) + b

    qk = synth.q4k_weights(3, 2, 6101)           # 3 rows x 512 columns of Q4_K: 3 * 2 * 144 bytes
    q0 = synth.q4_0_weights(2, 4, 6102)          # 2 rows x 128 columns of Q4_0: 2 * 4 * 18 bytes
    body = b"GGUF" + struct.pack("<IQQ", 3, 2, 3)
    body += gstr("general.architecture") + struct.pack("<I", 8) + gstr("llama")        # 8 = string
    body += gstr("llama.block_count") + struct.pack("<II", 4, 7)                       # 4 = uint32
    body += gstr("x.list") + struct.pack("<IIQ", 9, 5, 3) + struct.pack("<iii", -1, 0, 9)   # 9 = array of int32 (5)
    off0, off1 = 0, (len(qk) + 31) // 32 * 32
    body += gstr("a.weight") + struct.pack("<IQQ", 2, 512, 3) + struct.pack("<IQ", 12, off0)    # 12 = Q4_K
    body += gstr("b.weight") + struct.pack("<IQQ", 2, 128, 2) + struct.pack("<IQ", 2, off1)     # 2 = Q4_0
    body += b"\0" * (-len(body) % 32)
    data = qk.tobytes() + b"\0" * (off1 - len(qk)) + q0.tobytes()
    path = tmp_path / "by_hand.gguf"
    path.write_bytes(body + data)
    with gguf.GgufFile(path) as g:
        assert g.version == 3 and g.alignment == 32 and g.data_start == len(body)
        assert g.metadata == {"general.architecture": "llama", "llama.block_count": 7, "x.list": [-1, 0, 9]}
        a, b = g.tensors["a.weight"], g.tensors["b.weight"]
        assert (a.shape, a.type_name, a.nbytes) == ((512, 3), "Q4_K", 3 * 2 * 144)
        assert (b.shape, b.type_name, b.nbytes) == ((128, 2), "Q4_0", 2 * 4 * 18)
        assert np.array_equal(g.tensor_bytes("a.weight"), qk) and np.array_equal(g.tensor_bytes("b.weight"), q0)
        fmt, rows, n, qa = g.q4_matrix("a.weight")
        assert (fmt, rows, n) == ("q4k", 3, 2) and np.array_equal(np.asarray(qa).reshape(-1), qk)
        assert g.q4_matrix("b.weight")[:3] == ("q4_0", 2, 4)
