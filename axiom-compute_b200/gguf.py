"""GGUF tensor ingestion for the two 4-bit formats the kernels consume.

The byte layouts of the kernels' ``q`` buffers are ggml's ``block_q4_K`` (144 bytes per 256
weights) and ``block_q4_0`` (18 bytes per 32 weights), which is what the reference's kernels were
written against (the design notes of the reference repository, lines 442-451 of its top-level design file); a Q4_K / Q4_0 tensor stored in a GGUF file is
therefore consumed as it lies in the file: one row of the matrix = ``ne[0] / block`` consecutive
blocks, rows consecutive, no repacking.  This module reads the container (header, metadata,
tensor directory) and hands out such tensors as byte views plus the (rows, blocks per row) the
matvec entry points take.  The reference scopes GGUF ingestion out (its M2.5 / M2.6 milestones);
this is the step in front of the hot path.

The container format is restated from the published GGUF specification (version 3: little
endian; magic "GGUF"; uint32 version; uint64 tensor and metadata counts; metadata key/value
pairs; the tensor directory; tensor data aligned to ``general.alignment``, default 32).  No file
written by another tool is available here to pin the reader against, so it is checked only
against files written by ``write_gguf`` below: container parity is unpinned.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np

GGUF_MAGIC = 0x46554747          # "GGUF"
DEFAULT_ALIGNMENT = 32

# ggml tensor types this module knows the size of: id -> (name, weights per block, bytes per block)
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
    7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110),
    12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292),
}
GGML_TYPE_Q4_0, GGML_TYPE_Q4_K = 2, 12
SUPPORTED = {GGML_TYPE_Q4_0: "q4_0", GGML_TYPE_Q4_K: "q4k"}

# metadata value types
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


class GgufError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    shape: Tuple[int, ...]      # ggml order: shape[0] is the innermost dimension (columns of a matrix)
    ggml_type: int
    offset: int                 # from the start of the data section
    nbytes: int

    @property
    def type_name(self) -> str:
        return GGML_TYPES.get(self.ggml_type, (f"type{self.ggml_type}", 0, 0))[0]


class _Reader:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GgufError("truncated file")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GgufError("truncated string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", "replace")
        self.pos += n
        return s

    def value(self, vtype: int):
        if vtype in _SCALARS:
            return self.take(_SCALARS[vtype])
        if vtype == _T_STRING:
            return self.string()
        if vtype == _T_ARRAY:
            etype, count = self.take("<I"), self.take("<Q")
            if etype == _T_ARRAY:
                raise GgufError("nested arrays are not part of the format")
            return [self.value(etype) for _ in range(count)]
        raise GgufError(f"unknown metadata value type {vtype}")


class GgufFile:
    """A memory-mapped GGUF file: ``metadata`` (dict), ``tensors`` (name -> TensorInfo)."""

    def __init__(self, path):
        self.path = str(path)
        self._f = open(self.path, "rb")
        try:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError as exc:
            self._f.close()
            raise GgufError(f"cannot map {self.path}: {exc}") from None
        view = memoryview(self._map)
        try:
            self._parse(_Reader(view))
        except Exception:
            view.release()
            self.close()
            raise
        view.release()

    def _parse(self, r: "_Reader") -> None:
        if len(self._map) < 24 or r.take("<I") != GGUF_MAGIC:
            raise GgufError("not a GGUF file (bad magic)")
        self.version = r.take("<I")
        if self.version not in (2, 3):
            raise GgufError(f"GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors, n_kv = r.take("<Q"), r.take("<Q")
        self.metadata: Dict[str, object] = {}
        for _ in range(n_kv):
            key = r.string()
            self.metadata[key] = r.value(r.take("<I"))
        self.alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        if self.alignment <= 0 or self.alignment & (self.alignment - 1):
            raise GgufError("general.alignment must be a power of two")
        self.tensors: Dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = r.string()
            n_dims = r.take("<I")
            if n_dims > 4:
                raise GgufError(f"tensor {name}: {n_dims} dimensions")
            shape = tuple(r.take("<Q") for _ in range(n_dims))
            ttype, offset = r.take("<I"), r.take("<Q")
            n_elems = int(np.prod(shape, dtype=np.uint64)) if shape else 1
            _nm, per_block, block_bytes = GGML_TYPES.get(ttype, ("?", 0, 0))
            if per_block and shape and shape[0] % per_block:
                raise GgufError(f"tensor {name}: row length {shape[0]} is not a multiple of the block size {per_block}")
            nbytes = n_elems // per_block * block_bytes if per_block else 0
            if offset % self.alignment:
                raise GgufError(f"tensor {name}: offset {offset} is not aligned to {self.alignment}")
            self.tensors[name] = TensorInfo(name, shape, ttype, offset, nbytes)
        self.data_start = (r.pos + self.alignment - 1) // self.alignment * self.alignment
        for t in self.tensors.values():
            if t.nbytes and self.data_start + t.offset + t.nbytes > len(self._map):
                raise GgufError(f"tensor {t.name} extends past the end of the file")

    def close(self) -> None:
        """Unmap the file.  Views handed out by ``tensor_bytes`` keep the mapping alive until they
        are gone; closing while they exist only closes the file descriptor."""
        try:
            self._map.close()
        except BufferError:
            pass
        finally:
            self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def tensor_bytes(self, name: str) -> np.ndarray:
        """The tensor's bytes as a read-only uint8 view of the mapping (no copy)."""
        t = self.tensors[name]
        if not t.nbytes:
            raise GgufError(f"tensor {name}: type {t.type_name} has no known size")
        start = self.data_start + t.offset
        return np.frombuffer(self._map, dtype=np.uint8, count=t.nbytes, offset=start)

    def q4_matrix(self, name: str):
        """(fmt, rows, blocks_per_row, bytes) of a Q4_K / Q4_0 matrix, ready for the matvec entry
        points: fmt is "q4k" or "q4_0", bytes a uint8 view of rows x blocks_per_row blocks."""
        t = self.tensors[name]
        if t.ggml_type not in SUPPORTED:
            raise GgufError(f"tensor {name} is {t.type_name}; only Q4_K and Q4_0 feed these kernels")
        if len(t.shape) < 1:
            raise GgufError(f"tensor {name} has no dimensions")
        per_block = GGML_TYPES[t.ggml_type][1]
        cols = t.shape[0]
        rows = int(np.prod(t.shape[1:], dtype=np.uint64)) if len(t.shape) > 1 else 1
        return SUPPORTED[t.ggml_type], rows, cols // per_block, self.tensor_bytes(name)

    def q4_matrices(self) -> List[str]:
        return [n for n, t in self.tensors.items() if t.ggml_type in SUPPORTED]


def _put_string(out: bytearray, s: str) -> None:
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def _put_value(out: bytearray, v) -> None:
    if isinstance(v, bool):
        out += struct.pack("<I?", 7, v)
    elif isinstance(v, int):
        out += struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<IQ", 10, v) if v >= 2 ** 32 else struct.pack("<II", 4, v)
    elif isinstance(v, float):
        out += struct.pack("<If", 6, v)
    elif isinstance(v, str):
        out += struct.pack("<I", _T_STRING)
        _put_string(out, v)
    elif isinstance(v, (list, tuple)):
        if not v or not all(isinstance(e, type(v[0])) for e in v):
            raise GgufError("arrays must be non-empty and of one type")
        probe = bytearray()
        _put_value(probe, v[0])
        etype = struct.unpack_from("<I", probe)[0]
        out += struct.pack("<IIQ", _T_ARRAY, etype, len(v))
        for e in v:
            one = bytearray()
            _put_value(one, e)
            out += one[4:]          # the element without its type tag
    else:
        raise GgufError(f"cannot store metadata value of type {type(v).__name__}")


def write_gguf(path, tensors, metadata=None, alignment: int = DEFAULT_ALIGNMENT) -> None:
    """Write a GGUF v3 file.  tensors: iterable of (name, shape in ggml order, ggml_type, bytes-like).
    Used for synthetic checkpoints and for the reader's tests."""
    metadata = dict(metadata or {})
    if alignment != DEFAULT_ALIGNMENT:
        metadata["general.alignment"] = int(alignment)
    tensors = [(n, tuple(int(d) for d in s), int(t), np.ascontiguousarray(np.frombuffer(memoryview(b), dtype=np.uint8)))
               for n, s, t, b in tensors]
    head = bytearray(struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(metadata)))
    for k, v in metadata.items():
        _put_string(head, k)
        _put_value(head, v)
    offset, offsets = 0, []
    for _n, shape, ttype, data in tensors:
        _nm, per_block, block_bytes = GGML_TYPES[ttype]
        n_elems = int(np.prod(shape, dtype=np.uint64))
        if shape[0] % per_block or n_elems // per_block * block_bytes != data.size:
            raise GgufError("tensor bytes do not match its shape and type")
        offsets.append(offset)
        offset = (offset + data.size + alignment - 1) // alignment * alignment
    for (name, shape, ttype, _d), off in zip(tensors, offsets):
        _put_string(head, name)
        head += struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        head += struct.pack("<IQ", ttype, off)
    with open(path, "wb") as f:
        f.write(head)
        f.write(bytes(-len(head) % alignment))
        for (_n, _s, _t, data), off in zip(tensors, offsets):
            f.write(data.tobytes())
            f.write(bytes(-data.size % alignment))
