"""Decode sweep over a stack of Q4_K_M linear layers (the 70B-shaped workload).

The reference has no model; the sweep is this backend's end-to-end use of its matvec: one
token's pass through ``layers`` blocks of seven linears with the dataflow

    q, k, v = Wq h, Wk h, Wv h            (k and v are only checksummed)
    o       = Wo   . unitRMS(q)
    g, u    = Wgate . unitRMS(o),  Wup . unitRMS(o)
    d       = Wdown . unitRMS(g + u)
    h      <- unitRMS(d)                   unitRMS(v) = v / sqrt(mean(v^2)), fp32

Every elementwise step is folded into the matvec that consumes it (``axc_cuda_q4k_matvec_fused``:
x = a [+ b], unit RMS as one output scale), Wq/Wk/Wv and Wgate/Wup are stored as one matrix each,
so a layer is four launches.  With more than one GPU every linear is row-sharded and its
all-gather is fused into the producing kernel's epilogue.  How a linear's output becomes the
next linear's input is the ``mode``:

* ``"prepared"``: a small prepare kernel between the two (started while the producer is
  still running when the source is (value, epoch) words) assembles x once, quantises it to the
  digit-word image and leaves the sums of x^2; every CTA of the consumer reads its digit words
  straight into registers.
* ``"fused"``: every consumer CTA assembles and quantises x itself (``axc_cuda_q4k_matvec_fused``);
  with more than one GPU a finish kernel first unpacks the words into a plain vector.
* ``"mixed"`` (default on one GPU): "prepared" for the linears with K > 8192 (the down projection),
  "fused" for the others: the faster choice per shape on one GPU.  On several GPUs it runs (the
  prepare kernel then reads the words of gate+up) but measured slower than "fused" (5.92 against
  5.73 ms/token on two GPUs).
* ``"poll"``: as "fused", but every consumer CTA polls the (value, epoch) words itself (no launch in
  between, 2 x the bytes per CTA past L1: measured slower).
* ``"paired"`` (several GPUs only, the default there when the shape divides): the linears are sharded in pairs so that a layer has two exchanges
  instead of four.  qkv and gate+up are sharded by ROWS, each rank owning matching slices (its
  rows of q, k and v; its rows of g and of u); o and down are sharded by COLUMNS: a rank multiplies
  its column range of Wo with its own slice of q (of Wdown with its own g + u), which it has
  locally, and stores the full-length vector of partial sums into every rank's storage; a
  reduce-finish kernel sums the parts (same order on every rank) into the plain vector the next
  row-sharded linear stages.  The unit-RMS scale of q and of g + u never has to be exchanged:
  both feed a linear whose output is normalised again before use, and unitRMS(s v) = unitRMS(v).
  The sums of partial products are rounded differently from the one-GPU order, within the same
  bar; the vectors o and d held here are the unscaled sums.

Weights are synthetic (uniform nibbles and scale bytes, d and dmin = f16(|N(0,1)| * 0.01)),
generated on the device in eight row chunks per linear so that the global matrices are the same
for 1, 2, 4 and 8 ranks.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import _ffi
from .runtime import _raise_for

CHUNKS = 8   # generation granularity along rows = the largest supported world size


@dataclass(frozen=True)
class SweepShape:
    hidden: int
    kv: int
    ffn: int
    layers: int

    @property
    def linears(self):
        """(name, rows, K) of the four launches of a layer."""
        return (("qkv", self.hidden + 2 * self.kv, self.hidden), ("o", self.hidden, self.hidden),
                ("gate_up", 2 * self.ffn, self.hidden), ("down", self.hidden, self.ffn))

    @property
    def weights_per_layer(self) -> int:
        return sum(r * k for _n, r, k in self.linears)

    @property
    def bytes_per_layer(self) -> int:
        return self.weights_per_layer // 256 * 144

    @property
    def vector_words_per_layer(self) -> int:
        return sum(r for _n, r, _k in self.linears)


LLAMA_70B = SweepShape(hidden=8192, kv=1024, ffn=28672, layers=80)


def synth_chunk(rows: int, n_sb: int, seed: int, device) -> torch.Tensor:
    """`rows` rows of well-formed Q4_K_M superblocks, generated on `device`."""
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    nblk = rows * n_sb
    q = torch.randint(0, 256, (nblk, 144), dtype=torch.uint8, device=device, generator=g)
    hdr = (torch.randn((nblk, 2), device=device, generator=g).abs() * 0.01).to(torch.float16)
    q[:, :4] = hdr.view(torch.uint8)
    return q.view(-1)


def full_matrix(shape: SweepShape, seed: int, layer: int, j: int, device) -> torch.Tensor:
    """The whole matrix of linear j of `layer` (all row chunks), as ``DecodeSweep`` generates it."""
    _n, rows, k = shape.linears[j]
    return torch.cat([synth_chunk(rows // CHUNKS, k // 256, seed + (layer * 4 + j) * CHUNKS + c, device)
                      for c in range(CHUNKS)])


MODES = ("prepared", "fused", "poll", "mixed", "paired")


class DecodeSweep:
    """One rank's share of the stack plus the buffers and launches of a token."""

    def __init__(self, shape: SweepShape, device, seed: int = 0xA0C0 + 4 * 16, group=None, tuning=None,
                 mode: str = "auto"):
        if mode == "auto":   # the faster one as measured: mixed on one GPU, paired sharding on several
            multi = torch.distributed.is_available() and torch.distributed.is_initialized() \
                and torch.distributed.get_world_size(group) > 1
            mode = "mixed"
            if multi:
                w = torch.distributed.get_world_size(group)
                fits = shape.hidden % (256 * w) == 0 and shape.ffn % (256 * w) == 0 and shape.kv % w == 0
                mode = "paired" if fits else "fused"
        if mode not in MODES:
            raise ValueError(f"mode must be one of {MODES}")
        self.shape, self.device = shape, torch.device(device)
        self.mode, self.seed = mode, int(seed)
        self.consumer_polls = mode == "poll"
        self.world, self.rank = 1, 0
        self.tuning = tuning
        dist_on = group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()
                                        and torch.distributed.get_world_size() > 1)
        if dist_on:
            import torch.distributed as dist
            group = group if group is not None else dist.group.WORLD
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if CHUNKS % self.world:
            raise ValueError(f"world size must divide {CHUNKS}")
        self.parallelism = (f"rows of every linear sharded over {self.world} GPUs, all-gather fused into the "
                            "producer's epilogue (peer stores of (value, epoch) words)")
        for _n, rows, k in shape.linears:
            if rows % CHUNKS or k % 256 or k // 256 > 128:
                raise ValueError("every linear needs rows divisible by 8 and K a multiple of 256 up to 32768")
        if self.mode == "paired":
            self._init_paired(shape, seed, group)
            return
        per = CHUNKS // self.world
        # weights[layer][j]: this rank's contiguous rows of linear j
        self.weights: List[List[torch.Tensor]] = []
        for layer in range(shape.layers):
            row = []
            for j, (_n, rows, k) in enumerate(shape.linears):
                parts = [synth_chunk(rows // CHUNKS, k // 256, seed + (layer * 4 + j) * CHUNKS + c, self.device)
                         for c in range(self.rank * per, (self.rank + 1) * per)]
                row.append(torch.cat(parts) if len(parts) > 1 else parts[0])
            self.weights.append(row)
        # vectors: every linear's full output, per layer (k and v stay available for the checksum)
        words = shape.vector_words_per_layer * shape.layers
        self.offsets = []   # word offset of linear j of layer l
        off = 0
        for layer in range(shape.layers):
            o = []
            for _n, rows, _k in shape.linears:
                o.append(off)
                off += rows
            self.offsets.append(o)
        self.checkable_outputs = (0, 1, 2, 3)   # linears whose full output vector every rank holds
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.h = torch.zeros(shape.hidden, dtype=torch.float32, device=self.device)     # token input (plain)
        self.d_last = torch.zeros(shape.hidden, dtype=torch.float32, device=self.device)
        if self.world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            # Two copies of the (value, epoch) store, used alternately by even and odd tokens: a rank
            # that is already writing token t + 1 never touches words that a slower rank is still
            # reading for token t.  (Token t + 2 cannot start anywhere before every rank has sent its
            # last vector of token t + 1, which it does after it has read all of token t.)
            self.pairs = symm_mem.empty(2 * words, dtype=torch.int64, device=self.device)
            self.pairs.zero_()
            self._handle = symm_mem.rendezvous(self.pairs, group)
            ptrs = list(self._handle.buffer_ptrs)
            torch.cuda.synchronize(self.device)
            dist.barrier(group)
            self.ptr_table = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
        else:
            self.pairs = None
        self.parity_stride = words * 8
        self.vec = torch.zeros(words, dtype=torch.float32, device=self.device)
        if self.world == 1 and self.consumer_polls:
            raise ValueError("mode 'poll' needs more than one rank")
        # per linear: hand x over through a prepare kernel?  mixed: only where K is large (measured per
        # shape in strict order: 8192 x 28672 31.9 -> 28.2 us, but 8192 x 8192 11.0 -> 12.5 us)
        self.prepared_linear = [self.mode == "prepared" or (self.mode == "mixed" and k > 8192)
                                for _n, _r, k in shape.linears]
        # several ranks: does linear j's vector get its own finish kernel (words -> plain vector)?
        # Only where the consumer (the next linear) stages x itself from a plain vector.
        self.finish_after = [self.world > 1 and self.mode in ("fused", "mixed") and not self.prepared_linear[(j + 1) % 4]
                             for j in range(4)]
        k_max = max(k for _n, _r, k in shape.linears)
        img_bytes = int(_ffi.lib().axc_cuda_q4k_prepared_x_bytes(k_max // 256))
        self.images = [torch.zeros(img_bytes, dtype=torch.uint8, device=self.device) for _ in range(2)]
        self._img = 0
        if self.mode == "prepared":
            self.launches_per_token = 8 * shape.layers + (3 if self.world > 1 else 1)
        elif self.world == 1:
            self.launches_per_token = (4 + sum(self.prepared_linear)) * shape.layers + 1
        else:
            self.launches_per_token = (4 + sum(self.prepared_linear) + sum(self.finish_after)) * shape.layers + 2 \
                + (0 if all(self.finish_after) else 1)

    # -- helpers ---------------------------------------------------------------------------
    def _stream(self) -> int:
        return int(torch.cuda.current_stream(self.device).cuda_stream)

    def _linear(self, layer: int, j: int, xsrc: "_ffi.AxcXSrc") -> None:
        _n, rows, k = self.shape.linears[j]
        rows_local = rows // self.world
        w = self.weights[layer][j]
        off = self.offsets[layer][j]
        st = self.status.data_ptr()
        tn = C.byref(self.tuning) if self.tuning is not None else None
        if self.world > 1:
            g = _ffi.AxcGather(self.ptr_table.data_ptr(), off * 8, self.epoch.data_ptr(), self.world, self.rank,
                               self.rank * rows_local, self.parity_stride)
            rc = _ffi.lib().axc_cuda_q4k_matvec_fused(w.data_ptr(), C.byref(xsrc), None, rows_local, k // 256,
                                                      C.byref(g), self._stream(), st, tn)
            if rc == 0 and self.finish_after[j]:
                rc = _ffi.lib().axc_cuda_gather_finish(
                    self.pairs.data_ptr() + off * 8, self.epoch.data_ptr(), self.vec.data_ptr() + off * 4, rows,
                    self._stream(), st, _ffi.AXC_FINISH_OVERLAP_PREVIOUS, self.parity_stride, None)
        else:
            rc = _ffi.lib().axc_cuda_q4k_matvec_fused(w.data_ptr(), C.byref(xsrc), self.vec.data_ptr() + off * 4,
                                                      rows_local, k // 256, None, self._stream(), st, tn)
        _raise_for(rc)

    def _linear_prepared(self, layer: int, j: int, xsrc: "_ffi.AxcXSrc", rms: bool, overlap: bool) -> None:
        """prepare_x of the source into the next image buffer, then the matvec that reads it."""
        _n, rows, k = self.shape.linears[j]
        rows_local = rows // self.world
        w = self.weights[layer][j]
        off = self.offsets[layer][j]
        st = self.status.data_ptr()
        tn = C.byref(self.tuning) if self.tuning is not None else None
        self._img ^= 1
        img = self.images[self._img].data_ptr()
        L = _ffi.lib()
        _raise_for(L.axc_cuda_q4k_prepare_x(C.byref(xsrc), img, None, k // 256, self._stream(), st,
                                            _ffi.AXC_FINISH_OVERLAP_PREVIOUS if overlap else 0))
        if self.world > 1:
            g = _ffi.AxcGather(self.ptr_table.data_ptr(), off * 8, self.epoch.data_ptr(), self.world, self.rank,
                               self.rank * rows_local, self.parity_stride)
            rc = L.axc_cuda_q4k_matvec_prepared(w.data_ptr(), img, 1 if rms else 0, None, rows_local, k // 256,
                                                C.byref(g), self._stream(), st, tn)
            if rc == 0 and self.finish_after[j]:
                rc = L.axc_cuda_gather_finish(self.pairs.data_ptr() + off * 8, self.epoch.data_ptr(),
                                              self.vec.data_ptr() + off * 4, rows, self._stream(), st,
                                              _ffi.AXC_FINISH_OVERLAP_PREVIOUS, self.parity_stride, None)
        else:
            rc = L.axc_cuda_q4k_matvec_prepared(w.data_ptr(), img, 1 if rms else 0,
                                                self.vec.data_ptr() + off * 4, rows_local, k // 256, None,
                                                self._stream(), st, tn)
        _raise_for(rc)

    def _src(self, layer: int, j: int, word: int = 0, second: Optional[int] = None, rms: bool = True):
        """x source = output of linear j of `layer` starting at `word` (+ the vector at `second`):
        the plain vector where a finish kernel unpacked it, else the (value, epoch) words."""
        base = self.offsets[layer][j] + word
        if self.world > 1 and not self.finish_after[j]:
            p = self.pairs.data_ptr()
            return _ffi.AxcXSrc(None, None, p + base * 8,
                                None if second is None else p + (self.offsets[layer][j] + second) * 8,
                                self.epoch.data_ptr(), 1 if rms else 0, self.parity_stride)
        p = self.vec.data_ptr()
        return _ffi.AxcXSrc(p + base * 4, None if second is None else p + (self.offsets[layer][j] + second) * 4,
                            None, None, None, 1 if rms else 0, 0)

    # -- one token --------------------------------------------------------------------------
    def token(self, normalise_input: bool = True) -> None:
        """Enqueue one token: reads ``self.h`` (normalised first unless told otherwise, which is
        how the previous token's d becomes this token's h), leaves the last layer's d in
        ``self.d_last`` and every linear's output in the vector store."""
        sh = self.shape
        if self.mode == "paired":
            return self._token_paired(normalise_input)
        with torch.cuda.device(self.device):
            if self.world > 1:
                _raise_for(_ffi.lib().axc_cuda_gather_next_epoch(self.epoch.data_ptr(), self._stream()))
            # The prepare kernel waits for the launch before it even when its sources are epoch words (it
            # could start behind its producer and poll, but that measured 3 us slower per linear).
            ov = False
            for layer in range(sh.layers):
                if layer == 0:
                    x = _ffi.AxcXSrc(self.h.data_ptr(), None, None, None, None, 1 if normalise_input else 0, 0)
                else:
                    x = self._src(layer - 1, 3)                         # h = unitRMS(d of the layer before)
                sources = (x,                                            # q, k, v = W h
                           self._src(layer, 0),                          # o = Wo . unitRMS(q): first `hidden` words
                           self._src(layer, 1),                          # g, u = W . unitRMS(o)
                           self._src(layer, 2, 0, sh.ffn))               # d = Wdown . unitRMS(g + u)
                for j, src in enumerate(sources):
                    rms = normalise_input or layer > 0 or j > 0
                    if self.prepared_linear[j]:
                        self._linear_prepared(layer, j, src, rms, ov and (layer > 0 or j > 0))
                    else:
                        self._linear(layer, j, src)
            last = self.offsets[sh.layers - 1][3]
            if self.world > 1 and not all(self.finish_after):
                # some vectors were never unpacked: every vector (k and v included) in one pass
                _raise_for(_ffi.lib().axc_cuda_gather_finish(
                    self.pairs.data_ptr(), self.epoch.data_ptr(), self.vec.data_ptr(),
                    sh.vector_words_per_layer * sh.layers, self._stream(), self.status.data_ptr(), 0,
                    self.parity_stride, None))
            self.d_last.copy_(self.vec[last:last + sh.hidden])

    # -- paired sharding (rows for qkv and gate+up, columns for o and down) -------------------
    def _init_paired(self, shape: SweepShape, seed: int, group) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        W, r, dev = self.world, self.rank, self.device
        if W < 2:
            raise ValueError("mode 'paired' needs more than one rank")
        hid, kv, ffn = shape.hidden, shape.kv, shape.ffn
        if hid % (256 * W) or ffn % (256 * W) or kv % W:
            raise ValueError("paired sharding needs hidden and ffn divisible by 256 * world and kv by world")
        hq, hk, hf = hid // W, kv // W, ffn // W
        self.slices = (hq, hk, hf)
        self.parallelism = (f"qkv and gate+up sharded by rows, o and down by columns over {W} GPUs: two exchanges "
                            "per layer (partial sums stored into every rank by the producer's epilogue, summed by a "
                            "reduce-finish kernel)")
        self.weights = []
        for layer in range(shape.layers):
            row = []
            for j, (_n, rows, k) in enumerate(shape.linears):
                n_sb = k // 256
                full = full_matrix(shape, seed, layer, j, dev).view(rows, n_sb, 144)
                if j == 0:      # this rank's rows of q, of k and of v
                    part = torch.cat([full[r * hq:(r + 1) * hq], full[hid + r * hk:hid + (r + 1) * hk],
                                      full[hid + kv + r * hk:hid + kv + (r + 1) * hk]])
                elif j == 2:    # this rank's rows of g and of u
                    part = torch.cat([full[r * hf:(r + 1) * hf], full[ffn + r * hf:ffn + (r + 1) * hf]])
                else:           # this rank's columns (whole superblocks) of every row
                    per = n_sb // W
                    part = full[:, r * per:(r + 1) * per]
                row.append(part.contiguous().view(-1))
                del full, part
            self.weights.append(row)
        L = shape.layers
        # (value, epoch) storage: per layer W parts of o partial sums and W parts of d partial sums, two copies
        self._words_layer = 2 * W * hid
        words = self._words_layer * L
        self.pairs = symm_mem.empty(2 * words, dtype=torch.int64, device=dev)
        self.pairs.zero_()
        self._handle = symm_mem.rendezvous(self.pairs, group if group is not None else dist.group.WORLD)
        ptrs = list(self._handle.buffer_ptrs)
        torch.cuda.synchronize(dev)
        dist.barrier(group)
        self.ptr_table = torch.tensor(ptrs, dtype=torch.int64, device=dev)
        self.parity_stride = words * 8
        # plain local vectors, per layer: [q k v slices | o sum | g u slices | d sum]
        self._loc = (hq + 2 * hk, hid, 2 * hf, hid)
        self._loc_off = [0, self._loc[0], self._loc[0] + hid, self._loc[0] + hid + 2 * hf]
        self._loc_layer = sum(self._loc)
        self.vec = torch.zeros(self._loc_layer * L, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.h = torch.zeros(hid, dtype=torch.float32, device=dev)
        self.d_last = torch.zeros(hid, dtype=torch.float32, device=dev)
        self.checkable_outputs = ()        # full q/k/v and g/u exist nowhere; o and d are unscaled sums
        self.prepared_linear = [False] * 4
        self.finish_after = [False, True, False, True]
        self.launches_per_token = 6 * L + 2
        self._group = group

    def _vec_ptr(self, layer: int, part: int, off: int = 0) -> int:
        return self.vec.data_ptr() + (layer * self._loc_layer + self._loc_off[part] + off) * 4

    def _token_paired(self, normalise_input: bool) -> None:
        sh, W, r = self.shape, self.world, self.rank
        hq, hk, hf = self.slices
        hid = sh.hidden
        L = _ffi.lib()
        st = self.status.data_ptr()
        tn = C.byref(self.tuning) if self.tuning is not None else None
        ep = self.epoch.data_ptr()
        stream = self._stream
        with torch.cuda.device(self.device):
            _raise_for(L.axc_cuda_gather_next_epoch(ep, stream()))
            for layer in range(sh.layers):
                wq, wo, wgu, wd = self.weights[layer]
                base = layer * self._words_layer          # word offset of this layer's parts
                # qkv (rows): x = h (first layer) or the summed d of the layer before, unit RMS
                if layer == 0:
                    x = _ffi.AxcXSrc(self.h.data_ptr(), None, None, None, None, 1 if normalise_input else 0, 0)
                else:
                    x = _ffi.AxcXSrc(self._vec_ptr(layer - 1, 3), None, None, None, None, 1, 0)
                _raise_for(L.axc_cuda_q4k_matvec_fused(wq.data_ptr(), C.byref(x), self._vec_ptr(layer, 0), hq + 2 * hk,
                                                       hid // 256, None, stream(), st, tn))
                # o (columns): this rank's slice of q times its columns of Wo -> part `rank` on every rank
                x = _ffi.AxcXSrc(self._vec_ptr(layer, 0), None, None, None, None, 0, 0)
                g = _ffi.AxcGather(self.ptr_table.data_ptr(), (base + r * hid) * 8, ep, W, r, 0, self.parity_stride)
                _raise_for(L.axc_cuda_q4k_matvec_fused(wo.data_ptr(), C.byref(x), None, hid, hq // 256, C.byref(g),
                                                       stream(), st, tn))
                _raise_for(L.axc_cuda_gather_reduce_finish(self.pairs.data_ptr() + base * 8, ep, self._vec_ptr(layer, 1), hid,
                                                           W, hid * 8, stream(), st, _ffi.AXC_FINISH_OVERLAP_PREVIOUS,
                                                           self.parity_stride))
                # gate+up (rows): x = summed o, unit RMS
                x = _ffi.AxcXSrc(self._vec_ptr(layer, 1), None, None, None, None, 1, 0)
                _raise_for(L.axc_cuda_q4k_matvec_fused(wgu.data_ptr(), C.byref(x), self._vec_ptr(layer, 2), 2 * hf,
                                                       hid // 256, None, stream(), st, tn))
                # down (columns): (g + u) slice times this rank's columns of Wdown -> parts of d
                x = _ffi.AxcXSrc(self._vec_ptr(layer, 2), self._vec_ptr(layer, 2, hf), None, None, None, 0, 0)
                g = _ffi.AxcGather(self.ptr_table.data_ptr(), (base + (W + r) * hid) * 8, ep, W, r, 0, self.parity_stride)
                _raise_for(L.axc_cuda_q4k_matvec_fused(wd.data_ptr(), C.byref(x), None, hid, hf // 256, C.byref(g),
                                                       stream(), st, tn))
                _raise_for(L.axc_cuda_gather_reduce_finish(self.pairs.data_ptr() + (base + W * hid) * 8, ep,
                                                           self._vec_ptr(layer, 3), hid, W, hid * 8, stream(), st,
                                                           _ffi.AXC_FINISH_OVERLAP_PREVIOUS, self.parity_stride))
            last = (sh.layers - 1) * self._loc_layer + self._loc_off[3]
            self.d_last.copy_(self.vec[last:last + hid])

    def local_output(self, layer: int, part: int) -> torch.Tensor:
        """paired mode: this rank's plain vectors of `layer`: 0 = its slices of q, k, v; 1 = the summed o;
        2 = its slices of g, u; 3 = the summed d (o and d without the unit-RMS scale of their input)."""
        o = layer * self._loc_layer + self._loc_off[part]
        return self.vec[o:o + self._loc[part]]

    def _plain_store(self) -> torch.Tensor:
        return self.vec

    def advance(self) -> None:
        """h of the next token = d of this one (normalised by the next token's first launch)."""
        self.h.copy_(self.d_last)

    # -- results ----------------------------------------------------------------------------
    def output(self, layer: int, j: int) -> torch.Tensor:
        """Full output vector of linear j of `layer` (after ``token()`` has completed)."""
        off = self.offsets[layer][j]
        return self._plain_store()[off:off + self.shape.linears[j][1]]

    def kv_checksum(self) -> torch.Tensor:
        """Sum of every layer's k and v entries (fp64, on the device)."""
        sh = self.shape
        if self.mode == "paired":      # every rank holds its slices of k and v: sum them over the ranks
            import torch.distributed as dist
            hq, hk, _hf = self.slices
            v = self.vec.view(sh.layers, self._loc_layer)[:, hq:hq + 2 * hk].double().sum()
            dist.all_reduce(v, group=self._group)
            return v
        per = sh.vector_words_per_layer
        v = self._plain_store().view(sh.layers, per)[:, sh.hidden:sh.hidden + 2 * sh.kv]
        return v.double().sum()

    def hidden_out(self) -> torch.Tensor:
        """h after the token: unitRMS(d of the last layer)."""
        d = self.d_last
        return d / torch.sqrt(torch.mean(d * d))
