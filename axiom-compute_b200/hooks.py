"""The timing hooks that drive the backend: ``bench_variant`` and ``grid_search``.

Mirrors, for the two Q4 kernels, what the reference's agent-facing tools do around
``VulkanContext``:

* ``bench_variant`` -- crates/axc-driver/src/mcp/tools/bench_variant.rs:170-320: prepare the
  kernel once, run ``sample_count`` timed ``dispatch_handle`` calls (every sample re-uploads all
  inputs), ``median_ns = sorted[len / 2]``, a tri-state correctness verdict and machine metadata.
* ``grid_search`` -- crates/axc-optimize/src/grid_search.rs:54-164,166-283 and
  crates/axc-driver/src/mcp/tools/grid_search.rs:206-410: enumerate the Cartesian product of the
  strategy holes in mixed-radix order, check, time, rank, pick the fastest, fall back to the
  lowest ordinals, append a JSONL history record under an exclusive file lock.

Differences, all forced by what this backend is:

* there is no compiler here: a request names the kernel through its ``KernelMetadata`` (or the
  path of the JSON sidecar) instead of ``.axc`` source, and the holes are the launch tunables of
  the ahead-of-time CUDA kernel (``TUNABLE_HOLES``), applied with ``KernelHandle.set_tuning``;
* the reference leaves both Q4 kernels ``NotChecked`` and derives a meaningless grid from the
  byte length of ``q`` (bench_variant.rs:64-80,111-127,395-400).  Here the verdict is real: the
  fast kernel's y is compared with the reference-order kernel (same operation order as the
  reference's CPU function, run on the GPU by a strict handle), and the grid is derived from the
  buffer sizes and the push constant (rows = what q, x and y can hold);
* a response also carries ``device_median_ns``, the kernel's device time from CUDA events;
* variant ids are a 64-bit BLAKE2b of the reference's canonical encoding (u32-LE name length,
  name, i64-LE value), not xxh3: ids are only compared within one history file.

Nothing here has a CPU fallback: without the CUDA library or a GPU every entry point raises.
"""
from __future__ import annotations

import base64
import datetime
import fcntl
import hashlib
import itertools
import json
import os
import struct
from dataclasses import dataclass, field, asdict
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from . import _ffi, runtime, synth
from .errors import DispatchError
from .runtime import (CudaContext, KernelMetadata, ParamBindingPlan, captured_icd_path,
                      load_kernel_metadata, q4_matvec_binding_plan)

Q4_KERNELS = {"q4km_dequant_matvec": (144, 256), "q4_0_dequant_matvec": (18, 32)}  # block bytes, weights
TUNABLE_HOLES = ("ctas_per_sm", "tile_rows", "stages", "threads", "evict_first", "pdl", "resident")
CARTESIAN_WARN_THRESHOLD = 100          # crates/axc-optimize/src/enumerator.rs:42
DEFAULT_REL_TOL = 1e-3                  # the reference's GPU-vs-CPU bar (AT-1324 / AT-918: rel < 1e-3)


class InvalidParams(ValueError):
    """``McpToolError::InvalidParams``."""


# ------------------------------------------------------------------ correctness verdict

@dataclass
class CorrectnessStatus:
    """bench_variant.rs:30-49: ``Ok`` | ``Failed{reason}`` | ``NotChecked{reason}``."""
    kind: str
    reason: str = ""

    def to_json_obj(self):
        """serde form of the reference: tag ``status`` in snake case (bench_variant.rs:27-49)."""
        if self.kind == "Ok":
            return {"status": "ok"}
        return {"status": "failed" if self.kind == "Failed" else "not_checked", "reason": self.reason}

    @staticmethod
    def ok():
        return CorrectnessStatus("Ok")

    @staticmethod
    def failed(reason):
        return CorrectnessStatus("Failed", reason)

    @staticmethod
    def not_checked(reason):
        return CorrectnessStatus("NotChecked", reason)


def pick_reference(kernel_name: str, plan: ParamBindingPlan) -> Optional[str]:
    """bench_variant.rs:62-80 for this backend: which check a kernel gets."""
    if kernel_name in Q4_KERNELS and len(plan.buffers) == 3 and len(plan.scalars) == 1:
        return "strict_order_kernel"
    return None


# ------------------------------------------------------------------ inputs and grid

def compute_variant_id(assignments: Dict[str, int]) -> int:
    """Fingerprint of the canonical encoding (enumerator.rs:88-105); 0 for no assignments
    (bench_variant.rs:323-335)."""
    if not assignments:
        return 0
    enc = bytearray()
    for name in sorted(assignments):
        nb = name.encode("utf-8")
        enc += struct.pack("<I", len(nb)) + nb + struct.pack("<q", int(assignments[name]))
    return int.from_bytes(hashlib.blake2b(bytes(enc), digest_size=8).digest(), "little")


def seeded_inputs(input_sizes: Sequence[int], variant_id: int) -> List[bytes]:
    """bench_variant.rs:88-101: binding i gets `size` bytes from a generator seeded with
    ``variant_id ^ i`` (here numpy's Philox; the reference uses rand's StdRng)."""
    out = []
    for i, size in enumerate(input_sizes):
        rng = np.random.Generator(np.random.Philox(key=(int(variant_id) ^ i) & 0xFFFFFFFFFFFFFFFF))
        out.append(rng.integers(0, 256, int(size), dtype=np.uint8).tobytes())
    return out


def seeded_q4_inputs(kernel_name: str, input_sizes: Sequence[int], n: int, variant_id: int) -> List[bytes]:
    """Well-formed inputs for the Q4 kernels: uniformly random bytes put Inf/NaN into the f16
    scales, which makes any comparison of sums meaningless, so q holds whole rows of valid
    blocks (finite scales, uniform nibbles), x is N(0, 1) and y is zero."""
    blk, _elems = Q4_KERNELS[kernel_name]
    q_len, x_len, y_len = (int(v) for v in input_sizes)
    rows = q_len // (n * blk) if n else 0
    seed = (int(variant_id) ^ 0x51A7) & 0x7FFFFFFF
    if rows:
        q = synth.q4k_weights(rows, n, seed) if kernel_name == "q4km_dequant_matvec" \
            else synth.q4_0_weights(rows, n, seed)
        qb = q.tobytes() + bytes(q_len - q.nbytes)
    else:
        qb = bytes(q_len)
    x = synth.activations(x_len // 4, seed + 1).tobytes() + bytes(x_len % 4)
    return [qb, x, bytes(y_len)]


def derive_workgroups(input_sizes: Sequence[int], workgroup_size: Sequence[int],
                      override: Optional[Sequence[int]] = None, *, kernel_name: Optional[str] = None,
                      push_constants: bytes = b"", output_sizes: Optional[Sequence[int]] = None) -> List[int]:
    """bench_variant.rs:111-127, plus the rule the Q4 kernels need.  An override wins.  For a Q4
    kernel the grid is the row count the buffers hold: ``min(q_len / (n * block), y_len / 4)``
    (n from the push constant), at least 1.  Otherwise the reference's rule: axis 0 =
    ``ceil(input_sizes[0] / 4 / workgroup_size[0])``; ``[1, 1, 1]`` when there is nothing to go by."""
    if override is not None:
        return [int(v) for v in override]
    if kernel_name in Q4_KERNELS and len(input_sizes) == 3 and len(push_constants) >= 4:
        blk, _ = Q4_KERNELS[kernel_name]
        n = struct.unpack_from("<I", push_constants)[0]
        y_len = (output_sizes or input_sizes)[2]
        rows = min(input_sizes[0] // (n * blk), y_len // 4) if n else 1
        return [max(int(rows), 1), 1, 1]
    if not input_sizes or not workgroup_size or workgroup_size[0] == 0:
        return [1, 1, 1]
    n_elems = int(input_sizes[0]) // 4
    wg_x = int(workgroup_size[0])
    return [max((n_elems + wg_x - 1) // wg_x, 1), 1, 1]


def build_push_constants(push_constants_base64: Optional[str], pc_size: int) -> bytes:
    """bench_variant.rs:338-360: decoded length must equal the plan's size; zero-filled if absent."""
    if push_constants_base64 is None:
        return bytes(pc_size)
    try:
        decoded = base64.b64decode(push_constants_base64, validate=True)
    except Exception as exc:
        raise InvalidParams(f"push_constants_base64: {exc}") from None
    if len(decoded) != pc_size:
        raise InvalidParams(f"push_constants_base64 decoded to {len(decoded)} bytes, but kernel expects {pc_size}")
    return decoded


def tuning_from_assignments(assignments: Dict[str, int]):
    """Hole assignments -> launch tunables; unknown hole names are an error."""
    unknown = sorted(set(assignments) - set(TUNABLE_HOLES))
    if unknown:
        raise InvalidParams(f"unknown tunable(s) {unknown}; this kernel's holes are {list(TUNABLE_HOLES)}")
    t = _ffi.AxcTuning(0, 0, 0, 0, -1, -1, 0)
    for k, v in assignments.items():
        setattr(t, k, int(v))
    return t


# ------------------------------------------------------------------ machine metadata

@dataclass
class MachineMetadata:
    """bench_variant.rs:131-146 (``icd_path`` is always None: there is no Vulkan loader)."""
    device_name: str
    driver_version: int = 0
    api_version: int = 0
    physical_device_index: int = 0
    icd_path: Optional[str] = None
    git_sha: Optional[str] = None


def build_machine_metadata(ctx: CudaContext, git_sha: Optional[str] = None) -> MachineMetadata:
    icd = captured_icd_path()
    return MachineMetadata(ctx.physical_device_name(), 0, int(_ffi.lib().axc_cuda_version()),
                           ctx.device_index(), icd or None, git_sha)


class OnceCuda:
    """crates/axc-driver/src/mcp/dispatch.rs:78-129 (``OnceVulkan``): the context is created on
    first use and a failure is cached and re-raised, never retried."""

    def __init__(self, options=None):
        self._options, self._ctx, self._err = options, None, None

    def get_or_init(self) -> CudaContext:
        if self._err is not None:
            raise self._err
        if self._ctx is None:
            try:
                self._ctx = CudaContext(self._options)
            except DispatchError as exc:
                self._err = exc
                raise
        return self._ctx


@dataclass
class McpContext:
    cuda: OnceCuda = field(default_factory=OnceCuda)
    git_sha: Optional[str] = None
    history_dir: Optional[str] = None


# ------------------------------------------------------------------ bench_variant

@dataclass
class BenchVariantRequest:
    """bench_variant.rs:160-186 with ``metadata`` / ``path`` naming the kernel's JSON sidecar."""
    input_sizes: Sequence[int]
    sample_count: int
    metadata: Optional[KernelMetadata] = None
    path: Optional[str] = None
    assignments: Dict[str, int] = field(default_factory=dict)
    workgroup_override: Optional[Sequence[int]] = None
    push_constants_base64: Optional[str] = None
    output_sizes: Optional[Sequence[int]] = None
    input_seed: Optional[int] = None   # inputs are seeded by the variant id (bench_variant.rs:252-256) unless a
                                       # caller that compares variants with each other fixes the seed


@dataclass
class BenchVariantResponse:
    median_ns: int
    samples: List[int]
    correctness: CorrectnessStatus
    machine: MachineMetadata
    device_median_ns: int = 0
    device_samples: List[int] = field(default_factory=list)
    workgroups: List[int] = field(default_factory=list)
    output_bytes: Optional[bytes] = None    # y of the last sample (for policies that compare variants); not serialised

    def to_json_obj(self):
        d = asdict(self)
        d.pop("output_bytes", None)
        d["correctness"] = self.correctness.to_json_obj()
        return d


def q4_metadata(kernel_name: str) -> KernelMetadata:
    """The sidecar the reference's compiler writes for either Q4 kernel (workgroup 64,1,1)."""
    plan = q4_matvec_binding_plan(kernel_name)
    return KernelMetadata.new(kernel_name, [64, 1, 1], plan, kernel_name)


def _resolve_metadata(req) -> KernelMetadata:
    if (req.metadata is None) == (req.path is None):
        raise InvalidParams("exactly one of `metadata` and `path` must be given")
    return req.metadata if req.metadata is not None else load_kernel_metadata(req.path)


def _median(values: Sequence[int]) -> int:
    s = sorted(values)
    return int(s[len(s) // 2])


def check_against_strict(ctx: CudaContext, meta: KernelMetadata, workgroups, inputs, output_sizes,
                         push_constants, outputs, rel_tol: float = DEFAULT_REL_TOL) -> CorrectnessStatus:
    """y of the fast kernel against the reference-order kernel on the same inputs.  Rows whose
    own magnitude is small against the vector's RMS are cancellation-dominated, so the error of
    row i is measured against ``max(|ref_i|, rms(ref))``."""
    if pick_reference(meta.kernel_name, meta.binding_plan) is None:
        return CorrectnessStatus.not_checked(
            f"no reference registered for kernel `{meta.kernel_name}`; variant is valid and timed"
            " -- proceed with caution")
    if outputs is None or len(outputs) < 3 or len(outputs[2]) < 4:
        return CorrectnessStatus.not_checked("no output data to check")
    strict = ctx.prepare_kernel([0x07230203, 0x5EC], meta.binding_plan,
                                meta.binding_plan.push_constant_total_bytes, meta.entry_point)
    try:
        strict.set_strict_order(True)
        ref_out = ctx.dispatch_handle(strict, workgroups, inputs, output_sizes, push_constants)
    finally:
        strict.drop()
    got = np.frombuffer(bytes(outputs[2]), dtype=np.float32)
    ref = np.frombuffer(bytes(ref_out[2]), dtype=np.float32)
    if got.shape != ref.shape:
        return CorrectnessStatus.failed(f"output length {got.size} != reference length {ref.size}")
    if not np.isfinite(ref).all():
        return CorrectnessStatus.not_checked("reference output is not finite (malformed scales in q?)")
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))) if ref.size else 0.0
    denom = np.maximum(np.abs(ref.astype(np.float64)), max(rms, 1e-30))
    err = np.abs(got.astype(np.float64) - ref) / denom
    bad = int((~(err <= rel_tol)).sum())
    if bad:
        return CorrectnessStatus.failed(
            f"{bad}/{ref.size} rows exceeded relative tolerance {rel_tol:g} (worst {float(np.nanmax(err)):.3e})")
    return CorrectnessStatus.ok()


def bench_variant(req: BenchVariantRequest, ctx: McpContext) -> BenchVariantResponse:
    """bench_variant.rs:214-320."""
    if int(req.sample_count) < 1:
        raise InvalidParams("sample_count must be >= 1")
    meta = _resolve_metadata(req)
    plan = meta.binding_plan
    if len(req.input_sizes) != len(plan.buffers):
        raise InvalidParams(f"input_sizes.len() == {len(req.input_sizes)} but kernel has "
                            f"{len(plan.buffers)} buffer bindings")
    tuning = tuning_from_assignments(req.assignments) if req.assignments else None
    cuda = ctx.cuda.get_or_init()
    pc = build_push_constants(req.push_constants_base64, plan.push_constant_total_bytes)
    output_sizes = list(req.output_sizes) if req.output_sizes is not None else list(req.input_sizes)
    workgroups = derive_workgroups(req.input_sizes, meta.workgroup_size, req.workgroup_override,
                                   kernel_name=meta.kernel_name, push_constants=pc, output_sizes=output_sizes)
    variant_id = compute_variant_id(req.assignments)
    seed = variant_id if req.input_seed is None else int(req.input_seed)
    if meta.kernel_name in Q4_KERNELS and len(pc) >= 4:
        inputs = seeded_q4_inputs(meta.kernel_name, req.input_sizes, struct.unpack_from("<I", pc)[0], seed)
    else:
        inputs = seeded_inputs(req.input_sizes, seed)
    # Distinct spirv words per variant keep the cache keys of differently tuned handles apart.
    handle = cuda.prepare_kernel([0x07230203, variant_id & 0xFFFFFFFF, variant_id >> 32], plan,
                                 plan.push_constant_total_bytes, meta.entry_point)
    try:
        handle.set_tuning(tuning)
        median_ns, samples, dev_ns, outputs = cuda.bench_dispatch(
            handle, workgroups, inputs, output_sizes, pc, int(req.sample_count))
        correctness = check_against_strict(cuda, meta, workgroups, inputs, output_sizes, pc, outputs)
    finally:
        handle.drop()
    y_bytes = bytes(outputs[2]) if outputs is not None and len(outputs) > 2 else None
    return BenchVariantResponse(median_ns, samples, correctness,
                                build_machine_metadata(cuda, ctx.git_sha),
                                _median(dev_ns) if dev_ns else 0, dev_ns, workgroups, y_bytes)


# ------------------------------------------------------------------ grid search (axc-optimize)

@dataclass
class CorrectnessPolicy:
    """grid_search.rs:54-66: ``None`` | ``BitExact`` | ``EquivFpTol{ulp}``."""
    kind: str = "None"
    ulp: int = 0

    @staticmethod
    def parse(text: str) -> "CorrectnessPolicy":
        """crates/axc-driver/src/optimize.rs:121-135: "none", "bit-exact", "fp-tol:<ulp>"."""
        if text == "bit-exact":
            return CorrectnessPolicy("BitExact")
        if text.startswith("fp-tol:"):
            digits = text[7:]
            ok = digits.isascii() and digits.isdigit() and int(digits) <= 0xFFFFFFFF
            return CorrectnessPolicy("EquivFpTol", int(digits) if ok else 4)   # an unparsable count means 4
        return CorrectnessPolicy("None")


@dataclass
class SampleStats:
    median_ns: int
    min_ns: int
    max_ns: int
    n_samples: int


@dataclass
class StrategyVariant:
    ordinal: int
    variant_id: int
    assignments: Dict[str, int]


@dataclass
class VariantResult:
    """``outcome`` is ("Ok", SampleStats) | ("Failed", reason) | ("CorrectnessRejected", failure)."""
    ordinal: int
    variant_id: int
    assignments: Dict[str, int]
    outcome: tuple


@dataclass
class GridSearchResult:
    winner_ordinal: int
    winner_variant_id: int
    winner_assignments: Dict[str, int]
    results: List[VariantResult]
    fallback_used: bool
    warnings: List[str]


class GridSearchError(Exception):
    pass


def enumerate_strategy(holes: Dict[str, Sequence[int]]) -> List[StrategyVariant]:
    """enumerator.rs:63-128: alphabetical keys, candidates in the given order, the last key
    varies fastest."""
    if not holes:
        raise GridSearchError("EmptyStrategy")
    keys = sorted(holes)
    out = []
    for ordinal, combo in enumerate(itertools.product(*[list(holes[k]) for k in keys])):
        a = {k: int(v) for k, v in zip(keys, combo)}
        out.append(StrategyVariant(ordinal, compute_variant_id(a), a))
    return out


def grid_search(holes: Optional[Dict[str, Sequence[int]]], policy: CorrectnessPolicy,
                correctness_fn: Optional[Callable[[Dict[str, int]], Optional[tuple]]],
                bench_fn: Callable[[Dict[str, int]], SampleStats]) -> GridSearchResult:
    """grid_search.rs:166-283.  ``bench_fn(assignments)`` returns ``SampleStats`` or raises;
    ``correctness_fn(assignments)`` returns None when the variant is right or a failure tuple
    such as ``("UlpExceeded", count, max_ulp)``; it is consulted only when the policy is not None."""
    if holes is None:
        raise GridSearchError("NoStrategy")
    variants = enumerate_strategy(holes)
    warnings = []
    if len(variants) > CARTESIAN_WARN_THRESHOLD:
        warnings.append(f"Cartesian product size {len(variants)} exceeds CARTESIAN_WARN_THRESHOLD "
                        f"({CARTESIAN_WARN_THRESHOLD}); grid search may take a long time")
    results = []
    for v in variants:
        if policy.kind != "None" and correctness_fn is not None:
            failure = correctness_fn(v.assignments)
            if failure is not None:
                results.append(VariantResult(v.ordinal, v.variant_id, v.assignments, ("CorrectnessRejected", failure)))
                continue
        try:
            outcome = ("Ok", bench_fn(v.assignments))
        except Exception as exc:  # a failed variant is a result, not the end of the search
            outcome = ("Failed", str(exc))
        results.append(VariantResult(v.ordinal, v.variant_id, v.assignments, outcome))
    ok = sorted((r for r in results if r.outcome[0] == "Ok"), key=lambda r: r.outcome[1].median_ns)
    if not ok:
        for fo in (0, 1, 2, 3):
            for r in results:
                if r.ordinal == fo:
                    return GridSearchResult(r.ordinal, r.variant_id, dict(r.assignments), results, True, warnings)
        raise GridSearchError("NoSuccessfulVariants")
    w = ok[0]
    return GridSearchResult(w.ordinal, w.variant_id, dict(w.assignments), results, False, warnings)


# ------------------------------------------------------------------ the grid_search tool

def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between fp32 arrays (monotone integer mapping)."""
    def key(v):
        i = v.view(np.int32).astype(np.int64)
        return np.where(i < 0, -(i & 0x7FFFFFFF), i)
    return np.abs(key(np.ascontiguousarray(a, np.float32)) - key(np.ascontiguousarray(b, np.float32)))


@dataclass
class GridSearchRequest:
    """mcp/tools/grid_search.rs:206-240 for the Q4 kernels."""
    input_sizes: Sequence[int]
    sample_count: int
    holes: Dict[str, Sequence[int]]
    metadata: Optional[KernelMetadata] = None
    path: Optional[str] = None
    correctness: str = "none"
    workgroup_override: Optional[Sequence[int]] = None
    push_constants_base64: Optional[str] = None
    output_sizes: Optional[Sequence[int]] = None


@dataclass
class RankedVariant:
    ordinal: int
    variant_id: int
    assignments: Dict[str, int]
    median_ns: Optional[int]
    correctness: CorrectnessStatus
    outcome: str
    device_median_ns: Optional[int] = None


@dataclass
class GridSearchResponse:
    winner_variant_id: int
    winner_assignments: Dict[str, int]
    winner_median_ns: int
    ranked: List[RankedVariant]
    machine: MachineMetadata
    fallback_used: bool = False
    warnings: List[str] = field(default_factory=list)
    history_path: Optional[str] = None


def append_history_entry(path: str, entry: dict) -> None:
    """mcp/tools/grid_search.rs:166-200: one JSON line appended under an exclusive flock."""
    line = json.dumps(entry, sort_keys=True)
    assert "\n" not in line
    with open(path, "a", encoding="utf-8") as f:
        fcntl.flock(f.fileno(), fcntl.LOCK_EX)
        f.write(line + "\n")
        f.flush()


def policy_failure(policy: CorrectnessPolicy, got: Optional[bytes], ref: Optional[bytes]) -> Optional[tuple]:
    """The policy applied to a variant's output bytes against those of the ordinal-0 variant, as
    the reference does (grid_search.rs:54-75): ``BitExact`` rejects any differing element with
    ``("BitMismatch", count)``; ``EquivFpTol{ulp}`` rejects elements further than `ulp` units in the
    last place with ``("UlpExceeded", count, max_ulp)``.  None = accepted."""
    if policy.kind == "None":
        return None
    if got is None or ref is None:
        return ("OracleError", "no output to compare")
    if len(got) != len(ref):
        return ("OracleError", f"output length {len(got)} != reference length {len(ref)}")
    a = np.frombuffer(got[:len(got) // 4 * 4], dtype=np.float32)
    b = np.frombuffer(ref[:len(ref) // 4 * 4], dtype=np.float32)
    if policy.kind == "BitExact":
        count = int((a.view(np.uint32) != b.view(np.uint32)).sum())
        return ("BitMismatch", count) if count else None
    d = ulp_distance(a, b)
    d = np.where(np.isnan(a) | np.isnan(b), np.where(a.view(np.uint32) == b.view(np.uint32), 0, 1 << 31), d)
    count = int((d > policy.ulp).sum())
    return ("UlpExceeded", count, int(min(int(d.max()), 0xFFFFFFFF))) if count else None


def grid_search_tool(req: GridSearchRequest, ctx: McpContext) -> GridSearchResponse:
    """Every variant = one ``bench_variant`` with its assignments; ranked by wall-clock median
    like the reference (device medians are reported beside them)."""
    meta = _resolve_metadata(req)
    policy = CorrectnessPolicy.parse(req.correctness)
    responses: Dict[int, BenchVariantResponse] = {}

    first = enumerate_strategy(dict(req.holes))[0].assignments if req.holes else {}
    # a policy that compares variants needs all of them to see the same inputs: those of ordinal 0
    shared_seed = compute_variant_id(first) if policy.kind != "None" else None

    def run(assignments) -> BenchVariantResponse:
        vid = compute_variant_id(assignments)
        if vid not in responses:
            responses[vid] = bench_variant(BenchVariantRequest(
                req.input_sizes, req.sample_count, metadata=meta, assignments=dict(assignments),
                workgroup_override=req.workgroup_override, push_constants_base64=req.push_constants_base64,
                output_sizes=req.output_sizes, input_seed=shared_seed), ctx)
        return responses[vid]

    def bench_fn(assignments) -> SampleStats:
        r = run(assignments)
        return SampleStats(r.median_ns, min(r.samples), max(r.samples), len(r.samples))

    def correctness_fn(assignments):
        r = run(assignments)
        if r.correctness.kind == "Failed":     # wrong against the reference-order kernel: never a winner
            return ("OracleError", r.correctness.reason)
        # the stated policy: this variant's output against the ordinal-0 variant's
        return policy_failure(policy, r.output_bytes, run(first).output_bytes)

    result = grid_search(dict(req.holes), policy, correctness_fn, bench_fn)
    ranked = []
    for r in result.results:
        resp = responses.get(r.variant_id)
        if r.outcome[0] == "Ok":
            ranked.append(RankedVariant(r.ordinal, r.variant_id, r.assignments, r.outcome[1].median_ns,
                                        resp.correctness, "ok", resp.device_median_ns))
        elif r.outcome[0] == "Failed":
            ranked.append(RankedVariant(r.ordinal, r.variant_id, r.assignments, None,
                                        CorrectnessStatus.not_checked("variant did not run"),
                                        f"failed: {r.outcome[1]}"))
        else:
            ranked.append(RankedVariant(r.ordinal, r.variant_id, r.assignments, None,
                                        resp.correctness if resp else CorrectnessStatus.failed(str(r.outcome[1])),
                                        f"correctness_rejected: {r.outcome[1]}"))
    ranked.sort(key=lambda v: (v.median_ns is None, v.median_ns or 0, v.ordinal))
    winner = responses.get(result.winner_variant_id)
    cuda = ctx.cuda.get_or_init()
    out = GridSearchResponse(result.winner_variant_id, result.winner_assignments,
                             winner.median_ns if winner else 0, ranked,
                             build_machine_metadata(cuda, ctx.git_sha), result.fallback_used, result.warnings)
    if ctx.history_dir:
        os.makedirs(ctx.history_dir, exist_ok=True)
        ident = json.dumps([meta.kernel_name, meta.entry_point, meta.binding_plan.to_json_obj()], sort_keys=True)
        key = hashlib.blake2b(ident.encode(), digest_size=8).hexdigest()
        out.history_path = os.path.join(ctx.history_dir, f"{key}.jsonl")
        now = datetime.datetime.now(datetime.timezone.utc)
        append_history_entry(out.history_path, {
            "timestamp": now.strftime("%Y-%m-%dT%H:%M:%S.") + f"{now.microsecond // 1000:03d}Z",
            "git_sha": ctx.git_sha, "source_xxh3": key,
            "grid_search": {
                "winner_variant_id": out.winner_variant_id, "winner_assignments": out.winner_assignments,
                "winner_median_ns": out.winner_median_ns,
                "ranked": [{**{k: v for k, v in asdict(rv).items() if k != "correctness"},
                            "correctness": rv.correctness.to_json_obj()} for rv in ranked],
                "machine": asdict(out.machine)}})
    return out


# ------------------------------------------------------------------ axc optimize

def strategy_sidecar_path(output: str) -> str:
    """crates/axc-driver/src/optimize.rs:114-125: ``out.spv`` -> ``out.spv.axc.strategy.json``."""
    return str(output) + ".axc.strategy.json"


def run_optimize(req: GridSearchRequest, output: str, ctx: McpContext) -> GridSearchResponse:
    """The ``axc optimize`` flow (crates/axc-driver/src/optimize.rs:41-112) with a real bench
    function in place of the reference's fixed 1000 ns mock: grid-search the kernel's launch
    tunables on the device, then write the winner where the reference writes the winning SPIR-V --
    here the tuned kernel's metadata sidecar, since the kernel itself is compiled ahead of time --
    and the search result as ``<output>.axc.strategy.json``."""
    meta = _resolve_metadata(req)
    resp = grid_search_tool(req, ctx)
    meta.save(output)
    record = {
        "winner_variant_id": resp.winner_variant_id,
        "winner_assignments": {"values": resp.winner_assignments},
        "winner_median_ns": resp.winner_median_ns,
        "fallback_used": resp.fallback_used,
        "warnings": resp.warnings,
        "results": [{"ordinal": rv.ordinal, "variant_id": rv.variant_id, "assignments": {"values": rv.assignments},
                     "median_ns": rv.median_ns, "device_median_ns": rv.device_median_ns, "outcome": rv.outcome,
                     "correctness": rv.correctness.to_json_obj()} for rv in sorted(resp.ranked, key=lambda v: v.ordinal)],
        "machine": asdict(resp.machine),
    }
    with open(strategy_sidecar_path(output), "w", encoding="utf-8") as f:
        json.dump(record, f, indent=2, sort_keys=True)
    return resp
