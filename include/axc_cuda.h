/*
 * axc_cuda.h -- C ABI of libaxc_cuda.so, the B200 (sm_100a) backend for AXIOM-Compute's
 * quantised dequant-matvec path.
 *
 * Two layers:
 *   1. A runtime layer that mirrors axc-runtime's context / kernel-handle / dispatch API one
 *      to one (host buffers in, host buffers out, typed error codes), so a Rust `cuda`
 *      backend module can implement VulkanContext's method set by calling it.
 *   2. A device layer that launches the kernels on caller-owned device memory and a caller's
 *      stream, for callers that keep weights and activations resident (decode loops,
 *      multi-GPU drivers, benchmarks).
 *
 * Conventions: every function returning `int` returns an axc_status (0 = AXC_OK).  No C++
 * exception crosses this boundary.  After a non-zero status, axc_cuda_last_error_detail()
 * gives a thread-local, human-readable detail string and axc_cuda_last_error_fields() the
 * typed fields of the matching DispatchError variant.  All functions are thread-safe;
 * dispatches on one kernel handle serialise on a per-handle mutex, different handles may run
 * concurrently (crates/axc-runtime/src/context.rs:494-497).
 *
 * Paths cited below are relative to the AXIOM-Compute repository.
 */
#ifndef AXC_CUDA_H
#define AXC_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* One code per DispatchError variant that this backend can raise
 * (crates/axc-runtime/src/error.rs:27-195), plus AXC_ERR_INVALID_ARGUMENT for a null or
 * malformed argument at the C boundary itself (unrepresentable in the Rust API). */
typedef enum axc_status {
    AXC_OK = 0,
    AXC_ERR_NO_SUPPORTED_DEVICE = 3,              /* NoSupportedDevice */
    AXC_ERR_DEVICE_CREATION_FAILED = 5,           /* DeviceCreationFailed(String) */
    AXC_ERR_PIPELINE_CREATION_FAILED = 10,        /* PipelineCreationFailed(String) */
    AXC_ERR_BUFFER_ALLOCATION_FAILED = 11,        /* BufferAllocationFailed{binding,size,reason} */
    AXC_ERR_QUEUE_SUBMIT_FAILED = 15,             /* QueueSubmitFailed(String) */
    AXC_ERR_FENCE_TIMEOUT = 16,                   /* FenceTimeout{timeout_ns} */
    AXC_ERR_READBACK_FAILED = 17,                 /* ReadbackFailed{binding,reason} */
    AXC_ERR_BINDING_COUNT_MISMATCH = 18,          /* BindingCountMismatch{expected,provided} */
    AXC_ERR_PUSH_CONSTANT_SIZE_MISMATCH = 19,     /* PushConstantSizeMismatch{expected,provided} */
    AXC_ERR_WORKGROUP_COUNT_EXCEEDS_LIMIT = 20,   /* WorkgroupCountExceedsDeviceLimit{requested,max} */
    AXC_ERR_STAGING_COPY_FAILED = 25,             /* StagingCopyFailed{binding,direction,reason} */
    AXC_ERR_INVALID_ARGUMENT = 100
} axc_status;

/* CopyDirection (crates/axc-runtime/src/error.rs:14-20). */
enum { AXC_COPY_HOST_TO_DEVICE = 0, AXC_COPY_DEVICE_TO_HOST = 1 };

/* Typed payload of the last error on this thread (fields unused by a variant are zero). */
typedef struct axc_error_fields {
    uint32_t binding;
    uint32_t direction;      /* AXC_COPY_* */
    uint64_t size;
    uint64_t expected;
    uint64_t provided;
    uint64_t timeout_ns;
    uint32_t requested[3];
    uint32_t max[3];
} axc_error_fields;

typedef struct axc_ctx axc_ctx;       /* <-> VulkanContext  (context.rs:160-373) */
typedef struct axc_kernel axc_kernel; /* <-> KernelHandle   (kernel_handle.rs:44-151) */

/* <-> VulkanContextOptions (context.rs:76-109). */
typedef struct axc_ctx_opts {
    int32_t physical_device_index; /* CUDA ordinal; -1 = AXC_PHYSICAL_DEVICE_INDEX or 0 */
    uint64_t fence_timeout_ms;     /* 0 = AXC_FENCE_TIMEOUT_MS, read per dispatch, else 10 000 */
    const char* pipeline_cache_path; /* accepted and ignored: kernels are compiled ahead of time */
} axc_ctx_opts;

/* Element type / access of one buffer binding (axc-hir ScalarTy / BufferAccess,
 * crates/axc-hir/src/ty.rs:13-26, crates/axc-hir/src/buffer.rs:16-49). */
enum { AXC_TY_U8 = 1, AXC_TY_F32 = 2, AXC_TY_U32 = 3, AXC_TY_OTHER = 0 };
enum { AXC_ACCESS_READ_ONLY = 1, AXC_ACCESS_READ_WRITE = 2, AXC_ACCESS_WRITE_ONLY = 3 };

/* One BufferBindingSlot of the ParamBindingPlan (crates/axc-hir/src/param.rs:66-78). */
typedef struct axc_buf_desc {
    uint32_t elem_ty;          /* AXC_TY_* */
    uint32_t access;           /* AXC_ACCESS_* */
    uint32_t buffer_position;  /* = descriptor binding index */
    uint32_t position;         /* position in the kernel's parameter list */
} axc_buf_desc;

/* Device-side timing of one dispatch (CUDA events on the context's stream). */
typedef struct axc_dispatch_stats {
    uint64_t h2d_ns;
    uint64_t kernel_ns;
    uint64_t d2h_ns;
    uint64_t total_device_ns;
    uint32_t rows_effective;   /* rows actually computed after clamping to the buffer sizes */
    uint32_t blocks_per_row;   /* push constant n_superblocks / n_blocks */
} axc_dispatch_stats;

/* ---- availability (crates/axc-runtime/src/icd.rs:22-80) ---- */

/* <-> probe_vulkan_available(): 1 if at least one compute-capability-10.x device exists. */
int axc_cuda_probe(void);
/* <-> gpu_tests_enabled(): 1 iff AXC_ENABLE_GPU_TESTS == "1". */
int axc_cuda_gpu_tests_enabled(void);
/* Number of CUDA devices (0 when the driver is absent). */
int axc_cuda_device_count(void);

/* ---- context (context.rs:160-373, 569-625) ---- */

/* <-> VulkanContext::new_with_options; opts == NULL <-> VulkanContext::new() (from_env). */
int axc_cuda_ctx_create(const axc_ctx_opts* opts, axc_ctx** out);
/* <-> Drop for VulkanContext: waits for the device to go idle, then releases.  Kernel
 * handles stay valid afterwards (kernel_handle_outlives_context, AT-827). */
void axc_cuda_ctx_destroy(axc_ctx* ctx);
/* <-> physical_device_name(): NUL-terminated copy into buf; returns the full length. */
size_t axc_cuda_ctx_device_name(const axc_ctx* ctx, char* buf, size_t cap);
/* <-> max_compute_work_group_count(). */
void axc_cuda_ctx_max_grid(const axc_ctx* ctx, uint32_t out[3]);
int axc_cuda_ctx_device_index(const axc_ctx* ctx);
int axc_cuda_ctx_sm_count(const axc_ctx* ctx);

/* ---- kernel handles (context.rs:392-486, kernel_handle.rs:44-151,216-246) ---- */

/* <-> prepare_kernel(spirv, plan, pc_total, entry_point).  The SPIR-V is not consumed; its
 * xxh3 hash and the plan's hash form the cache key with pc_total_bytes, exactly as in
 * make_cache_key.  Two calls with the same key while the first handle is alive return the
 * same object with one more reference.  entry_point selects the kernel:
 * "q4km_dequant_matvec" or "q4_0_dequant_matvec" with buffers [U8 RO, F32 RO, F32 RW] and a
 * 4-byte push-constant block; anything else is AXC_ERR_PIPELINE_CREATION_FAILED. */
int axc_cuda_prepare_kernel(axc_ctx* ctx, const char* entry_point, const axc_buf_desc* bufs,
                            uint32_t n_bufs, uint32_t pc_total_bytes, uint64_t spirv_hash,
                            uint64_t plan_hash, axc_kernel** out);
void axc_cuda_kernel_retain(axc_kernel* k);   /* <-> KernelHandle::clone */
void axc_cuda_kernel_release(axc_kernel* k);  /* <-> Drop for KernelHandle */
/* <-> KernelHandle::buffer_sizes(): device size of each allocated binding slot; returns the
 * number of slots (may exceed cap; only cap entries are written). */
uint32_t axc_cuda_kernel_buffer_sizes(const axc_kernel* k, uint64_t* out, uint32_t cap);
/* <-> KernelHandle::cache_key(): (spirv_hash, plan_hash, pc bytes). */
void axc_cuda_kernel_cache_key(const axc_kernel* k, uint64_t* spirv_hash, uint64_t* plan_hash,
                               uint32_t* pc_total_bytes);
/* Strict mode: when non-zero the handle runs the reference-order kernel whose y is
 * bit-identical to the CPU reference (one thread per row; slow).  Default 0. */
void axc_cuda_kernel_set_strict_order(axc_kernel* k, int strict);
/* Launch tunables the handle's later dispatches use (struct axc_tuning below; NULL = defaults).
 * This is what a grid search over the kernel's tunables sets per variant: the reference's
 * `assignments` of strategy holes (crates/axc-optimize/src/enumerator.rs:44-61) select a
 * compiled variant, here they select launch geometry of the one ahead-of-time kernel.  A
 * combination the launcher cannot realise makes the dispatch return QueueSubmitFailed. */
struct axc_tuning;
void axc_cuda_kernel_set_tuning(axc_kernel* k, const struct axc_tuning* tuning);

/* ---- dispatch (context.rs:498-547, kernel_handle.rs:295-393,410-738, dispatch.rs:56-132) ----
 *
 * <-> dispatch_handle(handle, workgroups, inputs, output_sizes, push_constants).
 *   inputs[i] / input_lens[i]: host bytes for binding i; length 0 skips the upload and the
 *     device buffer keeps its contents (resident weights).
 *   outputs[i] / output_sizes[i]: caller-allocated host buffers; size 0 skips the readback
 *     (outputs[i] may then be NULL).  The Rust side wraps them into Vec<Vec<u8>>.
 *   Validation order, before any allocation: n_inputs, n_outputs, pc_len, workgroup limits.
 *   Device buffers grow to round_up_pow2(max(in, out, 4)) and never shrink.
 *   Rows come from the grid: rows = workgroups[0]; the push constant keeps its reference
 *   meaning (n_superblocks / n_blocks PER ROW).  rows is clamped to what the q and y buffers
 *   hold; workgroups = [1,1,1] is exactly the reference's single-output behaviour, and
 *   n = 0 writes y[0] = +0.0.
 *   The wait for completion is bounded by the fence timeout -> AXC_ERR_FENCE_TIMEOUT.
 *   Two ways through a dispatch, with the same results.  With stats == NULL, resident or freshly given
 *   inputs, at least 64 rows, no input binding read back and a row length the streaming kernel serves
 *   (Q4_K_M up to 128 superblocks, Q4_0 an even number of blocks up to 1024), a dispatch is ONE kernel
 *   launch: x is read from its pinned, device-mapped staging buffer by the kernel's first CTAs, y is copied
 *   into mapped host memory by its last CTA, and completion is a sequence number polled in mapped host
 *   memory (no copy-engine transfer, no event).  Otherwise (device timing asked for, strict handles, other
 *   shapes, or AXC_DISPATCH_FAST=0 in the environment) inputs go through cudaMemcpyAsync and completion
 *   through a CUDA event.
 */
int axc_cuda_dispatch(axc_ctx* ctx, axc_kernel* k, const uint32_t workgroups[3],
                      const void* const* inputs, const size_t* input_lens, uint32_t n_inputs,
                      void* const* outputs, const size_t* output_sizes, uint32_t n_outputs,
                      const void* push_constants, size_t pc_len, axc_dispatch_stats* stats);

/* <-> VulkanContext::dispatch(DispatchRequest) (dispatch.rs:109-132): validate, prepare,
 * dispatch once, release. */
int axc_cuda_dispatch_oneshot(axc_ctx* ctx, const char* entry_point, const axc_buf_desc* bufs,
                              uint32_t n_bufs, uint32_t pc_total_bytes, uint64_t spirv_hash,
                              uint64_t plan_hash, const uint32_t workgroups[3],
                              const void* const* inputs, const size_t* input_lens,
                              uint32_t n_inputs, void* const* outputs, const size_t* output_sizes,
                              uint32_t n_outputs, const void* push_constants, size_t pc_len,
                              axc_dispatch_stats* stats);

/* <-> the timing loop of bench_variant (crates/axc-driver/src/mcp/tools/bench_variant.rs:
 * 284-301): sample_count wall-clock timed dispatch_handle calls; samples_ns receives each
 * sample, *median_ns = sorted[len/2].  device_kernel_ns (nullable) receives the per-sample
 * device time of the kernel alone. */
int axc_cuda_bench_dispatch(axc_ctx* ctx, axc_kernel* k, const uint32_t workgroups[3],
                            const void* const* inputs, const size_t* input_lens, uint32_t n_inputs,
                            void* const* outputs, const size_t* output_sizes, uint32_t n_outputs,
                            const void* push_constants, size_t pc_len, uint32_t sample_count,
                            uint64_t* samples_ns, uint64_t* median_ns, uint64_t* device_kernel_ns);

/* ---- errors (error.rs) ---- */
const char* axc_cuda_strerror(int status);
size_t axc_cuda_last_error_detail(char* buf, size_t cap);
void axc_cuda_last_error_fields(axc_error_fields* out);

/* ---- device layer: kernels on caller-owned device memory ----
 *
 * q, x, y are device pointers (16-byte aligned), stream is a cudaStream_t (NULL = default
 * stream), status is an optional device uint32 that receives kernel error bits.  These are
 * the same kernels axc_cuda_dispatch launches for examples/q4km_dequant_matvec.axc and
 * examples/q4_0_dequant_matvec.axc, generalised from one row to `rows` rows.
 */
typedef struct axc_tuning {
    int32_t ctas_per_sm; /* 0 = default */
    int32_t tile_rows;
    int32_t stages;
    int32_t threads;
    int32_t evict_first; /* -1 = default */
    int32_t pdl;         /* programmatic dependent launch: 0 off, 1 on, 2 on with the weight
                            stream started before the dependency wait (default: an ORDERED
                            launch, which lets the launch behind it be scheduled only after its
                            own wait, i.e. once everything before it in the stream is complete),
                            3 = an INDEPENDENT launch: the caller asserts that x is not written,
                            and y neither read nor written, by any launch of this stream that may
                            still be in flight, which is every launch from the most recent ordered
                            one (inclusive; any kernel not of this library counts as ordered) up
                            to this call.  Only the final store of y waits for the launch before,
                            and the launch is shaped for a RUN of such launches (one small CTA on
                            every second SM, up to four launches resident per SM): a lone
                            independent launch uses half the machine.  Example: producer of x, then
                            the matrices that consume it, the first with pdl 2, the others with
                            pdl 3. */
    int32_t resident;    /* CTAs per SM the shared-memory budget is cut for; 0 = default */
} axc_tuning;

int axc_cuda_q4k_matvec(const void* q, const float* x, float* y, uint32_t rows,
                        uint32_t n_superblocks, void* stream, uint32_t* status,
                        const axc_tuning* tuning);
int axc_cuda_q4_0_matvec(const void* q, const float* x, float* y, uint32_t rows,
                         uint32_t n_blocks, void* stream, uint32_t* status,
                         const axc_tuning* tuning);
/* Reference-order variants: y bit-identical to q4km_dequant_matvec_cpu /
 * q4_0_dequant_matvec_cpu (common_helpers.rs:411-461, benches/common.rs:212-259). */
int axc_cuda_q4k_matvec_seq(const void* q, const float* x, float* y, uint32_t rows,
                            uint32_t n_superblocks, void* stream);
int axc_cuda_q4_0_matvec_seq(const void* q, const float* x, float* y, uint32_t rows,
                             uint32_t n_blocks, void* stream);
/* Dequantised weights, bit-identical to the reference's per-element values, shape
 * [rows][n * 256] (Q4_K_M) or [rows][n * 32] (Q4_0) in x-index order. */
int axc_cuda_q4k_dequant(const void* q, float* w, uint32_t rows, uint32_t n_superblocks,
                         void* stream);
int axc_cuda_q4_0_dequant(const void* q, float* w, uint32_t rows, uint32_t n_blocks,
                          void* stream);
/* Row-sharded matvec with the all-gather of y fused into the kernel (one process per GPU).
 * The reference has no multi-GPU path; this is the exchange step of sharding its rows over the
 * GPUs of one node.  Every rank computes `rows_local` rows and stores them at
 * [row_offset, row_offset + rows_local) of EVERY rank's full-length vector through peer-mapped
 * memory (plain stores over NVLink).  A vector is stored as one 8-byte word per global row:
 * the fp32 value in the low half, the epoch of the step in the high half, written by a single
 * store, so a reader that finds the epoch has the value.  The producer needs no fence, no flag
 * and never waits.  Before anything reads an assembled vector, axc_cuda_gather_finish must run
 * in the same stream: it waits (bounded to about two seconds per missing word, after which bit 4
 * of *status is set) until every word carries the current epoch and writes the values out as a
 * plain fp32 vector, so the exchange latency overlaps with the calls in between.
 *   y_peer_bases: DEVICE array of `world` addresses (this process's mappings of each rank's
 *     pair storage; entry `rank` is the local buffer; the storage is zero before first use);
 *   y_offset_bytes: where this call's vector (8 bytes per global row) starts in that storage;
 *   epoch: this rank's epoch counter (one device uint32, zero before first use), advanced by
 *     axc_cuda_gather_next_epoch once per step (one step = one pass over the vectors in use).
 * All ranks issue the same sequence of calls.  A vector may be rewritten only once every rank has
 * finished the step that read it.  Nothing in the producer waits for that, so a caller whose ranks
 * can drift apart by a step keeps TWO copies of the storage, parity_stride_bytes apart (0 = one
 * copy): every kernel of this family then uses the copy selected by the low bit of the epoch it
 * read, and the end-of-step handshake of axc_cuda_gather_finish (axc_gather_sync) keeps any rank
 * from starting step e + 2 before every rank has consumed step e.  A reader that meets a word
 * from a LATER epoch than its own sets bit 8 of *status instead of accepting it. */
typedef struct axc_gather {
    const uint64_t* y_peer_bases;
    uint64_t y_offset_bytes;
    const uint32_t* epoch;
    uint32_t world, rank, row_offset;
    uint64_t parity_stride_bytes;
} axc_gather;
int axc_cuda_q4k_matvec_allgather(const void* q, const float* x, uint32_t rows_local,
                                  uint32_t n_superblocks, const axc_gather* g, void* stream,
                                  uint32_t* status, const axc_tuning* tuning);
/* Batched prefill (M > 1), the one place where the path is a dense contraction and runs on the
 * tensor cores (tcgen05, accumulators in tensor memory):
 *   C[m][n] = sum_k A[m][k] * bf16(W[n][k]),  fp32 accumulate,
 * A = m_tokens x (n_superblocks * 256) bf16 (row-major, as uint16 bit patterns), W = n_rows rows
 * of n_superblocks Q4_K_M superblocks (the matvec's q layout), C = m_tokens x n_rows fp32
 * row-major.  bf16(W) is the reference's fp32 dequantised weight (same operations and rounding
 * points as examples/q4km_dequant_matvec.axc:91-112) rounded to nearest even.  All pointers are
 * 16-byte aligned device memory.  The reference has no M > 1 kernel; the comparison is its CPU
 * dequantisation followed by a GEMM (tolerance 1e-2 relative).  *status receives bit 0 if a
 * bounded wait inside the kernel ran out. */
int axc_cuda_q4k_prefill(const void* q, const uint16_t* a_bf16, float* c, uint32_t m_tokens,
                         uint32_t n_rows, uint32_t n_superblocks, void* stream, uint32_t* status);
/* The same with the kernel form chosen by the caller: 0 = the library's choice, 1 = one CTA per
 * 128-row tile (tcgen05.mma.cta_group::1), 2 = a pair of CTAs per 256 rows (cta_group::2).
 * flags: AXC_PREFILL_INDEPENDENT = the caller states that q and a are not written, and c not read
 * or written, by any launch of the stream from the most recent one made without this flag
 * (inclusive) up to this call (say the up projection right after the gate projection of the same
 * activations): the call may then start on SMs the previous call leaves idle; only its stores of
 * c wait.  A call without the flag lets the next launch be scheduled only after its own wait. */
#define AXC_PREFILL_INDEPENDENT 1u
int axc_cuda_q4k_prefill_form(const void* q, const uint16_t* a_bf16, float* c, uint32_t m_tokens,
                              uint32_t n_rows, uint32_t n_superblocks, void* stream, uint32_t* status, int form,
                              uint32_t flags);

/* Q4_K_M matvec whose activations are assembled inside the kernel: x = a [+ b], where a and b
 * are each a plain fp32 vector (x, x2) or a vector of (value, epoch) words that the all-gather
 * epilogue of an earlier call wrote (x_pairs, x2_pairs: the kernel itself polls, bounded, until
 * every word carries the epoch read from `epoch`, so no separate finish launch is needed
 * between dependent calls); with unit_rms != 0 the result is the matvec of x / sqrt(mean(x^2))
 * (fp32).  y receives the rows when g is NULL; with g the rows go into every rank's vector as
 * for axc_cuda_q4k_matvec_allgather.  No counterpart in the reference (it has neither a
 * multi-GPU path nor a model); this is the linear layer of the 70B-shaped decode sweep. */
#define AXC_FINISH_OVERLAP_PREVIOUS 1u
#define AXC_FINISH_LET_NEXT_START 2u
typedef struct axc_xsrc {
    const float* x;
    const float* x2;
    const uint64_t* x_pairs;
    const uint64_t* x2_pairs;
    const uint32_t* epoch;
    uint32_t unit_rms;
    uint64_t parity_stride_bytes; /* (value, epoch) sources: distance of the odd-epoch copy, 0 = one copy */
} axc_xsrc;
int axc_cuda_q4k_matvec_fused(const void* q, const axc_xsrc* xs, float* y, uint32_t rows,
                              uint32_t n_superblocks, const axc_gather* g, void* stream,
                              uint32_t* status, const axc_tuning* tuning);
/* The same work split in two launches, for vectors that many CTAs consume: prepare_x assembles
 * x = a [+ b] once (one CTA per 64 x 64 columns), quantises it to the digit-word image the matvec
 * kernels otherwise build per CTA in shared memory, stores the per-group sums of x^2 behind it and
 * optionally writes x out as a plain fp32 vector (plain_out may be NULL); matvec_prepared then
 * reads its digit words straight into registers (no staging, no CTA-wide barrier) and, with
 * unit_rms != 0, scales by 1 / sqrt(mean(x^2)).  image: axc_cuda_q4k_prepared_x_bytes(n) bytes of
 * 16-byte aligned device memory.  flags: AXC_FINISH_OVERLAP_PREVIOUS (epoch-word sources only)
 * lets prepare_x start before the launch directly before it has completed.  matvec_prepared
 * must directly follow the prepare_x of its image in the same stream, or a launch that does not
 * write the image.  No counterpart in the reference. */
size_t axc_cuda_q4k_prepared_x_bytes(uint32_t n_superblocks);
int axc_cuda_q4k_prepare_x(const axc_xsrc* xs, void* image, float* plain_out, uint32_t n_superblocks,
                           void* stream, uint32_t* status, uint32_t flags);
int axc_cuda_q4k_matvec_prepared(const void* q, const void* image, uint32_t unit_rms, float* y, uint32_t rows,
                                 uint32_t n_superblocks, const axc_gather* g, void* stream, uint32_t* status,
                                 const axc_tuning* tuning);
/* *epoch += 1, in stream order (a one-thread kernel). */
int axc_cuda_gather_next_epoch(uint32_t* epoch, void* stream);
/* Consumer side: pairs = this rank's own pair storage (n words; the copy for odd epochs
 * parity_stride_bytes further on when that is non-zero), out = n fp32 values.
 * flags: AXC_FINISH_OVERLAP_PREVIOUS lets the kernel start before the launch directly before it
 * in the stream has completed (it polls for that launch's words anyway); the caller guarantees
 * that launch neither advances the epoch nor reads or writes `out`.
 * AXC_FINISH_LET_NEXT_START (axc_cuda_gather_finish only) keeps the wait for the launch before it
 * but lets the launches BEHIND it be scheduled at once, as an independent matvec launch
 * (tuning.pdl = 3) does: the caller states that those launches, up to the next ordered one, read
 * neither `out` nor anything else a launch still in flight writes before their own dependency
 * wait.  The matvec launches of the next step then stream their weights while this launch waits for
 * the step's words, and a stream (or a CUDA graph) of several steps never drains at the end of a
 * step; their stores still wait for this launch, and so for the epoch it advances.  Without the
 * flag the launch is ordered: nothing behind it starts before everything before it is complete.
 * sync (nullable): the end-of-step handshake for callers whose ranks are not kept in step by the
 * data they exchange.  The last CTA of the launch stores the epoch it consumed into entry `rank`
 * of every rank's done array (a peer store), waits (bounded, then bit 4 of *status) until its own
 * done array shows that every rank has consumed the epoch before, and only then advances *epoch
 * itself: the caller issues no axc_cuda_gather_next_epoch.  With two copies of the storage this
 * makes the reuse of a copy two steps later safe.  The epoch counter starts at 1 for this
 * protocol; done arrays and arrive_counter are zero before first use.  n may be 0 (handshake only). */
typedef struct axc_gather_sync {
    const uint64_t* done_peer_bases; /* DEVICE array of `world` addresses: each rank's uint32 done[world] */
    const uint32_t* done_local;      /* this rank's own done[world] */
    uint32_t* arrive_counter;        /* one device uint32 of scratch */
    uint32_t* epoch;                 /* the epoch counter, read and advanced */
    uint32_t world, rank;
} axc_gather_sync;
int axc_cuda_gather_finish(const uint64_t* pairs, const uint32_t* epoch, float* out, uint32_t n,
                           void* stream, uint32_t* status, uint32_t flags, uint64_t parity_stride_bytes,
                           const axc_gather_sync* sync);

/* Consumer side of a linear sharded by COLUMNS (K) instead of rows: rank r multiplies its column
 * range of every row with its slice of x and stores the full-length vector of partial sums into
 * part r of every rank's pair storage (axc_cuda_q4k_matvec_fused with an axc_gather whose
 * row_offset is 0 and whose y_offset_bytes selects part r: parts lie part_stride_bytes apart).
 * This call waits (bounded, as axc_cuda_gather_finish) until all n_parts words of each of the n
 * elements carry the current epoch and writes their sum, taken in part order on every rank so
 * that all ranks obtain the same bits, to out as plain fp32.  flags and parity_stride_bytes as for
 * axc_cuda_gather_finish.  No counterpart in the reference. */
int axc_cuda_gather_reduce_finish(const uint64_t* pairs, const uint32_t* epoch, float* out, uint32_t n,
                                  uint32_t n_parts, uint64_t part_stride_bytes, void* stream, uint32_t* status,
                                  uint32_t flags, uint64_t parity_stride_bytes);

/* Launch geometry the matvec launchers would use (no launch). */
int axc_cuda_q4k_matvec_plan(uint32_t rows, uint32_t n_superblocks, const axc_tuning* tuning,
                             int32_t sm_count, int32_t out_grid_block_smem_tile_stages[5]);

/* Q4_K_M matvec that allocates nothing.  It has no counterpart in the reference; it exists for
 * callers that may not create device memory when they need a matvec: a plug-in inside a host
 * program that owns the GPU's memory pool and bans driver allocations after start-up, or a
 * latency-critical decode thread that must avoid cudaMalloc / cudaFree because they synchronise
 * the device.  q, x, y are the caller's 16-byte aligned device pointers as for
 * axc_cuda_q4k_matvec; the quantised form of x that the kernel consumes is kept in a fixed
 * 139 520-byte array inside the library (held by every GPU that loads the library until the
 * process exits).  Limit: n_superblocks <= AXC_STATIC_MAX_SUPERBLOCKS (K <= 32768); longer rows
 * return AXC_ERR_BUFFER_ALLOCATION_FAILED, nothing is launched.  The first call on each device
 * looks up the array's device address (cudaGetSymbolAddress) and should therefore be made with
 * that device current and before any stream capture begins.  All calls on a device share the
 * one array: calls whose kernels could overlap on the GPU (different streams) race on it and
 * must be ordered by the caller; calls in one stream are safe, each call rewrites every word it
 * later reads.  The entry point itself calls no cudaMalloc, cudaFree or allocating library
 * routine; but the CUDA runtime loads a kernel (and the module that holds the array) the first
 * time it is used on a device, and that load may allocate device memory and synchronise.  Call
 * axc_cuda_q4k_matvec_static_warmup() once per device at start-up, with that device current and
 * outside any stream capture: it looks up the array and loads every kernel this entry point can
 * launch (the quantiser and the three tile heights of the matvec) without launching anything, so
 * that later calls of any shape find everything resident. */
#define AXC_STATIC_MAX_SUPERBLOCKS 128
int axc_cuda_q4k_matvec_static_warmup(void);
int axc_cuda_q4k_matvec_static(const void* q, const float* x, float* y, uint32_t rows,
                               uint32_t n_superblocks, void* stream);

/* Library version: major * 10000 + minor * 100 + patch. */
int axc_cuda_version(void);

#ifdef __cplusplus
}
#endif
#endif /* AXC_CUDA_H */
