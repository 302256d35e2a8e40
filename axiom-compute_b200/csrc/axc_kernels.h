// Internal launch interface between the C-ABI layer and the sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace axc {

// Fused all-gather epilogue of the streaming matvec (one process per GPU, peer-mapped memory).
struct GatherArgs {
    const uint64_t* y_peer_bases;  // device array [world]: base address of each rank's pair storage
    uint64_t y_offset_bytes;       // this call's vector (8 bytes per global row) inside that storage
    const uint32_t* epoch_ptr;     // this rank's epoch counter
    uint32_t world, rank, row_offset;
    uint64_t parity_stride_bytes = 0;  // odd epochs use a second copy of the storage this far behind the first
};

// End-of-step handshake of the fused all-gather (see gather_finish_kernel).
struct GatherSync {
    const uint64_t* done_peer_bases;  // device array [world]: address of each rank's uint32 done[world]
    const uint32_t* done_local;       // this rank's own done[world]
    uint32_t* arrive_counter;         // device uint32, zero before first use
    uint32_t* epoch_rw;               // the epoch counter (advanced by the finish kernel)
    uint32_t world, rank;
};

// Where the streaming matvec takes its activations from when they are not one plain vector:
// x = a [+ b]; a and b are each a plain fp32 vector or a vector of (value, epoch) words written by
// the all-gather epilogue of an earlier call (the reader polls, bounded, until the epoch read
// from `epoch_ptr` has arrived); unit_rms divides x by sqrt(mean(x^2)).
struct XSource {
    const float* x = nullptr;
    const float* x2 = nullptr;
    const uint64_t* x_pairs = nullptr;
    const uint64_t* x2_pairs = nullptr;
    const uint32_t* epoch_ptr = nullptr;
    int unit_rms = 0;
    uint64_t parity_stride_bytes = 0;  // (value, epoch) sources: second copy for odd epochs
};

// Completion signal of the streaming matvec for a host that polls a word in mapped host memory
// instead of waiting on an event: the last CTA to finish writes `seq` to `flag` once y is visible
// to the host.  `counter` is one device word, zero before first use.
struct DoneSignal {
    uint32_t* counter;
    uint32_t* flag;
    uint32_t seq;
    float* y_host;   // optional: y is device memory; the last CTA copies it here (mapped host memory) before `flag`
};

// Single-launch host dispatch: x lies in mapped host memory; the launch's first CTAs quantise it
// into the image named by MatvecTuning::x_prepared and publish `seq` in `ready` (device words,
// zero before first use), which all CTAs wait for (bounded) before reading the image.
struct HostX {
    const float* x_host;   // device view of the mapped host buffer
    uint32_t* ready;
    uint32_t* counter;
    uint32_t seq;
};

// Tunables of the streaming matvec kernels.  0 = let the launcher choose.
struct MatvecTuning {
    int ctas_per_sm = 0;  // resident CTAs per SM the grid is sized for
    int tile_rows = 0;    // rows per shared-memory stage
    int stages = 0;       // stages in the ring
    int threads = 0;      // threads per CTA (Q4_0 only; Q4_K derives it from the row length)
    int evict_first = -1; // L2 evict-first hint on the weight stream (-1 = default)
    int pdl = -1;         // programmatic dependent launch: 0 off, 1 on, 2 on + weights before the wait (-1 = default)
    int resident = 0;     // CTAs per SM the shared-memory budget is cut for (0 = default)
    int dry_run = 0;      // compute the launch geometry only, launch nothing
    const void* x_prepared = nullptr;  // activations already quantised by a prepare kernel
    int x_prepared_rms = 0;            // with x_prepared: scale y by 1 / sqrt(mean(x^2))
    const GatherArgs* gather = nullptr;  // all-gather fused into the epilogue (y is ignored)
    const XSource* xsrc = nullptr;       // fused activation source (Q4_K_M only; x is ignored)
    const DoneSignal* done = nullptr;    // completion signal for a polling host (streaming kernels only)
    const HostX* host_x = nullptr;       // with x_prepared: the launch produces the image itself from host memory
};

// True when launch_q4k_matvec / launch_q4_0_matvec take the streaming kernel for this row length
// (the kernel that supports x_prepared, gather, xsrc and done).
inline bool q4k_uses_stream_kernel(uint32_t n_sb) { return n_sb >= 1 && n_sb <= 128; }
inline bool q4_0_uses_stream_kernel(uint32_t n_blocks) { return n_blocks >= 2 && !(n_blocks & 1u) && n_blocks <= 1024u; }

struct LaunchInfo {
    int grid = 0, block = 0;
    size_t smem = 0;
    int tile_rows = 0, stages = 0, seg = 0, n_seg = 0;
};

// y[r] = dot(dequant(q row r), x) for r < rows; row r starts at q + r * n_sb * 144.
// `status` is a device word that receives error bits (may be null).
cudaError_t launch_q4k_matvec(const uint8_t* q, const float* x, float* y, uint32_t rows,
                              uint32_t n_sb, uint32_t* status, cudaStream_t stream,
                              const MatvecTuning& tune, int sm_count, LaunchInfo* info);
// Same results as the reference's sequential fp32 loop, bit for bit (one thread per row).
cudaError_t launch_q4k_matvec_seq(const uint8_t* q, const float* x, float* y, uint32_t rows,
                                  uint32_t n_sb, cudaStream_t stream);
// w[r][i] = bit-exact dequantised weight i of row r (x-index order).
cudaError_t launch_q4k_dequant(const uint8_t* q, float* w, uint32_t rows, uint32_t n_sb,
                               cudaStream_t stream);

// C[m][n] = sum_k A[m][k] * bf16(W[n][k]) on the tensor cores (tcgen05): A [m_tokens][n_sb * 256]
// bf16, W [n_rows][n_sb] Q4_K_M superblocks, C [m_tokens][n_rows] fp32.
cudaError_t launch_q4k_prefill(const uint8_t* q, const uint16_t* a_bf16, float* c, uint32_t m_tokens,
                               uint32_t n_rows, uint32_t n_sb, uint32_t* status, cudaStream_t stream,
                               int form = 0 /* 0 choose, 1 single CTA per tile, 2 CTA pair */,
                               bool independent = false /* inputs / C untouched by the launch before */);

cudaError_t launch_gather_finish(const uint64_t* pairs, const uint32_t* epoch_ptr, float* out, uint32_t n,
                                 uint32_t* status, cudaStream_t stream, bool overlap, uint64_t parity_stride = 0,
                                 const GatherSync* sync = nullptr, bool let_next_start = false);
cudaError_t launch_gather_next_epoch(uint32_t* epoch_ptr, cudaStream_t stream);
// out[i] = sum over parts r < n_parts of the value of word pairs[r * part_stride / 8 + i] (K-sharded linears).
cudaError_t launch_gather_reduce_finish(const uint64_t* pairs, const uint32_t* epoch_ptr, float* out, uint32_t n,
                                        uint32_t n_parts, uint64_t part_stride, uint32_t* status, cudaStream_t stream,
                                        bool overlap, uint64_t parity_stride);

// Quantised form of x for `n_pos` 64-column positions (see q4_stream.cu): bytes needed and the
// kernel that fills them; a matvec launched with tuning.x_prepared set reads it instead of x.
size_t q4_prepared_x_bytes(uint32_t n_pos);
cudaError_t preload_q4k_prepared_path();   // load those kernels on the current device, launch nothing
cudaError_t launch_q4_quantize_x(const float* x, void* out, uint32_t n_pos, cudaStream_t stream);
// The same from a fused source, one CTA per 64 positions, with the per-group sums of x^2 behind
// the image (for the unit-RMS scale) and optionally x written out as a plain vector.
cudaError_t launch_q4_prepare_x(const XSource& src, void* image, float* plain_out, uint32_t n_pos, uint32_t* status,
                                cudaStream_t stream, bool overlap);

cudaError_t launch_q4_0_matvec(const uint8_t* q, const float* x, float* y, uint32_t rows,
                               uint32_t n_blocks, uint32_t* status, cudaStream_t stream,
                               const MatvecTuning& tune, int sm_count, LaunchInfo* info);
cudaError_t launch_q4_0_matvec_seq(const uint8_t* q, const float* x, float* y, uint32_t rows,
                                   uint32_t n_blocks, cudaStream_t stream);
cudaError_t launch_q4_0_dequant(const uint8_t* q, float* w, uint32_t rows, uint32_t n_blocks,
                                cudaStream_t stream);

}  // namespace axc
