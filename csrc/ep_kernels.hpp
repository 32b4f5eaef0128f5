// Parameter blocks and launch entry points of the dispatch/combine kernels (torch-free).
//
// Every kernel exists as one device body with two __global__ wrappers: the production wrapper
// takes the parameter block by value for one rank; the multi-rank wrapper reads the block of
// logical rank blockIdx.y from a device array, so a whole group can run as ONE launch on one GPU
// (ranks that wait on one another must never be separate launches on the same device).
//
// Protocol (differs from the reference's push + epilogue design, csrc/dispatch_main.cuh:356-453):
//   dispatch = stage (copy tokens into the own window, count, exchange counts, peer barrier)
//              -> plan (fresh only: receivers scan the sources' routing and assign rows/slots)
//              -> pull (receivers bulk-load rows from the sources' windows straight into the
//                 final compact / expert-major output, zero padding included)
//   combine  = ONE kernel: transfer warps bulk-store result rows into the sources' return partitions
//              (optional FP32 local pre-reduction) and flag each row on arrival; reduce warps of the
//              same launch sum a source token as soon as all of its rows are flagged.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "layout.hpp"

namespace nep {

struct CommonParams {
    void* peers[kMaxRanks];  // window base of every rank as mapped in this process
    WindowLayout layout;
    int rank;
    uint64_t timeout_ns;
    uint32_t* status_dev;
    volatile uint32_t* status_host;
};

struct StageParams {
    CommonParams c;
    const __nv_bfloat16* x;   // [T,H]
    const int64_t* topk;      // [T,K] global expert ids or -1 (fresh only)
    const float* weights;     // [T,K] or null
    int tokens;
    int fresh;
    int parity;
    int alignment;
    int skip_copy;  // single-rank groups: the pull reads x directly, nothing is staged
    int fused;      // stage + pull in one launch: blocks wait for the barrier result instead of exiting
    uint64_t epoch;
    // handle tensors written by a fresh dispatch
    int64_t* snapshot;          // [T,K] copy of topk
    int64_t* dst_slots;         // [T,R] staging row read by destination d, or -1
    int64_t* send_counts;       // [R]
    int64_t* recv_rank_prefix;  // [R] inclusive
    int64_t* expert_counts;     // [L]
    int64_t* expert_offsets;    // [L+1]
    volatile int64_t* mailbox;  // mapped host: [0]=N, [1]=C (negative = failure)
    // Optional diagnostics (null = off), %globaltimer nanoseconds: [0] earliest start, [1] routing counted,
    // [2] rows staged, [3] peer barrier passed, [4] end of the tail block.
    unsigned long long* trace;
};

struct PlanParams {
    CommonParams c;
    int parity;
    int expand;
};

struct PullParams {
    CommonParams c;
    const int* meta;  // [N,K+2] plan scratch (fresh) or handle metadata (cached)
    int rows;
    int parity;
    int expand;
    int zero_padding;
    int write_meta;
    int stages;
    __nv_bfloat16* x_out;
    int64_t* topk_out;   // compact [N,K]
    float* w_out;        // compact [N,K] / expanded [C], or null
    int* meta_out;       // fresh: handle metadata [N,K+2]
    int* slot_map;       // expanded: [C] -> row*K+k, -1 for padding
    const int64_t* expert_counts;
    const int64_t* expert_offsets;
    const int64_t* recv_rank_prefix;  // [R] inclusive receive rows by source
    // Slot-ordered walk (expert-major layout): items are the output slots in ascending order and a
    // row is transferred when its lowest slot comes up, so row blocks fill front to back.
    const int* slot_src;  // [C] slot -> row*K+k (-1 = gap) or null for the row-ordered walk
    int capacity;
    // Rows whose source is this rank may be read from the caller's tensors instead of the staged copy.
    const __nv_bfloat16* x_local;  // [T,H] or null
    const float* w_local;          // [T,K] or null
    uint64_t data_epoch;  // fresh dispatch: wait until every source has signalled its staged rows with this epoch (0: no wait)
    int* tile_ready;  // optional: [C/128] counters, +1 per expert-major row (data or zero padding) once it is in memory
};

enum PushMode : int { kPushCompact = 0, kPushExpanded = 1, kPushExpandedReduce = 2 };

// One launch per combine.  Every CTA holds `push_warps` transfer warps (shared-memory ring, bulk copies), one
// publisher warp and reduce warps.  Transfer warps return this rank's expert outputs to the source ranks'
// return partitions; once a row's bulk store has completed the publisher warp writes the combine's tag into
// the row's arrival flag (one system-scope release per sweep, off the transfer warps' path).  Reduce warps
// walk this rank's own source tokens, wait (bounded) until every partition a token expects carries the tag,
// and write the FP32 sum.  No barrier sits between the two: the only cross-rank waits are the flags.
struct CombineParams {
    CommonParams c;
    // expert side
    const __nv_bfloat16* y;  // [N,H] or [C,H]
    const float* w;          // [N,K] or [C] or null
    const int* meta;         // [N,K+2]
    const int64_t* recv_rank_prefix;  // [R] inclusive receive rows by source
    int rows;                // N
    int capacity;            // C
    int mode;                // PushMode
    int stages;
    int push_warps;
    // source side
    const int64_t* topk;           // [T,K] source routing snapshot
    const __nv_bfloat16* bias;     // [T,H] or null
    __nv_bfloat16* out;            // [T,H]
    float* w_out;                  // [T,K] or null
    int tokens;
    int sum_all_choices;  // 1: one partition per valid k; 0: one per destination rank
    uint64_t epoch;       // signalled to every peer when this rank's pushes and reduction are done
    uint64_t wait_epoch;  // peers must have signalled this much before their return area is overwritten (0: nothing to wait for)
    int reduce_group;     // register path: reduce warps that share one source token (1 .. reduce warps per CTA)
    // Shared-memory path of the source-side sum (reduce_stages >= 2; 0 selects the register path): the returned rows
    // of a token are bulk-loaded into a ring of reduce_stages stages, reduce_chunk_bytes of every partition per stage.
    int reduce_stages;
    int reduce_chunk_bytes;
    int store_depth;      // bulk stores a transfer warp may have pending before it waits (2, 4, 6, 8 or 12; anything else means 2)
    // Optional diagnostics (null = off): [0] earliest start, [1] latest end of the transfer warps, [2] of the
    // publisher warps, [3] of the reduce warps, as %globaltimer nanoseconds; [4] nanoseconds the reduce groups spent
    // waiting for arrivals, summed over groups, [5] nanoseconds they spent summing, [6] tokens summed, [7] the longest
    // single token (nanoseconds in the upper half, its start after [0] in the lower), [8] when the last token's rows
    // were seen.  A kernel profiler cannot be attached to a multi-process run, and events cannot see inside one launch.
    unsigned long long* trace;
};

// Source-side reduction alone, for a combine whose rows were pushed by another kernel (the scatter epilogue of
// the down-projection GEMM) and made visible by a peer barrier.
struct ReduceParams {
    CommonParams c;
    const int64_t* topk;           // [T,K] source routing snapshot
    const __nv_bfloat16* bias;     // [T,H] or null
    __nv_bfloat16* out;            // [T,H]
    float* w_out;                  // [T,K] or null
    int tokens;
    int sum_all_choices;  // 1: one partition per valid k; 0: one per destination rank
};

// Single-rank combine: every contribution is local, so the expert outputs are summed straight into
// the result (same FP32 order and rounding points as push + reduce).
struct LocalCombineParams {
    CommonParams c;
    const __nv_bfloat16* y;      // [N,H] or [C,H]
    const float* w;              // receive-layout weights or null
    const int* meta;             // [N,K+2]
    const int64_t* topk;         // [T,K] source routing snapshot
    const __nv_bfloat16* bias;   // [T,H] or null
    __nv_bfloat16* out;          // [T,H]
    float* w_out;                // [T,K] or null
    int rows, capacity, tokens;
    int expand;
    int round_partial;  // expanded + multiple reduction: bf16 round of the local sum before bias
};

struct BarrierParams {
    CommonParams c;
    uint64_t epoch;
    int signal_only;  // 1: publish the epoch to every peer and return (nobody waits here)
};

struct LaunchShape {
    int grid_x;
    int ranks_y;  // 1 = production wrapper, >1 = multi-rank wrapper (params is then a device array)
};

// Each returns the CUDA error of the launch.  `params` points to one block (ranks_y == 1, host
// memory) or to a device array of ranks_y blocks.
cudaError_t launch_stage(const StageParams* params, LaunchShape shape, size_t smem, cudaStream_t stream);
cudaError_t launch_plan(const PlanParams* params, LaunchShape shape, size_t smem, cudaStream_t stream);
cudaError_t launch_pull(const PullParams* params, LaunchShape shape, int warps, size_t smem, cudaStream_t stream);
// Fresh dispatch for small calls: stage, plan and pull in ONE cooperative launch; outputs sized at an upper bound.
cudaError_t launch_fused_fresh_dispatch(const StageParams* stage, const PlanParams* plan, const PullParams* pull, LaunchShape shape, int warps,
                                        size_t smem, cudaStream_t stream);
// `cooperative`: every block must be resident at once (a whole logical group in one launch waits on itself).
cudaError_t launch_combine(const CombineParams* params, LaunchShape shape, size_t smem, cudaStream_t stream, bool cooperative);
cudaError_t launch_reduce(const ReduceParams* params, LaunchShape shape, cudaStream_t stream);
cudaError_t launch_barrier(const BarrierParams* params, LaunchShape shape, cudaStream_t stream);
// Cached dispatch for small calls: stage, peer barrier and pull in ONE cooperative launch (all blocks
// resident; the block that finishes staging last runs the barrier and releases the others).
cudaError_t launch_fused_cached_dispatch(const StageParams* stage, const PullParams* pull, LaunchShape shape, int warps, size_t smem,
                                         cudaStream_t stream);
// Test utility: one thread that waits (bounded) until gate[0] != 0; gate is pinned host memory that the host writes.
cudaError_t launch_gate(int* gate, uint64_t timeout_ns, cudaStream_t stream);
cudaError_t launch_local_combine(const LocalCombineParams* params, LaunchShape shape, cudaStream_t stream);

// Shared-memory plan of the pull/push rings: `warps` independent rings of `stages` row buffers.
struct RingPlan {
    int warps, stages;
    size_t smem_bytes;
};
RingPlan plan_ring(int64_t row_bytes, int max_smem_bytes);
// Shared memory of a combine CTA: the transfer warps' rings, the flag board and (reduce_stages >= 2) the reduce
// pipeline.  reduce_chunk_bytes == 0 lets the plan pick the chunk.
struct CombinePlan {
    RingPlan ring;
    int reduce_stages, reduce_chunk_bytes;
};
CombinePlan plan_combine(int64_t row_bytes, int parts, int max_smem_bytes, int reduce_stages, int reduce_chunk_bytes);
constexpr int kCombineThreads = 512;  // transfer warps + reduce warps of one combine CTA
int stage_smem_bytes(const WindowLayout& l);
int plan_smem_bytes(const WindowLayout& l);

// Table of kernels for diagnostics (name, registers, static smem, max threads), filled from
// cudaFuncGetAttributes on the current device.
struct KernelInfo {
    const char* name;
    int regs, static_smem, max_threads, const_bytes;
};
int kernel_table(KernelInfo* out, int capacity);

}  // namespace nep
