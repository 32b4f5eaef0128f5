/* Allocation-free receive planning.
 *
 * This entry point has no counterpart in the reference library.  It exists for host code that is
 * not allowed to obtain device memory at the moment it needs a receive plan: an inference-engine
 * plugin inside its enqueue callback, a component running under a fixed memory budget negotiated at
 * start-up, or a latency-critical loop where cudaMalloc/cudaFree (which may synchronise the whole
 * device) cannot be tolerated.  Such callers own their input and output buffers already; what they
 * lack is the few kilobytes of cursor storage the planning kernel needs.  Here that storage is a
 * fixed array inside the library image, so the call performs no cudaMalloc, no cudaFree and uses no
 * allocating library routine.
 *
 * The computation is the one the dispatch "plan" phase performs for ONE source rank: keep the
 * tokens that chose an expert in [expert_lo, expert_lo + local_experts), give each a receive row,
 * and write one metadata row [source, token, v_0 .. v_{K-1}] per kept token, where v_k is the local
 * expert id (expand == 0) or an expert-major slot taken from expert_offsets (expand != 0), and -1
 * for choices that are masked or live elsewhere.  Row order and the order of slots inside one
 * expert's range are unspecified.
 *
 * Limits and rules
 *   - local_experts <= NEP_NOALLOC_MAX_LOCAL_EXPERTS (4096), topk <= 32, tokens <= 2^24.  Larger
 *     requests are rejected with NEP_NOALLOC_TOO_LARGE and nothing is launched.
 *   - The cursor array (NEP_NOALLOC_SCRATCH_BYTES = 16640 bytes) lives in every GPU that loads this
 *     library, from load to process exit.
 *   - The first call on each device looks up the device address of that array (the device must be
 *     current, as for every call) and, when the CUDA runtime loads modules lazily, also loads this
 *     library's device code, which the driver may back with memory of its own.  Make that first call
 *     during start-up: before any stream capture begins and before a phase in which nothing may be
 *     allocated.
 *   - Every call on a device shares the one array and starts by clearing it on `stream`.  Two calls
 *     that overlap on the GPU (different streams, no ordering) race on it; order them.
 *   - All pointers are device pointers valid on the current device; `stream` is a cudaStream_t.
 */
#ifndef NEP_PLAN_ROWS_NOALLOC_H
#define NEP_PLAN_ROWS_NOALLOC_H

#ifdef __cplusplus
extern "C" {
#endif

#define NEP_NOALLOC_MAX_LOCAL_EXPERTS 4096
#define NEP_NOALLOC_SCRATCH_BYTES ((NEP_NOALLOC_MAX_LOCAL_EXPERTS + 64) * 4)

enum {
    NEP_NOALLOC_OK = 0,
    NEP_NOALLOC_TOO_LARGE = 1,   /* a size exceeds the stated maximum */
    NEP_NOALLOC_BAD_ARGUMENT = 2, /* null pointer or non-positive dimension */
    NEP_NOALLOC_CUDA_ERROR = 3    /* a CUDA call failed; see nep_noalloc_last_error() */
};

/* topk_i32        [tokens, topk] int32 global expert ids, -1 = masked
 * expert_offsets  [local_experts + 1] int32 exclusive padded offsets (read only when expand != 0)
 * meta_out        [>= kept tokens, topk + 2] int32; size it for `tokens` rows to be safe
 * row_count_out   one int32: number of rows written, or -1 when expert_offsets do not fit the routing
 *                 (a slot fell outside its expert's range; such choices are written as -1)
 * Returns one of the codes above.  Work is enqueued on `stream`; outputs are valid once it drains. */
int nep_plan_rows_noalloc(const int* topk_i32, int tokens, int topk, int source_rank, int expert_lo, int local_experts,
                          const int* expert_offsets, int expand, int* meta_out, int* row_count_out, void* stream);

/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char* nep_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
