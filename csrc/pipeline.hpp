// Host entry points of the native extension (see pipeline.cpp).
#pragma once
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/util/Optional.h>

#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "peer_window.hpp"

namespace nep {

// Completion of an asynchronous operation: an event recorded on the comm stream plus the tensors
// a consumer stream must be registered with before it may use (and later free) them.  Mirrors the
// reference's CompletionEvent (csrc/include/nano_ep/event.hpp:12-28).
struct CompletionEvent {
    at::cuda::CUDAEvent event;
    std::vector<at::Tensor> protect;
    void wait(const c10::cuda::CUDAStream& stream);
    void current_stream_wait();
    bool query() const;
};

struct DispatchOut {
    // per rank: [x, topk_idx (compact) or empty, topk_weights or empty]
    std::vector<std::vector<at::Tensor>> outputs;
    // per rank: [recv_metadata, expert_counts, expert_offsets, dst_slots, send_counts, topk_idx,
    //            recv_rank_prefix, slot_map]
    std::vector<std::vector<at::Tensor>> metadata;
    std::vector<std::pair<int64_t, int64_t>> counts;  // (N, C)
    std::shared_ptr<CompletionEvent> event;            // null unless async_op
};

struct CombineOut {
    std::vector<std::vector<at::Tensor>> outputs;  // per rank: [x, topk_weights or empty]
    std::shared_ptr<CompletionEvent> event;
};

DispatchOut dispatch(const std::vector<PeerWindow*>& wins, const std::vector<at::Tensor>& xs,
                     const std::vector<c10::optional<at::Tensor>>& topks, const std::vector<c10::optional<at::Tensor>>& weights,
                     const std::vector<std::vector<at::Tensor>>& cached_meta, const std::vector<int64_t>& cached_capacity,
                     int64_t alignment, bool expand, bool zero_padding, int64_t num_sms, int64_t comm_stream, int64_t previous_event,
                     bool async_op, double mailbox_timeout_s, const std::vector<c10::optional<at::Tensor>>& tile_ready = {},
                     int64_t ring_smem_limit = 0);

CombineOut combine(const std::vector<PeerWindow*>& wins, const std::vector<at::Tensor>& xs, const std::vector<std::vector<at::Tensor>>& meta,
                   const std::vector<int64_t>& capacity, const std::vector<c10::optional<at::Tensor>>& weights,
                   const std::vector<c10::optional<at::Tensor>>& bias, bool expand, bool allow_multiple_reduction, int64_t num_sms,
                   int64_t comm_stream, int64_t previous_event, bool async_op);

std::vector<at::Tensor> combine_finish(const std::vector<PeerWindow*>& wins, const std::vector<std::vector<at::Tensor>>& meta,
                                       const std::vector<c10::optional<at::Tensor>>& bias);

// Per-phase device times (name, microseconds) of the operations issued since the last call.
// Token threshold and grid bound of the single-launch cached dispatch for small calls (see pipeline.cpp).
struct FusedLimits {
    int64_t dispatch_tokens, blocks, fresh_tokens;
};
FusedLimits fused_limits();
// Negative token values / blocks < 1 leave the respective setting unchanged.
void set_fused_limits(int64_t dispatch_tokens, int64_t blocks, int64_t fresh_tokens);

// In-kernel time stamps of the next combines of this process (single-rank calls): microseconds from the
// kernel's first block to the end of its transfer warps, its flag publishers and its reduce warps.
// `store_depth` (0 = default) sets how many bulk stores a transfer warp keeps pending, `reduce_group` (0 = default)
// how the source-side sum runs: N > 0 = in registers with N reduce warps per token, a negative value
// -(stages * 1000 + chunk bytes / 128) = through a shared-memory ring of that many stages (chunk 0 = chosen by the
// plan).  take_combine_trace() returns those three stamps followed by the
// reduce groups' totals: microseconds waited, microseconds summing, tokens summed, the longest token, when it began
// and when the last token's rows were seen.
void set_combine_trace(bool enabled, int64_t store_depth, int64_t reduce_group);
std::vector<double> take_combine_trace();
// The same for the stage kernel of the last fresh dispatch: microseconds until the routing was counted, the rows
// were staged, the peer barrier was passed and the tail block finished.
std::vector<double> take_stage_trace();
// Test hook: with a pinned host int32[2] tensor set, every dispatch holds its pull behind a kernel that waits (at most
// `timeout_s`) until the host writes word[0] != 0; word[1] becomes 1 if that wait ran out.  None switches it off.
// (The word lives in host memory so that opening the gate needs no GPU work: a kernel or copy issued to open it could
// queue up behind the very kernels the gate holds back.)
void set_test_gate(const c10::optional<at::Tensor>& word, double timeout_s);
void set_phase_timing(bool enabled);
std::vector<std::pair<std::string, double>> take_phase_timings();

void group_barrier(const std::vector<PeerWindow*>& wins, int64_t stream);

}  // namespace nep
