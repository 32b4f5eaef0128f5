// Byte layout of one rank's peer window and of the rows that cross NVLink.
//
// One header shared by host and device code so both sides compute identical offsets.  The
// reference keeps the same "single source of truth" idea in csrc/layout.hpp:59-98, but the
// regions here serve a different protocol: senders *stage* their tokens in their own window
// and receivers pull them; the dispatch regions that peers touch exist twice (parity = dispatch
// sequence & 1) so that one peer barrier per dispatch is enough; the combine return area is a
// single [P partitions][Tmax] array written by the expert ranks, with one arrival flag per
// (partition, token) that carries the writing operation's tag.  P = K, or min(R, K) when the
// buffer pre-reduces per rank (the reference sizes its return area the same way,
// csrc/layout.hpp:51-57).
#pragma once
#include <cstdint>
#include <stdexcept>

#if defined(__CUDACC__)
#define NEP_HD __host__ __device__ __forceinline__
#else
#define NEP_HD inline
#endif

namespace nep {

constexpr int kMaxRanks = 32;
constexpr int kMaxTopk = 32;
constexpr int64_t kRegionAlign = 256;

NEP_HD constexpr int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Staged (wire) row of one source token: bf16 x[H] followed by fp32 gate weights[K], padded to
// 16 bytes so a single bulk copy can move the whole row.
NEP_HD constexpr int64_t wire_weights_offset(int hidden) { return int64_t(hidden) * 2; }
NEP_HD constexpr int64_t wire_row_bytes(int hidden, int topk) { return align_up(int64_t(hidden) * 2 + int64_t(topk) * 4, 16); }

// Per (source -> destination) count message: [0] deduplicated rows, [1] source token count,
// [2 + l] assignments to local expert l of the destination.
NEP_HD constexpr int64_t count_msg_ints(int local_experts) { return 2 + int64_t(local_experts); }

struct WindowLayout {
    int ranks, hidden, topk, local_experts;
    int64_t max_tokens, num_experts;
    // Region offsets (bytes from the window base).  Regions marked [2] hold two parity copies,
    // `*_stride` apart.
    int64_t signal_offset;       // u64[kMaxRanks]   epoch written by each peer
    int64_t data_signal_offset;  // u64[kMaxRanks]   epoch of the fresh dispatch whose rows peer p has finished staging
    int64_t ctrl_offset;         // local scratch: tickets, count accumulators, cursors, prefixes
    int64_t counts_in_offset;    // [2] i32[R][2+L]  count messages written by the sources
    int64_t counts_in_stride;
    int64_t routing_in_offset;   // [2] i32[R][Tmax][K] every source's routing, written by the sources
    int64_t routing_in_stride;
    int64_t chunks_in_offset;    // [2] i32[R][ceil(Tmax/32)] rows each source sends here per chunk of 32 of its tokens
    int64_t chunks_in_stride;    //     (written by the sources; turned into an exclusive prefix by the receiver)
    int64_t stage_rows_offset;   // [2] u8[Tmax][wire_row_bytes] staged tokens, pulled by the receivers
    int64_t stage_rows_stride;
    int ret_parts;               // P: return partitions per token
    int rank_indexed;            // 1: partition = expert rank (P == R); 0: partition = index of the choice
    int64_t ret_w_offset;        // f32[Tmax][K] gate-weight payload returned by combine
    int64_t ret_flag_offset;     // u32[P][Tmax] tag of the combine that last wrote (partition, token)
    int64_t ret_offset;          // bf16[P][Tmax][H] expert outputs pushed back by combine
    int64_t meta_scratch_offset; // i32[R*Tmax][K+2] receive plan of a fresh dispatch (local only)
    int64_t slot_scratch_offset; // i32[slot_scratch_ints] expert-major slot -> row*K+k of a fresh dispatch (local only)
    int64_t slot_scratch_ints;
    int64_t num_bytes;

    // ctrl sub-layout, in int32 units from ctrl_offset.
    // words 4..6: status; word 9: the combine's shared position in its row walk (reset by the combine's last block)
    static constexpr int kTicketStage = 0, kTicketCombine = 1, kGoWord = 2, kTicketCopy = 3, kTicketPlan = 7, kGoWordPlan = 8, kWorkCursor = 9, kCtrlHeaderInts = 16;
    NEP_HD int64_t ctrl_count_acc() const { return kCtrlHeaderInts; }                         // i32[R + E]
    NEP_HD int64_t ctrl_row_cursor() const { return ctrl_count_acc() + ranks + num_experts; }  // i32[R] (reserved; rows are placed by chunk prefixes)
    NEP_HD int64_t ctrl_expert_cursor() const { return ctrl_row_cursor() + ranks; }            // i32[L]
    NEP_HD int64_t ctrl_recv_prefix() const { return ctrl_expert_cursor() + local_experts; }   // i32[R+1] exclusive
    NEP_HD int64_t ctrl_expert_offsets() const { return ctrl_recv_prefix() + ranks + 1; }      // i32[L+1]
    NEP_HD int64_t ctrl_expert_counts() const { return ctrl_expert_offsets() + local_experts + 1; }  // i32[L]
    NEP_HD int64_t ctrl_src_tokens() const { return ctrl_expert_counts() + local_experts; }    // i32[R]
    NEP_HD int64_t ctrl_chunk_acc() const { return ctrl_src_tokens() + ranks; }                // i32[R][chunks_per_rank()]
    NEP_HD int64_t ctrl_ints() const { return ctrl_chunk_acc() + int64_t(ranks) * chunks_per_rank(); }
    NEP_HD int64_t chunks_per_rank() const { return (max_tokens + 31) / 32; }

    NEP_HD int64_t row_bytes() const { return wire_row_bytes(hidden, topk); }
    NEP_HD int64_t msg_ints() const { return count_msg_ints(local_experts); }

    static WindowLayout make(int ranks, int64_t max_tokens, int hidden, int topk, int64_t num_experts, bool per_rank_reduction = false) {
        if (ranks <= 0 || ranks > kMaxRanks || (ranks & (ranks - 1)) != 0)
            throw std::invalid_argument("world size must be a power of two in [1,32]");
        if (max_tokens <= 0 || hidden <= 0 || topk <= 0 || topk > kMaxTopk)
            throw std::invalid_argument("window needs positive capacity/hidden and topk in [1,32]");
        if (hidden % 8 != 0) throw std::invalid_argument("hidden must be a multiple of 8 (16-byte rows)");
        if (num_experts <= 0 || num_experts % ranks != 0)
            throw std::invalid_argument("num_experts must be positive and divisible by the world size");
        if (max_tokens > (int64_t(1) << 24) || num_experts > (int64_t(1) << 20))
            throw std::invalid_argument("capacity or expert count too large for 32-bit metadata");
        WindowLayout w{};
        w.ranks = ranks;
        w.hidden = hidden;
        w.topk = topk;
        w.max_tokens = max_tokens;
        w.num_experts = num_experts;
        w.local_experts = int(num_experts / ranks);
        int64_t at = 0;
        auto take = [&](int64_t bytes) {
            int64_t here = at;
            at = align_up(at + bytes, kRegionAlign);
            return here;
        };
        w.signal_offset = take(kMaxRanks * 8);
        w.data_signal_offset = take(kMaxRanks * 8);
        w.ctrl_offset = take(w.ctrl_ints() * 4);
        w.counts_in_stride = align_up(int64_t(ranks) * w.msg_ints() * 4, kRegionAlign);
        w.counts_in_offset = take(2 * w.counts_in_stride);
        w.routing_in_stride = align_up(int64_t(ranks) * max_tokens * topk * 4, kRegionAlign);
        w.routing_in_offset = take(2 * w.routing_in_stride);
        w.chunks_in_stride = align_up(int64_t(ranks) * w.chunks_per_rank() * 4, kRegionAlign);
        w.chunks_in_offset = take(2 * w.chunks_in_stride);
        w.stage_rows_stride = align_up(max_tokens * w.row_bytes(), kRegionAlign);
        w.stage_rows_offset = take(2 * w.stage_rows_stride);
        // One row per (token, expert rank) comes back when the buffer pre-reduces per rank: min(R, K) partitions
        // are enough, indexed by the expert rank when every rank has its own.
        w.ret_parts = per_rank_reduction ? (ranks < topk ? ranks : topk) : topk;
        w.rank_indexed = (per_rank_reduction && ranks <= topk) ? 1 : 0;
        w.ret_w_offset = take(max_tokens * topk * 4);
        w.ret_flag_offset = take(int64_t(w.ret_parts) * max_tokens * 4);
        w.ret_offset = take(int64_t(w.ret_parts) * max_tokens * hidden * 2);
        w.meta_scratch_offset = take(int64_t(ranks) * max_tokens * (topk + 2) * 4);
        w.slot_scratch_ints = int64_t(ranks) * max_tokens * topk + int64_t(w.local_experts) * 128;
        w.slot_scratch_offset = take(w.slot_scratch_ints * 4);
        w.num_bytes = at;
        return w;
    }
};

// Sticky device-side error codes (status word 0); word 1 carries a detail value.
enum Status : uint32_t {
    kOk = 0,
    kBarrierTimeout = 1,   // a peer did not signal the epoch within the wait limit
    kBadExpertId = 2,      // topk_idx outside [-1, E)
    kCopyTimeout = 3,      // a bulk copy's mbarrier did not complete within the wait limit
    kSlotOverflow = 4,     // receive row or expert slot beyond the planned capacity
    kBadMetadata = 5,      // handle metadata names an impossible rank/token/slot
};

}  // namespace nep
