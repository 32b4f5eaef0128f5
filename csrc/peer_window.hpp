// Per-rank peer window: device allocation shared through CUDA IPC, peer address table, epoch and
// parity bookkeeping, mapped host mailbox and status words.
//
// Counterpart of the reference's PeerRuntime (csrc/peer.cu:17-283, include/nano_ep/peer.hpp:18-65).
// Differences: failures inside kernels arrive as status codes in mapped host memory instead of a
// device trap; a window can also adopt other windows of the same process as "logical peers" so a
// whole group runs on one GPU; operation parities select between the two copies of each region.
#pragma once
#include <cstdint>
#include <string>
#include <utility>
#include <vector>
#include <cuda_runtime.h>
#include "ep_kernels.hpp"
#include "layout.hpp"

namespace nep {

class PeerWindow {
public:
    PeerWindow(int rank, int world, const WindowLayout& layout, double wait_timeout_s);
    ~PeerWindow();
    PeerWindow(const PeerWindow&) = delete;
    PeerWindow& operator=(const PeerWindow&) = delete;

    int rank() const { return rank_; }
    int world() const { return world_; }
    int device() const { return device_; }
    const WindowLayout& layout() const { return layout_; }
    void* base() const { return base_; }
    int64_t num_bytes() const { return layout_.num_bytes; }
    bool connected() const { return connected_; }
    bool closed() const { return closed_; }

    // 64 raw bytes of the CUDA IPC memory handle of the local window.
    std::string export_handle();
    // Map every peer's window (index = rank; the own entry is ignored).  `peer_devices[p]` is the CUDA ordinal of
    // rank p's GPU in THIS process (-1 when it is not visible here); visible peers are checked for P2P access first.
    void import_handles(const std::vector<std::string>& handles, const std::vector<int>& peer_devices = {});
    // Same-process alternative: use other PeerWindow objects (one per logical rank) as peers.
    void adopt_peers(const std::vector<PeerWindow*>& group);
    // Two-phase teardown: every importer unmaps first; only then may owners free.
    void close_peer_mappings();
    void close();

    // Monotone barrier epochs; all ranks reserve in the same order.
    uint64_t reserve_epochs(int count);
    uint64_t last_epoch() const { return epoch_; }
    int next_dispatch_parity() { return int(dispatch_seq_++ & 1); }
    // A combine reserves one epoch, which it signals to every peer when its pushes and its reduction are done,
    // and learns the epoch of the previous combine: before writing into a peer's (single) return area it waits
    // until that peer has signalled at least that epoch, i.e. has finished reading the previous contents.
    struct CombineEpochs {
        uint64_t epoch, wait_epoch;  // wait_epoch 0: no earlier combine
    };
    CombineEpochs begin_combine() {
        const uint64_t previous = last_combine_epoch_;
        last_combine_epoch_ = reserve_epochs(1);
        return CombineEpochs{last_combine_epoch_, previous};
    }

    CommonParams common() const;
    void set_wait_timeout(double seconds) { timeout_ns_ = uint64_t(seconds * 1e9); }

    // Fresh-dispatch count mailbox (mapped pinned host memory written by the stage kernel).
    volatile int64_t* mailbox() const { return mailbox_; }
    volatile int64_t* mailbox_device() const { return mailbox_dev_; }
    void arm_mailbox();
    // Spin until both counts are published; polls the stream for asynchronous errors and gives up
    // after `timeout_s`.  Throws std::runtime_error on failure and latches the window as failed.
    std::pair<int64_t, int64_t> wait_mailbox(cudaStream_t stream, double timeout_s);

    // Device-reported status: 0 when clean.  `check_status` throws with a decoded message.
    uint32_t status_code() const { return status_host_[0]; }
    void check_status() const;
    void clear_status(cudaStream_t stream);

    // Standalone barrier on `stream` (shares the epoch sequence with the fused barriers).
    void barrier(cudaStream_t stream);

    // Operations of one window must reach the GPU in the order in which they reserved their epochs, whatever
    // stream each runs on: signals only grow, and a region's parity copy is reused two operations later.
    // Called at the start of every operation with the stream it will run on: when the previous operation ran
    // on another stream, `stream` is made to wait for everything enqueued on that stream so far.
    void order_after_last(cudaStream_t stream);

    // Launch counter for diagnostics and benchmarks.
    static int64_t launches;

private:
    int rank_, world_, device_;
    WindowLayout layout_;
    void* base_ = nullptr;
    void* peers_[kMaxRanks] = {};
    bool imported_[kMaxRanks] = {};
    bool connected_ = false, closed_ = false, unmapped_ = false, failed_ = false;
    uint64_t epoch_ = 0, dispatch_seq_ = 0, last_combine_epoch_ = 0;
    uint64_t timeout_ns_;
    volatile int64_t* mailbox_ = nullptr;       // host pointer
    volatile int64_t* mailbox_dev_ = nullptr;   // device alias
    volatile uint32_t* status_host_ = nullptr;  // host pointer
    volatile uint32_t* status_host_dev_ = nullptr;
    void* pinned_ = nullptr;
    cudaStream_t last_stream_ = nullptr;
    bool has_last_ = false;
    cudaEvent_t order_event_ = nullptr;
};

// Empty when `own_device` may use `peer_device`'s window, else the reason (distinct GPUs and peer access are required).
std::string peer_access_error(int own_rank, int peer_rank, int own_device, int peer_device, bool can_access, bool access_supported);
const char* status_name(uint32_t code);
std::string format_status(uint32_t code, uint32_t detail, uint32_t tag, int rank);

}  // namespace nep
