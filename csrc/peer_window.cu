#include "peer_window.hpp"

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <string>
#include <stdexcept>
#include <thread>

namespace nep {

int64_t PeerWindow::launches = 0;

namespace {
void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        const std::string message = std::string(what) + ": " + cudaGetErrorString(e);
        cudaGetLastError();
        throw std::runtime_error(message);
    }
}
}  // namespace

const char* status_name(uint32_t code) {
    switch (code) {
        case kOk: return "ok";
        case kBarrierTimeout: return "peer barrier timed out (a rank did not reach the collective)";
        case kBadExpertId: return "topk_idx holds an expert id outside [-1, num_experts)";
        case kCopyTimeout: return "bulk copy did not complete within the wait limit";
        case kSlotOverflow: return "receive row or expert slot beyond the planned capacity";
        case kBadMetadata: return "handle metadata names an impossible rank, token or slot";
        default: return "unknown device status";
    }
}

PeerWindow::PeerWindow(int rank, int world, const WindowLayout& layout, double wait_timeout_s)
    : rank_(rank), world_(world), layout_(layout), timeout_ns_(uint64_t(wait_timeout_s * 1e9)) {
    if (world != layout.ranks || rank < 0 || rank >= world) throw std::invalid_argument("rank/world do not match the window layout");
    check(cudaGetDevice(&device_), "cudaGetDevice");
    check(cudaMalloc(&base_, size_t(layout.num_bytes)), "cudaMalloc(peer window)");
    cudaError_t e = cudaMemset(base_, 0, size_t(layout.num_bytes));
    if (e == cudaSuccess) e = cudaHostAlloc(&pinned_, 256, cudaHostAllocMapped | cudaHostAllocPortable);
    if (e == cudaSuccess) {
        std::memset(pinned_, 0, 256);
        mailbox_ = static_cast<volatile int64_t*>(pinned_);
        status_host_ = reinterpret_cast<volatile uint32_t*>(static_cast<char*>(pinned_) + 64);
        void* dev = nullptr;
        e = cudaHostGetDevicePointer(&dev, pinned_, 0);
        mailbox_dev_ = static_cast<volatile int64_t*>(dev);
        status_host_dev_ = reinterpret_cast<volatile uint32_t*>(static_cast<char*>(dev) + 64);
    }
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&order_event_, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (order_event_) cudaEventDestroy(order_event_);
        if (pinned_) cudaFreeHost(pinned_);
        cudaFree(base_);
        base_ = nullptr;
        check(e, "peer window initialisation");
    }
    peers_[rank_] = base_;
}

PeerWindow::~PeerWindow() {
    // Never free a window that peers may still map: an un-closed window leaks on purpose.
    if (!closed_ && base_ != nullptr && !connected_) {
        cudaFree(base_);
        if (pinned_) cudaFreeHost(pinned_);
    } else if (!closed_ && base_ != nullptr) {
        std::fprintf(stderr, "nanoep_b200: PeerWindow destroyed without close(); leaking the window\n");
    }
}

std::string peer_access_error(int own_rank, int peer_rank, int own_device, int peer_device, bool can_access, bool access_supported) {
    char buf[256];
    if (peer_device == own_device) {
        std::snprintf(buf, sizeof(buf), "rank %d and rank %d share CUDA device %d; every rank needs its own GPU", own_rank, peer_rank, own_device);
        return buf;
    }
    if (!can_access || !access_supported) {
        std::snprintf(buf, sizeof(buf), "CUDA device %d (rank %d) has no peer access to device %d (rank %d); NVLink or PCIe P2P is required",
                      own_device, own_rank, peer_device, peer_rank);
        return buf;
    }
    return std::string();
}

std::string PeerWindow::export_handle() {
    if (closed_) throw std::runtime_error("peer window is closed");
    cudaIpcMemHandle_t h;
    check(cudaIpcGetMemHandle(&h, base_), "cudaIpcGetMemHandle");
    return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void PeerWindow::import_handles(const std::vector<std::string>& handles, const std::vector<int>& peer_devices) {
    if (closed_ || connected_) throw std::runtime_error("peer window already connected or closed");
    if (int(handles.size()) != world_) throw std::invalid_argument("need one IPC handle per rank");
    if (!peer_devices.empty() && int(peer_devices.size()) != world_) throw std::invalid_argument("need one device ordinal per rank");
    try {
        for (int p = 0; p < world_; ++p) {
            if (p == rank_) continue;
            // Where the peer's GPU is visible to this process, check before mapping that it is another GPU and that
            // this GPU may load from, store to and bulk-copy into it (same role as the reference's checks,
            // csrc/peer.cu:95-126).  A peer GPU outside this process's visible set can only be judged by the mapping call.
            const int peer_device = peer_devices.empty() ? -1 : peer_devices[p];
            if (peer_device >= 0) {
                int can = 0, supported = 0;
                if (peer_device != device_) {
                    check(cudaDeviceCanAccessPeer(&can, device_, peer_device), "cudaDeviceCanAccessPeer");
                    check(cudaDeviceGetP2PAttribute(&supported, cudaDevP2PAttrAccessSupported, device_, peer_device), "cudaDeviceGetP2PAttribute");
                }
                const std::string problem = peer_access_error(rank_, p, device_, peer_device, can != 0, supported != 0);
                if (!problem.empty()) throw std::runtime_error(problem);
            }
            if (handles[p].size() != sizeof(cudaIpcMemHandle_t)) throw std::invalid_argument("IPC handle must be 64 bytes");
            cudaIpcMemHandle_t h;
            std::memcpy(&h, handles[p].data(), sizeof(h));
            void* mapped = nullptr;
            check(cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
            peers_[p] = mapped;
            imported_[p] = true;
        }
    } catch (...) {
        for (int p = 0; p < world_; ++p)
            if (imported_[p]) {
                cudaIpcCloseMemHandle(peers_[p]);
                imported_[p] = false;
                peers_[p] = nullptr;
            }
        cudaGetLastError();
        throw;
    }
    connected_ = true;
}

void PeerWindow::adopt_peers(const std::vector<PeerWindow*>& group) {
    if (closed_ || connected_) throw std::runtime_error("peer window already connected or closed");
    if (int(group.size()) != world_) throw std::invalid_argument("need one window per logical rank");
    for (int p = 0; p < world_; ++p) {
        if (group[p] == nullptr || group[p]->rank() != p || group[p]->layout().num_bytes != layout_.num_bytes)
            throw std::invalid_argument("logical peer windows must be ordered by rank and share one layout");
        peers_[p] = group[p]->base();
    }
    connected_ = true;
}

void PeerWindow::close_peer_mappings() {
    if (unmapped_) return;
    cudaError_t first = cudaSuccess;
    for (int p = 0; p < world_; ++p)
        if (imported_[p]) {
            cudaError_t e = cudaIpcCloseMemHandle(peers_[p]);
            if (first == cudaSuccess) first = e;
            imported_[p] = false;
            peers_[p] = nullptr;
        }
    unmapped_ = true;
    check(first, "cudaIpcCloseMemHandle");
}

void PeerWindow::close() {
    if (closed_) return;
    if (connected_ && !unmapped_) throw std::runtime_error("close_peer_mappings() must run on every rank before close()");
    cudaError_t e = cudaFree(base_);
    if (pinned_) cudaFreeHost(pinned_);
    if (order_event_) cudaEventDestroy(order_event_);
    order_event_ = nullptr;
    base_ = nullptr;
    pinned_ = nullptr;
    closed_ = true;
    check(e, "cudaFree(peer window)");
}

uint64_t PeerWindow::reserve_epochs(int count) {
    if (closed_) throw std::runtime_error("peer window is closed");
    if (failed_) throw std::runtime_error("peer window is in a failed state after an earlier error");
    const uint64_t first = epoch_ + 1;
    epoch_ += uint64_t(count);
    return first;
}

CommonParams PeerWindow::common() const {
    CommonParams c{};
    for (int p = 0; p < kMaxRanks; ++p) c.peers[p] = peers_[p];
    c.layout = layout_;
    c.rank = rank_;
    c.timeout_ns = timeout_ns_;
    c.status_dev = reinterpret_cast<uint32_t*>(static_cast<char*>(base_) + layout_.ctrl_offset) + 4;
    c.status_host = status_host_dev_;
    return c;
}

void PeerWindow::arm_mailbox() {
    mailbox_[0] = -1;
    mailbox_[1] = -1;
    std::atomic_thread_fence(std::memory_order_seq_cst);
}

std::pair<int64_t, int64_t> PeerWindow::wait_mailbox(cudaStream_t stream, double timeout_s) {
    using clock = std::chrono::steady_clock;
    const auto start = clock::now();
    auto last_query = start;
    for (;;) {
        const int64_t n = mailbox_[0], c = mailbox_[1];
        if (n != -1 && c != -1) {
            if (n < 0 || c < 0) {
                failed_ = true;
                check_status();
                throw std::runtime_error("dispatch count exchange failed on the device");
            }
            return {n, c};
        }
        const auto now = clock::now();
        if (now - last_query > std::chrono::milliseconds(1)) {
            last_query = now;
            cudaError_t q = cudaStreamQuery(stream);
            if (q != cudaSuccess && q != cudaErrorNotReady) {
                failed_ = true;
                check(q, "dispatch count exchange (stream error)");
            }
            if (q == cudaSuccess && (mailbox_[0] == -1 || mailbox_[1] == -1)) {
                failed_ = true;
                throw std::runtime_error("dispatch kernels finished without publishing receive counts");
            }
            if (std::chrono::duration<double>(now - start).count() > timeout_s) {
                failed_ = true;
                throw std::runtime_error("timed out waiting for dispatch receive counts");
            }
        }
    }
}

std::string format_status(uint32_t code, uint32_t detail, uint32_t tag, int rank) {
    // snprintf on purpose: numeric operator<< on iostreams is avoided throughout this extension.
    char buf[320];
    std::snprintf(buf, sizeof(buf), "nanoep_b200 device status %u (%s), detail %u, kernel tag %u, rank %d", code, status_name(code), detail,
                  tag, rank);
    return std::string(buf);
}

void PeerWindow::check_status() const {
    const uint32_t code = status_host_[0];
    if (code == kOk) return;
    const uint32_t detail = status_host_[1], tag = status_host_[2];
    throw std::runtime_error(format_status(code, detail, tag, rank_));
}

void PeerWindow::clear_status(cudaStream_t stream) {
    check(cudaMemsetAsync(static_cast<char*>(base_) + layout_.ctrl_offset + 16, 0, 16, stream), "clear status");
    check(cudaStreamSynchronize(stream), "clear status sync");
    status_host_[0] = status_host_[1] = status_host_[2] = 0;
    failed_ = false;
}

void PeerWindow::order_after_last(cudaStream_t stream) {
    if (has_last_ && last_stream_ != stream) {
        check(cudaEventRecord(order_event_, last_stream_), "record previous operation's stream");
        check(cudaStreamWaitEvent(stream, order_event_, 0), "order behind previous operation");
    }
    last_stream_ = stream;
    has_last_ = true;
}

void PeerWindow::barrier(cudaStream_t stream) {
    order_after_last(stream);
    BarrierParams p{};
    p.c = common();
    p.epoch = reserve_epochs(1);
    ++launches;
    check(launch_barrier(&p, LaunchShape{1, 1}, stream), "barrier launch");
}

}  // namespace nep
