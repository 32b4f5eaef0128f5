// Host pipeline: validation, stream choreography, allocation and kernel launches for
// dispatch() and combine().
//
// Same responsibilities as the reference's host pipeline (csrc/pipeline.cu:26-489 plus
// dispatch_epilogue.cpp / combine_epilogue.cpp): one native call per Python operation; inputs are
// ordered behind the caller's stream or an explicit event; outputs are allocated with their exact
// size in the consumer stream's allocator pool; the only host wait is the N/C mailbox of a fresh
// dispatch.  Every entry point takes a *list* of ranks: one element in production, R elements when a
// whole logical group shares one GPU (tests) -- then each phase is a single multi-rank launch.
#include "pipeline.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <sstream>

namespace nep {

namespace {

constexpr int kFusedDispatchDefaultTokens = 64;
constexpr int kFusedFreshDefaultTokens = 0;  // single-launch fresh dispatch: off unless asked for (the host waits for N and C either way)
constexpr int64_t kFusedFreshMaxOutputBytes = int64_t(256) << 20;  // single-launch fresh dispatch: largest bound-sized output
constexpr int kFusedDefaultBlocks = 1024;  // i.e. bounded by the SM budget and co-residency only

void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    }
}

// Optional per-phase device timing: events recorded on the comm stream between launches.  Off by
// default; switched on from Python for benchmarks (multi-GPU runs cannot use a kernel profiler).
struct PhaseMarks {
    bool enabled = false;
    std::vector<std::pair<std::string, cudaEvent_t>> marks;
    std::vector<cudaEvent_t> pool;
    void mark(const char* name, cudaStream_t stream) {
        if (!enabled) return;
        cudaEvent_t ev;
        if (!pool.empty()) {
            ev = pool.back();
            pool.pop_back();
        } else {
            cuda_check(cudaEventCreate(&ev), "cudaEventCreate");
        }
        cuda_check(cudaEventRecord(ev, stream), "cudaEventRecord");
        marks.emplace_back(name, ev);
    }
};
PhaseMarks g_marks;

// In-kernel time stamps of the combine kernel (see CombineParams::trace): a small device buffer, reset before
// every traced combine and read on request.
struct CombineTrace {
    bool enabled = false;
    at::Tensor words;  // uint64 x 9 as int64
    at::Tensor stage_words;  // uint64 x 5 as int64 (stage kernel of a fresh dispatch)
    // Tuning of the combine kernel: bulk stores pending per transfer warp and the form of the source-side sum
    // (see set_combine_trace); 0 = default.
    // NANOEP_COMBINE_STORE_DEPTH / NANOEP_COMBINE_REDUCE_GROUP set the process-wide start values.
    int depth = 0;
    int group = 0;
    CombineTrace() {
        if (const char* env = std::getenv("NANOEP_COMBINE_STORE_DEPTH")) depth = std::atoi(env);
        if (const char* env = std::getenv("NANOEP_COMBINE_REDUCE_GROUP")) group = std::atoi(env);
    }
};
CombineTrace g_trace;
// Shared-memory pipeline with two stages and a chunk of about half of shared memory / 2 / partitions (whole rows at
// hidden 7168 x 8 partitions): same time as the register path at 4096 tokens per rank, 10-14 us less from 1 to 128.
constexpr int kDefaultReduceSetting = -2000;

// Test hook: while set, every dispatch of this process launches a gate kernel between its planning kernels and its
// pull, so a test can keep one rank's pull pending (a "slow reader") while its peers run ahead.
struct TestGate {
    at::Tensor word;  // pinned host int32[2]: [0] release (written by the host), [1] set by the kernel when its wait ran out
    double timeout_s = 0;
};
TestGate g_gate;

// Single-launch paths for small calls.  Cached dispatches of at most `dispatch_tokens` tokens per rank run
// stage, peer barrier and pull as one cooperative launch; fresh dispatches of at most `fresh_tokens` tokens run
// stage, plan and pull as one (NANOEP_FUSED_FRESH_TOKENS, default 0 = off); `blocks` bounds their grids (every block must be
// resident at once and spins on one word while the last block runs the peer barrier).  Defaults come from
// NANOEP_FUSED_DISPATCH_TOKENS / NANOEP_FUSED_BLOCKS (0 tokens switches the path off) and can be changed
// at run time.  (A combine is one launch at every size.)
struct FusedLimitsState {
    std::atomic<int64_t> dispatch_tokens, blocks, fresh_tokens;
    FusedLimitsState() {
        auto read = [](const char* name, int64_t fallback) {
            const char* env = std::getenv(name);
            return env != nullptr ? std::atoll(env) : fallback;
        };
        dispatch_tokens = std::max<int64_t>(0, read("NANOEP_FUSED_DISPATCH_TOKENS", kFusedDispatchDefaultTokens));
        blocks = std::max<int64_t>(1, read("NANOEP_FUSED_BLOCKS", kFusedDefaultBlocks));
        fresh_tokens = std::max<int64_t>(0, read("NANOEP_FUSED_FRESH_TOKENS", kFusedFreshDefaultTokens));
    }
};
FusedLimitsState& fused_state() {
    static FusedLimitsState state;
    return state;
}
int64_t fused_dispatch_max_tokens() { return fused_state().dispatch_tokens.load(std::memory_order_relaxed); }
int64_t fused_fresh_max_tokens() { return fused_state().fresh_tokens.load(std::memory_order_relaxed); }
int64_t fused_max_blocks() { return fused_state().blocks.load(std::memory_order_relaxed); }

struct DeviceLimits {
    int sms;
    int smem_optin;
};
DeviceLimits device_limits() {
    const auto* prop = at::cuda::getCurrentDeviceProperties();
    return DeviceLimits{prop->multiProcessorCount, int(prop->sharedMemPerBlockOptin)};
}

void check_payload(const at::Tensor& x, const c10::optional<at::Tensor>& topk, const c10::optional<at::Tensor>& weights,
                   const WindowLayout& L, int device) {
    TORCH_CHECK(x.is_cuda() && x.get_device() == device, "x must live on this rank's GPU");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16, "x must be bfloat16");
    TORCH_CHECK(x.dim() == 2 && x.size(1) == L.hidden, "x must be [T, hidden]");
    TORCH_CHECK(x.is_contiguous(), "x must be contiguous");
    TORCH_CHECK(x.size(0) <= L.max_tokens, "x has more tokens than num_max_tokens_per_rank");
    TORCH_CHECK(x.numel() == 0 || reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "x must be 16-byte aligned; clone() an offset view");
    if (topk.has_value()) {
        const auto& t = *topk;
        TORCH_CHECK(t.is_cuda() && t.get_device() == device && t.scalar_type() == at::kLong && t.is_contiguous(),
                    "topk_idx must be a contiguous int64 tensor on this rank's GPU");
        TORCH_CHECK(t.dim() == 2 && t.size(0) == x.size(0) && t.size(1) == L.topk, "topk_idx must be [T, num_topk]");
    }
    if (weights.has_value()) {
        const auto& w = *weights;
        TORCH_CHECK(w.is_cuda() && w.get_device() == device && w.scalar_type() == at::kFloat && w.is_contiguous(),
                    "weights must be a contiguous float32 tensor on this rank's GPU");
        TORCH_CHECK(w.dim() == 2 && w.size(0) == x.size(0) && w.size(1) == L.topk, "weights must be [T, num_topk]");
    }
}

void check_meta_tensor(const at::Tensor& t, at::ScalarType dtype, at::IntArrayRef shape, int device, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.get_device() == device && t.scalar_type() == dtype && t.is_contiguous() && t.sizes() == shape,
                "handle metadata '", name, "' has the wrong device, dtype, shape or layout");
}

// [recv_metadata, expert_counts, expert_offsets, dst_slots, send_counts, topk_idx, recv_rank_prefix, slot_map]
void check_handle_meta(const std::vector<at::Tensor>& m, const WindowLayout& L, int64_t tokens, bool expand, int64_t capacity, int device) {
    TORCH_CHECK(m.size() == 8, "handle metadata must hold 8 tensors");
    const int64_t n = m[0].dim() == 2 ? m[0].size(0) : -1;
    TORCH_CHECK(n >= 0 && n <= int64_t(L.ranks) * L.max_tokens, "handle receive count out of range");
    check_meta_tensor(m[0], at::kInt, {n, L.topk + 2}, device, "recv_metadata");
    check_meta_tensor(m[1], at::kLong, {L.local_experts}, device, "expert_counts");
    check_meta_tensor(m[2], at::kLong, {L.local_experts + 1}, device, "expert_offsets");
    check_meta_tensor(m[3], at::kLong, {tokens, L.ranks}, device, "dst_slots");
    check_meta_tensor(m[4], at::kLong, {L.ranks}, device, "send_counts");
    check_meta_tensor(m[5], at::kLong, {tokens, L.topk}, device, "topk_idx");
    check_meta_tensor(m[6], at::kLong, {L.ranks}, device, "recv_rank_prefix");
    check_meta_tensor(m[7], at::kInt, {expand ? capacity : 0}, device, "slot_map");
}

// Upload a host array of parameter blocks for a multi-rank launch.  The device buffer comes from the
// comm stream's pool, so its reuse is ordered behind the launch that reads it.
template <typename P>
const P* upload(const std::vector<P>& host, std::vector<at::Tensor>& keep, cudaStream_t stream) {
    if (host.size() == 1) return host.data();
    auto buf = at::empty({int64_t(host.size() * sizeof(P))}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA));
    cuda_check(cudaMemcpyAsync(buf.data_ptr(), host.data(), host.size() * sizeof(P), cudaMemcpyHostToDevice, stream), "parameter upload");
    keep.push_back(buf);
    return static_cast<const P*>(buf.data_ptr());
}

struct Streams {
    c10::cuda::CUDAStream compute, comm;
    c10::cuda::CUDAStream work;  // where this operation's kernels run
};

// Asynchronous operations run on the buffer's communication stream behind the caller's stream (or
// behind `previous_event`).  Synchronous operations run directly on the caller's stream - no stream
// hop on either side, which is what small (decode-size) calls are made of - after whatever earlier
// asynchronous operation is still on the communication stream, so operations of one rank never overlap.
// A reusable event per thread for the stream hand-over below (creating and destroying an event per call
// costs microseconds, which small calls notice).
cudaEvent_t handover_event() {
    static thread_local cudaEvent_t event = nullptr;
    if (event == nullptr) cuda_check(cudaEventCreateWithFlags(&event, cudaEventDisableTiming), "cudaEventCreate");
    return event;
}

Streams order_inputs(const std::vector<PeerWindow*>& wins, int64_t comm_handle, int64_t previous_event, int device, bool async_op) {
    auto compute = c10::cuda::getCurrentCUDAStream(device);
    auto comm = c10::cuda::getStreamFromExternal(reinterpret_cast<cudaStream_t>(comm_handle), device);
    const c10::cuda::CUDAStream work = async_op ? comm : compute;
    if (async_op) {
        if (previous_event != -1) {
            cuda_check(cudaStreamWaitEvent(comm.stream(), reinterpret_cast<cudaEvent_t>(previous_event), 0), "wait previous_event");
        } else {
            cudaEvent_t ready = handover_event();
            cuda_check(cudaEventRecord(ready, compute.stream()), "record caller stream");
            cuda_check(cudaStreamWaitEvent(comm.stream(), ready, 0), "wait caller stream");
        }
    } else if (previous_event != -1) {
        cuda_check(cudaStreamWaitEvent(compute.stream(), reinterpret_cast<cudaEvent_t>(previous_event), 0), "wait previous_event");
    }
    // Behind the window's previous operation, whichever stream that ran on (free when it is the same stream).
    for (PeerWindow* w : wins) w->order_after_last(work.stream());
    return Streams{compute, comm, work};
}

// Every operation carries its barrier epoch and buffer parity as kernel arguments, so a captured
// launch could not be replayed; fail clearly instead of recording a graph that deadlocks later.
void reject_graph_capture(int device, const char* why) {
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    cuda_check(cudaStreamIsCapturing(c10::cuda::getCurrentCUDAStream(device).stream(), &capture), "capture query");
    TORCH_CHECK(capture == cudaStreamCaptureStatusNone, "nanoep_b200 operations cannot be captured in a CUDA graph: ", why);
}

void validate_group(const std::vector<PeerWindow*>& wins) {
    TORCH_CHECK(!wins.empty(), "no ranks given");
    const int n = int(wins.size());
    TORCH_CHECK(n == 1 || n == wins[0]->world(), "a multi-rank call must cover the whole logical group");
    for (int i = 0; i < n; ++i) {
        TORCH_CHECK(wins[i] != nullptr && !wins[i]->closed() && wins[i]->connected(), "peer window is closed or not connected");
        TORCH_CHECK(n == 1 || wins[i]->rank() == i, "logical ranks must be passed in rank order");
    }
}

std::shared_ptr<CompletionEvent> finish(const Streams& s, bool async_op, std::vector<at::Tensor> inputs, std::vector<at::Tensor> results) {
    if (!async_op) return nullptr;  // the work already sits on the caller's stream
    // Inputs were produced on another stream's pool; tell the allocator the comm stream used them.
    for (auto& t : inputs)
        if (t.defined() && t.numel() > 0) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), s.comm);
    auto done = std::make_shared<CompletionEvent>();
    done->event.record(s.comm);
    done->protect = std::move(results);
    return done;
}

}  // namespace

void CompletionEvent::wait(const c10::cuda::CUDAStream& stream) {
    event.block(stream);
    for (auto& t : protect)
        if (t.defined() && t.numel() > 0) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), stream);
}
void CompletionEvent::current_stream_wait() { wait(c10::cuda::getCurrentCUDAStream()); }
bool CompletionEvent::query() const { return event.query(); }

DispatchOut dispatch(const std::vector<PeerWindow*>& wins, const std::vector<at::Tensor>& xs,
                     const std::vector<c10::optional<at::Tensor>>& topks, const std::vector<c10::optional<at::Tensor>>& weights,
                     const std::vector<std::vector<at::Tensor>>& cached_meta, const std::vector<int64_t>& cached_capacity,
                     int64_t alignment, bool expand, bool zero_padding, int64_t num_sms, int64_t comm_stream, int64_t previous_event,
                     bool async_op, double mailbox_timeout_s, const std::vector<c10::optional<at::Tensor>>& tile_ready,
                     int64_t ring_smem_limit) {
    validate_group(wins);
    const int n = int(wins.size());
    TORCH_CHECK(int(xs.size()) == n && int(topks.size()) == n && int(weights.size()) == n && int(cached_meta.size()) == n &&
                    int(cached_capacity.size()) == n,
                "per-rank argument lists must have one entry per rank");
    const WindowLayout& L = wins[0]->layout();
    const int device = wins[0]->device();
    c10::cuda::CUDAGuard device_guard(device);
    const bool fresh = cached_meta[0].empty();
    const bool weighted = weights[0].has_value();
    TORCH_CHECK(alignment > 0 && alignment <= (int64_t(1) << 20), "alignment must be a positive integer");
    for (int i = 0; i < n; ++i) {
        TORCH_CHECK(cached_meta[i].empty() == fresh && weights[i].has_value() == weighted, "ranks disagree on cached/weights mode");
        TORCH_CHECK(fresh == topks[i].has_value(), "fresh dispatch needs topk_idx; cached dispatch uses the handle snapshot");
        check_payload(xs[i], topks[i], weights[i], L, device);
        if (!fresh) check_handle_meta(cached_meta[i], L, xs[i].size(0), expand, cached_capacity[i], device);
        wins[i]->check_status();
    }
    const DeviceLimits lim = device_limits();
    TORCH_CHECK(num_sms >= 1 && num_sms <= lim.sms, "num_sms out of range");
    // A smaller ring leaves shared memory for a compute kernel that shares the SMs with the pull.
    const int ring_budget = ring_smem_limit > 0 ? int(std::min<int64_t>(ring_smem_limit, lim.smem_optin)) : lim.smem_optin;
    const RingPlan ring = plan_ring(L.row_bytes(), ring_budget);
    TORCH_CHECK(ring.warps >= 1, "hidden size too large for the shared-memory row ring");
    reject_graph_capture(device, fresh ? "fresh dispatch waits for receive counts on the host" : "barrier epochs and buffer parities are kernel arguments");

    const Streams s = order_inputs(wins, comm_stream, previous_event, device, async_op);
    // Outputs live in the consumer stream's pool: the caller's stream when the call completes on it,
    // the comm stream when completion is handed over through an event.
    const c10::cuda::CUDAStream consumer = async_op ? s.comm : s.compute;
    const auto i64 = at::TensorOptions().dtype(at::kLong).device(at::kCUDA, device);
    const auto i32 = at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device);
    const auto f32 = at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, device);
    const auto bf16 = at::TensorOptions().dtype(at::kBFloat16).device(at::kCUDA, device);

    DispatchOut out;
    out.metadata.resize(n);
    out.outputs.resize(n);
    out.counts.resize(n);
    std::vector<at::Tensor> keep;
    std::vector<StageParams> stage(n);
    std::vector<int> parity(n);
    const cudaStream_t cs = s.work.stream();

    {
        c10::cuda::CUDAStreamGuard pool(consumer);
        for (int i = 0; i < n; ++i) {
            const int64_t T = xs[i].size(0);
            auto& m = out.metadata[i];
            if (fresh) {
                // one allocation, six views: allocator calls sit on the host's critical path of a small fresh dispatch
                m.resize(8);
                const int64_t Le = L.local_experts, R = L.ranks, K = L.topk;
                at::Tensor block = at::empty({Le + (Le + 1) + T * R + R + T * K + R}, i64);
                int64_t at_ = 0;
                auto take = [&](int64_t count) {
                    at::Tensor view = block.narrow(0, at_, count);
                    at_ += count;
                    return view;
                };
                m[1] = take(Le);
                m[2] = take(Le + 1);
                m[3] = take(T * R).view({T, R});
                m[4] = take(R);
                m[5] = take(T * K).view({T, K});
                m[6] = take(R);
            } else {
                m = cached_meta[i];
            }
            parity[i] = wins[i]->next_dispatch_parity();
            StageParams& p = stage[i];
            p.c = wins[i]->common();
            p.x = reinterpret_cast<const __nv_bfloat16*>(xs[i].data_ptr());
            p.topk = fresh ? topks[i]->data_ptr<int64_t>() : nullptr;
            p.weights = weighted ? weights[i]->data_ptr<float>() : nullptr;
            p.tokens = int(T);
            p.fresh = fresh;
            p.parity = parity[i];
            p.alignment = int(alignment);
            p.skip_copy = L.ranks == 1 ? 1 : 0;
            p.epoch = wins[i]->reserve_epochs(1);
            if (fresh) {
                p.snapshot = m[5].data_ptr<int64_t>();
                p.dst_slots = m[3].data_ptr<int64_t>();
                p.send_counts = m[4].data_ptr<int64_t>();
                p.recv_rank_prefix = m[6].data_ptr<int64_t>();
                p.expert_counts = m[1].data_ptr<int64_t>();
                p.expert_offsets = m[2].data_ptr<int64_t>();
                wins[i]->arm_mailbox();
                p.mailbox = wins[i]->mailbox_device();
                if (g_trace.enabled && n == 1) {
                    if (!g_trace.stage_words.defined())
                        g_trace.stage_words = at::empty({5}, at::TensorOptions().dtype(at::kLong).device(at::kCUDA, device));
                    p.trace = reinterpret_cast<unsigned long long*>(g_trace.stage_words.data_ptr<int64_t>());
                }
            }
        }
    }
    int64_t max_tokens_now = 0;
    for (int i = 0; i < n; ++i) max_tokens_now = std::max<int64_t>(max_tokens_now, xs[i].size(0));
    // Small cached calls: stage, peer barrier and pull go out as ONE cooperative launch.
    bool gated = false;
    for (const auto& t : tile_ready) gated = gated || t.has_value();
    const bool fuse_small = !fresh && !gated && max_tokens_now <= fused_dispatch_max_tokens();
    // Small fresh calls: stage, plan and pull as ONE cooperative launch writing into outputs sized at an upper bound
    // (every rank may send all of its Tmax tokens here), trimmed to N / C once the mailbox has them.  Only when that
    // bound is modest, i.e. for buffers configured for small batches.
    const int64_t bound_rows_n = int64_t(L.ranks) * L.max_tokens;
    const int64_t bound_rows_c = bound_rows_n * std::min<int64_t>(L.topk, L.local_experts) + int64_t(L.local_experts) * (alignment - 1);
    const int64_t bound_bytes = (expand ? bound_rows_c : bound_rows_n) * L.hidden * 2;
    const bool fuse_fresh = fresh && !gated && !g_gate.word.defined() && max_tokens_now <= fused_fresh_max_tokens() &&
                            bound_bytes <= kFusedFreshMaxOutputBytes && (!expand || bound_rows_c <= L.slot_scratch_ints) &&
                            ring.warps >= 2 && ring.smem_bytes >= size_t(stage_smem_bytes(L)) &&
                            ring.smem_bytes >= size_t(ring.warps) * 32 * L.topk * 4;
    const StageParams* stage_dev = nullptr;
    const PlanParams* plan_dev = nullptr;
    std::vector<PlanParams> plan(fresh ? n : 0);  // outlives the launches: a single-rank call passes it by host pointer
    {
        c10::cuda::CUDAStreamGuard on_comm(s.work);
        for (int i = 0; i < n; ++i) stage[i].fused = (fuse_small || fuse_fresh) ? 1 : 0;
        stage_dev = upload(stage, keep, cs);
        if (fresh && g_trace.enabled && n == 1) {
            const int64_t init[5] = {INT64_MAX, 0, 0, 0, 0};
            cuda_check(cudaMemcpyAsync(g_trace.stage_words.data_ptr(), init, sizeof(init), cudaMemcpyHostToDevice, cs), "trace reset");
        }
        g_marks.mark("begin", cs);
        if (!fuse_small && !fuse_fresh) {
            PeerWindow::launches += 1;
            // 16 warps per block, 4 row quarters per token: small calls get small grids
            const int stage_grid = int(std::max<int64_t>(1, std::min<int64_t>(2 * num_sms, (max_tokens_now * 4 + 15) / 16)));
            cuda_check(launch_stage(stage_dev, LaunchShape{stage_grid, n}, size_t(stage_smem_bytes(L)), cs), "stage launch");
            g_marks.mark("stage", cs);
        }
        if (fresh) {
            for (int i = 0; i < n; ++i) {
                plan[i].c = stage[i].c;
                plan[i].parity = parity[i];
                plan[i].expand = expand;
            }
            const int chunks = L.ranks * int((L.max_tokens + 31) / 32);
            const int grid = std::max(1, std::min((chunks + 7) / 8, 4 * lim.sms));
            plan_dev = upload(plan, keep, cs);
            if (!fuse_fresh) {
                PeerWindow::launches += 1;
                cuda_check(launch_plan(plan_dev, LaunchShape{grid, n}, size_t(plan_smem_bytes(L)), cs), "plan launch");
                g_marks.mark("plan", cs);
            }
        }
    }
    for (int i = 0; i < n; ++i) {
        if (fuse_fresh) {
            out.counts[i] = {bound_rows_n, expand ? bound_rows_c : 0};  // allocation sizes; the real counts follow the launch
        } else if (fresh) {
            std::pair<int64_t, int64_t> nc;
            {
                pybind11::gil_scoped_release release;
                nc = wins[i]->wait_mailbox(cs, mailbox_timeout_s);
            }
            out.counts[i] = {nc.first, nc.second};
        } else {
            out.counts[i] = {cached_meta[i][0].size(0), cached_capacity[i]};
        }
    }
    std::vector<PullParams> pull(n);
    {
        c10::cuda::CUDAStreamGuard pool(consumer);
        for (int i = 0; i < n; ++i) {
            const int64_t N = out.counts[i].first, C = out.counts[i].second;
            auto& m = out.metadata[i];
            if (fresh) {
                const int64_t cells = N * (L.topk + 2), slots = expand ? C : 0;
                at::Tensor block = at::empty({cells + slots}, i32);
                m[0] = block.narrow(0, 0, cells).view({N, L.topk + 2});
                m[7] = block.narrow(0, cells, slots);
            }
            auto& o = out.outputs[i];
            o.resize(3);
            o[0] = at::empty({expand ? C : N, L.hidden}, bf16);
            o[1] = expand ? at::empty({0}, i64) : at::empty({N, L.topk}, i64);
            o[2] = !weighted ? at::empty({0}, f32) : expand ? at::empty({C}, f32) : at::empty({N, L.topk}, f32);
            PullParams& p = pull[i];
            p.c = stage[i].c;
            p.meta = fresh ? reinterpret_cast<const int*>(static_cast<char*>(wins[i]->base()) + L.meta_scratch_offset) : m[0].data_ptr<int>();
            p.rows = int(N);
            p.parity = parity[i];
            p.data_epoch = (fresh && L.ranks > 1) ? stage[i].epoch : 0;  // a single-rank group pulls from the caller's tensor
            p.expand = expand;
            p.zero_padding = zero_padding;
            p.write_meta = fresh;
            p.stages = ring.stages;
            p.x_out = reinterpret_cast<__nv_bfloat16*>(o[0].data_ptr());
            p.topk_out = expand ? nullptr : o[1].data_ptr<int64_t>();
            p.w_out = weighted ? o[2].data_ptr<float>() : nullptr;
            p.meta_out = fresh ? m[0].data_ptr<int>() : nullptr;
            p.slot_map = (expand && fresh) ? m[7].data_ptr<int>() : nullptr;
            p.expert_counts = m[1].data_ptr<int64_t>();
            p.expert_offsets = m[2].data_ptr<int64_t>();
            p.recv_rank_prefix = m[6].data_ptr<int64_t>();
            p.x_local = reinterpret_cast<const __nv_bfloat16*>(xs[i].data_ptr());
            p.w_local = weighted ? weights[i]->data_ptr<float>() : nullptr;
            if (int(tile_ready.size()) == n && tile_ready[i].has_value()) {
                const auto& t = *tile_ready[i];
                TORCH_CHECK(expand && zero_padding, "tile counters need the expert-major layout with zero padding");
                TORCH_CHECK(t.is_cuda() && t.get_device() == device && t.scalar_type() == at::kInt && t.is_contiguous() &&
                                t.numel() * 128 >= C,
                            "tile_ready must be a zeroed CUDA int32 tensor with one entry per 128 expert-major rows");
                p.tile_ready = t.data_ptr<int>();
                // Consumers gated by the counters want row blocks to complete front to back.
                if (!fresh || C <= L.slot_scratch_ints) {
                    p.slot_src = fresh ? reinterpret_cast<const int*>(static_cast<char*>(wins[i]->base()) + L.slot_scratch_offset)
                                       : m[7].data_ptr<int>();
                    p.capacity = int(C);
                }
            }
        }
    }
    {
        c10::cuda::CUDAStreamGuard on_comm(s.work);
        const PullParams* dev = upload(pull, keep, cs);
        if (g_gate.word.defined())
            cuda_check(launch_gate(g_gate.word.data_ptr<int>(), uint64_t(g_gate.timeout_s * 1e9), cs), "test gate launch");
        g_marks.mark("host_gap", cs);
        PeerWindow::launches += 1;
        int64_t max_items = 1;
        for (int i = 0; i < n; ++i) max_items = std::max<int64_t>(max_items, expand ? out.counts[i].second : out.counts[i].first * L.ranks);
        const int pull_grid = int(std::max<int64_t>(1, std::min<int64_t>(num_sms, (max_items + ring.warps - 1) / ring.warps)));
        if (fuse_fresh) {
            const int64_t work = std::max<int64_t>(max_tokens_now * int64_t(L.ranks) * (expand ? std::min<int64_t>(L.topk, L.local_experts) : 1),
                                                   max_tokens_now * 4);
            const int fused_grid = int(std::max<int64_t>(1, std::min<int64_t>({int64_t(num_sms), int64_t(lim.sms / n), fused_max_blocks(),
                                                                               (work + ring.warps - 1) / ring.warps})));
            cuda_check(launch_fused_fresh_dispatch(stage_dev, plan_dev, dev, LaunchShape{fused_grid, n}, ring.warps, ring.smem_bytes, cs),
                       "fused fresh dispatch launch");
            g_marks.mark("fused_fresh_dispatch", cs);
        } else if (fuse_small) {
            // every block must be resident at once (one block per SM with this ring): bound the grid
            const int64_t work = std::max<int64_t>(max_items, max_tokens_now * 4);
            const int fused_grid = int(std::max<int64_t>(1, std::min<int64_t>({int64_t(num_sms), int64_t(lim.sms / n), fused_max_blocks(),
                                                                               (work + ring.warps - 1) / ring.warps})));
            cuda_check(launch_fused_cached_dispatch(stage_dev, dev, LaunchShape{fused_grid, n}, ring.warps, ring.smem_bytes, cs),
                       "fused cached dispatch launch");
            g_marks.mark("fused_dispatch", cs);
        } else {
            cuda_check(launch_pull(dev, LaunchShape{pull_grid, n}, ring.warps, ring.smem_bytes, cs), "pull launch");
            g_marks.mark("pull", cs);
        }
    }
    if (fuse_fresh) {
        // The kernel is on its way; now wait for N and C and trim the outputs to their exact sizes (leading-dimension
        // views of the bound-sized allocations: contiguous, same storage).
        for (int i = 0; i < n; ++i) {
            std::pair<int64_t, int64_t> nc;
            {
                pybind11::gil_scoped_release release;
                nc = wins[i]->wait_mailbox(cs, mailbox_timeout_s);
            }
            const int64_t N = nc.first, C = nc.second;
            TORCH_CHECK(N <= bound_rows_n && (!expand || C <= bound_rows_c), "receive counts exceed the single-launch bound");
            out.counts[i] = {N, C};
            auto& m = out.metadata[i];
            auto& o = out.outputs[i];
            m[0] = m[0].narrow(0, 0, N);
            if (expand) m[7] = m[7].narrow(0, 0, C);
            o[0] = o[0].narrow(0, 0, expand ? C : N);
            if (!expand) o[1] = o[1].narrow(0, 0, N);
            if (weighted) o[2] = o[2].narrow(0, 0, expand ? C : N);
        }
    }
    std::vector<at::Tensor> inputs, results;
    for (int i = 0; i < n; ++i) {
        inputs.push_back(xs[i]);
        if (topks[i].has_value()) inputs.push_back(*topks[i]);
        if (weighted) inputs.push_back(*weights[i]);
        for (auto& t : out.outputs[i]) results.push_back(t);
        for (auto& t : out.metadata[i]) results.push_back(t);
    }
    out.event = finish(s, async_op, std::move(inputs), std::move(results));
    return out;
}

CombineOut combine(const std::vector<PeerWindow*>& wins, const std::vector<at::Tensor>& xs, const std::vector<std::vector<at::Tensor>>& meta,
                   const std::vector<int64_t>& capacity, const std::vector<c10::optional<at::Tensor>>& weights,
                   const std::vector<c10::optional<at::Tensor>>& bias, bool expand, bool allow_multiple_reduction, int64_t num_sms,
                   int64_t comm_stream, int64_t previous_event, bool async_op) {
    validate_group(wins);
    const int n = int(wins.size());
    TORCH_CHECK(int(xs.size()) == n && int(meta.size()) == n && int(capacity.size()) == n && int(weights.size()) == n && int(bias.size()) == n,
                "per-rank argument lists must have one entry per rank");
    const WindowLayout& L = wins[0]->layout();
    const int device = wins[0]->device();
    c10::cuda::CUDAGuard device_guard(device);
    const bool weighted = weights[0].has_value();
    for (int i = 0; i < n; ++i) {
        const auto& m = meta[i];
        TORCH_CHECK(m.size() == 8, "handle metadata must hold 8 tensors");
        const int64_t T = m[5].dim() == 2 ? m[5].size(0) : -1;
        TORCH_CHECK(T >= 0 && T <= L.max_tokens, "handle source token count out of range");
        check_handle_meta(m, L, T, expand, capacity[i], device);
        const int64_t rows = expand ? capacity[i] : m[0].size(0);
        const auto& x = xs[i];
        TORCH_CHECK(x.is_cuda() && x.get_device() == device && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2 &&
                        x.size(0) == rows && x.size(1) == L.hidden,
                    "combine x must be contiguous CUDA bfloat16 with the handle's exact receive shape");
        TORCH_CHECK(x.numel() == 0 || reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "combine x must be 16-byte aligned");
        TORCH_CHECK(weights[i].has_value() == weighted, "ranks disagree on weights presence");
        if (weighted) {
            const auto& w = *weights[i];
            const bool shape_ok = expand ? (w.dim() == 1 && w.size(0) == rows) : (w.dim() == 2 && w.size(0) == rows && w.size(1) == L.topk);
            TORCH_CHECK(w.is_cuda() && w.get_device() == device && w.scalar_type() == at::kFloat && w.is_contiguous() && shape_ok,
                        "combine weights must be contiguous CUDA float32 with the handle's receive layout");
        }
        if (bias[i].has_value()) {
            const auto& b = *bias[i];
            TORCH_CHECK(b.is_cuda() && b.get_device() == device && b.scalar_type() == at::kBFloat16 && b.is_contiguous() && b.dim() == 2 &&
                            b.size(0) == T && b.size(1) == L.hidden,
                        "combine bias must be contiguous source [T,H] bfloat16 on this buffer's device");
            TORCH_CHECK(b.numel() == 0 || reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0, "combine bias must be 16-byte aligned");
        }
        wins[i]->check_status();
    }
    const DeviceLimits lim = device_limits();
    TORCH_CHECK(num_sms >= 1 && num_sms <= lim.sms, "num_sms out of range");
    // How the source-side sum runs: a positive setting = register path with that many warps per token; a negative one
    // = shared-memory pipeline, -(stages * 1000 + chunk bytes / 128) with chunk 0 = chosen by the plan; 0 = default.
    const int reduce_setting = g_trace.group != 0 ? g_trace.group : kDefaultReduceSetting;
    const int pipe_stages = reduce_setting < 0 ? (-reduce_setting) / 1000 : 0;
    const int pipe_chunk = reduce_setting < 0 ? ((-reduce_setting) % 1000) * 128 : 0;
    const CombinePlan plan = plan_combine(int64_t(L.hidden) * 2, L.ret_parts, lim.smem_optin, pipe_stages, pipe_chunk);
    const RingPlan ring = plan.ring;
    TORCH_CHECK(ring.warps >= 1, "hidden size too large for the shared-memory row ring");
    reject_graph_capture(device, "barrier epochs and buffer parities are kernel arguments");

    const Streams s = order_inputs(wins, comm_stream, previous_event, device, async_op);
    const c10::cuda::CUDAStream consumer = async_op ? s.comm : s.compute;
    const cudaStream_t cs = s.work.stream();
    const auto f32 = at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, device);
    const auto bf16 = at::TensorOptions().dtype(at::kBFloat16).device(at::kCUDA, device);

    CombineOut out;
    out.outputs.resize(n);
    if (L.ranks == 1) {
        // Everything is local: one kernel sums the expert outputs straight into the result.
        LocalCombineParams p{};
        {
            c10::cuda::CUDAStreamGuard pool(consumer);
            const auto& m = meta[0];
            const int64_t T = m[5].size(0);
            auto& o = out.outputs[0];
            o.resize(2);
            o[0] = at::empty({T, L.hidden}, bf16);
            o[1] = weighted ? at::empty({T, L.topk}, f32) : at::empty({0}, f32);
            p.c = wins[0]->common();
            p.y = reinterpret_cast<const __nv_bfloat16*>(xs[0].data_ptr());
            p.w = weighted ? weights[0]->data_ptr<float>() : nullptr;
            p.meta = m[0].data_ptr<int>();
            p.topk = m[5].data_ptr<int64_t>();
            p.bias = bias[0].has_value() ? reinterpret_cast<const __nv_bfloat16*>(bias[0]->data_ptr()) : nullptr;
            p.out = reinterpret_cast<__nv_bfloat16*>(o[0].data_ptr());
            p.w_out = weighted ? o[1].data_ptr<float>() : nullptr;
            p.rows = int(m[0].size(0));
            p.capacity = int(capacity[0]);
            p.tokens = int(T);
            p.expand = expand;
            p.round_partial = (expand && allow_multiple_reduction) ? 1 : 0;
        }
        {
            c10::cuda::CUDAStreamGuard on_comm(s.work);
            g_marks.mark("begin", cs);
            PeerWindow::launches += 1;
            cuda_check(launch_local_combine(&p, LaunchShape{2 * lim.sms, 1}, cs), "local combine launch");
            g_marks.mark("local_combine", cs);
        }
        std::vector<at::Tensor> inputs{xs[0]}, results;
        if (weighted) inputs.push_back(*weights[0]);
        if (bias[0].has_value()) inputs.push_back(*bias[0]);
        for (auto& t : meta[0]) inputs.push_back(t);
        for (auto& t : out.outputs[0]) results.push_back(t);
        out.event = finish(s, async_op, std::move(inputs), std::move(results));
        return out;
    }
    std::vector<CombineParams> params(n);
    std::vector<at::Tensor> keep;
    TORCH_CHECK(ring.stages >= 2 && ring.warps >= 1 && ring.warps <= 8, "combine ring plan out of range");
    {
        c10::cuda::CUDAStreamGuard pool(consumer);
        for (int i = 0; i < n; ++i) {
            const auto& m = meta[i];
            const int64_t T = m[5].size(0);
            const PeerWindow::CombineEpochs epochs = wins[i]->begin_combine();
            auto& o = out.outputs[i];
            o.resize(2);
            o[0] = at::empty({T, L.hidden}, bf16);
            o[1] = weighted ? at::empty({T, L.topk}, f32) : at::empty({0}, f32);
            CombineParams& p = params[i];
            p.c = wins[i]->common();
            p.y = reinterpret_cast<const __nv_bfloat16*>(xs[i].data_ptr());
            p.w = weighted ? weights[i]->data_ptr<float>() : nullptr;
            p.meta = m[0].data_ptr<int>();
            p.recv_rank_prefix = m[6].data_ptr<int64_t>();
            p.rows = int(m[0].size(0));
            p.capacity = int(capacity[i]);
            p.mode = !expand ? kPushCompact : allow_multiple_reduction ? kPushExpandedReduce : kPushExpanded;
            p.stages = ring.stages;
            p.push_warps = ring.warps;
            p.topk = m[5].data_ptr<int64_t>();
            p.bias = bias[i].has_value() ? reinterpret_cast<const __nv_bfloat16*>(bias[i]->data_ptr()) : nullptr;
            p.out = reinterpret_cast<__nv_bfloat16*>(o[0].data_ptr());
            p.w_out = weighted ? o[1].data_ptr<float>() : nullptr;
            p.tokens = int(T);
            p.sum_all_choices = (expand && !allow_multiple_reduction) ? 1 : 0;
            p.epoch = epochs.epoch;
            p.wait_epoch = epochs.wait_epoch;
            p.store_depth = g_trace.depth;
            // Register path: two reduce warps share a token (measured at 2 and 8 GPUs: one or two per token finish the
            // kernel soonest; larger groups hold fewer tokens at a time).
            p.reduce_group = reduce_setting > 0 ? reduce_setting : 2;
            p.reduce_stages = plan.reduce_stages;
            p.reduce_chunk_bytes = plan.reduce_chunk_bytes;
            if (g_trace.enabled && n == 1) {
                if (!g_trace.words.defined()) g_trace.words = at::empty({9}, at::TensorOptions().dtype(at::kLong).device(at::kCUDA, device));
                p.trace = reinterpret_cast<unsigned long long*>(g_trace.words.data_ptr<int64_t>());
            }
            TORCH_CHECK(p.sum_all_choices == 0 || L.ret_parts == L.topk, "this buffer's return area holds one partition per rank only");
        }
    }
    {
        c10::cuda::CUDAStreamGuard on_comm(s.work);
        int64_t max_transfers = 1, max_tokens_now = 1;
        for (int i = 0; i < n; ++i) {
            max_transfers = std::max<int64_t>(max_transfers, expand && !allow_multiple_reduction ? capacity[i] : meta[i][0].size(0));
            max_tokens_now = std::max<int64_t>(max_tokens_now, meta[i][5].size(0));
        }
        // Every block holds transfer warps and a group of reduce warps that sums one token at a time: enough blocks
        // for the larger of the two jobs.
        const int groups = plan.reduce_stages >= 2 ? 1 : std::max(1, (kCombineThreads / 32 - ring.warps - 1) / params[0].reduce_group);
        const int64_t wanted = std::max<int64_t>((max_transfers + ring.warps - 1) / ring.warps, (max_tokens_now + groups - 1) / groups);
        // A whole logical group in one launch waits on itself: all its blocks must be resident (cooperative launch).
        const bool group_launch = n > 1;
        const int64_t cap = group_launch ? std::min<int64_t>(num_sms, lim.sms / n) : num_sms;
        const int grid = int(std::max<int64_t>(1, std::min<int64_t>(cap, wanted)));
        const CombineParams* dev = upload(params, keep, cs);
        if (g_trace.enabled && n == 1) {
            const int64_t init[9] = {INT64_MAX, 0, 0, 0, 0, 0, 0, 0, 0};  // [0] takes the minimum, [1..3] and [7] the maximum, [4..6] are sums
            cuda_check(cudaMemcpyAsync(g_trace.words.data_ptr(), init, sizeof(init), cudaMemcpyHostToDevice, cs), "trace reset");
        }
        g_marks.mark("begin", cs);
        PeerWindow::launches += 1;
        cuda_check(launch_combine(dev, LaunchShape{grid, n}, ring.smem_bytes, cs, group_launch), "combine launch");
        g_marks.mark("combine", cs);
    }
    std::vector<at::Tensor> inputs, results;
    for (int i = 0; i < n; ++i) {
        inputs.push_back(xs[i]);
        if (weighted) inputs.push_back(*weights[i]);
        if (bias[i].has_value()) inputs.push_back(*bias[i]);
        for (auto& t : meta[i]) inputs.push_back(t);
        for (auto& t : out.outputs[i]) results.push_back(t);
    }
    out.event = finish(s, async_op, std::move(inputs), std::move(results));
    return out;
}

std::vector<at::Tensor> combine_finish(const std::vector<PeerWindow*>& wins, const std::vector<std::vector<at::Tensor>>& meta,
                                       const std::vector<c10::optional<at::Tensor>>& bias) {
    // Second half of a combine whose push was done by another kernel (the scatter epilogue of the
    // down-projection GEMM): peer barrier, then the source-side reduction, on the current stream.
    validate_group(wins);
    const int n = int(wins.size());
    TORCH_CHECK(int(meta.size()) == n && int(bias.size()) == n, "per-rank argument lists must have one entry per rank");
    const WindowLayout& L = wins[0]->layout();
    const int device = wins[0]->device();
    c10::cuda::CUDAGuard device_guard(device);
    const cudaStream_t cs = c10::cuda::getCurrentCUDAStream(device).stream();
    for (PeerWindow* w : wins) w->order_after_last(cs);
    const DeviceLimits lim = device_limits();
    std::vector<BarrierParams> barrier(n);
    std::vector<ReduceParams> reduce(n);
    std::vector<at::Tensor> outs(n), keep;
    for (int i = 0; i < n; ++i) {
        TORCH_CHECK(meta[i].size() == 8, "handle metadata must hold 8 tensors");
        const int64_t T = meta[i][5].size(0);
        wins[i]->check_status();
        barrier[i].c = wins[i]->common();
        barrier[i].epoch = wins[i]->reserve_epochs(1);
        TORCH_CHECK(L.ret_parts == L.topk, "this buffer's return area holds one partition per rank only");
        outs[i] = at::empty({T, L.hidden}, at::TensorOptions().dtype(at::kBFloat16).device(at::kCUDA, device));
        ReduceParams& r = reduce[i];
        r.c = barrier[i].c;
        r.topk = meta[i][5].data_ptr<int64_t>();
        if (bias[i].has_value()) {
            const auto& b = *bias[i];
            TORCH_CHECK(b.is_cuda() && b.scalar_type() == at::kBFloat16 && b.is_contiguous() && b.dim() == 2 && b.size(0) == T &&
                            b.size(1) == L.hidden,
                        "bias must be contiguous source [T,H] bfloat16");
            r.bias = reinterpret_cast<const __nv_bfloat16*>(b.data_ptr());
        }
        r.out = reinterpret_cast<__nv_bfloat16*>(outs[i].data_ptr());
        r.tokens = int(T);
        r.sum_all_choices = 1;
    }
    const BarrierParams* bdev = upload(barrier, keep, cs);
    PeerWindow::launches += 1;
    cuda_check(launch_barrier(bdev, LaunchShape{1, n}, cs), "barrier launch");
    const ReduceParams* rdev = upload(reduce, keep, cs);
    PeerWindow::launches += 1;
    cuda_check(launch_reduce(rdev, LaunchShape{2 * lim.sms, n}, cs), "reduce launch");
    // Tell every peer that this rank has finished reading its return area (nobody waits): the next combine kernel
    // waits for this epoch before it overwrites the area, exactly as it does after a combine kernel.
    std::vector<BarrierParams> done(n);
    for (int i = 0; i < n; ++i) {
        done[i].c = barrier[i].c;
        done[i].epoch = wins[i]->begin_combine().epoch;
        done[i].signal_only = 1;
    }
    const BarrierParams* ddev = upload(done, keep, cs);
    PeerWindow::launches += 1;
    cuda_check(launch_barrier(ddev, LaunchShape{1, n}, cs), "end-of-combine signal launch");
    return outs;
}

FusedLimits fused_limits() { return FusedLimits{fused_dispatch_max_tokens(), fused_max_blocks(), fused_fresh_max_tokens()}; }

void set_fused_limits(int64_t dispatch_tokens, int64_t blocks, int64_t fresh_tokens) {
    if (dispatch_tokens >= 0) fused_state().dispatch_tokens = dispatch_tokens;
    if (fresh_tokens >= 0) fused_state().fresh_tokens = fresh_tokens;
    if (blocks >= 1) fused_state().blocks = blocks;
}

void set_phase_timing(bool enabled) { g_marks.enabled = enabled; }

void set_test_gate(const c10::optional<at::Tensor>& word, double timeout_s) {
    if (!word.has_value()) {
        g_gate.word = at::Tensor();
        return;
    }
    TORCH_CHECK(word->is_pinned() && word->scalar_type() == at::kInt && word->numel() >= 2 && word->is_contiguous(),
                "the gate word must be a pinned host int32 tensor with two entries");
    g_gate.word = *word;
    g_gate.timeout_s = timeout_s;
}

void set_combine_trace(bool enabled, int64_t store_depth, int64_t reduce_group) {
    g_trace.enabled = enabled;
    g_trace.depth = int(store_depth);
    g_trace.group = int(reduce_group);
}

std::vector<double> take_stage_trace() {
    std::vector<double> out;
    if (!g_trace.stage_words.defined()) return out;
    const at::Tensor host = g_trace.stage_words.cpu();
    const int64_t* w = host.data_ptr<int64_t>();
    if (w[0] == INT64_MAX) return out;
    for (int i = 1; i < 5; ++i) out.push_back(w[i] > w[0] ? double(w[i] - w[0]) * 1e-3 : 0.0);
    return out;
}

std::vector<double> take_combine_trace() {
    std::vector<double> out;
    if (!g_trace.words.defined()) return out;
    const at::Tensor host = g_trace.words.cpu();  // synchronises with the stream that ran the combine
    const int64_t* w = host.data_ptr<int64_t>();
    if (w[0] == INT64_MAX) return out;
    for (int i = 1; i < 4; ++i) out.push_back(w[i] > w[0] ? double(w[i] - w[0]) * 1e-3 : 0.0);
    // reduce groups: microseconds waited and summed (totals over all groups), tokens summed, longest token
    out.push_back(double(w[4]) * 1e-3);
    out.push_back(double(w[5]) * 1e-3);
    out.push_back(double(w[6]));
    out.push_back(double(uint64_t(w[7]) >> 32) * 1e-3);
    out.push_back(double(uint64_t(w[7]) & 0xffffffffull) * 1e-3);  // when that token started
    out.push_back(w[8] > w[0] ? double(w[8] - w[0]) * 1e-3 : 0.0);  // when the last token's rows were seen
    return out;
}

std::vector<std::pair<std::string, double>> take_phase_timings() {
    std::vector<std::pair<std::string, double>> out;
    auto& m = g_marks.marks;
    if (!m.empty()) cuda_check(cudaEventSynchronize(m.back().second), "phase timing sync");
    for (size_t i = 0; i < m.size(); ++i) {
        if (m[i].first != "begin" && i > 0) {
            float ms = 0.f;
            cuda_check(cudaEventElapsedTime(&ms, m[i - 1].second, m[i].second), "cudaEventElapsedTime");
            out.emplace_back(m[i].first, double(ms) * 1e3);
        }
    }
    for (auto& e : m) g_marks.pool.push_back(e.second);
    m.clear();
    return out;
}

void group_barrier(const std::vector<PeerWindow*>& wins, int64_t stream) {
    validate_group(wins);
    const int n = int(wins.size());
    c10::cuda::CUDAGuard device_guard(wins[0]->device());
    const cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
    if (n == 1) {
        wins[0]->barrier(cs);
        return;
    }
    std::vector<BarrierParams> b(n);
    for (int i = 0; i < n; ++i) {
        wins[i]->order_after_last(cs);
        b[i].c = wins[i]->common();
        b[i].epoch = wins[i]->reserve_epochs(1);
    }
    std::vector<at::Tensor> keep;
    c10::cuda::CUDAStreamGuard on(c10::cuda::getStreamFromExternal(cs, wins[0]->device()));
    const BarrierParams* dev = upload(b, keep, cs);
    PeerWindow::launches += 1;
    cuda_check(launch_barrier(dev, LaunchShape{1, n}, cs), "barrier launch");
}

}  // namespace nep
