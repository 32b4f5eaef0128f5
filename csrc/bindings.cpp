// pybind11 module `nanoep_b200._C`: PeerWindow, CompletionEvent, dispatch/combine, layout and
// diagnostics.  Same boundary as the reference's csrc/bindings.cpp:11-86.
#include <torch/extension.h>

#include "gemm_api.hpp"
#include "pipeline.hpp"

namespace py = pybind11;
using nep::PeerWindow;

namespace {

// Routing metadata of one handle kept on the native side, so that cached dispatch and combine pass
// one opaque object instead of converting eight tensors in and out of Python on every call.
struct HandleState {
    std::vector<at::Tensor> metadata;  // same order as DispatchOut::metadata
    int64_t capacity;
    bool expand;
};

py::dict layout_dict(const nep::WindowLayout& w) {
    py::dict d;
    d["signal_offset"] = w.signal_offset;
    d["data_signal_offset"] = w.data_signal_offset;
    d["ctrl_offset"] = w.ctrl_offset;
    d["counts_in_offset"] = w.counts_in_offset;
    d["counts_in_stride"] = w.counts_in_stride;
    d["routing_in_offset"] = w.routing_in_offset;
    d["routing_in_stride"] = w.routing_in_stride;
    d["chunks_in_offset"] = w.chunks_in_offset;
    d["chunks_in_stride"] = w.chunks_in_stride;
    d["stage_rows_offset"] = w.stage_rows_offset;
    d["stage_rows_stride"] = w.stage_rows_stride;
    d["ret_parts"] = w.ret_parts;
    d["rank_indexed"] = w.rank_indexed;
    d["ret_w_offset"] = w.ret_w_offset;
    d["ret_flag_offset"] = w.ret_flag_offset;
    d["ret_offset"] = w.ret_offset;
    d["meta_scratch_offset"] = w.meta_scratch_offset;
    d["slot_scratch_offset"] = w.slot_scratch_offset;
    d["num_bytes"] = w.num_bytes;
    d["row_bytes"] = w.row_bytes();
    d["msg_ints"] = w.msg_ints();
    return d;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "nanoep_b200 native runtime (sm_100a)";

    m.def(
        "window_layout",
        [](int ranks, int64_t max_tokens, int hidden, int topk, int64_t num_experts, bool per_rank_reduction) {
            return layout_dict(nep::WindowLayout::make(ranks, max_tokens, hidden, topk, num_experts, per_rank_reduction));
        },
        py::arg("ranks"), py::arg("max_tokens"), py::arg("hidden"), py::arg("topk"), py::arg("num_experts"),
        py::arg("per_rank_reduction") = false);

    py::class_<PeerWindow>(m, "PeerWindow")
        .def(py::init([](int rank, int world, int64_t max_tokens, int hidden, int topk, int64_t num_experts, double wait_timeout_s,
                         bool per_rank_reduction) {
                 return new PeerWindow(rank, world, nep::WindowLayout::make(world, max_tokens, hidden, topk, num_experts, per_rank_reduction),
                                       wait_timeout_s);
             }),
             py::arg("rank"), py::arg("world"), py::arg("max_tokens"), py::arg("hidden"), py::arg("topk"), py::arg("num_experts"),
             py::arg("wait_timeout_s") = 10.0, py::arg("per_rank_reduction") = false)
        .def_property_readonly("rank", &PeerWindow::rank)
        .def_property_readonly("world", &PeerWindow::world)
        .def_property_readonly("device", &PeerWindow::device)
        .def_property_readonly("num_bytes", &PeerWindow::num_bytes)
        .def_property_readonly("connected", &PeerWindow::connected)
        .def_property_readonly("closed", &PeerWindow::closed)
        .def_property_readonly("last_epoch", &PeerWindow::last_epoch)
        .def_property_readonly("status_code", &PeerWindow::status_code)
        .def("layout", [](const PeerWindow& w) { return layout_dict(w.layout()); })
        .def("export_handle", [](PeerWindow& w) { return py::bytes(w.export_handle()); })
        .def("import_handles",
             [](PeerWindow& w, const std::vector<py::bytes>& handles, const std::vector<int>& peer_devices) {
                 std::vector<std::string> raw;
                 for (const auto& h : handles) raw.emplace_back(std::string(h));
                 w.import_handles(raw, peer_devices);
             },
             py::arg("handles"), py::arg("peer_devices") = std::vector<int>{})
        .def("adopt_peers", &PeerWindow::adopt_peers)
        .def("close_peer_mappings", &PeerWindow::close_peer_mappings)
        .def("close", &PeerWindow::close)
        .def("reserve_epochs", &PeerWindow::reserve_epochs)
        .def("set_wait_timeout", &PeerWindow::set_wait_timeout)
        .def("check_status", &PeerWindow::check_status)
        .def("clear_status", [](PeerWindow& w, int64_t stream) { w.clear_status(reinterpret_cast<cudaStream_t>(stream)); })
        .def("barrier", [](PeerWindow& w, int64_t stream) { w.barrier(reinterpret_cast<cudaStream_t>(stream)); })
        .def("local_window", [](PeerWindow& w) {
            // Borrowed uint8 view of the whole window (tests and diagnostics); invalid after close().
            return at::from_blob(w.base(), {w.num_bytes()}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, w.device()));
        });

    py::class_<nep::CompletionEvent, std::shared_ptr<nep::CompletionEvent>>(m, "CompletionEvent")
        .def("current_stream_wait", &nep::CompletionEvent::current_stream_wait)
        .def("wait_stream", [](nep::CompletionEvent& e, int64_t stream, int device) {
            e.wait(c10::cuda::getStreamFromExternal(reinterpret_cast<cudaStream_t>(stream), device));
        })
        .def("query", &nep::CompletionEvent::query);

    m.def(
        "dispatch",
        [](const std::vector<PeerWindow*>& wins, const std::vector<at::Tensor>& xs, const std::vector<c10::optional<at::Tensor>>& topks,
           const std::vector<c10::optional<at::Tensor>>& weights, const std::vector<std::vector<at::Tensor>>& cached_meta,
           const std::vector<int64_t>& cached_capacity, int64_t alignment, bool expand, bool zero_padding, int64_t num_sms,
           int64_t comm_stream, int64_t previous_event, bool async_op, double mailbox_timeout_s,
           const std::vector<c10::optional<at::Tensor>>& tile_ready, int64_t ring_smem_limit) {
            auto out = nep::dispatch(wins, xs, topks, weights, cached_meta, cached_capacity, alignment, expand, zero_padding, num_sms,
                                     comm_stream, previous_event, async_op, mailbox_timeout_s, tile_ready, ring_smem_limit);
            return py::make_tuple(out.outputs, out.metadata, out.counts, out.event);
        },
        py::arg("windows"), py::arg("x"), py::arg("topk_idx"), py::arg("weights"), py::arg("cached_metadata"), py::arg("cached_capacity"),
        py::arg("alignment"), py::arg("expand"), py::arg("zero_padding"), py::arg("num_sms"), py::arg("comm_stream"),
        py::arg("previous_event"), py::arg("async_op"), py::arg("mailbox_timeout_s") = 60.0,
        py::arg("tile_ready") = std::vector<c10::optional<at::Tensor>>{}, py::arg("ring_smem_limit") = 0);

    m.def(
        "combine",
        [](const std::vector<PeerWindow*>& wins, const std::vector<at::Tensor>& xs, const std::vector<std::vector<at::Tensor>>& meta,
           const std::vector<int64_t>& capacity, const std::vector<c10::optional<at::Tensor>>& weights,
           const std::vector<c10::optional<at::Tensor>>& bias, bool expand, bool allow_multiple_reduction, int64_t num_sms,
           int64_t comm_stream, int64_t previous_event, bool async_op) {
            auto out = nep::combine(wins, xs, meta, capacity, weights, bias, expand, allow_multiple_reduction, num_sms, comm_stream,
                                    previous_event, async_op);
            return py::make_tuple(out.outputs, out.event);
        },
        py::arg("windows"), py::arg("x"), py::arg("metadata"), py::arg("capacity"), py::arg("weights"), py::arg("bias"), py::arg("expand"),
        py::arg("allow_multiple_reduction"), py::arg("num_sms"), py::arg("comm_stream"), py::arg("previous_event"), py::arg("async_op"));

    py::class_<HandleState, std::shared_ptr<HandleState>>(m, "HandleState")
        .def(py::init([](std::vector<at::Tensor> metadata, int64_t capacity, bool expand) {
            return std::make_shared<HandleState>(HandleState{std::move(metadata), capacity, expand});
        }))
        .def_readonly("metadata", &HandleState::metadata)
        .def_readonly("capacity", &HandleState::capacity)
        .def_readonly("expand", &HandleState::expand);

    // Single-rank fast paths (the list-based entry points above stay the general interface).
    m.def(
        "dispatch_cached",
        [](PeerWindow& window, const at::Tensor& x, const c10::optional<at::Tensor>& weights, const std::shared_ptr<HandleState>& state,
           bool zero_padding, int64_t num_sms, int64_t comm_stream, int64_t previous_event, bool async_op, double mailbox_timeout_s,
           const c10::optional<at::Tensor>& tile_ready, int64_t ring_smem_limit) {
            auto out = nep::dispatch({&window}, {x}, {c10::nullopt}, {weights}, {state->metadata}, {state->capacity}, 1, state->expand,
                                     zero_padding, num_sms, comm_stream, previous_event, async_op, mailbox_timeout_s, {tile_ready},
                                     ring_smem_limit);
            auto& o = out.outputs[0];
            return py::make_tuple(o[0], o[1], o[2], out.event);
        },
        py::arg("window"), py::arg("x"), py::arg("weights"), py::arg("state"), py::arg("zero_padding"), py::arg("num_sms"),
        py::arg("comm_stream"), py::arg("previous_event"), py::arg("async_op"), py::arg("mailbox_timeout_s") = 60.0,
        py::arg("tile_ready") = c10::nullopt, py::arg("ring_smem_limit") = 0);
    m.def(
        "combine_single",
        [](PeerWindow& window, const at::Tensor& x, const std::shared_ptr<HandleState>& state, const c10::optional<at::Tensor>& weights,
           const c10::optional<at::Tensor>& bias, bool allow_multiple_reduction, int64_t num_sms, int64_t comm_stream, int64_t previous_event,
           bool async_op) {
            auto out = nep::combine({&window}, {x}, {state->metadata}, {state->capacity}, {weights}, {bias}, state->expand,
                                    allow_multiple_reduction, num_sms, comm_stream, previous_event, async_op);
            return py::make_tuple(out.outputs[0][0], out.outputs[0][1], out.event);
        },
        py::arg("window"), py::arg("x"), py::arg("state"), py::arg("weights"), py::arg("bias"), py::arg("allow_multiple_reduction"),
        py::arg("num_sms"), py::arg("comm_stream"), py::arg("previous_event"), py::arg("async_op"));

    m.def("combine_finish", &nep::combine_finish);
    m.def("group_barrier", &nep::group_barrier);
    m.def("fused_limits", [] {
        const nep::FusedLimits f = nep::fused_limits();
        return py::make_tuple(f.dispatch_tokens, f.blocks, f.fresh_tokens);
    });
    m.def("set_fused_limits", &nep::set_fused_limits, py::arg("dispatch_tokens") = -1, py::arg("blocks") = -1, py::arg("fresh_tokens") = -1);
    m.def("set_test_gate", &nep::set_test_gate, py::arg("word"), py::arg("timeout_s") = 10.0);
    m.def("set_phase_timing", &nep::set_phase_timing);
    m.def(
        "combine_plan",
        [](int64_t hidden, int64_t parts, int64_t max_smem_bytes, int64_t reduce_stages, int64_t reduce_chunk_bytes) {
            const nep::CombinePlan plan = nep::plan_combine(hidden * 2, int(parts), int(max_smem_bytes), int(reduce_stages), int(reduce_chunk_bytes));
            return std::make_tuple(plan.ring.warps, plan.ring.stages, int64_t(plan.ring.smem_bytes), plan.reduce_stages, plan.reduce_chunk_bytes);
        },
        py::arg("hidden"), py::arg("parts"), py::arg("max_smem_bytes"), py::arg("reduce_stages") = 2, py::arg("reduce_chunk_bytes") = 0,
        "Shared-memory plan of a combine CTA: (transfer warps, ring stages, dynamic bytes, reduce stages, reduce chunk bytes)");
    m.def("set_combine_trace", &nep::set_combine_trace, py::arg("enabled"), py::arg("store_depth") = 0, py::arg("reduce_group") = 0);
    m.def("take_combine_trace", &nep::take_combine_trace);
    m.def("take_stage_trace", &nep::take_stage_trace);
    m.def("take_phase_timings", &nep::take_phase_timings);
    m.def("launch_count", [] { return PeerWindow::launches; });
    m.def("format_status", &nep::format_status);
    m.def("peer_access_error", &nep::peer_access_error, py::arg("own_rank"), py::arg("peer_rank"), py::arg("own_device"),
          py::arg("peer_device"), py::arg("can_access"), py::arg("access_supported"));
    m.def("status_name", [](uint32_t code) { return std::string(nep::status_name(code)); });
    m.def("kernel_table", [] {
        nep::KernelInfo info[32];
        const int n = nep::kernel_table(info, 32);
        py::list out;
        for (int i = 0; i < n; ++i) {
            py::dict d;
            d["name"] = info[i].name;
            d["registers"] = info[i].regs;
            d["static_smem"] = info[i].static_smem;
            d["max_threads"] = info[i].max_threads;
            out.append(d);
        }
        return out;
    });

    nep::bind_gemm(m);
}
