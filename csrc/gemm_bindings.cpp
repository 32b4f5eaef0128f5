// Python bindings of the tcgen05 grouped GEMM and helpers (tensor-map construction lives here).
#include "gemm_api.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "grouped_gemm_sm100.hpp"
#include "peer_window.hpp"

namespace nep {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result);
        TORCH_CHECK(e == cudaSuccess && result == cudaDriverEntryPointSuccess && ptr != nullptr, "cuTensorMapEncodeTiled is not available");
        return reinterpret_cast<EncodeFn>(ptr);
    }();
    return fn;
}

// Row-major bf16 [rows, cols]; box = 64 columns (128 bytes, one swizzle row) x 128 rows.
CUtensorMap make_map(const void* base, int64_t rows, int64_t cols) {
    TORCH_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0 && (cols * 2) % 16 == 0, "TMA operand must be 16-byte aligned with 16-byte row pitch");
    CUtensorMap map;
    const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(cols) * 2};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed");
    return map;
}

void check_bf16(const at::Tensor& t, int dims, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.dim() == dims, name,
                " must be a contiguous CUDA bfloat16 tensor of the expected rank");
}

struct GemmCommon {
    gemm::Args args{};
    CUtensorMap map_a, map_b;
    int grid = 0;
};

GemmCommon prepare(const at::Tensor& a, const at::Tensor& w, const at::Tensor& expert_offsets, const at::Tensor& status, int mode,
                   double timeout_s) {
    check_bf16(a, 2, "activations");
    check_bf16(w, 3, "weights");
    TORCH_CHECK(expert_offsets.is_cuda() && expert_offsets.scalar_type() == at::kLong && expert_offsets.is_contiguous() &&
                    expert_offsets.dim() == 1 && expert_offsets.size(0) == w.size(0) + 1,
                "expert_offsets must be a CUDA int64 tensor of num_experts + 1 entries");
    TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 2, "status must be a CUDA int32 tensor");
    const int64_t rows = a.size(0), K = a.size(1), E = w.size(0), NW = w.size(1);
    TORCH_CHECK(w.size(2) == K, "weights must be [experts, N, K] with the activations' K");
    TORCH_CHECK(rows % 128 == 0, "row count must be a multiple of 128 (dispatch with alignment=128)");
    TORCH_CHECK(K % 64 == 0 && K >= 64, "K must be a multiple of 64");
    TORCH_CHECK(E >= 1 && E <= 1024, "1..1024 experts per rank");
    GemmCommon g;
    g.args.expert_offsets = expert_offsets.data_ptr<int64_t>();
    g.args.num_experts = int(E);
    g.args.m_blocks = int(rows / 128);
    g.args.k_blocks = int(K / 64);
    g.args.b_rows_per_expert = int(NW);
    if (mode == gemm::kSwiGLU) {
        TORCH_CHECK(NW % 256 == 0, "SwiGLU weight must be [experts, 2*I, K] with I a multiple of 128");
        g.args.swiglu_up_row_offset = int(NW / 2);
        g.args.n_tiles = int(NW / 2 / 128);
    } else {
        TORCH_CHECK(NW % 256 == 0, "N must be a multiple of 256");
        g.args.n_tiles = int(NW / 256);
    }
    g.args.status = reinterpret_cast<uint32_t*>(status.data_ptr<int>());
    g.args.timeout_ns = uint64_t(timeout_s * 1e9);
    if (rows > 0) g.map_a = make_map(a.data_ptr(), rows, K);
    g.map_b = make_map(w.data_ptr(), E * NW, K);
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    g.grid = std::max(1, std::min(sms, g.args.m_blocks * g.args.n_tiles));
    return g;
}

}  // namespace

void bind_gemm(pybind11::module_& m) {
    // out = A @ W[e]^T per 128-row block (mode 0) or silu(gate) * up with W = [E, 2I, K] (mode 1).
    m.def(
        "grouped_gemm",
        [](const at::Tensor& a, const at::Tensor& w, const at::Tensor& expert_offsets, at::Tensor& out, at::Tensor& status, int64_t mode,
           c10::optional<at::Tensor> tile_ready, c10::optional<at::Tensor> tile_expected, int64_t max_ctas, double timeout_s,
           c10::optional<at::Tensor> row_scale, int64_t stages, bool pair) {
            c10::cuda::CUDAGuard guard(a.device());
            TORCH_CHECK(mode == gemm::kPlain || mode == gemm::kSwiGLU, "mode must be 0 (plain) or 1 (SwiGLU)");
            auto g = prepare(a, w, expert_offsets, status, int(mode), timeout_s);
            check_bf16(out, 2, "out");
            const int64_t n_out = mode == gemm::kSwiGLU ? w.size(1) / 2 : w.size(1);
            TORCH_CHECK(out.size(0) == a.size(0) && out.size(1) == n_out, "out has the wrong shape");
            g.args.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
            g.args.ldo = int(n_out);
            if (tile_ready.has_value()) {
                TORCH_CHECK(tile_expected.has_value() && tile_ready->scalar_type() == at::kInt && tile_expected->scalar_type() == at::kInt &&
                                tile_ready->numel() >= g.args.m_blocks && tile_expected->numel() >= g.args.m_blocks &&
                                tile_ready->is_cuda() && tile_expected->is_cuda() && tile_ready->device() == a.device() &&
                                tile_expected->device() == a.device() && tile_ready->is_contiguous() && tile_expected->is_contiguous(),
                            "tile_ready/tile_expected must be contiguous int32 tensors on the activations' device with one entry per 128-row block");
                g.args.tile_ready = tile_ready->data_ptr<int>();
                g.args.tile_expected = tile_expected->data_ptr<int>();
            }
            if (row_scale.has_value()) {
                TORCH_CHECK(mode == gemm::kPlain && row_scale->is_cuda() && row_scale->scalar_type() == at::kFloat &&
                                row_scale->is_contiguous() && row_scale->numel() == a.size(0),
                            "row_scale must be float32 [rows] (plain mode only)");
                g.args.row_scale = row_scale->data_ptr<float>();
            }
            TORCH_CHECK(stages == 3 || stages == 4, "stages must be 3 or 4 (single-CTA) or 4 for the gated CTA-pair kernel");
            if (a.size(0) == 0) return;
            const int grid = max_ctas > 0 ? std::min<int>(g.grid, int(max_ctas)) : g.grid;
            PeerWindow::launches += 1;
            if (pair) {
                const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
                const int pair_grid = max_ctas > 0 ? std::min<int>(sms, int(max_ctas)) : sms;
                // gated by tile counters = meant to share the SMs with the pull kernel: shorter pipeline
                cudaError_t pe = gemm::launch_pair(g.map_a, g.map_b, g.args, int(mode), pair_grid, c10::cuda::getCurrentCUDAStream().stream(),
                                                   tile_ready.has_value() ? 4 : 6);
                TORCH_CHECK(pe == cudaSuccess, "grouped GEMM (CTA pairs) launch failed: ", cudaGetErrorString(pe));
                return;
            }
            cudaError_t e = gemm::launch(g.map_a, g.map_b, g.args, int(mode), int(stages), grid, c10::cuda::getCurrentCUDAStream().stream());
            TORCH_CHECK(e == cudaSuccess, "grouped GEMM launch failed: ", cudaGetErrorString(e));
        },
        pybind11::arg("a"), pybind11::arg("w"), pybind11::arg("expert_offsets"), pybind11::arg("out"), pybind11::arg("status"),
        pybind11::arg("mode"), pybind11::arg("tile_ready") = c10::nullopt, pybind11::arg("tile_expected") = c10::nullopt,
        pybind11::arg("max_ctas") = 0, pybind11::arg("timeout_s") = 5.0, pybind11::arg("row_scale") = c10::nullopt,
        pybind11::arg("stages") = 4, pybind11::arg("pair") = false);

    // Down projection fused with the combine push: row r of (A @ W[e]^T) * slot_weight[r] is stored
    // (bf16) into the return partition of the row's source rank; padding rows are skipped.  The return area
    // exists once: a dispatch (whose peer barrier every rank passes only after its previous reduction) must lie
    // between two such calls, as it does in a layer's forward pass.
    m.def(
        "grouped_gemm_scatter",
        [](PeerWindow& window, const at::Tensor& a, const at::Tensor& w, const at::Tensor& expert_offsets,
           const at::Tensor& slot_map, const at::Tensor& recv_metadata, c10::optional<at::Tensor> slot_weights, at::Tensor& status,
           int64_t max_ctas, double timeout_s, bool pair) {
            c10::cuda::CUDAGuard guard(a.device());
            auto g = prepare(a, w, expert_offsets, status, gemm::kScatter, timeout_s);
            const WindowLayout& L = window.layout();
            TORCH_CHECK(w.size(1) == L.hidden, "down-projection N must equal the buffer's hidden size");
            TORCH_CHECK(slot_map.is_cuda() && slot_map.scalar_type() == at::kInt && slot_map.numel() == a.size(0) && slot_map.is_contiguous(),
                        "slot_map must be contiguous int32 [rows]");
            TORCH_CHECK(recv_metadata.is_cuda() && recv_metadata.scalar_type() == at::kInt && recv_metadata.dim() == 2 &&
                            recv_metadata.size(1) == L.topk + 2 && recv_metadata.is_contiguous(),
                        "recv_metadata must be int32 [N, topk + 2]");
            g.args.slot_map = slot_map.data_ptr<int>();
            g.args.recv_metadata = recv_metadata.data_ptr<int>();
            if (slot_weights.has_value()) {
                TORCH_CHECK(slot_weights->is_cuda() && slot_weights->scalar_type() == at::kFloat && slot_weights->numel() == a.size(0),
                            "slot_weights must be float32 [rows]");
                g.args.slot_weights = slot_weights->data_ptr<float>();
            }
            const CommonParams c = window.common();
            for (int p = 0; p < kMaxRanks; ++p) g.args.peers[p] = c.peers[p];
            TORCH_CHECK(L.ret_parts == L.topk, "the fused combine epilogue needs one return partition per choice (allow_multiple_reduction=False)");
            g.args.ret_offset = L.ret_offset;
            g.args.max_tokens = L.max_tokens;
            g.args.topk = L.topk;
            g.args.ranks = L.ranks;
            g.args.recv_rows = int(recv_metadata.size(0));
            g.args.ldo = L.hidden;
            if (a.size(0) == 0) return;
            const int grid = max_ctas > 0 ? std::min<int>(g.grid, int(max_ctas)) : g.grid;
            PeerWindow::launches += 1;
            cudaError_t e;
            if (pair) {
                const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
                e = gemm::launch_pair(g.map_a, g.map_b, g.args, gemm::kScatter, max_ctas > 0 ? std::min<int>(sms, int(max_ctas)) : sms,
                                      c10::cuda::getCurrentCUDAStream().stream());
            } else {
                e = gemm::launch(g.map_a, g.map_b, g.args, gemm::kScatter, 3, grid, c10::cuda::getCurrentCUDAStream().stream());
            }
            TORCH_CHECK(e == cudaSuccess, "grouped GEMM (scatter) launch failed: ", cudaGetErrorString(e));
        },
        pybind11::arg("window"), pybind11::arg("a"), pybind11::arg("w"), pybind11::arg("expert_offsets"),
        pybind11::arg("slot_map"), pybind11::arg("recv_metadata"), pybind11::arg("slot_weights"), pybind11::arg("status"),
        pybind11::arg("max_ctas") = 0, pybind11::arg("timeout_s") = 5.0, pybind11::arg("pair") = true);

    m.def("gemm_kernel_registers", [](int64_t mode) { return gemm::kernel_registers(int(mode)); });
    m.def("gemm_shared_bytes", [](int64_t mode, int64_t stages) { return int64_t(gemm::shared_bytes(int(mode), int(stages))); });
}

}  // namespace nep
